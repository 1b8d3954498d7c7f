// VQ linear layer:  y[b,m] = (sum_g LUT_b[g, codes[m,g]]) * scales[m] (+ bias[m]) + CSR row m . x_b
// Replaces SplitManifoldLinear::forward_cpu + forward_outliers_cpu
// (split_manifold_lut_experiment/native/src/ojasx_lut_cpu.cpp:104-206) and the three kernels of
// split_manifold_lut_experiment/native/src/ojasx_lut_cuda.cu:28-162 with one persistent kernel:
// table build, code gather and CSR outlier add all happen in the CTA that owns the rows, and y
// is written once.
#include "lut_core.cuh"
#include "lut_chain.cuh"
#include "launch.h"
#include "handles.h"
#include "peer.cuh"

#include <cstdlib>

namespace ojx {

__device__ __forceinline__ const LinearProblem& find_problem(const LinearProblem* probs, int nprobs, int item) {
    int lo = 0, hi = nprobs - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (probs[mid].item_begin <= item) lo = mid; else hi = mid - 1;
    }
    return probs[lo];
}

constexpr int kChainMinRows = 32 * kWarps;

template <int D>
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
lut_linear_kernel(const LinearProblem* __restrict__ probs, int nprobs, int total_items,
                  const __grid_constant__ LinearProblem single, int chain_walk, const __grid_constant__ PeerLink link) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    CoreSmem& sm = *reinterpret_cast<CoreSmem*>(smem_raw);

    for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
        const LinearProblem P = probs ? find_problem(probs, nprobs, item) : single;
        const int local = item - P.item_begin;
        const int b = local / P.tiles, t = local - b * P.tiles;
        const int r0 = P.row_start + t * P.tile_rows;
        const int n = min(P.tile_rows, P.row_stop - r0);
        const int rows_out = P.row_stop - P.row_start;
        const size_t esz = P.io_dtype == OJX_BF16 ? 2 : 4;

        RowSet rs;
        rs.base0 = P.codes + (size_t)r0 * P.G;
        rs.base1 = rs.base0;
        rs.n0 = n;
        rs.n = n;
        rs.G = P.G;
        rs.aligned = ((P.G & 15) == 0) && ((reinterpret_cast<uintptr_t>(P.codes) & 15) == 0);
        const XLoad xl{static_cast<const char*>(P.x) + (size_t)b * P.K * esz, P.K, P.io_dtype};

        // Lanes share a row (conflict-free gathers) whenever the code rows split into 16-byte pieces.
        bool chain = false;
        // (a chain needs 31 steps to fill and drain per slice: below 32 rows per warp the row-per-lane walk wins)
        if constexpr (D <= 16) chain = chain_walk && n >= kChainMinRows && ChainWalker<D>::usable(smem_raw, rs.base0, P.codebook, P.G);
        float* accp = sm.acc;
        float* area = sm.lut;
        int* rp = reinterpret_cast<int*>(sm.ring);
        if constexpr (D <= 16) {
            if (chain) {
                const ChainWalker<D> cw(smem_raw, rs.base0, n, P.G);
                accp = cw.acc();
                area = cw.table();
                rp = cw.ring_hi_ints();
            }
        }
        // A work item that took the shared-row walk ends without a barrier (its warps finish their rows on their
        // own); the next one starts with loads into registers and meets the others at its first table build.
        // Anything that writes shared memory earlier than that waits here for the slower warps.
        if (!chain || P.G == 0) __syncthreads();
        if (P.G == 0)
            for (int lr = threadIdx.x; lr < n; lr += kThreads) accp[lr] = 0.0f;
        // (Asking L2 for the outlier arrays ahead of the epilogue was measured and costs 5 %: with the code stream
        // running close to the DRAM limit the lines are gone again before they are used.)
        auto ask_l2 = [&]() {};
        // With the shared-row walk every warp streams the outlier entries of its own rows in the epilogue; where they
        // begin and end is read under the last walk.
        int jbw = 0, jew = 0;
        bool stream = false;
        if constexpr (D <= 16) {
            if (chain) {
                const ChainWalker<D> cw(smem_raw, rs.base0, n, P.G);
                stream = P.csr.nnz > 0 && P.K <= kCsrXFloats && ChainWalker<D>::stream_ok(P.csr);
                auto entry_range = [&]() {
                    if (stream && cw.warp_row_count() > 0) {
                        jbw = P.csr.row_ptrs[r0 + cw.warp_first_row()];
                        jew = P.csr.row_ptrs[r0 + cw.warp_first_row() + cw.warp_row_count()];
                    }
                };
                cw.run(xl, P.codebook, P.Kcb, entry_range);
                if (cw.nslices == 0) entry_range();
            }
            else RowWalker<D>(sm, rs).run(xl, P.codebook, P.Kcb, ask_l2);
        } else {
            RowWalker<D>(sm, rs).run(xl, P.codebook, P.Kcb, ask_l2);
        }
        __syncthreads();

        // Epilogue (ojasx_lut_cpu.cpp:178-182 then :117-127): scale, bias, outlier row, one store.
        // With a link the result also goes to the same place in every other rank's copy of the output buffer
        // (the all-gather of a row-split layer, fused into the epilogue).
        auto store_y = [&](int m, float res) {
            const size_t o = P.y_full ? (size_t)b * P.y_ld + m : (size_t)b * rows_out + (m - P.row_start);
            if (P.io_dtype == OJX_BF16) peer_store(link, reinterpret_cast<__nv_bfloat16*>(P.y) + o, __float2bfloat16_rn(res));
            else peer_store(link, reinterpret_cast<float*>(P.y) + o, res);
        };
        if constexpr (D <= 16) {
            if (chain) {
                // every warp finishes the rows it walked; only the staging of x needs the whole CTA
                const ChainWalker<D> cw(smem_raw, rs.base0, n, P.G);
                const float* xsm = nullptr;
                if (P.csr.nnz > 0 && P.K <= kCsrXFloats) {
                    float* xw = cw.epilogue_x();
                    for (int k = threadIdx.x; k < P.K; k += kThreads) xw[k] = xl(k);
                    __syncthreads();
                    xsm = xw;
                }
                if (stream) cw.warp_epilogue_stream(P.csr, r0, P.scales, P.bias, xsm, jbw, jew, store_y);
                else cw.warp_epilogue(P.csr, r0, P.scales, P.bias, xsm, xl, store_y);
                continue;
            }
        }
        if (P.csr.nnz > 0) csr_rows_to_area(area, rp, P.csr, r0, n, 0, xl);
        for (int lr = threadIdx.x; lr < n; lr += kThreads) {
            const int m = r0 + lr;
            float res = accp[lr];
            if (P.scales) res = __fmul_rn(res, P.scales[m]);
            if (P.bias) res = __fadd_rn(res, P.bias[m]);
            if (P.csr.nnz > 0) res = __fadd_rn(res, area[lr]);
            store_y(m, res);
        }
        __syncthreads();
    }
    peer_signal_when_last(link, gridDim.x);
}

using LinearKernel = void (*)(const LinearProblem*, int, int, const LinearProblem, int, const PeerLink);

static LinearKernel pick_linear_kernel(int D) {
    switch (D) {
        case 4: return lut_linear_kernel<4>;
        case 8: return lut_linear_kernel<8>;
        case 16: return lut_linear_kernel<16>;
        case 32: return lut_linear_kernel<32>;
        default: return nullptr;
    }
}

static int prepare_kernel(LinearKernel k) {
    // Opt in to the large dynamic shared-memory carve-out once per kernel per device.
    static thread_local LinearKernel done[8] = {};
    static thread_local int done_dev[8] = {};
    int dev = 0;
    OJX_CUDA_TRY(cudaGetDevice(&dev));
    for (int i = 0; i < 8; ++i)
        if (done[i] == k && done_dev[i] == dev + 1) return OJX_OK;
    OJX_CUDA_TRY(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(CoreSmem)));
    for (int i = 0; i < 8; ++i)
        if (done[i] == nullptr) { done[i] = k; done_dev[i] = dev + 1; break; }
    return OJX_OK;
}

int plan_tile_rows(int rows, int parallel_items) {
    // Spread one problem over the SMs when it is alone; otherwise keep tiles large so the table
    // build (replicated per tile) is amortised over many rows.
    const int sms = kCtasPerSm * num_sms();
    int tiles_wanted = sms / (parallel_items > 0 ? parallel_items : 1);
    if (tiles_wanted < 1) tiles_wanted = 1;
    int tr = round_up((rows + tiles_wanted - 1) / tiles_wanted, 32);
    if (tr < 32) tr = 32;
    if (tr > kAccRows) tr = kAccRows;
    return tr;
}

// OJASX_B200_LINEAR_KERNEL=persistent keeps single problems on the persistent kernel (used by
// the tests to cover both kernels on the same inputs).
static bool force_persistent() {
    const char* e = getenv("OJASX_B200_LINEAR_KERNEL");
    return e && e[0] == 'p';
}
bool linear_cluster_disabled() { return force_persistent(); }

// OJASX_B200_LINEAR_WALK=rows keeps the walk that gives every lane a row of its own (RowWalker).
static int chain_walk_enabled() {
    const char* e = getenv("OJASX_B200_LINEAR_WALK");
    return !(e && e[0] == 'r');
}

int validate_linear(const LinearProblem& P) {
    if (!P.codes || !P.codebook || !P.x || !P.y) return OJX_ERR_ARG;
    if (P.batch <= 0 || P.K <= 0 || P.G < 0 || P.row_stop <= P.row_start || P.row_start < 0) return OJX_ERR_ARG;
    if (P.Kcb <= 0 || P.Kcb > 256) return OJX_ERR_UNSUPPORTED;
    if (!pick_linear_kernel(P.D)) return OJX_ERR_UNSUPPORTED;
    if (P.csr.nnz > 0 && (!P.csr.row_ptrs || !P.csr.cols || !P.csr.vals)) return OJX_ERR_ARG;
    return OJX_OK;
}

int launch_linear(LinearProblem P, cudaStream_t stream, const PeerLink* link) {
    int rc = validate_linear(P);
    if (rc != OJX_OK) return rc;
    const PeerLink none{};
    const PeerLink& L = link ? *link : none;
    const int rows = P.row_stop - P.row_start;
    if (P.tile_rows <= 0 && !force_persistent()) {
        // Small single problems: the cluster kernel spreads the table build over the GPU.
        rc = try_launch_linear_cluster(P, stream, link);
        if (rc != OJX_ERR_UNSUPPORTED) return rc;
    }
    if (P.tile_rows <= 0) P.tile_rows = plan_tile_rows(rows, P.batch);
    P.tiles = (rows + P.tile_rows - 1) / P.tile_rows;
    P.item_begin = 0;
    const int total = P.tiles * P.batch;
    LinearKernel k = pick_linear_kernel(P.D);
    rc = prepare_kernel(k);
    if (rc != OJX_OK) return rc;
    const int cap = kCtasPerSm * num_sms();
    const int grid = total < cap ? total : cap;
    k<<<grid, kThreads, sizeof(CoreSmem), stream>>>(nullptr, 0, total, P, chain_walk_enabled(), L);
    count_launch(1);
    OJX_CUDA_TRY(cudaGetLastError());
    return OJX_OK;
}

int launch_linear_group(const LinearProblem* d_probs, int nprobs, int total_items, int D, cudaStream_t stream,
                        const PeerLink* link) {
    if (!d_probs || nprobs <= 0 || total_items <= 0) return OJX_ERR_ARG;
    LinearKernel k = pick_linear_kernel(D);
    if (!k) return OJX_ERR_UNSUPPORTED;
    int rc = prepare_kernel(k);
    if (rc != OJX_OK) return rc;
    const int cap = kCtasPerSm * num_sms();
    const int grid = total_items < cap ? total_items : cap;
    LinearProblem dummy{};
    const PeerLink none{};
    k<<<grid, kThreads, sizeof(CoreSmem), stream>>>(d_probs, nprobs, total_items, dummy, chain_walk_enabled(), link ? *link : none);
    count_launch(1);
    OJX_CUDA_TRY(cudaGetLastError());
    return OJX_OK;
}

}  // namespace ojx
