// Latency-oriented VQ linear for ONE small problem (decode-time layers: a few thousand rows,
// batch of a few tokens), where the persistent kernel of linear.cu would spend most of its time
// rebuilding the whole lookup table in every CTA.
//
// A thread-block cluster of C CTAs shares one tile of rows.  CTA s of the cluster owns a slice of
// the group axis: it builds only that slice of the table (so each table entry is built by
// n_clusters CTAs instead of by every CTA), gathers LUT[g, code[row, g]] for all rows of the tile
// and its groups, and sends each gathered value straight into the shared memory of the CTA that
// owns the row (st.shared::cluster, distributed shared memory).  After one cluster barrier every
// CTA holds, for its rows, the G gathered values in group order and adds them with one fp32
// accumulator per row, g ascending -- the reference's order (ojasx_lut_cpu.cpp:161-175) -- then
// applies scale, bias and the CSR outlier row sum.  Results are bit-identical to linear.cu.
#include "lut_core.cuh"
#include "launch.h"
#include "handles.h"
#include "peer.cuh"

namespace ojx {


constexpr int kClThreads = 512;
constexpr int kClProd = 2048;   // CSR products staged per pass

struct ClusterPlan {
    int C;        // CTAs per cluster
    int cpc;      // 16-group chunks per CTA
    int R;        // rows per tile (multiple of 32); the largest of the problems' tiles in a grouped launch
    int RO;       // rows of a tile owned by one CTA for the ordered sum (of the largest tile)
    int stride;   // bytes per staged code row (odd multiple of 16: conflict-free 128-bit reads)
    int n_tiles;
    int n_clusters;
    size_t smem;
};

// Up to kClMaxGroup problems with the same K, G, block_dim and batch in one launch (q/k/v of an attention
// block, gate/up of an MLP): every cluster works on one problem, clusters [first[p], first[p+1]) on
// problem p with that problem's own tile size.  Passed by value, so a launch needs no device-side table.
constexpr int kClMaxGroup = 8;
struct ClusterGroup {
    LinearProblem P[kClMaxGroup];
    int first[kClMaxGroup + 1];
    int R[kClMaxGroup], RO[kClMaxGroup], n_tiles[kClMaxGroup];
    int count;
};

__device__ __forceinline__ unsigned cluster_ctarank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ unsigned mapa_shared(unsigned addr, unsigned rank) {
    unsigned r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_cluster_v4(unsigned addr, float a, float b, float c, float d) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <int D>
__global__ void __launch_bounds__(kClThreads, 1)
lut_linear_cluster_kernel(const __grid_constant__ ClusterGroup grp, const __grid_constant__ ClusterPlan plan,
                          const __grid_constant__ PeerLink link) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int C = plan.C;
    const int cid_all = blockIdx.x / C;
    int pi = 0;
    while (pi + 1 < grp.count && cid_all >= grp.first[pi + 1]) ++pi;   // same for every CTA of a cluster
    const LinearProblem& P = grp.P[pi];
    const int G = P.G, RO = grp.RO[pi], R = grp.R[pi], n_tiles = grp.n_tiles[pi];
    const int n_clusters = grp.first[pi + 1] - grp.first[pi];
    const int ngp = plan.cpc * 16;                                       // groups of a full slice
    float* lut = reinterpret_cast<float*>(smem_raw);                     // [ngp][256]
    const int Gp = G + 4;                                                // padded row of gathered values
    float* recv = lut + (size_t)ngp * 256;                               // [plan.RO][Gp]
    uint8_t* codes_s = reinterpret_cast<uint8_t*>(recv + (size_t)Gp * plan.RO);  // [plan.R][stride]
    float* xs = reinterpret_cast<float*>(codes_s + (size_t)plan.R * plan.stride);  // [ngp*D]
    float* oacc_s = xs + (size_t)ngp * D;                                          // [plan.RO]
    int* rp_s = reinterpret_cast<int*>(oacc_s + plan.RO);                          // [plan.RO + 1]
    float* prod_s = reinterpret_cast<float*>(rp_s + plan.RO + 1);                  // [kClProd]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int rank = (int)cluster_ctarank();
    const int cid = cid_all - grp.first[pi];
    const int b = blockIdx.y;
    const int g0 = rank * ngp;
    const int ng = max(0, min(G, g0 + ngp) - g0);
    const int rows_out = P.row_stop - P.row_start;
    const size_t esz = P.io_dtype == OJX_BF16 ? 2 : 4;
    const XLoad xl{static_cast<const char*>(P.x) + (size_t)b * P.K * esz, P.K, P.io_dtype};
    const unsigned recv_addr = static_cast<unsigned>(__cvta_generic_to_shared(recv));

    auto stage_codes = [&](int tile) {
        const int r0 = P.row_start + tile * R;
        const int nR = min(R, P.row_stop - r0);
        const int ppr = ng >> 4;  // 16-byte pieces per row
        for (int i = tid; i < nR * ppr; i += kClThreads) {
            const int row = i / ppr, c = i - row * ppr;
            cp_async16(codes_s + (size_t)row * plan.stride + c * 16, P.codes + (size_t)(r0 + row) * G + g0 + c * 16, 16);
        }
        cp_async_commit();
    };

    // CSR outlier sums of the rows this CTA owns in `tile` (reference order,
    // ojasx_lut_cpu.cpp:117-126).  The entries of those rows are contiguous: all threads load
    // (col, val) coalesced and multiply in parallel into shared memory, then one thread per row
    // adds its products in entry order -- three memory round trips whatever the row count.  It
    // depends only on x, so it runs while the tile's code bytes are still in flight.
    auto outlier_sums = [&](int tile) {
        if (P.csr.nnz <= 0) return;
        const int r0 = P.row_start + tile * R;
        const int nR = min(R, P.row_stop - r0);
        const int first = rank * RO;
        const int mine = max(0, min(RO, nR - first));
        for (int i = tid; i <= mine; i += kClThreads) rp_s[i] = mine > 0 ? P.csr.row_ptrs[r0 + first + i] : 0;
        __syncthreads();
        const int jb = rp_s[0], je = rp_s[mine];
        float acc = 0.0f;
        for (int jc = jb; jc < je; jc += kClProd) {
            const int ce = min(jc + kClProd, je);
            for (int j = jc + tid; j < ce; j += kClThreads) prod_s[j - jc] = __fmul_rn(P.csr.vals[j], xl(P.csr.cols[j]));
            __syncthreads();
            if (tid < mine) {
                const int s = max(rp_s[tid], jc), e = min(rp_s[tid + 1], ce);
                for (int j = s; j < e; ++j) acc = __fadd_rn(acc, prod_s[j - jc]);
            }
            __syncthreads();
        }
        if (tid < mine) oacc_s[tid] = acc;
    };

    int tile = cid;
    if (tile < n_tiles) {
        stage_codes(tile);
        outlier_sums(tile);
    }

    // table slice for my groups (same arithmetic as RowWalker::build_slice)
    for (int i = tid; i < ng * D; i += kClThreads) xs[i] = xl(g0 * D + i);
    __syncthreads();
    {
        const int kc = tid & 255;
        float c[D];
#pragma unroll
        for (int d = 0; d < D; ++d) c[d] = kc < P.Kcb ? P.codebook[kc * D + d] : 0.0f;
        for (int gl = tid >> 8; gl < ng; gl += kClThreads / 256) {
            const float* xg = xs + gl * D;
            float dot = __fmul_rn(xg[0], c[0]);
#pragma unroll
            for (int d = 1; d < D; ++d) dot = __fadd_rn(dot, __fmul_rn(xg[d], c[d]));
            lut[gl * 256 + kc] = kc < P.Kcb ? dot : 0.0f;
        }
    }

    for (; tile < n_tiles; tile += n_clusters) {
        const int r0 = P.row_start + tile * R;
        const int nR = min(R, P.row_stop - r0);
        cp_async_wait<0>();
        __syncthreads();  // codes landed, table built

        // gather: lane = row; every value goes to the CTA that owns the row
        const int nrb = (nR + 31) >> 5;
        for (int rb = warp; rb < nrb; rb += kClThreads / 32) {
            const int lr = rb * 32 + lane;
            if (lr < nR) {
                const int owner = lr / RO, slot = lr - owner * RO;
                const unsigned dst = mapa_shared(recv_addr, (unsigned)owner) + (unsigned)(((size_t)slot * Gp + g0) * 4);
                const uint8_t* row = codes_s + (size_t)lr * plan.stride;
                for (int c16 = 0; c16 < (ng >> 4); ++c16) {
                    const uint4 w = *reinterpret_cast<const uint4*>(row + c16 * 16);
                    const unsigned ws[4] = {w.x, w.y, w.z, w.w};
                    const float* lp = lut + c16 * 16 * 256;
                    float v[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const unsigned code = (ws[j >> 2] >> ((j & 3) * 8)) & 0xffu;
                        v[j] = lp[j * 256 + code];
                    }
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        st_cluster_v4(dst + (unsigned)((c16 * 16 + q * 4) * 4), v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                }
            }
        }
        cluster_sync_all();  // all values of this tile are in their owners' shared memory

        // next tile's codes can stream in while this one is summed (codes_s is no longer read)
        if (tile + n_clusters < n_tiles) stage_codes(tile + n_clusters);

        // ordered sums for my rows of the tile
        const int first = rank * RO;
        const int mine = max(0, min(RO, nR - first));
        float res = 0.0f;
        if (tid < mine) {
            float acc = 0.0f;
            const float4* rp = reinterpret_cast<const float4*>(recv + (size_t)tid * Gp);
            for (int g4 = 0; g4 < (G >> 2); g4 += 4) {  // G is a multiple of 16
                float4 v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) v[u] = rp[g4 + u];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    acc = __fadd_rn(acc, v[u].x);
                    acc = __fadd_rn(acc, v[u].y);
                    acc = __fadd_rn(acc, v[u].z);
                    acc = __fadd_rn(acc, v[u].w);
                }
            }
            const int m = r0 + first + tid;
            res = acc;
            if (P.scales) res = __fmul_rn(res, P.scales[m]);
            if (P.bias) res = __fadd_rn(res, P.bias[m]);
        }
        if (P.csr.nnz > 0 && tid < mine) res = __fadd_rn(res, oacc_s[tid]);
        if (tid < mine) {
            const int m = r0 + first + tid;
            const size_t o = P.y_full ? (size_t)b * P.y_ld + m : (size_t)b * rows_out + (size_t)(m - P.row_start);
            if (P.io_dtype == OJX_BF16) peer_store(link, reinterpret_cast<__nv_bfloat16*>(P.y) + o, __float2bfloat16_rn(res));
            else peer_store(link, reinterpret_cast<float*>(P.y) + o, res);
        }
        __syncthreads();     // oacc_s of this tile has been consumed
        if (tile + n_clusters < n_tiles) outlier_sums(tile + n_clusters);
        cluster_sync_all();  // recv may be overwritten by the next tile; nobody exits while peers may still write
    }
    peer_signal_when_last(link, gridDim.x * gridDim.y);
}

template <int D>
static int launch_cluster_t(const ClusterGroup& grp, ClusterPlan plan, cudaStream_t stream, bool dry_run, const PeerLink& link) {
    auto kern = lut_linear_cluster_kernel<D>;
    // query_max_clusters<D> already opted this kernel in to kClSmemCap bytes of dynamic shared memory on
    // this device (plans never exceed it), so nothing has to be set per launch.
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(kClThreads);
    cfg.dynamicSmemBytes = plan.smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = plan.C;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cfg.gridDim = dim3(plan.C * plan.n_clusters, grp.P[0].batch);
    if (dry_run) return OJX_OK;
    OJX_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, grp, plan, link));
    count_launch(1);
    return OJX_OK;
}

constexpr size_t kClSmemCap = 220 * 1024;

template <int D>
static int query_max_clusters(int C) {
    auto kern = lut_linear_cluster_kernel<D>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kClSmemCap) != cudaSuccess) return 0;
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(kClThreads);
    cfg.dynamicSmemBytes = kClSmemCap;
    cfg.gridDim = dim3(C * 64, 1);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = C;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n;
}

// Clusters of C CTAs (one CTA per SM at this shared-memory size) that can be resident at once;
// a cluster must sit inside one GPC, so this is less than num_sms / C.  Cached per device.
static int max_active_clusters(int D, int C) {
    static int cache[8][4][9] = {};  // [device][D index][C], 0 = unknown, -1 = cannot launch
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 8) dev = 0;
    const int di = D == 4 ? 0 : D == 8 ? 1 : D == 16 ? 2 : 3;
    int& slot = cache[dev][di][C];
    if (slot == 0) {
        int n = D == 4 ? query_max_clusters<4>(C) : D == 8 ? query_max_clusters<8>(C)
              : D == 16 ? query_max_clusters<16>(C) : query_max_clusters<32>(C);
        slot = n > 0 ? n : -1;
    }
    return slot > 0 ? slot : 0;
}

// Picks cluster size, group slice and row tiles for `count` problems that share K, G, block_dim, batch and
// io dtype; returns false when they do not suit this kernel (unaligned code rows, too large a table
// slice, too many rows or problems).  The resident clusters are shared out in proportion to the rows.
static bool plan_cluster_group(const LinearProblem* Ps, int count, ClusterPlan* out, ClusterGroup* grp) {
    if (count <= 0 || count > kClMaxGroup) return false;
    const LinearProblem& P0 = Ps[0];
    long long rows_total = 0;
    for (int p = 0; p < count; ++p) {
        const LinearProblem& P = Ps[p];
        if (P.G != P0.G || P.K != P0.K || P.D != P0.D || P.batch != P0.batch || P.io_dtype != P0.io_dtype || P.Kcb != P0.Kcb) return false;
        if ((P.G & 15) || (reinterpret_cast<uintptr_t>(P.codes) & 15) || P.G == 0 || P.row_stop <= P.row_start) return false;
        rows_total += P.row_stop - P.row_start;
    }
    if (P0.D != 4 && P0.D != 8 && P0.D != 16 && P0.D != 32) return false;
    // Measured on B200 (2560->6912): 12.5 us against 22.7 us for the persistent kernel at batch 1,
    // but 33 us against 24.7 us at batch 4, where the persistent kernel's larger tiles win.
    if (P0.batch > 2 || rows_total * P0.batch > 32768) return false;
    const int TC = P0.G / 16, sms = num_sms();
    double best = 1e30;
    bool found = false;
    for (int C = 1; C <= 8; ++C) {
        ClusterPlan pl{};
        ClusterGroup g{};
        pl.C = C;
        pl.cpc = (TC + C - 1) / C;
        if ((C - 1) * pl.cpc >= TC && C > 1) continue;  // would leave the last CTA without groups
        int resident = max_active_clusters(P0.D, C);
        if (resident <= 0) continue;
        if (resident > sms / C) resident = sms / C;
        const int ncl_max = resident / P0.batch > 0 ? resident / P0.batch : 1;
        if (ncl_max < count) continue;
        pl.stride = pl.cpc * 16 + ((pl.cpc & 1) ? 0 : 16);
        // clusters per problem: proportional to its rows, at least one, at most ncl_max in all
        int ncl[kClMaxGroup], used = 0;
        for (int p = 0; p < count; ++p) {
            const long long rows = Ps[p].row_stop - Ps[p].row_start;
            ncl[p] = (int)std::max<long long>(1, rows * (ncl_max - count) / rows_total + 1);
            used += ncl[p];
        }
        while (used > ncl_max) {   // rounding: take from the problem with the fewest rows per cluster
            int w = -1;
            double least = 1e30;
            for (int p = 0; p < count; ++p) {
                const double per = double(Ps[p].row_stop - Ps[p].row_start) / ncl[p];
                if (ncl[p] > 1 && per < least) { least = per; w = p; }
            }
            if (w < 0) break;
            --ncl[w]; --used;
        }
        if (used > ncl_max) continue;
        int Rmax = 0;
        for (int p = 0; p < count; ++p) {
            const int rows = Ps[p].row_stop - Ps[p].row_start;
            g.R[p] = round_up((rows + ncl[p] - 1) / ncl[p], 32);
            Rmax = std::max(Rmax, g.R[p]);
        }
        for (;;) {   // shrink the largest tiles until the shared memory fits
            pl.R = Rmax;
            pl.RO = (pl.R + C - 1) / C;
            pl.smem = sizeof(float) * ((size_t)pl.cpc * 16 * 256 + (size_t)(P0.G + 4) * pl.RO + (size_t)pl.cpc * 16 * P0.D + 2 * pl.RO + 1 + kClProd) +
                      (size_t)pl.R * pl.stride;
            if (pl.smem <= kClSmemCap || Rmax <= 32) break;
            Rmax -= 32;
        }
        if (pl.smem > kClSmemCap) continue;
        int waves = 1, first = 0;
        for (int p = 0; p < count; ++p) {
            const int rows = Ps[p].row_stop - Ps[p].row_start;
            g.P[p] = Ps[p];
            g.R[p] = std::min(g.R[p], Rmax);
            g.RO[p] = (g.R[p] + C - 1) / C;
            g.n_tiles[p] = (rows + g.R[p] - 1) / g.R[p];
            const int n = std::min(ncl[p], g.n_tiles[p]);
            g.first[p] = first;
            first += n;
            waves = std::max(waves, (g.n_tiles[p] + n - 1) / n);
        }
        g.first[count] = first;
        g.count = count;
        pl.n_clusters = first;
        pl.n_tiles = 0;
        // crude cost in clocks: table slice build + per-tile gather and ordered sum
        const double cost = pl.cpc * 16 * 75.0 + waves * (pl.R * pl.cpc * 16 / 6.0 + P0.G * 6.0 + 1500.0);
        if (cost < best) { best = cost; *out = pl; *grp = g; found = true; }
    }
    return found;
}

static int launch_cluster_group(const ClusterGroup& grp, const ClusterPlan& plan, cudaStream_t stream, const PeerLink* lk) {
    const PeerLink none{};
    const PeerLink& link = lk ? *lk : none;
    switch (grp.P[0].D) {
        case 4: return launch_cluster_t<4>(grp, plan, stream, false, link);
        case 8: return launch_cluster_t<8>(grp, plan, stream, false, link);
        case 16: return launch_cluster_t<16>(grp, plan, stream, false, link);
        case 32: return launch_cluster_t<32>(grp, plan, stream, false, link);
        default: return OJX_ERR_UNSUPPORTED;
    }
}

// Entry used by launch_linear(): returns OJX_ERR_UNSUPPORTED when the caller should fall back
// to the persistent kernel.
int try_launch_linear_cluster(const LinearProblem& P, cudaStream_t stream, const PeerLink* link) {
    ClusterPlan plan;
    ClusterGroup grp;
    if (!plan_cluster_group(&P, 1, &plan, &grp)) return OJX_ERR_UNSUPPORTED;
    return launch_cluster_group(grp, plan, stream, link);
}

// Same for a few problems at once (host copies of the problems; nothing is read from them after
// the call returns).  OJX_ERR_UNSUPPORTED: use the persistent grouped kernel.
int try_launch_linear_cluster_group(const LinearProblem* probs, int count, cudaStream_t stream, const PeerLink* link) {
    ClusterPlan plan;
    ClusterGroup grp;
    if (!plan_cluster_group(probs, count, &plan, &grp)) return OJX_ERR_UNSUPPORTED;
    return launch_cluster_group(grp, plan, stream, link);
}

}  // namespace ojx

