// Top-k MoE over VQ-coded experts: only the routed experts' code rows are read.
// Replaces SplitManifoldMoE::forward_cpu
// (split_manifold_lut_experiment/native/src/ojasx_lut_cpu.cpp:213-365) and adds the router of
// split_manifold_lut_experiment/tools/run_full_48_layers_and_generate.py:172-175.
//
// Stages (all on one stream, no host round trip):
//   router   : logits -> softmax -> top-k -> renormalise           (moe_router_*)
//   gate/up  : per (token, expert) pair and tile of intermediate indices, one table pass over
//              the expert's gate rows and up rows, then inter = silu(gate) * up
//   down     : per pair and tile of hidden rows, table of `inter` against the down codebook
//   combine  : y[t] = sum over the token's pairs in caller order of expert_out * weight
// The combine is a separate ordered pass so that the sum over experts has the reference's
// order whatever SM finished first.
#include <cstdlib>
#include "lut_core.cuh"
#include "lut_chain.cuh"
#include "launch.h"
#include "handles.h"
#include "peer.cuh"
#include "../../include/ojasx_lut_b200.h"

#include <mutex>

namespace ojx {

// silu(v) = v / (1 + exp(-v))  (ojasx_lut_cpu.cpp:209-211).  exp is evaluated in double and
// rounded once, which reproduces a correctly rounded expf in all but ~1e-9 of arguments.
__device__ __forceinline__ float silu_ref(float v) {
    const float e = (float)exp((double)(-v));
    return __fdiv_rn(v, __fadd_rn(1.0f, e));
}

struct MoePair {
    int token, expert;  // expert is the LOCAL expert index, or -1 when the pair is skipped
};

__device__ __forceinline__ MoePair decode_pair(const MoeProblem& P, int pair) {
    MoePair r;
    r.token = pair / P.k_active;
    const int e = P.topk_idx[pair] - P.expert_offset;
    const float w = P.topk_w[pair];
    // ojasx_lut_cpu.cpp:284-286: ids outside the expert table and |w| < 1e-8 are skipped.
    r.expert = (e < 0 || e >= P.E || fabsf(w) < 1e-8f) ? -1 : e;
    return r;
}

template <int D>
__global__ void __launch_bounds__(kThreads, kCtasPerSm) moe_gate_up_kernel(const __grid_constant__ MoeProblem P) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    CoreSmem& sm = *reinterpret_cast<CoreSmem*>(smem_raw);
    const int total = (P.pair_list ? P.pair_list[0] : P.n_tokens * P.k_active) * P.gu_tiles;
    const size_t esz = P.io_dtype == OJX_BF16 ? 2 : 4;
    for (int item = blockIdx.x; item < total; item += gridDim.x) {
        const int slot = item / P.gu_tiles, tile = item - slot * P.gu_tiles;
        const int pair = P.pair_list ? P.pair_list[1 + slot] : slot;
        const MoePair pr = decode_pair(P, pair);
        if (pr.expert < 0) continue;  // uniform across the CTA
        const int i0 = tile * P.gu_tile, n = min(P.gu_tile, P.I - i0);
        const size_t row0 = (size_t)pr.expert * 2 * P.I;
        RowSet rs;
        rs.base0 = P.gu_codes + (row0 + i0) * P.G;
        rs.base1 = P.gu_codes + (row0 + P.I + i0) * P.G;
        rs.n0 = n;
        rs.n = 2 * n;
        rs.G = P.G;
        rs.aligned = ((P.G & 15) == 0) && ((reinterpret_cast<uintptr_t>(P.gu_codes) & 15) == 0);
        const XLoad xl{static_cast<const char*>(P.x) + (size_t)pr.token * P.H * esz, P.H, P.io_dtype};
        RowWalker<D> walker(sm, rs);
        if (walker.nslices == 0)
            for (int lr = threadIdx.x; lr < 2 * n; lr += kThreads) sm.acc[lr] = 0.0f;
        walker.run(xl, P.cb_in, P.Kcb, [&]() {
            if (P.gu_csr.nnz > 0) {
                csr_prefetch_l2(P.gu_csr, (int)(row0 + i0), n);
                csr_prefetch_l2(P.gu_csr, (int)(row0 + P.I + i0), n);
            }
        }, P.lut_in ? P.lut_in + (size_t)pr.token * P.G * 256 : nullptr);
        __syncthreads();
        if (P.gu_csr.nnz > 0) {
            csr_rows_to_smem(sm, P.gu_csr, (int)(row0 + i0), n, 0, xl);
            csr_rows_to_smem(sm, P.gu_csr, (int)(row0 + P.I + i0), n, n, xl);
        }
        for (int lr = threadIdx.x; lr < n; lr += kThreads) {
            const size_t rg = row0 + i0 + lr, ru = row0 + P.I + i0 + lr;
            float gate = sm.acc[lr], up = sm.acc[n + lr];
            if (P.gu_scales) { gate = __fmul_rn(gate, P.gu_scales[rg]); up = __fmul_rn(up, P.gu_scales[ru]); }
            if (P.gu_csr.nnz > 0) {
                gate = __fadd_rn(gate, sm.lut[lr]);
                up = __fadd_rn(up, sm.lut[n + lr]);
            }
            if (P.gate_limit > 0.0f) {
                gate = fminf(gate, P.gate_limit);
                up = fminf(fmaxf(up, -P.gate_limit), P.gate_limit);
            }
            P.inter[(size_t)pair * P.I + i0 + lr] = __fmul_rn(silu_ref(gate), up);
        }
        __syncthreads();
    }
}

template <int D>
__global__ void __launch_bounds__(kThreads, kCtasPerSm) moe_down_kernel(const __grid_constant__ MoeProblem P,
                                                                        const __grid_constant__ PeerLink link) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    CoreSmem& sm = *reinterpret_cast<CoreSmem*>(smem_raw);
    const int total = (P.pair_list ? P.pair_list[0] : P.n_tokens * P.k_active) * P.dn_tiles;
    for (int item = blockIdx.x; item < total; item += gridDim.x) {
        const int slot = item / P.dn_tiles, tile = item - slot * P.dn_tiles;
        const int pair = P.pair_list ? P.pair_list[1 + slot] : slot;
        const MoePair pr = decode_pair(P, pair);
        if (pr.expert < 0) continue;
        const int h0 = tile * P.dn_tile, n = min(P.dn_tile, P.H - h0);
        const size_t row0 = (size_t)pr.expert * P.H;
        RowSet rs;
        rs.base0 = P.dn_codes + (row0 + h0) * P.Gi;
        rs.base1 = rs.base0;
        rs.n0 = n;
        rs.n = n;
        rs.G = P.Gi;
        rs.aligned = ((P.Gi & 15) == 0) && ((reinterpret_cast<uintptr_t>(P.dn_codes) & 15) == 0);
        const XLoad xl{P.inter + (size_t)pair * P.I, P.I, OJX_F32};
        RowWalker<D> walker(sm, rs);
        if (walker.nslices == 0)
            for (int lr = threadIdx.x; lr < n; lr += kThreads) sm.acc[lr] = 0.0f;
        walker.run(xl, P.cb_down, P.Kcb, [&]() { if (P.dn_csr.nnz > 0) csr_prefetch_l2(P.dn_csr, (int)(row0 + h0), n); });
        __syncthreads();
        if (P.dn_csr.nnz > 0) csr_rows_to_smem(sm, P.dn_csr, (int)(row0 + h0), n, 0, xl);
        for (int lr = threadIdx.x; lr < n; lr += kThreads) {
            const size_t r = row0 + h0 + lr;
            float v = sm.acc[lr];
            if (P.dn_scales) v = __fmul_rn(v, P.dn_scales[r]);
            if (P.dn_csr.nnz > 0) v = __fadd_rn(v, sm.lut[lr]);
            peer_store(link, P.expert_out + (size_t)pair * P.H + h0 + lr, v);   // expert-parallel: every rank gets the pair's output
        }
        __syncthreads();
    }
    peer_signal_when_last(link, gridDim.x);
}

// ---- gate/up with the lanes of a warp sharing a row (ChainWalker), for batches where a work item is a whole expert
// (2I rows, gate rows then up rows, contiguous in the code matrix) of one token.  The token's table slices come as
// ready-made images of the table area (moe_chain_prebuild_kernel) through one bulk copy per slice; every warp finishes
// the rows it walked (scale, outlier rows) in place, then inter = silu(gate) * up.  Same bits as moe_gate_up_kernel.
// One work item of the gate/up pass: the routed pair in slot `slot` of the work list (all threads of the CTA; ends
// with a barrier).
template <int D>
__device__ __forceinline__ void moe_gate_up_chain_item(const MoeProblem& P, unsigned char* smem_raw, int slot) {
    const size_t esz = P.io_dtype == OJX_BF16 ? 2 : 4;
    const int nslices = (P.G + ChainWalker<D>::SG - 1) / ChainWalker<D>::SG;
    const int pair = P.pair_list ? P.pair_list[1 + slot] : slot;
    const MoePair pr = decode_pair(P, pair);
    if (pr.expert < 0) return;  // uniform across the CTA
    const int n = 2 * P.I;
    const size_t row0 = (size_t)pr.expert * n;
    const ChainWalker<D> cw(smem_raw, P.gu_codes + row0 * P.G, n, P.G);
    const XLoad xl{static_cast<const char*>(P.x) + (size_t)pr.token * P.H * esz, P.H, P.io_dtype};
    // Everything the epilogue reads from global memory is asked for while the row walk still hides the latency:
    // the token's activations wait in registers, the expert's row pointers in the (idle) activation area behind
    // the copy barrier, the outlier entries and the scales are asked into L2 under the last walk.
    constexpr int kXr = kCsrXFloats / kThreads, kRpMax = kXsFloats - 4;
    const bool has = P.gu_csr.nnz > 0;
    const bool x_regs = has && P.H <= kCsrXFloats, rp_early = has && n + 1 <= kRpMax;
    float xr[kXr];
#pragma unroll
    for (int q = 0; q < kXr; ++q) {
        const int k = threadIdx.x + q * kThreads;
        xr[q] = (x_regs && k < P.H) ? xl(k) : 0.0f;
    }
    int* rp_s = cw.template at<int>(kChXs) + 4;
    int jb = 0, je = 0;
    if (has) { jb = P.gu_csr.row_ptrs[row0]; je = P.gu_csr.row_ptrs[row0 + n]; }
    if (rp_early) {
        for (int b0 = threadIdx.x; b0 <= n; b0 += kThreads * 4) {
            int v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = b0 + u * kThreads <= n ? P.gu_csr.row_ptrs[row0 + b0 + u * kThreads] : 0;
#pragma unroll
            for (int u = 0; u < 4; ++u) if (b0 + u * kThreads <= n) rp_s[b0 + u * kThreads] = v[u];
        }
    }
    cw.run_prebuilt(P.lut_in + (size_t)pr.token * nslices * ChainWalker<D>::kImageFloats, [&]() {
        for (int j = (jb & ~31) + threadIdx.x * 32; j < je; j += kThreads * 32) {
            asm volatile("prefetch.global.L2 [%0];" ::"l"(P.gu_csr.cols + j));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(P.gu_csr.vals + j));
        }
        if (has && !rp_early)
            for (int r = threadIdx.x * 32; r <= n; r += kThreads * 32) asm volatile("prefetch.global.L2 [%0];" ::"l"(P.gu_csr.row_ptrs + row0 + r));
        if (P.gu_scales)
            for (int r = threadIdx.x * 32; r < n; r += kThreads * 32) asm volatile("prefetch.global.L2 [%0];" ::"l"(P.gu_scales + row0 + r));
    });   // ends with a barrier: the table area is scratch now
    const float* xsm = nullptr;
    if (x_regs) {
        float* xw = cw.epilogue_x();
#pragma unroll
        for (int q = 0; q < kXr; ++q) {
            const int k = threadIdx.x + q * kThreads;
            if (k < P.H) xw[k] = xr[q];
        }
        __syncthreads();
        xsm = xw;
    }
    float* acc = cw.acc();
    cw.warp_epilogue(P.gu_csr, (int)row0, P.gu_scales, nullptr, xsm, xl, [&](int m, float res) { acc[m - (int)row0] = res; }, rp_early ? rp_s : nullptr);
    __syncthreads();
    for (int i = threadIdx.x; i < P.I; i += kThreads) {
        float gate = acc[i], up = acc[P.I + i];
        if (P.gate_limit > 0.0f) {
            gate = fminf(gate, P.gate_limit);
            up = fminf(fmaxf(up, -P.gate_limit), P.gate_limit);
        }
        P.inter[(size_t)pair * P.I + i] = __fmul_rn(silu_ref(gate), up);
    }
    __syncthreads();   // the sums are parked again by the next work item
}

template <int D>
__global__ void __launch_bounds__(kThreads, kCtasPerSm) moe_gate_up_chain_kernel(const __grid_constant__ MoeProblem P) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int total = P.pair_list ? P.pair_list[0] : P.n_tokens * P.k_active;
    if (!ChainWalker<D>::usable(smem_raw, P.gu_codes, P.cb_in, P.G)) {   // checked on the host as far as it can be; the
        if (threadIdx.x == 0) atomicExch(&g_bulk_copy_timeout, 2);      // shared-memory base only shows here
        return;
    }
    for (int slot = blockIdx.x; slot < total; slot += gridDim.x) moe_gate_up_chain_item<D>(P, smem_raw, slot);
}

// ---- down projection of a routed pair by the chain walk: the pair's table is built in the kernel from its
// intermediate vector (it is the pair's own, so nothing can be shared), all H rows of the expert are one work item.
// Same bits as moe_down_kernel.
template <int D>
__device__ __forceinline__ void moe_down_chain_item(const MoeProblem& P, const PeerLink& link, unsigned char* smem_raw, int slot) {
    const int pair = P.pair_list ? P.pair_list[1 + slot] : slot;
    const MoePair pr = decode_pair(P, pair);
    if (pr.expert < 0) return;
    const int n = P.H;
    const size_t row0 = (size_t)pr.expert * n;
    const ChainWalker<D> cw(smem_raw, P.dn_codes + row0 * P.Gi, n, P.Gi);
    const XLoad xl{P.inter + (size_t)pair * P.I, P.I, OJX_F32};
    // what the epilogue reads from global memory is asked for before the walk (see moe_gate_up_chain_kernel); the
    // row pointers wait behind the parked sums
    constexpr int kXr = 4;
    const bool has = P.dn_csr.nnz > 0;
    const int rp_off = (n + 3) & ~3;
    const bool x_regs = has && P.I <= kXr * kThreads, rp_early = has && rp_off + n + 1 <= kAccRows;
    float xr[kXr];
#pragma unroll
    for (int q = 0; q < kXr; ++q) {
        const int k = threadIdx.x + q * kThreads;
        xr[q] = (x_regs && k < P.I) ? xl(k) : 0.0f;
    }
    int* rp_s = reinterpret_cast<int*>(cw.acc() + rp_off);
    int jb = 0, je = 0;
    if (has) { jb = P.dn_csr.row_ptrs[row0]; je = P.dn_csr.row_ptrs[row0 + n]; }
    if (rp_early) {
        for (int b0 = threadIdx.x; b0 <= n; b0 += kThreads * 4) {
            int v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = b0 + u * kThreads <= n ? P.dn_csr.row_ptrs[row0 + b0 + u * kThreads] : 0;
#pragma unroll
            for (int u = 0; u < 4; ++u) if (b0 + u * kThreads <= n) rp_s[b0 + u * kThreads] = v[u];
        }
    }
    cw.run(xl, P.cb_down, P.Kcb, [&]() {
        for (int j = (jb & ~31) + threadIdx.x * 32; j < je; j += kThreads * 32) {
            asm volatile("prefetch.global.L2 [%0];" ::"l"(P.dn_csr.cols + j));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(P.dn_csr.vals + j));
        }
        if (has && !rp_early)
            for (int r = threadIdx.x * 32; r <= n; r += kThreads * 32) asm volatile("prefetch.global.L2 [%0];" ::"l"(P.dn_csr.row_ptrs + row0 + r));
        if (P.dn_scales)
            for (int r = threadIdx.x * 32; r < n; r += kThreads * 32) asm volatile("prefetch.global.L2 [%0];" ::"l"(P.dn_scales + row0 + r));
    });
    __syncthreads();   // walks over: the table area is scratch now
    const float* xsm = nullptr;
    if (has && P.I <= kCsrXFloats) {
        float* xw = cw.epilogue_x();
        if (x_regs) {
#pragma unroll
            for (int q = 0; q < kXr; ++q) {
                const int k = threadIdx.x + q * kThreads;
                if (k < P.I) xw[k] = xr[q];
            }
        } else {
            for (int k = threadIdx.x; k < P.I; k += kThreads) xw[k] = xl(k);
        }
        __syncthreads();
        xsm = xw;
    }
    float* out = P.expert_out + (size_t)pair * P.H;
    cw.warp_epilogue(P.dn_csr, (int)row0, P.dn_scales, nullptr, xsm, xl,
                     [&](int m, float res) { peer_store(link, out + (m - (int)row0), res); },   // expert-parallel: every rank gets the pair's output
                     rp_early ? rp_s : nullptr);
    __syncthreads();   // the next work item parks row pointers and sums again
}

template <int D>
__global__ void __launch_bounds__(kThreads, kCtasPerSm) moe_down_chain_kernel(const __grid_constant__ MoeProblem P,
                                                                              const __grid_constant__ PeerLink link) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int total = P.pair_list ? P.pair_list[0] : P.n_tokens * P.k_active;
    const bool usable = ChainWalker<D>::usable(smem_raw, P.dn_codes, P.cb_down, P.Gi);
    if (!usable && threadIdx.x == 0) atomicExch(&g_bulk_copy_timeout, 2);
    for (int slot = blockIdx.x; usable && slot < total; slot += gridDim.x) moe_down_chain_item<D>(P, link, smem_raw, slot);
    peer_signal_when_last(link, gridDim.x);
}

// ---- both passes in one launch.  With a few routed pairs per CTA (32 tokens on one GPU, or a shard of an
// expert-parallel layer) two launches cost a rounded-up wave each: 320 pairs on 148 CTAs are three waves of gate/up and
// three of down where 4.3 would do.  Here the CTAs claim work items from one counter: first every pair's gate/up, then
// every pair's down, which waits (bounded) for the flag its gate/up item raised.  A down item is claimed only after
// all gate/up items have been claimed by CTAs that are running and never wait themselves, so the wait always ends.
// ctl[0] = claim counter, ctl[1 + slot] = "intermediate vector of the slot is written"; moe_plan_kernel zeroes both.
constexpr int kMoeFlagSpin = 1 << 22;
template <int D>
__global__ void __launch_bounds__(kThreads, kCtasPerSm) moe_experts_chain_kernel(const __grid_constant__ MoeProblem P,
                                                                                 const __grid_constant__ PeerLink link) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    // (no static shared memory: the walker needs the dynamic area at its fixed address; between two work items all of
    // it is free, so the claimed item is handed round through its first word)
    volatile int* s_item = reinterpret_cast<volatile int*>(smem_raw);
    const int total = P.pair_list[0];
    int* ctl = const_cast<int*>(P.chain_ctl);
    const bool usable = ChainWalker<D>::usable(smem_raw, P.gu_codes, P.cb_in, P.G) && ChainWalker<D>::usable(smem_raw, P.dn_codes, P.cb_down, P.Gi);
    if (!usable && threadIdx.x == 0) atomicExch(&g_bulk_copy_timeout, 2);
    while (usable) {
        if (threadIdx.x == 0) *s_item = atomicAdd(&ctl[0], 1);
        __syncthreads();
        const int item = *s_item;
        __syncthreads();   // everyone has read the claim before it is overwritten
        if (item >= 2 * total) break;
        if (item < total) {
            moe_gate_up_chain_item<D>(P, smem_raw, item);   // ends with a barrier: the intermediate vector is written
            if (threadIdx.x == 0) {
                __threadfence();
                asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(ctl + 1 + item), "r"(1) : "memory");
            }
        } else {
            const int slot = item - total;
            if (threadIdx.x == 0) {
                int seen = 0;
                for (int i = 0; i < kMoeFlagSpin && !seen; ++i) {
                    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(ctl + 1 + slot) : "memory");
                    if (!seen) __nanosleep(64);
                }
                if (!seen) atomicExch(&g_bulk_copy_timeout, 4);
            }
            __syncthreads();
            moe_down_chain_item<D>(P, link, smem_raw, slot);
        }
    }
    peer_signal_when_last(link, gridDim.x);
}

// Table slices of one activation vector as images of the chain walk's table area: image[s][h][k][jl][l] =
// <x[group s*SG + 4*l' + 2*h + jl], cb[k]> with l' = l, or l & 15 when the slice has at most 64 groups (stored twice).
// Arithmetic of RowWalker::build_slice (d ascending, separate multiply and add).  grid = (slices, vectors), 256
// threads: thread = (k half, h, jl, l); 32 lanes write 128 contiguous bytes per centroid.
template <int D>
__global__ void __launch_bounds__(256) moe_chain_prebuild_kernel(const void* __restrict__ x, int io_dtype, int K, int G,
                                                                 const float* __restrict__ codebook, int Kcb,
                                                                 float* __restrict__ out) {
    constexpr int SG = ChainWalker<D>::SG;
    __shared__ float cb_s[256 * D];
    const int s = blockIdx.x, t = blockIdx.y, nsl = gridDim.x;
    const int g0 = s * SG, ng = min(SG, G - g0);
    const size_t esz = io_dtype == OJX_BF16 ? 2 : 4;
    const XLoad xl{static_cast<const char*>(x) + (size_t)t * K * esz, K, io_dtype};
    for (int i = threadIdx.x; i < 256 * D; i += 256) cb_s[i] = (i / D) < Kcb ? codebook[i] : 0.0f;
    const int l = threadIdx.x & 31, jl = (threadIdx.x >> 5) & 1, h = (threadIdx.x >> 6) & 1, khalf = threadIdx.x >> 7;
    const int lpos = ng <= 64 ? (l & 15) : l;
    const int gl = 4 * lpos + 2 * h + jl;
    const bool mine = gl < ng;
    float xg[D];
#pragma unroll
    for (int d = 0; d < D; ++d) xg[d] = mine ? xl((g0 + gl) * D + d) : 0.0f;
    __syncthreads();
    float* img = out + ((size_t)t * nsl + s) * ChainWalker<D>::kImageFloats + (size_t)h * 16384 + jl * 32 + l;
    for (int k = khalf * 128; k < khalf * 128 + 128; ++k) {
        const float* c = cb_s + k * D;
        float dot = __fmul_rn(xg[0], c[0]);
#pragma unroll
        for (int d = 1; d < D; ++d) dot = __fadd_rn(dot, __fmul_rn(xg[d], c[d]));
        img[(size_t)k * 64] = (mine && k < Kcb) ? dot : 0.0f;
    }
}

// Work list of one forward: the (token, expert) pairs this handle evaluates -- expert held here,
// |w| >= 1e-8 -- grouped by expert so that pairs of one expert run close together in time and
// share its code rows in L2, and so that every CTA of the expert kernels gets real work (with
// expert-parallel shards most routed pairs belong to other ranks).  One CTA; a counting sort on
// the local expert id.  list[0] = count, list[1..] = pair ids.
__global__ void __launch_bounds__(1024) moe_plan_kernel(const __grid_constant__ MoeProblem P, int* __restrict__ list) {
    extern __shared__ int plan_smem[];
    int* cnt = plan_smem;          // [E] pairs per local expert
    int* start = plan_smem + P.E;  // [E] next free slot of the expert
    __shared__ int warp_tot[32];
    const int pairs = P.n_tokens * P.k_active;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    for (int e = threadIdx.x; e < P.E; e += blockDim.x) cnt[e] = 0;
    if (P.chain_ctl)   // claim counter and flags of the one-launch expert pass
        for (int i = threadIdx.x; i <= pairs; i += blockDim.x) const_cast<int*>(P.chain_ctl)[i] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = decode_pair(P, p).expert;
        if (e >= 0) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    // exclusive prefix: each thread owns a contiguous run of experts; warp-shuffle scans join the runs
    const int per = (P.E + (int)blockDim.x - 1) / (int)blockDim.x;
    const int lo = min(P.E, (int)threadIdx.x * per), hi = min(P.E, lo + per);
    int run = 0;
    for (int e = lo; e < hi; ++e) run += cnt[e];
    int inc = run;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, inc, off);
        if (lane >= off) inc += v;
    }
    if (lane == 31) warp_tot[wid] = inc;
    __syncthreads();
    if (wid == 0) {
        int t = lane < nwarp ? warp_tot[lane] : 0;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, t, off);
            if (lane >= off) t += v;
        }
        warp_tot[lane] = t;
    }
    __syncthreads();
    int base = inc - run + (wid > 0 ? warp_tot[wid - 1] : 0);
    for (int e = lo; e < hi; ++e) {
        start[e] = base;
        base += cnt[e];
    }
    if (threadIdx.x == 0) list[0] = warp_tot[nwarp - 1];
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = decode_pair(P, p).expert;
        if (e >= 0) list[1 + atomicAdd(&start[e], 1)] = p;
    }
}

// y[t,h] = sum_k expert_out[t*k+k', h] * w  in caller order (ojasx_lut_cpu.cpp:361-362).
__device__ __forceinline__ bool combine_takes(const MoeProblem& P, int pair) {
    if (!P.combine_all) return decode_pair(P, pair).expert >= 0;
    const int e = P.topk_idx[pair];
    return e >= 0 && e < P.E_total && fabsf(P.topk_w[pair]) >= 1e-8f;
}

__global__ void moe_combine_kernel(const __grid_constant__ MoeProblem P, const __grid_constant__ PeerLink link) {
    if (link.n > 0) {   // expert outputs of the other ranks land in expert_out: wait for every rank's flag first
        if (threadIdx.x < 32) peer_wait_warp(link);
        __syncthreads();
    }
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= P.n_tokens * P.H) return;
    const int t = idx / P.H, h = idx - t * P.H;
    float y = 0.0f;
    for (int k0 = 0; k0 < P.k_active; k0 += 8) {  // eight loads in flight, additions in caller order
        float v[8], w[8];
        bool ok[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int k = k0 + u, pair = t * P.k_active + k;
            ok[u] = k < P.k_active && combine_takes(P, pair);
            v[u] = ok[u] ? P.expert_out[(size_t)pair * P.H + h] : 0.0f;
            w[u] = ok[u] ? P.topk_w[pair] : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if (ok[u]) y = __fadd_rn(y, __fmul_rn(v[u], w[u]));
    }
    if (P.io_dtype == OJX_BF16) reinterpret_cast<__nv_bfloat16*>(P.y)[idx] = __float2bfloat16_rn(y);
    else reinterpret_cast<float*>(P.y)[idx] = y;
}

// ------------------------------------------------------------------------------- router
// logit[t,e] with 32 interleaved partial sums and a butterfly combine: lane j owns columns
// j, j+32, ... in ascending order (separate multiply and add), then v += shfl_xor(v, off) for
// off = 16..1.  One warp per expert (its row of W stays hot in L1 while the warp loops over the
// tokens of its blockIdx.y stripe).

// Experts [e_begin, e_end) only (an expert-parallel rank scores the experts it holds); with a link the logits go to
// every rank's copy of the logits buffer.
__device__ __forceinline__ void router_logits_block(const float* __restrict__ Wr, const void* __restrict__ x, int io_dtype,
                                                    int n_tokens, int H, int E, float* __restrict__ logits, int bx, int by,
                                                    int nby, int e_begin, int e_end, const PeerLink& link) {
    const int warp = e_begin + ((bx * 256 + threadIdx.x) >> 5), lane = threadIdx.x & 31;
    if (warp >= e_end) return;
    const float* w = Wr + (size_t)warp * H;
    const size_t esz = io_dtype == OJX_BF16 ? 2 : 4;
    for (int t = by; t < n_tokens; t += nby) {
        const XLoad xl{static_cast<const char*>(x) + (size_t)t * H * esz, H, io_dtype};
        float part = 0.0f;
        int c = lane;
        for (; c + 7 * 32 < H; c += 8 * 32) {  // eight loads in flight, additions still in column order
            float wv[8], xv[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) { wv[u] = w[c + 32 * u]; xv[u] = xl(c + 32 * u); }
#pragma unroll
            for (int u = 0; u < 8; ++u) part = __fadd_rn(part, __fmul_rn(wv[u], xv[u]));
        }
        for (; c < H; c += 32) part = __fadd_rn(part, __fmul_rn(w[c], xl(c)));
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) part = __fadd_rn(part, __shfl_xor_sync(0xffffffffu, part, off));
        if (lane == 0) peer_store(link, logits + (size_t)t * E + warp, part);
    }
}

__global__ void __launch_bounds__(256) moe_router_logits_kernel(const float* __restrict__ Wr, const void* __restrict__ x,
                                                                int io_dtype, int n_tokens, int H, int E,
                                                                float* __restrict__ logits, int e_begin, int e_end,
                                                                const __grid_constant__ PeerLink link) {
    router_logits_block(Wr, x, io_dtype, n_tokens, H, E, logits, blockIdx.x, blockIdx.y, gridDim.y, e_begin, e_end, link);
    peer_signal_when_last(link, gridDim.x * gridDim.y);
}

// Batches: a block scores eight experts (a warp each) for eight tokens at a time from a shared-memory tile of x, so a
// router row is read once per eight tokens instead of once per token.  Every (token, expert) sum is formed exactly as
// in router_logits_block: lane l adds columns l, l + 32, ... in order, then the same butterfly.
constexpr int kLogitTokens = 8, kLogitCols = 512;
__global__ void __launch_bounds__(256) moe_router_logits_tiled_kernel(const float* __restrict__ Wr, const void* __restrict__ x,
                                                                      int io_dtype, int n_tokens, int H, int E,
                                                                      float* __restrict__ logits, int e_begin, int e_end,
                                                                      const __grid_constant__ PeerLink link) {
    __shared__ __align__(16) float xs[kLogitTokens][kLogitCols];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = e_begin + blockIdx.x * 8 + warp, t0 = blockIdx.y * kLogitTokens;
    const bool live = e < e_end;
    const float* w = Wr + (size_t)(live ? e : e_begin) * H;
    const size_t esz = io_dtype == OJX_BF16 ? 2 : 4;
    float acc[kLogitTokens];
#pragma unroll
    for (int tt = 0; tt < kLogitTokens; ++tt) acc[tt] = 0.0f;
    for (int c0 = 0; c0 < H; c0 += kLogitCols) {
        const int nc = min(kLogitCols, H - c0);
        __syncthreads();   // the previous tile has been read
        if (io_dtype == OJX_F32 && (H & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {   // 16-byte pieces
            const float* xf = static_cast<const float*>(x);
            for (int i = threadIdx.x; i < kLogitTokens * kLogitCols / 4; i += 256) {
                const int tt = i / (kLogitCols / 4), j = (i - tt * (kLogitCols / 4)) * 4, t = t0 + tt;
                float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (t < n_tokens && j < nc) v = *reinterpret_cast<const float4*>(xf + (size_t)t * H + c0 + j);
                *reinterpret_cast<float4*>(&xs[tt][j]) = v;
            }
        } else {
            for (int i = threadIdx.x; i < kLogitTokens * kLogitCols; i += 256) {
                const int tt = i / kLogitCols, j = i - tt * kLogitCols, t = t0 + tt;
                float v = 0.0f;
                if (t < n_tokens && j < nc) {
                    const XLoad xl{static_cast<const char*>(x) + (size_t)t * H * esz, H, io_dtype};
                    v = xl(c0 + j);
                }
                xs[tt][j] = v;
            }
        }
        __syncthreads();
        if (live) {
            int cc = lane;
            for (; cc + 3 * 32 < nc; cc += 4 * 32) {   // four router weights in flight, additions still in column order
                float wv[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) wv[u] = __ldg(w + c0 + cc + 32 * u);
#pragma unroll
                for (int u = 0; u < 4; ++u)
#pragma unroll
                    for (int tt = 0; tt < kLogitTokens; ++tt) acc[tt] = __fadd_rn(acc[tt], __fmul_rn(wv[u], xs[tt][cc + 32 * u]));
            }
            for (; cc < nc; cc += 32) {
                const float wv = __ldg(w + c0 + cc);
#pragma unroll
                for (int tt = 0; tt < kLogitTokens; ++tt) acc[tt] = __fadd_rn(acc[tt], __fmul_rn(wv, xs[tt][cc]));
            }
        }
    }
#pragma unroll
    for (int tt = 0; tt < kLogitTokens; ++tt) {
        float part = acc[tt];
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) part = __fadd_rn(part, __shfl_xor_sync(0xffffffffu, part, off));
        if (live && lane == 0 && t0 + tt < n_tokens) peer_store(link, logits + (size_t)(t0 + tt) * E + e, part);
    }
    peer_signal_when_last(link, gridDim.x * gridDim.y);
}

// Router logits and the per-token gate/up tables in one launch: neither depends on the other, both
// depend only on x.  Blocks [0, lx*ly) are logits blocks (bx = b % lx, by = b / lx), the rest build
// tables (16 groups of one token each).
template <int D>
__global__ void __launch_bounds__(256) moe_logits_prebuild_kernel(const float* __restrict__ Wr, const void* __restrict__ x,
                                                                  int io_dtype, int n_tokens, int H, int E,
                                                                  float* __restrict__ logits, int lx, int ly, int G,
                                                                  const float* __restrict__ codebook, int Kcb,
                                                                  float* __restrict__ lut_out, int e_begin, int e_end,
                                                                  const __grid_constant__ PeerLink link) {
    __shared__ float xs[16 * D];
    const int b = blockIdx.x;
    if (b < lx * ly) {
        router_logits_block(Wr, x, io_dtype, n_tokens, H, E, logits, b % lx, b / lx, ly, e_begin, e_end, link);
    } else {
        const int j = b - lx * ly, px = (G + 15) / 16;
        lut_prebuild_block<D>(x, io_dtype, H, G, codebook, Kcb, lut_out, j % px, j / px, xs);
    }
    peer_signal_when_last(link, gridDim.x);
}

// One warp per token: softmax over E logits, k rounds of arg-max (ties to the lower index),
// renormalise.  The probabilities live in the warp's slice of shared memory.  The normaliser and
// the weight sum are accumulated sequentially in fp32 (lane 0), so the result does not depend on
// the thread count; max and arg-max are order-independent.
constexpr int kTopkWarps = 4;

__global__ void __launch_bounds__(kTopkWarps * 32) moe_router_topk_kernel(const float* __restrict__ logits, int n_tokens, int E,
                                                                         int k, int* __restrict__ idx_out,
                                                                         float* __restrict__ w_out,
                                                                         float* __restrict__ probs /* [n_tokens, E] scratch */,
                                                                         const __grid_constant__ PeerLink link) {
    extern __shared__ float topk_smem[];  // [kTopkWarps][E]
    if (link.n > 0) {   // the logits of the other ranks' experts arrive over the link
        if (threadIdx.x < 32) peer_wait_warp(link);
        __syncthreads();
    }
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int t = blockIdx.x * kTopkWarps + wid;
    if (t >= n_tokens) return;
    float* p = topk_smem + (size_t)wid * E;
    const float* l = logits + (size_t)t * E;
    float m = -INFINITY;
    for (int e = lane; e < E; e += 32) { const float v = l[e]; p[e] = v; m = fmaxf(m, v); }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    for (int e = lane; e < E; e += 32) p[e] = (float)exp((double)__fsub_rn(p[e], m));
    __syncwarp();
    float s = 0.0f;
    if (lane == 0)
        for (int e = 0; e < E; ++e) s = __fadd_rn(s, p[e]);
    s = __shfl_sync(0xffffffffu, s, 0);
    for (int e = lane; e < E; e += 32) {
        const float v = __fdiv_rn(p[e], s);
        p[e] = v;
        probs[(size_t)t * E + e] = v;
    }
    __syncwarp();
    float ws = 0.0f;
    for (int r = 0; r < k; ++r) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = p[e];
            if (v > bv) { bv = v; bi = e; }  // ascending e per lane keeps the lowest index on ties
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) {
            idx_out[(size_t)t * k + r] = bi;
            w_out[(size_t)t * k + r] = bv;
            p[bi] = -1.0f;  // taken (probabilities are >= 0)
        }
        ws = __fadd_rn(ws, bv);  // same value in every lane, selection order
        __syncwarp();
    }
    for (int r = lane; r < k; r += 32) w_out[(size_t)t * k + r] = __fdiv_rn(w_out[(size_t)t * k + r], ws);
}

// Same rule for E <= 32 * EPL: a lane keeps its EPL probabilities (experts lane, lane + 32, ...) in
// registers, so the k arg-max rounds touch no memory; only the sequential normaliser goes through
// shared memory.
template <int EPL>
__global__ void __launch_bounds__(kTopkWarps * 32) moe_router_topk_reg_kernel(const float* __restrict__ logits, int n_tokens,
                                                                             int E, int k, int* __restrict__ idx_out,
                                                                             float* __restrict__ w_out,
                                                                             float* __restrict__ probs,
                                                                             const __grid_constant__ PeerLink link) {
    extern __shared__ float topk_smem[];  // [kTopkWarps][E]
    if (link.n > 0) {   // the logits of the other ranks' experts arrive over the link
        if (threadIdx.x < 32) peer_wait_warp(link);
        __syncthreads();
    }
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int t = blockIdx.x * kTopkWarps + wid;
    if (t >= n_tokens) return;
    float* p = topk_smem + (size_t)wid * E;
    const float* l = logits + (size_t)t * E;
    float v[EPL];
    float m = -INFINITY;
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
        const int e = lane + 32 * j;
        v[j] = e < E ? l[e] : -INFINITY;
        m = fmaxf(m, v[j]);
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
        const int e = lane + 32 * j;
        if (e < E) {
            v[j] = (float)exp((double)__fsub_rn(v[j], m));
            p[e] = v[j];
        }
    }
    __syncwarp();
    float s = 0.0f;
    if (lane == 0) {
        int e = 0;
        for (; e + 8 <= E; e += 8) {   // loads ahead, additions in index order
            float q[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) q[u] = p[e + u];
#pragma unroll
            for (int u = 0; u < 8; ++u) s = __fadd_rn(s, q[u]);
        }
        for (; e < E; ++e) s = __fadd_rn(s, p[e]);
    }
    s = __shfl_sync(0xffffffffu, s, 0);
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
        const int e = lane + 32 * j;
        if (e < E) {
            v[j] = __fdiv_rn(v[j], s);
            probs[(size_t)t * E + e] = v[j];
        } else {
            v[j] = -1.0f;   // never selected (probabilities are >= 0)
        }
    }
    float ws = 0.0f, mine = 0.0f;   // lane r keeps the r-th selected weight
    for (int r = 0; r < k; ++r) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
#pragma unroll
        for (int j = 0; j < EPL; ++j)
            if (v[j] > bv) { bv = v[j]; bi = lane + 32 * j; }   // ascending index per lane keeps the lowest index on ties
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if ((bi & 31) == lane) {
#pragma unroll
            for (int j = 0; j < EPL; ++j)
                if (j == (bi >> 5)) v[j] = -1.0f;   // taken
        }
        if (lane == 0) idx_out[(size_t)t * k + r] = bi;
        if ((r & 31) == lane) mine = bv;
        ws = __fadd_rn(ws, bv);  // same value in every lane, selection order
        if ((r & 31) == 31 || r == k - 1) {   // every 32 rounds the lanes write their weights (each lane only ever
            const int r0 = r & ~31;            // touches indices = lane mod 32); normalised below
            if (r0 + lane <= r) w_out[(size_t)t * k + r0 + lane] = mine;
        }
    }
    __syncwarp();
    for (int r = lane; r < k; r += 32) w_out[(size_t)t * k + r] = __fdiv_rn(w_out[(size_t)t * k + r], ws);
}

// out = silu(gate) * up, elementwise, computed in fp32 with the expert kernels' silu and rounded once
// to the io dtype (the SwiGLU step of a dense VQ MLP block: gate and up are separate VQ linears).
__global__ void silu_mul_kernel(const void* __restrict__ gate, const void* __restrict__ up, void* __restrict__ out,
                                size_t n, int io_dtype) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    if (io_dtype == OJX_BF16) {
        const float g = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(gate)[i]);
        const float u = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(up)[i]);
        reinterpret_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(__fmul_rn(silu_ref(g), u));
    } else {
        reinterpret_cast<float*>(out)[i] = __fmul_rn(silu_ref(reinterpret_cast<const float*>(gate)[i]),
                                                     reinterpret_cast<const float*>(up)[i]);
    }
}

int launch_silu_mul(const void* gate, const void* up, void* out, size_t n, int io_dtype, cudaStream_t s) {
    if (!gate || !up || !out) return OJX_ERR_ARG;
    if (n == 0) return OJX_OK;
    silu_mul_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(gate, up, out, n, io_dtype);
    OJX_CUDA_TRY(cudaGetLastError());
    count_launch(1);
    return OJX_OK;
}

// ------------------------------------------------------------------------------- host side
template <typename K>
static int set_smem(K kern) {
    OJX_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(CoreSmem)));
    return OJX_OK;
}

constexpr int kMoePlanMinPairs = 64;

// Pairs this handle expects to evaluate: an expert-parallel shard sees its share of the routed pairs.
static int expected_pairs(const MoeProblem& P) {
    const int pairs = P.n_tokens * P.k_active;
    return P.E_total > P.E ? (int)(((long long)pairs * P.E + P.E_total - 1) / P.E_total) : pairs;
}

// Routed pairs expected on this handle from which the expert pass takes whole experts by the chain walk: measured
// faster than the tiled row-per-lane kernels from about half a pair per SM (80 pairs: 118 against 128 us per layer).
static int moe_chain_min_pairs() {
    const char* e = std::getenv("OJASX_B200_MOE_CHAIN_MIN_PAIRS");
    return e ? atoi(e) : (kCtasPerSm * num_sms() + 1) / 2;
}

// Gate/up by the chain walk (moe_gate_up_chain_kernel): a work item is a whole expert, which pays once there are
// enough expected pairs (moe_chain_min_pairs); the shape must fit the walker (16-byte pieces of code rows, all 2I
// sums parked at once).  OJASX_B200_MOE_CHAIN=0 keeps the row-per-lane kernel (for comparisons).
bool moe_chain_wanted(const MoeProblem& P) {
    if (!P.lut_in || P.D > 16 || (P.G & 15) != 0 || 2 * P.I > kAccRows || 2 * P.I < 512) return false;
    if (expected_pairs(P) < moe_chain_min_pairs()) return false;
    const char* e = std::getenv("OJASX_B200_MOE_CHAIN");
    return !(e && e[0] == '0');
}

static bool moe_chain_down_wanted(const MoeProblem& P) {
    if (P.D > 16 || (P.Gi & 15) != 0 || P.H > kAccRows || P.H < 512) return false;
    if (expected_pairs(P) < moe_chain_min_pairs()) return false;
    const char* e = std::getenv("OJASX_B200_MOE_CHAIN");
    return !(e && e[0] == '0');
}

size_t moe_table_bytes(int n_tokens, int G, int D) {
    const size_t plain = (size_t)G * 1024;
    const int sg = kXsFloats / D < kSliceGroups ? kXsFloats / D : kSliceGroups;
    const size_t images = (size_t)((G + sg - 1) / sg) * kSliceGroups * 1024;
    return (size_t)n_tokens * (plain > images ? plain : images);
}

template <int D>
static int launch_chain_images(const void* x, int io_dtype, int n_tokens, int H, int G, const float* cb, int Kcb, float* out, cudaStream_t s) {
    const int nsl = (G + ChainWalker<D>::SG - 1) / ChainWalker<D>::SG;
    moe_chain_prebuild_kernel<D><<<dim3(nsl, n_tokens), 256, 0, s>>>(x, io_dtype, H, G, cb, Kcb, out);
    OJX_CUDA_TRY(cudaGetLastError());
    count_launch(1);
    return OJX_OK;
}
int launch_moe_chain_images(const void* x, int io_dtype, int n_tokens, int H, int D, const float* cb, int Kcb, float* out, cudaStream_t s) {
    if (!x || !cb || !out || H % D != 0) return OJX_ERR_ARG;
    switch (D) {
        case 4: return launch_chain_images<4>(x, io_dtype, n_tokens, H, H / D, cb, Kcb, out, s);
        case 8: return launch_chain_images<8>(x, io_dtype, n_tokens, H, H / D, cb, Kcb, out, s);
        case 16: return launch_chain_images<16>(x, io_dtype, n_tokens, H, H / D, cb, Kcb, out, s);
        default: return OJX_ERR_UNSUPPORTED;
    }
}

template <int D>
static int launch_moe_experts_t(const MoeProblem& P, cudaStream_t s, const PeerLink& link) {
    int rc;
    if ((rc = set_smem(moe_gate_up_kernel<D>)) != OJX_OK) return rc;
    if ((rc = set_smem(moe_down_kernel<D>)) != OJX_OK) return rc;
    const int pairs = P.n_tokens * P.k_active, sms = kCtasPerSm * num_sms();
    const int gu_items = pairs * P.gu_tiles, dn_items = pairs * P.dn_tiles;
    int extra = 0;
    if (P.pair_list) {
        const size_t hs = sizeof(int) * 2 * (size_t)P.E;
        if (hs > 48 * 1024) OJX_CUDA_TRY(cudaFuncSetAttribute(moe_plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)hs));
        moe_plan_kernel<<<1, 1024, hs, s>>>(P, const_cast<int*>(P.pair_list));
        OJX_CUDA_TRY(cudaGetLastError());
        ++extra;
    }
    if constexpr (D <= 16) {
        if (P.lut_blocks == 2) {
            if (!P.lut_ready) {
                if ((rc = launch_chain_images<D>(P.x, P.io_dtype, P.n_tokens, P.H, P.G, P.cb_in, P.Kcb, const_cast<float*>(P.lut_in), s)) != OJX_OK) return rc;
            }
            const char* one = std::getenv("OJASX_B200_MOE_ONE_LAUNCH");
            if (P.pair_list && P.chain_ctl && P.dn_tiles == 1 && moe_chain_down_wanted(P) && !(one && one[0] == '0')) {
                // gate/up and down of every pair from one work queue (no rounded-up wave between the two passes)
                if ((rc = set_smem(moe_experts_chain_kernel<D>)) != OJX_OK) return rc;
                moe_experts_chain_kernel<D><<<pairs < sms ? pairs : sms, kThreads, sizeof(CoreSmem), s>>>(P, link);
                OJX_CUDA_TRY(cudaGetLastError());
                const int n = P.n_tokens * P.H;
                moe_combine_kernel<<<(n + 255) / 256, 256, 0, s>>>(P, link);
                OJX_CUDA_TRY(cudaGetLastError());
                count_launch(2 + extra);
                return OJX_OK;
            }
            if ((rc = set_smem(moe_gate_up_chain_kernel<D>)) != OJX_OK) return rc;
            moe_gate_up_chain_kernel<D><<<pairs < sms ? pairs : sms, kThreads, sizeof(CoreSmem), s>>>(P);
            OJX_CUDA_TRY(cudaGetLastError());
        }
    }
    if (P.lut_blocks != 2) {
        if (P.lut_in && !P.lut_ready) {
            lut_prebuild_kernel<D><<<dim3((P.G + 15) / 16, P.n_tokens), 256, 0, s>>>(P.x, P.io_dtype, P.H, P.G, P.cb_in, P.Kcb,
                                                                                    const_cast<float*>(P.lut_in));
            OJX_CUDA_TRY(cudaGetLastError());
            ++extra;
        }
        moe_gate_up_kernel<D><<<gu_items < sms ? gu_items : sms, kThreads, sizeof(CoreSmem), s>>>(P);
        OJX_CUDA_TRY(cudaGetLastError());
    }
    bool chain_down = false;
    if constexpr (D <= 16) {
        if (P.dn_tiles == 1 && moe_chain_down_wanted(P)) {
            if ((rc = set_smem(moe_down_chain_kernel<D>)) != OJX_OK) return rc;
            moe_down_chain_kernel<D><<<pairs < sms ? pairs : sms, kThreads, sizeof(CoreSmem), s>>>(P, link);
            chain_down = true;
        }
    }
    if (!chain_down) moe_down_kernel<D><<<dn_items < sms ? dn_items : sms, kThreads, sizeof(CoreSmem), s>>>(P, link);
    OJX_CUDA_TRY(cudaGetLastError());
    const int n = P.n_tokens * P.H;
    moe_combine_kernel<<<(n + 255) / 256, 256, 0, s>>>(P, link);
    OJX_CUDA_TRY(cudaGetLastError());
    count_launch(3 + extra);
    return OJX_OK;
}

// Layout of the token tables this forward wants (MoeProblem::lut_blocks).
int moe_table_layout(const MoeProblem& P) { return moe_fused_wanted(P) ? 1 : moe_chain_wanted(P) ? 2 : 0; }

int launch_moe_experts(MoeProblem P, cudaStream_t s, const PeerLink* lk) {
    if (!P.x || !P.y || !P.topk_idx || !P.topk_w || !P.inter || !P.expert_out) return OJX_ERR_ARG;
    if (P.n_tokens <= 0 || P.k_active <= 0) return OJX_ERR_ARG;
    const PeerLink none{};
    const PeerLink& link = lk ? *lk : none;
    P.combine_all = link.n > 0 ? 1 : 0;
    const int layout = moe_table_layout(P);
    if (P.lut_ready && P.lut_blocks != layout) P.lut_ready = 0;   // tables were built in another layout: rebuild
    P.lut_blocks = layout;
    // Whole-expert work items with gate/up and down fused (moe_fused.cu, opt-in); then the ordered combine.
    if (layout == 1) {
        const int rc = launch_moe_fused(P, s, lk);
        if (rc != OJX_ERR_UNSUPPORTED) {
            if (rc != OJX_OK) return rc;
            const int n = P.n_tokens * P.H;
            moe_combine_kernel<<<(n + 255) / 256, 256, 0, s>>>(P, link);
            OJX_CUDA_TRY(cudaGetLastError());
            count_launch(1);
            return OJX_OK;
        }
        P.lut_ready = 0;
        P.lut_blocks = moe_chain_wanted(P) ? 2 : 0;
    }
    const int pairs = P.n_tokens * P.k_active, sms = kCtasPerSm * num_sms();
    // Tiles: spread few pairs over the SMs, keep tiles whole when there are many pairs.
    const int expect = expected_pairs(P);
    // A handful of pairs: the work list (grouping by expert, dropping the pairs of other shards) buys nothing, so its
    // kernel is left out and the pairs are visited in order (pairs of other shards are skipped on sight).
    if (pairs <= kMoePlanMinPairs) P.pair_list = nullptr;
    int want = (sms + expect - 1) / (expect > 0 ? expect : 1);
    if (P.lut_blocks == 2) want = 1;   // the chain walk takes whole experts
    P.gu_tile = round_up((P.I + want - 1) / want, 16);
    if (P.gu_tile > kAccRows / 2) P.gu_tile = kAccRows / 2;
    P.gu_tiles = (P.I + P.gu_tile - 1) / P.gu_tile;
    P.dn_tile = round_up((P.H + want - 1) / want, 32);
    if (P.dn_tile > kAccRows) P.dn_tile = kAccRows;
    P.dn_tiles = (P.H + P.dn_tile - 1) / P.dn_tile;
    switch (P.D) {
        case 4: return launch_moe_experts_t<4>(P, s, link);
        case 8: return launch_moe_experts_t<8>(P, s, link);
        case 16: return launch_moe_experts_t<16>(P, s, link);
        case 32: return launch_moe_experts_t<32>(P, s, link);
        default: return OJX_ERR_UNSUPPORTED;
    }
}

// Lookup table of n activation vectors, out[t, g, k] = sum_d x[t, g*D + d] * cb[k, d] (kernel (a) on its own).
int launch_build_lut(const void* x, int io_dtype, int n_vectors, int K, int D, const float* codebook, int Kcb, float* out,
                     cudaStream_t s) {
    if (!x || !codebook || !out || n_vectors <= 0 || K <= 0 || D <= 0 || Kcb <= 0 || Kcb > 256) return OJX_ERR_ARG;
    const int G = (K + D - 1) / D;
    const dim3 grid((G + 15) / 16, n_vectors);
    switch (D) {
        case 4: lut_prebuild_kernel<4><<<grid, 256, 0, s>>>(x, io_dtype, K, G, codebook, Kcb, out); break;
        case 8: lut_prebuild_kernel<8><<<grid, 256, 0, s>>>(x, io_dtype, K, G, codebook, Kcb, out); break;
        case 16: lut_prebuild_kernel<16><<<grid, 256, 0, s>>>(x, io_dtype, K, G, codebook, Kcb, out); break;
        case 32: lut_prebuild_kernel<32><<<grid, 256, 0, s>>>(x, io_dtype, K, G, codebook, Kcb, out); break;
        default: return OJX_ERR_UNSUPPORTED;
    }
    OJX_CUDA_TRY(cudaGetLastError());
    count_launch(1);
    return OJX_OK;
}

int take_moe_bulk_copy_error(int* out) {
    int v = 0, zero = 0;
    OJX_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_bulk_copy_timeout, sizeof(int)));
    if (v) OJX_CUDA_TRY(cudaMemcpyToSymbol(g_bulk_copy_timeout, &zero, sizeof(int)));
    *out = v;
    return OJX_OK;
}

int launch_moe_router(const float* Wr, const void* x, int io_dtype, int n_tokens, int H, int E, int k,
                      float* logits, float* probs, int* idx_out, float* w_out, cudaStream_t s,
                      const float* codebook, int Kcb, int D, float* lut_out, int lut_blocks, const PeerLink* lk,
                      int e_begin, int e_end) {
    if (!Wr || !x || !logits || !probs || !idx_out || !w_out) return OJX_ERR_ARG;
    if (n_tokens <= 0 || k <= 0 || k > E) return OJX_ERR_ARG;
    // With a link every rank scores the experts [e_begin, e_end) it holds and stores their logits into every rank's
    // logits buffer; the top-k pass waits for all ranks.  Without one, all E experts are scored here.
    const PeerLink none{};
    const PeerLink& link = lk ? *lk : none;
    if (link.n <= 0) { e_begin = 0; e_end = E; }
    if (e_begin < 0 || e_end > E || e_begin > e_end) return OJX_ERR_ARG;
    if (lut_out && lut_blocks) {   // tables in a layout of one of the whole-expert kernels: a launch of their own
        const int rc = lut_blocks == 2 ? launch_moe_chain_images(x, io_dtype, n_tokens, H, D, codebook, Kcb, lut_out, s)
                                       : launch_moe_prebuild_blocks(x, io_dtype, n_tokens, H, D, codebook, Kcb, lut_out, s);
        if (rc != OJX_OK) return rc;
        lut_out = nullptr;
    }
    const int warps_per_block = 8;
    const int ne = e_end - e_begin > 0 ? e_end - e_begin : 1;
    const int lx = (ne + warps_per_block - 1) / warps_per_block, ly = n_tokens < 32 ? n_tokens : 32;
    if (lut_out) {   // the gate/up tables ride along (one launch less)
        if (!codebook || H % D != 0) return OJX_ERR_ARG;
        const int G = H / D, grid = lx * ly + (G + 15) / 16 * n_tokens;
        switch (D) {
            case 4: moe_logits_prebuild_kernel<4><<<grid, 256, 0, s>>>(Wr, x, io_dtype, n_tokens, H, E, logits, lx, ly, G, codebook, Kcb, lut_out, e_begin, e_end, link); break;
            case 8: moe_logits_prebuild_kernel<8><<<grid, 256, 0, s>>>(Wr, x, io_dtype, n_tokens, H, E, logits, lx, ly, G, codebook, Kcb, lut_out, e_begin, e_end, link); break;
            case 16: moe_logits_prebuild_kernel<16><<<grid, 256, 0, s>>>(Wr, x, io_dtype, n_tokens, H, E, logits, lx, ly, G, codebook, Kcb, lut_out, e_begin, e_end, link); break;
            case 32: moe_logits_prebuild_kernel<32><<<grid, 256, 0, s>>>(Wr, x, io_dtype, n_tokens, H, E, logits, lx, ly, G, codebook, Kcb, lut_out, e_begin, e_end, link); break;
            default: return OJX_ERR_UNSUPPORTED;
        }
    } else if (n_tokens >= kLogitTokens) {
        moe_router_logits_tiled_kernel<<<dim3(lx, (n_tokens + kLogitTokens - 1) / kLogitTokens), 256, 0, s>>>(Wr, x, io_dtype, n_tokens, H, E, logits,
                                                                                                          e_begin, e_end, link);
    } else {
        moe_router_logits_kernel<<<dim3(lx, ly), 256, 0, s>>>(Wr, x, io_dtype, n_tokens, H, E, logits, e_begin, e_end, link);
    }
    OJX_CUDA_TRY(cudaGetLastError());
    const size_t tsm = sizeof(float) * kTopkWarps * (size_t)E;
    if (tsm > 200 * 1024) return OJX_ERR_TOO_LARGE;
    if (tsm > 48 * 1024) OJX_CUDA_TRY(cudaFuncSetAttribute(moe_router_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tsm));
    const int tgrid = (n_tokens + kTopkWarps - 1) / kTopkWarps;
    if (E <= 512) moe_router_topk_reg_kernel<16><<<tgrid, kTopkWarps * 32, tsm, s>>>(logits, n_tokens, E, k, idx_out, w_out, probs, link);
    else moe_router_topk_kernel<<<tgrid, kTopkWarps * 32, tsm, s>>>(logits, n_tokens, E, k, idx_out, w_out, probs, link);
    OJX_CUDA_TRY(cudaGetLastError());
    count_launch(2);
    return OJX_OK;
}

}  // namespace ojx

// ---------------------------------------------------------------- no-allocation MoE forward
// Scratch for ojasx_b200_moe_forward_noalloc: a fixed array in this library's device image, so
// the call never has to obtain memory.  Every GPU that loads the library holds these 1 MiB
// until the process exits.
namespace ojx {
constexpr size_t kNoAllocScratchFloats = OJASX_B200_NOALLOC_SCRATCH_FLOATS;
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocScratchFloats];
}  // namespace ojx

extern "C" int ojasx_b200_moe_forward_noalloc(OjasxMoEHandle handle, const void* d_x, const int* d_topk_idx,
                                              const float* d_topk_w, void* d_y, int n_tokens, int k_active,
                                              int io_dtype, void* stream) {
    using namespace ojx;
    if (!handle || !d_x || !d_topk_idx || !d_topk_w || !d_y) return OJX_ERR_ARG;
    if (n_tokens <= 0 || k_active <= 0 || (io_dtype != OJX_F32 && io_dtype != OJX_BF16)) return OJX_ERR_ARG;
    auto* h = static_cast<MoeHandle*>(handle);
    const size_t need = (size_t)n_tokens * k_active * ((size_t)h->I + h->H);
    if (need > kNoAllocScratchFloats) {
        set_last_error_msg("ojasx_b200_moe_forward_noalloc: n_tokens*k_active*(intermediate+hidden) exceeds "
                           "OJASX_B200_NOALLOC_SCRATCH_FLOATS; use ojasx_b200_moe_forward for larger batches");
        return OJX_ERR_TOO_LARGE;
    }
    int dev = -1;
    OJX_CUDA_TRY(cudaGetDevice(&dev));
    if (dev != h->dev || dev < 0 || dev >= 64) {
        set_last_error_msg("ojasx_b200_moe_forward_noalloc: the handle's device must be the current device");
        return OJX_ERR_ARG;
    }
    // Set-up, once per device, with that device current: in host code `g_noalloc_scratch` is
    // only a stand-in for the symbol, so its device address is looked up here and that pointer,
    // not the symbol, is what the kernels receive.
    static std::mutex mu;
    static float* scratch_on[64] = {};
    float* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!scratch_on[dev]) {
            void* p = nullptr;
            OJX_CUDA_TRY(cudaGetSymbolAddress(&p, g_noalloc_scratch));
            scratch_on[dev] = static_cast<float*>(p);
        }
        scratch = scratch_on[dev];
    }
    MoeProblem P = h->problem(d_x, d_y, d_topk_idx, d_topk_w, n_tokens, k_active, io_dtype);
    // Nothing in the scratch has to start at zero: every (pair, index) slot that a later stage
    // reads was written by the stage before it in this same call, and slots of skipped pairs are
    // never read.  What an earlier call left there is therefore harmless.
    P.lut_in = nullptr;  // tables are rebuilt inside the gate/up kernel: no further scratch
    P.pair_list = nullptr;  // every pair is visited in order and skipped if it is not evaluated here
    P.plan = nullptr;
    P.chain_ctl = nullptr;
    P.inter = scratch;
    P.expert_out = scratch + (size_t)n_tokens * k_active * h->I;
    return launch_moe_experts(P, static_cast<cudaStream_t>(stream));
}
