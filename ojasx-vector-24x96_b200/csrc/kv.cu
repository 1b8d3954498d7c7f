// Quantized KV cache kernels.
//
// (1) Codebook-VQ cache ("kvq"): every head vector is stored as head_dim/block_dim uint8 codes
//     into a per-KV-head codebook.  Append = nearest centroid per sub-vector (rule of
//     ojasx_24x96/codec.py:217-224); decode = per-head query table LUT[g, code] = <q_g, C_k[code]>,
//     logit[t] = scale * sum_g LUT[g, k_code[t,g]] (structure of
//     split_manifold_lut_experiment/native/src/ojasx_lut_kv_cache.cpp:86-107), online softmax
//     over context chunks (ojasx_24x96/long_context.py:92-176) and value gather
//     out = sum_t p_t * C_v[v_code[t,g]].  The query heads that share a KV head (GQA) are
//     scored from one read of the code stream.
// (2) The reference's cache as shipped ("legacy"): int8 of each block's first coordinate with a
//     per-token abs-max scale (ojasx_lut_kv_cache.cpp:16-132, softmax of
//     ojasx_lut_c_api.cpp:178-191).
#include <algorithm>

#include "common.cuh"
#include "launch.h"
#include "peer.cuh"
#include "handles.h"

namespace ojx {

constexpr int kKvThreads = 256;
constexpr int kKvMaxGroups = 32;  // head_dim / block_dim


__device__ __forceinline__ float load_io(const void* p, size_t i, int dtype) {
    return dtype == OJX_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i])
                             : reinterpret_cast<const float*>(p)[i];
}

// ------------------------------------------------------------------------------ kvq append
// grid = (ceil(tasks / warps per CTA), B).  Task = (k|v, kv head, group); one warp per task scans
// the 256 centroids.  dist = (|v|^2 - 2 v.c) + |c|^2 with every dot product a sequential fp32 sum
// (separate multiply and add); arg-min takes the first minimum.  Every CTA counts itself done when
// its codes are written; the last one of a sequence advances that sequence's length (the others read
// the length before they count), so an append is one launch.
template <int D>
__global__ void __launch_bounds__(kKvThreads) kvq_append_kernel(const __grid_constant__ KvqProblem P) {
    const int b = blockIdx.y;
    const int T = P.seq_lens[b];
    if (T >= P.max_seq) {   // cache full: nothing is written, the error flag reports it
        if (blockIdx.x == 0 && threadIdx.x == 0) atomicExch(P.error_flag, 1);
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int G = P.G, hd = P.head_dim;
    const int tasks = 2 * P.Hkv * G;
    const int task = blockIdx.x * nwarps + warp;
    if (task < tasks) {
    const int which = task / (P.Hkv * G);
    const int rem = task - which * P.Hkv * G;
    const int h = rem / G, g = rem - h * G;
    const void* src = which ? P.new_v : P.new_k;
    const float* cb = (which ? P.v_cb : P.k_cb) + (size_t)h * P.Kcb * D;
    float v[D];
    float vv = 0.0f;
#pragma unroll
    for (int d = 0; d < D; ++d) {
        v[d] = load_io(src, ((size_t)b * P.Hkv + h) * hd + g * D + d, P.io_dtype);
        vv = __fadd_rn(vv, __fmul_rn(v[d], v[d]));
    }
    float bd = INFINITY;
    int bi = 0x7fffffff;
    for (int c = lane; c < P.Kcb; c += 32) {
        float cv[D];
#pragma unroll
        for (int d = 0; d < D; ++d) cv[d] = cb[(size_t)c * D + d];
        float vc = 0.0f, cc = 0.0f;
#pragma unroll
        for (int d = 0; d < D; ++d) vc = __fadd_rn(vc, __fmul_rn(v[d], cv[d]));
#pragma unroll
        for (int d = 0; d < D; ++d) cc = __fadd_rn(cc, __fmul_rn(cv[d], cv[d]));
        const float dist = __fadd_rn(__fsub_rn(vv, __fmul_rn(2.0f, vc)), cc);
        if (dist < bd) { bd = dist; bi = c; }
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        const float od = __shfl_xor_sync(0xffffffffu, bd, off);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
        if (od < bd || (od == bd && oi < bi)) { bd = od; bi = oi; }
    }
    if (lane == 0) {
        uint8_t* codes = which ? P.v_codes : P.k_codes;
        codes[(((size_t)b * P.Hkv + h) * P.max_seq + T) * G + g] = (uint8_t)bi;
    }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(&P.append_done[b], 1) == (int)gridDim.x - 1) {
            P.append_done[b] = 0;
            P.seq_lens[b] = T + 1;
        }
    }
}

// ------------------------------------------------------------------------------ kvq decode
// grid = (splits, Hkv, B); a CTA owns tokens [split*chunk, (split+1)*chunk) of one (sequence, KV head)
// and walks them in passes of kSub tokens with a running maximum (online softmax), so the query table
// [G,256,R] is built once per CTA however long its range is.
//
// The CTA's warps are split in two groups that work on consecutive passes at the same time:
//  * score warps: thread per token; its K codes (one 16-byte load when G is a multiple of 16) index the
//    query table, R heads per 128-bit gather; its V codes are stored as words of four groups,
//    [g / 4][token] (byte stores of different lanes into one word would be serialised); after a
//    barrier among the score warps every one of them knows the pass maximum, turns its scores into
//    probabilities exp(s - running max), and publishes the running maximum of the pass;
//  * value warps: thread = (group or pair of groups, token stripe); it gathers whole centroids of the
//    value codebook and keeps the R x D partial outputs of its groups in registers, rescaled when the
//    running maximum moves.  Two groups per thread (when the registers allow) halve the reads of the
//    probabilities and of the codes.
// Probabilities, transposed codes and the published maxima are double-buffered; the groups hand the
// buffers over with named barriers (full: score warps arrive, value warps wait; empty: the reverse).
//
// The kernel is bound by shared-memory wavefronts: a 128-bit gather is served eight lanes at a time, and
// eight random addresses over eight 16-byte bank groups collide (10.8 wavefronts per warp instead of 4,
// measured).  The value codebook is small, so when it fits it is stored eight times, copy q confined to
// bank group q, and lane l reads copy l % 8: those gathers are conflict-free.  While the score warps wait
// for their codes from global memory the value warps keep the shared-memory pipe busy.
//
// Threads per CTA: 512, or 256 where the R x D accumulators of a thread need more than 128 registers.
constexpr int kvq_decode_threads(int R, int D) { return R * D > 64 ? 256 : 512; }
constexpr int kKvVctPad = 4;                // words of padding per transposed code row (bank spread)
// named barriers (0 is __syncthreads)
constexpr int kBarScore = 1, kBarFull = 2 /* +buf */, kBarEmpty = 4 /* +buf */, kBarValue = 6;


__device__ __forceinline__ void named_bar_sync(int id, int count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void named_bar_arrive(int id, int count) {
    asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// R consecutive floats at a 4*R-byte aligned shared-memory address, as 128-bit (R % 4 == 0) or 64-bit (R == 2) accesses
template <int R>
__device__ __forceinline__ void ld_heads(const float* p, float (&o)[R]) {
    if constexpr (R % 4 == 0) {
#pragma unroll
        for (int q = 0; q < R / 4; ++q) {
            const float4 f = reinterpret_cast<const float4*>(p)[q];
            o[q * 4 + 0] = f.x; o[q * 4 + 1] = f.y; o[q * 4 + 2] = f.z; o[q * 4 + 3] = f.w;
        }
    } else if constexpr (R == 2) {
        const float2 f = *reinterpret_cast<const float2*>(p);
        o[0] = f.x; o[1] = f.y;
    } else {
#pragma unroll
        for (int r = 0; r < R; ++r) o[r] = p[r];
    }
}
template <int R>
__device__ __forceinline__ void st_heads(float* p, const float (&o)[R]) {
    if constexpr (R % 4 == 0) {
#pragma unroll
        for (int q = 0; q < R / 4; ++q) reinterpret_cast<float4*>(p)[q] = make_float4(o[q * 4], o[q * 4 + 1], o[q * 4 + 2], o[q * 4 + 3]);
    } else if constexpr (R == 2) {
        *reinterpret_cast<float2*>(p) = make_float2(o[0], o[1]);
    } else {
#pragma unroll
        for (int r = 0; r < R; ++r) p[r] = o[r];
    }
}

// Every CTA of a (sequence, KV head) calls this once its partial is written (all threads of the CTA).
// The CTA that arrives last merges the partials of the R query heads: M = max m_c, weights
// exp(m_c - M), splits in index order -- so a decode is one launch.  The counter returns to zero.
template <int R>
__device__ __forceinline__ void kvq_merge_if_last(const KvqProblem& P, int b, int h, const PeerLink& link) {
    __shared__ int s_last;
    __threadfence();   // this thread's partial is visible device-wide before the CTA is counted
    __syncthreads();
    if (threadIdx.x == 0) {
        int* cnt = P.split_done + (size_t)b * P.Hkv + h;
        const int last = atomicAdd(cnt, 1) == P.n_chunks - 1;
        if (last) *cnt = 0;
        s_last = last;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const int hd = P.head_dim;
    const float* base = P.partials + (((size_t)b * P.Hkv + h) * P.n_chunks) * R * (hd + 2);
    for (int i = threadIdx.x; i < R * hd; i += blockDim.x) {
        const int r = i / hd, col = i - r * hd;
        float M = -INFINITY;
        for (int c = 0; c < P.n_chunks; ++c) M = fmaxf(M, __ldcg(base + ((size_t)c * R + r) * (hd + 2)));
        float L = 0.0f, o = 0.0f;
        for (int c = 0; c < P.n_chunks; ++c) {
            const float* p = base + ((size_t)c * R + r) * (hd + 2);
            const float m = __ldcg(p);
            if (m != -INFINITY) {
                const float wgt = __expf(m - M);
                L += __ldcg(p + 1) * wgt;
                o = fmaf(__ldcg(p + 2 + col), wgt, o);
            }
        }
        o *= L > 0.0f ? 1.0f / L : 0.0f;
        // a KV-head shard writes its heads into the gathered output of every rank (link.n > 0)
        const int row_heads = P.out_heads > 0 ? P.out_heads : P.Hq;
        const size_t oi = ((size_t)b * row_heads + P.out_head0 + (size_t)h * R + r) * hd + col;
        if (P.io_dtype == OJX_BF16) peer_store(link, reinterpret_cast<__nv_bfloat16*>(P.out) + oi, __float2bfloat16_rn(o));
        else peer_store(link, reinterpret_cast<float*>(P.out) + oi, o);
    }
}

template <int R, int D>
__global__ void __launch_bounds__(kvq_decode_threads(R, D), 1) kvq_decode_kernel(const __grid_constant__ KvqProblem P,
                                                                                 const __grid_constant__ PeerLink link) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int kThreads = kvq_decode_threads(R, D), kHalf = kThreads / 2;   // score threads = value threads
    constexpr int kTpt = 2, kSub = kTpt * kHalf;                               // tokens per pass
    constexpr int kWarpsHalf = kHalf / 32, kPieces = D / 4;
    constexpr int kGp = R * D <= 32 ? 2 : 1;                                    // groups per value thread
    constexpr int kVu = 2;                                                      // tokens per step of a value thread
    const int G = P.G, hd = P.head_dim, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    float* lut = reinterpret_cast<float*>(smem_raw);               // [G][256][R], or [256][G][R] (see code_major)
    // One 16-byte entry (R = 4) per (group, centroid) and 16 groups: the table is kept centroid-major, so that the
    // entry of group g lies in 16-byte bank group g % 8 whatever the code is.  A score thread then walks the
    // groups starting at its own (g = (i + lane) & 15 in step i): the eight lanes that a 128-bit shared load
    // serves together read eight different bank groups, and the gather costs 4 wavefronts instead of 10.8.
    const bool code_major = R == 4 && G == 16;
    const int vrep = P.v_copies;                                   // 1 or 8 copies of the value codebook
    float* vcb = lut + (size_t)G * 256 * R;                        // [D/4][256][vrep] float4
    float* qs = vcb + 256 * D * vrep;                              // [R*hd]
    float* sc = qs + R * hd;                                       // [2][kSub*R] probabilities
    float* wred = sc + 2 * (size_t)kSub * R;                       // [2][score warps][R] warp maxima / normalisers
    float* mpub = wred + 2 * kWarpsHalf * R;                       // [2][R] running maximum after each pass
    float* lred = mpub + 2 * R;                                    // [score warps][R] normaliser partials, [R] final maximum
    float* mfin = lred + kWarpsHalf * R;
    uint32_t* vct = reinterpret_cast<uint32_t*>(mfin + R);         // [2][ceil(G/4)][kSub + pad] words of four codes
    const int vrow = kSub + kKvVctPad, Gq = (G + 3) >> 2;

    const int b = blockIdx.z, h = blockIdx.y, split = blockIdx.x;
    const int T = P.seq_lens[b];
    const int t_begin = split * P.chunk;
    const int t_end = min(T, t_begin + P.chunk);
    float* part = P.partials + ((((size_t)b * P.Hkv + h) * P.n_chunks + split) * R) * (hd + 2);
    if (t_begin >= t_end) {  // range beyond this sequence: neutral partial
        for (int i = tid; i < R * (hd + 2); i += kThreads) part[i] = (i % (hd + 2)) == 0 ? -INFINITY : 0.0f;
        kvq_merge_if_last<R>(P, b, h, link);
        peer_signal_when_last(link, gridDim.x * gridDim.y * gridDim.z);
        return;
    }
    const int n_passes = (t_end - t_begin + kSub - 1) / kSub;
    const uint8_t* kc = P.k_codes + (((size_t)b * P.Hkv + h) * P.max_seq) * G;
    const uint8_t* vc = P.v_codes + (((size_t)b * P.Hkv + h) * P.max_seq) * G;

    for (int i = tid; i < R * hd; i += kThreads) qs[i] = load_io(P.q, ((size_t)b * P.Hq + (size_t)h * R) * hd + i, P.io_dtype);
    for (int i0 = tid; i0 < 256 * kPieces * vrep; i0 += 4 * kThreads) {   // consecutive threads, consecutive 16-byte slots
        float4 val[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {   // loads first, then stores
            const int i = i0 + u * kThreads, slot = i / vrep, piece = slot >> 8, c = slot & 255;
            val[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (i < 256 * kPieces * vrep && c < P.Kcb)
                val[u] = *reinterpret_cast<const float4*>(P.v_cb + ((size_t)h * P.Kcb + c) * D + piece * 4);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (i0 + u * kThreads < 256 * kPieces * vrep) reinterpret_cast<float4*>(vcb)[i0 + u * kThreads] = val[u];
    }
    __syncthreads();
    // query table: kThreads / 256 threads per centroid, groups interleaved between them
    {
        const int cen = tid & 255;
        float c[D];
#pragma unroll
        for (int d = 0; d < D; ++d) c[d] = cen < P.Kcb ? P.k_cb[((size_t)h * P.Kcb + cen) * D + d] : 0.0f;
        for (int g = tid >> 8; g < G; g += kThreads / 256) {
            float e[R];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                float qv[D];   // D consecutive query values, 128-bit broadcast reads (D % 4 == 0, hd % 4 == 0)
                ld_heads<D>(qs + r * hd + g * D, qv);
                float dot = 0.0f;
#pragma unroll
                for (int d = 0; d < D; ++d) dot = fmaf(qv[d], c[d], dot);
                e[r] = dot;
            }
            st_heads<R>(lut + (code_major ? (size_t)cen * 16 + g : (size_t)g * 256 + cen) * R, e);
        }
    }
    __syncthreads();

    // value mapping: threads per unit (kGp groups) capped so that the stripe partials ([stripes][R][hd + 4])
    // fit in the area of the query table and the value codebook, both dead by then
    const int units = (G + kGp - 1) / kGp;
    const int stripes = min(kHalf / units, (int)((((size_t)G * R + (size_t)D * vrep) * 256) / ((size_t)R * (hd + 4))));
    float* stripe_out = lut;                       // [stripes][R][hd + 4]: padded so that stripes spread over the banks
    const int srow = hd + 4;
    const bool score_warp = warp < kWarpsHalf;
    const int vt_id = tid - kHalf;                 // value thread index (value warps only)
    const int vu = vt_id / stripes, vst = vt_id - vu * stripes;   // unit, stripe
    const int vg = vu * kGp;                                      // first group of the unit

    if (score_warp) {
        float m_run[R], l_loc[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            m_run[r] = -INFINITY;
            l_loc[r] = 0.0f;
        }
        // G == 16 (one 16-byte row per token): the rows of the next pass are fetched a pass ahead, so the
        // latency of global memory is off the score warps' critical path
        const bool ahead = G == 16;
        uint4 k_next[kTpt], v_next[kTpt];
        auto fetch = [&](int pass_base) {
#pragma unroll
            for (int j = 0; j < kTpt; ++j) {
                const int t = pass_base + tid + j * kHalf;
                const size_t row = (size_t)(t < t_end ? t : pass_base) * 16;
                k_next[j] = *reinterpret_cast<const uint4*>(kc + row);
                v_next[j] = *reinterpret_cast<const uint4*>(vc + row);
            }
        };
        if (ahead) fetch(t_begin);
        for (int it = 0; it < n_passes; ++it) {
            const int buf = it & 1, base = t_begin + it * kSub;
            const int n = min(kSub, t_end - base);
            float* scb = sc + (size_t)buf * kSub * R;
            float* wr = wred + buf * kWarpsHalf * R;
            uint32_t* vt = vct + (size_t)buf * Gq * vrow;
            if (it >= 2) named_bar_sync(kBarEmpty + buf, kThreads);   // the value warps are done with this buffer

            // both tokens of a thread go through the groups together, so that their gathers overlap; a token
            // beyond the pass reads row 0 of the pass and is discarded
            float s[kTpt][R], mloc[R];
            const uint8_t* krow[kTpt];
            const uint8_t* vrow_g[kTpt];
#pragma unroll
            for (int j = 0; j < kTpt; ++j) {
                const int t = tid + j * kHalf;
                const size_t row = (size_t)(base + (t < n ? t : 0)) * G;
                krow[j] = kc + row;
                vrow_g[j] = vc + row;
#pragma unroll
                for (int r = 0; r < R; ++r) s[j][r] = 0.0f;
            }
            // four groups: four gathers per token and one word of V codes
            auto quad = [&](int gq, const unsigned (&kword)[kTpt], const unsigned (&vword)[kTpt]) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    if (gq * 4 + q < G) {
#pragma unroll
                        for (int j = 0; j < kTpt; ++j) {
                            float e[R];
                            ld_heads<R>(lut + ((size_t)(gq * 4 + q) * 256 + ((kword[j] >> (8 * q)) & 255u)) * R, e);
#pragma unroll
                            for (int r = 0; r < R; ++r) s[j][r] += e[r];
                        }
                    }
                }
#pragma unroll
                for (int j = 0; j < kTpt; ++j) vt[(size_t)gq * vrow + tid + j * kHalf] = vword[j];
            };
            if (ahead && code_major) {
                uint4 kw[kTpt], vw[kTpt];
#pragma unroll
                for (int j = 0; j < kTpt; ++j) {
                    kw[j] = k_next[j];
                    vw[j] = v_next[j];
                }
                if (it + 1 < n_passes) fetch(base + kSub);
                // the 16 code bytes of a token, rotated so that byte i is the code of group (i + rot) & 15
                const int rot = tid & 15, sh = (rot & 3) * 8;
                unsigned rk[kTpt][4];
#pragma unroll
                for (int j = 0; j < kTpt; ++j) {
                    unsigned a0 = __funnelshift_r(kw[j].x, kw[j].y, sh), a1 = __funnelshift_r(kw[j].y, kw[j].z, sh);
                    unsigned a2 = __funnelshift_r(kw[j].z, kw[j].w, sh), a3 = __funnelshift_r(kw[j].w, kw[j].x, sh);
                    if (rot & 4) { const unsigned t = a0; a0 = a1; a1 = a2; a2 = a3; a3 = t; }
                    if (rot & 8) { unsigned t = a0; a0 = a2; a2 = t; t = a1; a1 = a3; a3 = t; }
                    rk[j][0] = a0; rk[j][1] = a1; rk[j][2] = a2; rk[j][3] = a3;
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int goff = ((i + rot) & 15) * R;
#pragma unroll
                    for (int j = 0; j < kTpt; ++j) {
                        const unsigned code = (rk[j][i >> 2] >> (8 * (i & 3))) & 255u;
                        float e[R];
                        ld_heads<R>(lut + code * (16 * R) + goff, e);
#pragma unroll
                        for (int r = 0; r < R; ++r) s[j][r] += e[r];
                    }
                }
#pragma unroll
                for (int j = 0; j < kTpt; ++j) {
                    vt[(size_t)0 * vrow + tid + j * kHalf] = vw[j].x;
                    vt[(size_t)1 * vrow + tid + j * kHalf] = vw[j].y;
                    vt[(size_t)2 * vrow + tid + j * kHalf] = vw[j].z;
                    vt[(size_t)3 * vrow + tid + j * kHalf] = vw[j].w;
                }
            } else if (ahead) {
                uint4 kw[kTpt], vw[kTpt];
#pragma unroll
                for (int j = 0; j < kTpt; ++j) {
                    kw[j] = k_next[j];
                    vw[j] = v_next[j];
                }
                if (it + 1 < n_passes) fetch(base + kSub);
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    unsigned ka[kTpt], va[kTpt];
#pragma unroll
                    for (int j = 0; j < kTpt; ++j) {
                        ka[j] = w == 0 ? kw[j].x : w == 1 ? kw[j].y : w == 2 ? kw[j].z : kw[j].w;
                        va[j] = w == 0 ? vw[j].x : w == 1 ? vw[j].y : w == 2 ? vw[j].z : vw[j].w;
                    }
                    quad(w, ka, va);
                }
            } else if ((G & 15) == 0) {
                for (int g = 0; g < G; g += 16) {
                    uint4 kw[kTpt], vw[kTpt];
#pragma unroll
                    for (int j = 0; j < kTpt; ++j) {
                        kw[j] = *reinterpret_cast<const uint4*>(krow[j] + g);
                        vw[j] = *reinterpret_cast<const uint4*>(vrow_g[j] + g);
                    }
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
                        unsigned ka[kTpt], va[kTpt];
#pragma unroll
                        for (int j = 0; j < kTpt; ++j) {
                            ka[j] = w == 0 ? kw[j].x : w == 1 ? kw[j].y : w == 2 ? kw[j].z : kw[j].w;
                            va[j] = w == 0 ? vw[j].x : w == 1 ? vw[j].y : w == 2 ? vw[j].z : vw[j].w;
                        }
                        quad((g >> 2) + w, ka, va);
                    }
                }
            } else {
                for (int gq = 0; gq < Gq; ++gq) {
                    unsigned ka[kTpt], va[kTpt];
#pragma unroll
                    for (int j = 0; j < kTpt; ++j) {
                        ka[j] = va[j] = 0u;
                        for (int q = 0; q < 4 && gq * 4 + q < G; ++q) {
                            ka[j] |= (unsigned)krow[j][gq * 4 + q] << (8 * q);
                            va[j] |= (unsigned)vrow_g[j][gq * 4 + q] << (8 * q);
                        }
                    }
                    quad(gq, ka, va);
                }
            }
#pragma unroll
            for (int r = 0; r < R; ++r) mloc[r] = -INFINITY;
#pragma unroll
            for (int j = 0; j < kTpt; ++j) {
                const bool live = tid + j * kHalf < n;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    s[j][r] = live ? s[j][r] * P.scale : -INFINITY;
                    mloc[r] = fmaxf(mloc[r], s[j][r]);
                }
            }
#pragma unroll
            for (int r = 0; r < R; ++r) {
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) mloc[r] = fmaxf(mloc[r], __shfl_xor_sync(0xffffffffu, mloc[r], off));
                if (lane == 0) wr[warp * R + r] = mloc[r];
            }
            named_bar_sync(kBarScore, kHalf);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                float m = m_run[r];
#pragma unroll
                for (int w = 0; w < kWarpsHalf; ++w) m = fmaxf(m, wr[w * R + r]);
                l_loc[r] *= __expf(m_run[r] - m);   // factor 0 on the first pass (m_run = -inf, m finite)
                m_run[r] = m;
            }
            if (tid == 0) {
#pragma unroll
                for (int r = 0; r < R; ++r) mpub[buf * R + r] = m_run[r];
            }
#pragma unroll
            for (int j = 0; j < kTpt; ++j) {
                const int t = tid + j * kHalf;
                if (t < n) {
                    float p[R];
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        p[r] = __expf(s[j][r] - m_run[r]);
                        l_loc[r] += p[r];
                    }
                    st_heads<R>(scb + (size_t)t * R, p);
                }
            }
            named_bar_arrive(kBarFull + buf, kThreads);
        }
        // normaliser: fixed-shape reduction (shuffle tree here, then the warps in order after the join)
#pragma unroll
        for (int r = 0; r < R; ++r) {
            float l = l_loc[r];
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) l += __shfl_xor_sync(0xffffffffu, l, off);
            if (lane == 0) lred[warp * R + r] = l;
            if (tid == 0) mfin[r] = m_run[r];
        }
    } else {
        float m_run[R], o[kGp][R][D];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            m_run[r] = -INFINITY;
#pragma unroll
            for (int i = 0; i < kGp; ++i)
#pragma unroll
                for (int d = 0; d < D; ++d) o[i][r][d] = 0.0f;
        }
        const float* vmine = vcb + (lane & (vrep - 1)) * 4;   // this lane's copy of the value codebook
        for (int it = 0; it < n_passes; ++it) {
            const int buf = it & 1, base = t_begin + it * kSub;
            const int n = min(kSub, t_end - base);
            const float* scb = sc + (size_t)buf * kSub * R;
            // the unit's codes of one token sit in one word (kGp divides 4)
            const uint8_t* codes = reinterpret_cast<const uint8_t*>(vct + (size_t)buf * Gq * vrow + (size_t)(vg >> 2) * vrow) + (vg & 3);
            named_bar_sync(kBarFull + buf, kThreads);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const float m = mpub[buf * R + r];
                const float alpha = __expf(m_run[r] - m);
                m_run[r] = m;
#pragma unroll
                for (int i = 0; i < kGp; ++i)
#pragma unroll
                    for (int d = 0; d < D; ++d) o[i][r][d] *= alpha;
            }
            if (vg < G) {
                // kVu tokens per step, loads first: a token beyond the pass re-reads this thread's first
                // token with probability 0
                for (int t = vst; t < n; t += kVu * stripes) {
                    float v[kVu][kGp][D], p[kVu][R];
#pragma unroll
                    for (int u = 0; u < kVu; ++u) {
                        const int tu = t + u * stripes;
                        const bool live = tu < n;
                        const int tt = live ? tu : t;
                        unsigned cc;   // kGp codes, one per byte (a group beyond G reads the zero padding of the word)
                        if constexpr (kGp == 2) cc = *reinterpret_cast<const uint16_t*>(codes + (size_t)tt * 4);
                        else cc = codes[(size_t)tt * 4];
#pragma unroll
                        for (int i = 0; i < kGp; ++i) {
                            const int c = (cc >> (8 * i)) & 255u;
#pragma unroll
                            for (int q = 0; q < kPieces; ++q) {
                                const float4 f = *reinterpret_cast<const float4*>(vmine + ((size_t)q * 256 + c) * vrep * 4);
                                v[u][i][q * 4 + 0] = f.x; v[u][i][q * 4 + 1] = f.y; v[u][i][q * 4 + 2] = f.z; v[u][i][q * 4 + 3] = f.w;
                            }
                        }
                        ld_heads<R>(scb + (size_t)tt * R, p[u]);
                        if (!live) {
#pragma unroll
                            for (int r = 0; r < R; ++r) p[u][r] = 0.0f;
                        }
                    }
#pragma unroll
                    for (int u = 0; u < kVu; ++u)
#pragma unroll
                        for (int i = 0; i < kGp; ++i)
#pragma unroll
                            for (int r = 0; r < R; ++r)
#pragma unroll
                                for (int d = 0; d < D; ++d) o[i][r][d] = fmaf(p[u][r], v[u][i][d], o[i][r][d]);
                }
            }
            if (it + 2 < n_passes) named_bar_arrive(kBarEmpty + buf, kThreads);   // only if a score pass will wait for it
        }
        // Every value warp is past its last pass, and so are the score warps (that pass was handed over by
        // all of them): the query table and the value codebook are dead, their area takes the stripe partials.
        named_bar_sync(kBarValue, kHalf);
        if (vg < G) {
#pragma unroll
            for (int i = 0; i < kGp; ++i) {
                if (vg + i < G) {
#pragma unroll
                    for (int r = 0; r < R; ++r) st_heads<D>(stripe_out + ((size_t)vst * R + r) * srow + (vg + i) * D, o[i][r]);
                }
            }
        }
    }

    __syncthreads();
    for (int i = tid; i < R * hd; i += kThreads) {   // stripes of one group are added in a fixed order
        const int r = i / hd, c = i - r * hd;
        float acc = 0.0f;
        for (int s2 = 0; s2 < stripes; ++s2) acc += stripe_out[((size_t)s2 * R + r) * srow + c];
        part[(size_t)r * (hd + 2) + 2 + c] = acc;
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        if (tid == r) {
            float l = 0.0f;
            for (int w = 0; w < kWarpsHalf; ++w) l += lred[w * R + r];
            part[(size_t)r * (hd + 2) + 0] = mfin[r];
            part[(size_t)r * (hd + 2) + 1] = l;
        }
    }
    kvq_merge_if_last<R>(P, b, h, link);
    peer_signal_when_last(link, gridDim.x * gridDim.y * gridDim.z);
}

static size_t kvq_decode_smem_copies(const KvqProblem& P, int R, int copies) {
    const int threads = kvq_decode_threads(R, P.D), sub = threads;   // two tokens per score thread, half the threads score
    return sizeof(float) * ((size_t)P.G * 256 * R + 256 * (size_t)P.D * copies + (size_t)R * P.head_dim +
                            2 * (size_t)sub * R + 3 * (threads / 64) * (size_t)R + 3 * (size_t)R) +
           2 * sizeof(uint32_t) * (size_t)((P.G + 3) / 4) * (sub + kKvVctPad);
}

// Copies of the value codebook the decode kernel keeps in shared memory: 8 when that fits, else 1.
int kvq_decode_v_copies(const KvqProblem& P, int R) { return kvq_decode_smem_copies(P, R, 8) + 64 <= 227 * 1024 ? 8 : 1; }

size_t kvq_decode_smem(const KvqProblem& P, int R) { return kvq_decode_smem_copies(P, R, kvq_decode_v_copies(P, R)); }

// Splits of the context: a CTA's range is a multiple of 64 tokens; among the split counts the one with
// the least (waves of CTAs, one per SM) x (range + the table set-up and the fill and drain of the
// score/value pipeline, together worth about 1000 tokens) wins.
void plan_kvq_decode(KvqProblem& P, int T, int sms) {
    const int heads = P.B * P.Hkv, slots = sms;
    const int max_s = std::min(kKvMaxSplits, (T + 255) / 256);
    long best = -1;
    P.chunk = round_up(std::max(T, 1), 64);
    P.n_chunks = 1;
    for (int s = 1; s <= max_s; ++s) {
        const int span = round_up((T + s - 1) / s, 64);
        const int n = (T + span - 1) / span;
        const long waves = ((long)heads * n + slots - 1) / slots;
        const long cost = waves * (span + 1000);
        if (best < 0 || cost < best) {
            best = cost;
            P.chunk = span;
            P.n_chunks = n;
        }
    }
}

template <int D>
static int launch_append_t(const KvqProblem& P, cudaStream_t s) {
    const int tasks = 2 * P.Hkv * P.G, wpb = kKvThreads / 32;
    kvq_append_kernel<D><<<dim3((tasks + wpb - 1) / wpb, P.B), kKvThreads, 0, s>>>(P);
    OJX_CUDA_TRY(cudaGetLastError());
    count_launch(1);
    return OJX_OK;
}

int launch_kvq_append(const KvqProblem& P, cudaStream_t s) {
    if (!P.new_k || !P.new_v || !P.k_codes || !P.v_codes || !P.seq_lens) return OJX_ERR_ARG;
    if (P.G > kKvMaxGroups) return OJX_ERR_UNSUPPORTED;
    switch (P.D) {
        case 4: return launch_append_t<4>(P, s);
        case 8: return launch_append_t<8>(P, s);
        case 16: return launch_append_t<16>(P, s);
        default: return OJX_ERR_UNSUPPORTED;
    }
}

template <int R, int D>
static int launch_decode_t(const KvqProblem& P, cudaStream_t s, const PeerLink& link) {
    const size_t smem = kvq_decode_smem(P, R);
    if (smem + 64 > 227 * 1024) return OJX_ERR_TOO_LARGE;   // 64: the kernel's few static bytes
    KvqProblem Q = P;
    Q.v_copies = kvq_decode_v_copies(P, R);
    static thread_local size_t configured[64] = {};  // largest opt-in made for this instantiation, per device
    int cur_dev = 0;
    OJX_CUDA_TRY(cudaGetDevice(&cur_dev));
    if (cur_dev < 0 || cur_dev >= 64 || smem > configured[cur_dev]) {
        OJX_CUDA_TRY(cudaFuncSetAttribute(kvq_decode_kernel<R, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (cur_dev >= 0 && cur_dev < 64) configured[cur_dev] = smem;
    }
    kvq_decode_kernel<R, D><<<dim3(P.n_chunks, P.Hkv, P.B), kvq_decode_threads(R, D), smem, s>>>(Q, link);
    OJX_CUDA_TRY(cudaGetLastError());
    count_launch(1);
    return OJX_OK;
}

template <int R>
static int launch_decode_r(const KvqProblem& P, cudaStream_t s, const PeerLink& link) {
    switch (P.D) {
        case 4: return launch_decode_t<R, 4>(P, s, link);
        case 8: return launch_decode_t<R, 8>(P, s, link);
        case 16: return launch_decode_t<R, 16>(P, s, link);
        default: return OJX_ERR_UNSUPPORTED;
    }
}

int launch_kvq_decode(const KvqProblem& P, cudaStream_t s, const PeerLink* lk) {
    const PeerLink none{};
    const PeerLink& link = lk ? *lk : none;
    if (!P.q || !P.out || !P.partials || !P.seq_lens) return OJX_ERR_ARG;
    if (P.G > kKvMaxGroups || P.Hq % P.Hkv != 0) return OJX_ERR_UNSUPPORTED;
    if (P.head_dim > 2 * kKvThreads || P.head_dim % 4 != 0) return OJX_ERR_UNSUPPORTED;
    switch (P.Hq / P.Hkv) {
        case 1: return launch_decode_r<1>(P, s, link);
        case 2: return launch_decode_r<2>(P, s, link);
        case 4: return launch_decode_r<4>(P, s, link);
        case 8: return launch_decode_r<8>(P, s, link);
        default: return OJX_ERR_UNSUPPORTED;
    }
}

// ------------------------------------------------------------------------------ legacy cache
// ojasx_lut_kv_cache.cpp:16-65 for one head: abs-max scale, then per block the first coordinate
// as round(val/scale) clamped to [-128,127], stored +128.
__global__ void legacy_append_kernel(const float* __restrict__ k, const float* __restrict__ v, int head_dim,
                                     int block_dim, uint8_t* k_row, uint8_t* v_row, float* k_scale, float* v_scale) {
    __shared__ float red[128];
    const int G = head_dim / block_dim;
    for (int which = 0; which < 2; ++which) {
        const float* src = which ? v : k;
        float m = 1e-8f;
        for (int d = threadIdx.x; d < head_dim; d += blockDim.x) m = fmaxf(m, fabsf(src[d]));
        red[threadIdx.x] = m;
        __syncthreads();
        for (int s = blockDim.x / 2; s > 0; s >>= 1) {
            if (threadIdx.x < s) red[threadIdx.x] = fmaxf(red[threadIdx.x], red[threadIdx.x + s]);
            __syncthreads();
        }
        const float scale = __fdiv_rn(red[0], 127.0f);
        __syncthreads();
        if (threadIdx.x == 0) *(which ? v_scale : k_scale) = scale;
        for (int g = threadIdx.x; g < G; g += blockDim.x) {
            int q = (int)roundf(__fdiv_rn(src[g * block_dim], scale));
            q = max(-128, min(127, q));
            (which ? v_row : k_row)[g] = (uint8_t)(q + 128);
        }
    }
}

// Attention of one head over T cached tokens (ojasx_lut_kv_cache.cpp:67-132 and the softmax of
// ojasx_lut_c_api.cpp:178-191), one CTA.  logits live in global scratch [T].
__global__ void __launch_bounds__(256) legacy_attention_kernel(const float* __restrict__ q, int head_dim, int block_dim, int T,
                                                               const uint8_t* __restrict__ k_codes,
                                                               const uint8_t* __restrict__ v_codes,
                                                               const float* __restrict__ k_scales,
                                                               const float* __restrict__ v_scales, float scale_factor,
                                                               float* __restrict__ logits, float* __restrict__ out) {
    extern __shared__ float lut[];  // [G*256]
    __shared__ float red[256];
    const int G = head_dim / block_dim, tid = threadIdx.x;
    if (scale_factor <= 0.0f) scale_factor = __fdiv_rn(1.0f, sqrtf((float)head_dim));
    for (int i = tid; i < G * 256; i += blockDim.x) lut[i] = __fmul_rn(q[(i >> 8) * block_dim], (float)((i & 255) - 128));
    __syncthreads();
    float m = -INFINITY;
    for (int t = tid; t < T; t += blockDim.x) {
        float s = 0.0f;
        for (int g = 0; g < G; ++g) s = __fadd_rn(s, lut[g * 256 + k_codes[(size_t)t * G + g]]);
        const float l = __fmul_rn(__fmul_rn(s, k_scales[t]), scale_factor);
        logits[t] = l;
        m = fmaxf(m, l);
    }
    red[tid] = m;
    __syncthreads();
    for (int s = blockDim.x / 2; s > 0; s >>= 1) {
        if (tid < s) red[tid] = fmaxf(red[tid], red[tid + s]);
        __syncthreads();
    }
    m = red[0];
    __syncthreads();
    float sum = 0.0f;
    for (int t = tid; t < T; t += blockDim.x) {
        const float e = (float)exp((double)__fsub_rn(logits[t], m));
        logits[t] = e;
        sum += e;
    }
    red[tid] = sum;
    __syncthreads();
    for (int s = blockDim.x / 2; s > 0; s >>= 1) {
        if (tid < s) red[tid] += red[tid + s];
        __syncthreads();
    }
    const float inv = __fdiv_rn(1.0f, red[0]);
    __syncthreads();
    for (int d = tid; d < head_dim; d += blockDim.x) out[d] = 0.0f;
    __syncthreads();
    // context: warp per group, lanes over tokens, fixed-shape shuffle reduction
    const int warp = tid >> 5, lane = tid & 31, nw = blockDim.x >> 5;
    for (int g = warp; g < G; g += nw) {
        float acc = 0.0f;
        for (int t = lane; t < T; t += 32) {
            const float w = __fmul_rn(__fmul_rn(logits[t], inv), v_scales[t]);
            acc += (float)((int)v_codes[(size_t)t * G + g] - 128) * w;
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
        if (lane == 0) out[g * block_dim] = acc;
    }
}

int launch_legacy_append(const float* k, const float* v, int head_dim, int block_dim, uint8_t* k_row, uint8_t* v_row,
                         float* k_scale, float* v_scale, cudaStream_t s) {
    legacy_append_kernel<<<1, 128, 0, s>>>(k, v, head_dim, block_dim, k_row, v_row, k_scale, v_scale);
    OJX_CUDA_TRY(cudaGetLastError());
    count_launch(1);
    return OJX_OK;
}

int launch_legacy_attention(const float* q, int head_dim, int block_dim, int T, const uint8_t* k_codes,
                            const uint8_t* v_codes, const float* k_scales, const float* v_scales, float scale_factor,
                            float* logits, float* out, cudaStream_t s) {
    const int G = head_dim / block_dim;
    if (G > 128) return OJX_ERR_UNSUPPORTED;
    const size_t smem = sizeof(float) * (size_t)G * 256;
    if (smem > 48 * 1024)
        OJX_CUDA_TRY(cudaFuncSetAttribute(legacy_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    legacy_attention_kernel<<<1, 256, smem, s>>>(q, head_dim, block_dim, T, k_codes, v_codes, k_scales, v_scales,
                                                 scale_factor, logits, out);
    OJX_CUDA_TRY(cudaGetLastError());
    count_launch(1);
    return OJX_OK;
}

}  // namespace ojx

