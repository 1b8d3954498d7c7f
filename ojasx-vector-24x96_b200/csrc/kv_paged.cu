// Paged int8 KV cache (the reference's PagedCompressedKVCache, ojasx_24x96/long_context.py:212-279):
// every cached token's key and value vector is int8 with one symmetric scale per token (abs-max / 127,
// stored as fp16), pages hold up to page_size tokens, and the host keeps the list of resident pages
// (sink pages + sliding window).
//
// paged_quantize_kernel: one warp per token vector; abs-max by shuffles, q = clamp(rint(t / scale), +-127)
// with the fp32 scale and IEEE division, exactly the arithmetic of _quantize_int8 (:236-241).
//
// paged_decode_kernel: attention of one new query over all resident tokens, straight on the int8 pages
// (the reference dequantises page after page and feeds OnlineSoftmaxBlockAttention, :259-267).  grid =
// (context splits, query heads, batch).  A warp takes one token at a time: each lane holds D/32 query
// values and loads the matching D/32 bytes of the key row and of the value row (one coalesced row per
// warp), the dot product is a shuffle tree, and the warp keeps its own running maximum, normaliser and
// output slice (online softmax).  The warps of a CTA are merged in shared memory, the splits of a
// (sequence, head) by the CTA that finishes last (atomic count after a device-wide fence).  Bound: HBM
// (2 * (D + 2) bytes per token and KV head).
#include <cuda_fp16.h>

#include "common.cuh"
#include "launch.h"
#include "handles.h"
#include "../../include/ojasx_lut_b200.h"

namespace ojx {

constexpr int kPgThreads = 256;
constexpr int kPgWarps = kPgThreads / 32;
constexpr int kPgUnroll = 4;   // tokens a warp has in flight

__device__ __forceinline__ float pg_load(const void* p, size_t i, int dt) {
    return dt == OJX_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]) : reinterpret_cast<const float*>(p)[i];
}

// src [n_vectors, D] io dtype -> q8 [n_vectors, D] int8, scales [n_vectors] fp16
__global__ void __launch_bounds__(kPgThreads) paged_quantize_kernel(const void* __restrict__ src, int io_dtype, size_t n_vectors,
                                                                    int D, int8_t* __restrict__ q8, __half* __restrict__ scales) {
    const size_t v = ((size_t)blockIdx.x * kPgThreads + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (v >= n_vectors) return;
    float amax = 0.0f;
    for (int d = lane; d < D; d += 32) amax = fmaxf(amax, fabsf(pg_load(src, v * D + d, io_dtype)));
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    const float scale = __fdiv_rn(fmaxf(amax, 1e-8f), 127.0f);
    for (int d = lane; d < D; d += 32) {
        const float r = rintf(__fdiv_rn(pg_load(src, v * D + d, io_dtype), scale));   // round half to even, like torch.round
        q8[v * D + d] = (int8_t)fminf(fmaxf(r, -127.0f), 127.0f);
    }
    if (lane == 0) scales[v] = __float2half_rn(scale);
}

struct PagedDecodeProblem {
    const void* q;            // [B, Hq, D] io dtype
    void* out;                // [B, Hq, D] io dtype
    const int8_t* k_pool;     // [slots, B, Hkv, page_size, D]
    const int8_t* v_pool;
    const __half* ks_pool;    // [slots, B, Hkv, page_size]
    const __half* vs_pool;
    const int* page_slot;     // [n_pages] pool slot of each resident page, oldest first
    const int* page_start;    // [n_pages + 1] first token of each page in the resident order (prefix sums)
    float* partials;          // [B, Hq, n_chunks, D + 2]
    int* done;                // [B, Hq] zeroed counters (they return to zero)
    int n_pages, B, Hq, Hkv, D, page_size, io_dtype, chunk, n_chunks;
    float scale;
};

// EPL int8 values of one lane, kept packed in a register word until they are used
template <int EPL> struct PackedWord;
template <> struct PackedWord<2> { using type = unsigned short; };
template <> struct PackedWord<4> { using type = unsigned; };
template <> struct PackedWord<8> { using type = unsigned long long; };

template <int EPL>
struct PackedRow {
    using word = typename PackedWord<EPL>::type;
    word k, v;
    float ks, vs;
    __device__ static __forceinline__ float get(word w, int e) { return (float)(signed char)((w >> (8 * e)) & 0xff); }
};

template <int EPL>   // elements per lane = D / 32
__global__ void __launch_bounds__(kPgThreads) paged_decode_kernel(const __grid_constant__ PagedDecodeProblem P) {
    __shared__ float sm_m[kPgWarps], sm_l[kPgWarps];
    __shared__ float sm_o[kPgWarps][32 * EPL];
    __shared__ int s_last;
    using Packed = PackedRow<EPL>;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int split = blockIdx.x, hq = blockIdx.y, b = blockIdx.z;
    const int hkv = hq / (P.Hq / P.Hkv), D = 32 * EPL;
    const int total = P.page_start[P.n_pages];
    const int t0 = split * P.chunk, t1 = min(total, t0 + P.chunk);
    float qv[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) qv[e] = pg_load(P.q, ((size_t)b * P.Hq + hq) * D + lane * EPL + e, P.io_dtype) * P.scale;
    float m = -INFINITY, l = 0.0f, o[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) o[e] = 0.0f;
    // pages that overlap [t0, t1); inside a page tokens are consecutive rows
    for (int p = 0; p < P.n_pages; ++p) {
        const int ps = P.page_start[p], pe = P.page_start[p + 1];
        if (pe <= t0 || ps >= t1) continue;
        const size_t row0 = (((size_t)P.page_slot[p] * P.B + b) * P.Hkv + hkv) * P.page_size;
        const int first = max(ps, t0) - ps, last = min(pe, t1) - ps;
        // kPgUnroll tokens of this warp per step: their bytes and scales are requested together (and stay packed
        // in registers until used; more registers per thread cost more in occupancy than a deeper pipeline gains)
        Packed cur[kPgUnroll];
        auto fetch = [&](int rb, Packed (&dst)[kPgUnroll]) {
#pragma unroll
            for (int u = 0; u < kPgUnroll; ++u) {
                const int r = rb + u * kPgWarps;
                const bool live = r < last;
                const size_t row = row0 + (live ? r : first);
                dst[u].k = *reinterpret_cast<const typename Packed::word*>(P.k_pool + row * D + lane * EPL);
                dst[u].v = *reinterpret_cast<const typename Packed::word*>(P.v_pool + row * D + lane * EPL);
                dst[u].ks = live ? __half2float(P.ks_pool[row]) : 0.0f;
                dst[u].vs = live ? __half2float(P.vs_pool[row]) : 0.0f;
            }
        };
        for (int rb = first + warp; rb < last; rb += kPgWarps * kPgUnroll) {
            fetch(rb, cur);
            float sc[kPgUnroll], mn = m;
#pragma unroll
            for (int u = 0; u < kPgUnroll; ++u) {
                float dot = 0.0f;
#pragma unroll
                for (int e = 0; e < EPL; ++e) dot = fmaf(qv[e], Packed::get(cur[u].k, e), dot);
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
                sc[u] = rb + u * kPgWarps < last ? dot * cur[u].ks : -INFINITY;
                mn = fmaxf(mn, sc[u]);
            }
            const float alpha = __expf(m - mn);   // the first token of the step is always live, so mn is finite
            l *= alpha;
#pragma unroll
            for (int e = 0; e < EPL; ++e) o[e] *= alpha;
#pragma unroll
            for (int u = 0; u < kPgUnroll; ++u) {
                const float pr = __expf(sc[u] - mn);   // 0 for a token beyond the range
                const float pv = pr * cur[u].vs;
                l += pr;
#pragma unroll
                for (int e = 0; e < EPL; ++e) o[e] = fmaf(pv, Packed::get(cur[u].v, e), o[e]);
            }
            m = mn;
        }
    }
    // merge the warps (each lane owns EPL output columns)
    if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
#pragma unroll
    for (int e = 0; e < EPL; ++e) sm_o[warp][lane * EPL + e] = o[e];
    __syncthreads();
    float* part = P.partials + (((size_t)b * P.Hq + hq) * P.n_chunks + split) * (D + 2);
    float M = -INFINITY;
    for (int w = 0; w < kPgWarps; ++w) M = fmaxf(M, sm_m[w]);
    if (tid < D) {
        float acc = 0.0f;
        for (int w = 0; w < kPgWarps; ++w)
            if (sm_m[w] != -INFINITY) acc = fmaf(sm_o[w][tid], __expf(sm_m[w] - M), acc);
        part[2 + tid] = acc;
    }
    if (tid == 0) {
        float L = 0.0f;
        for (int w = 0; w < kPgWarps; ++w)
            if (sm_m[w] != -INFINITY) L += sm_l[w] * __expf(sm_m[w] - M);
        part[0] = M;
        part[1] = L;
    }
    // the CTA that finishes last merges the splits of this (sequence, head)
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        int* cnt = P.done + (size_t)b * P.Hq + hq;
        const int last = atomicAdd(cnt, 1) == P.n_chunks - 1;
        if (last) *cnt = 0;
        s_last = last;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const float* base = P.partials + (((size_t)b * P.Hq + hq) * P.n_chunks) * (D + 2);
    if (tid < D) {
        float MM = -INFINITY;
        for (int c = 0; c < P.n_chunks; ++c) MM = fmaxf(MM, __ldcg(base + (size_t)c * (D + 2)));
        float LL = 0.0f, acc = 0.0f;
        for (int c = 0; c < P.n_chunks; ++c) {
            const float* pc = base + (size_t)c * (D + 2);
            const float mc = __ldcg(pc);
            if (mc != -INFINITY) {
                const float wgt = __expf(mc - MM);
                LL += __ldcg(pc + 1) * wgt;
                acc = fmaf(__ldcg(pc + 2 + tid), wgt, acc);
            }
        }
        acc *= LL > 0.0f ? 1.0f / LL : 0.0f;
        const size_t oi = ((size_t)b * P.Hq + hq) * D + tid;
        if (P.io_dtype == OJX_BF16) reinterpret_cast<__nv_bfloat16*>(P.out)[oi] = __float2bfloat16_rn(acc);
        else reinterpret_cast<float*>(P.out)[oi] = acc;
    }
}

}  // namespace ojx

using namespace ojx;

extern "C" {

int ojasx_b200_paged_kv_quantize(const void* d_src, int io_dtype, size_t n_vectors, int head_dim, int8_t* d_q8,
                                 void* d_scales_f16, void* stream) {
    if (!d_src || !d_q8 || !d_scales_f16 || head_dim <= 0) return OJX_ERR_ARG;
    if (io_dtype != OJX_F32 && io_dtype != OJX_BF16) return OJX_ERR_ARG;
    if (n_vectors == 0) return OJX_OK;
    const size_t blocks = (n_vectors * 32 + kPgThreads - 1) / kPgThreads;
    if (blocks > 0x7fffffffULL) return OJX_ERR_TOO_LARGE;
    paged_quantize_kernel<<<(unsigned)blocks, kPgThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        d_src, io_dtype, n_vectors, head_dim, d_q8, static_cast<__half*>(d_scales_f16));
    OJX_CUDA_TRY(cudaGetLastError());
    count_launch(1);
    return OJX_OK;
}

int ojasx_b200_paged_kv_scratch_floats(int batch, int q_heads, int head_dim, int max_tokens) {
    const int max_chunks = (max_tokens + 255) / 256;
    return batch * q_heads * max_chunks * (head_dim + 2);
}

int ojasx_b200_paged_kv_decode(const void* d_q, void* d_out, const int8_t* d_k_pool, const int8_t* d_v_pool,
                               const void* d_k_scales_f16, const void* d_v_scales_f16, const int* d_page_slot,
                               const int* d_page_start, int n_pages, int total_tokens, int batch, int q_heads, int kv_heads,
                               int head_dim, int page_size, float scale, int io_dtype, float* d_scratch, int* d_counters,
                               void* stream) {
    if (!d_q || !d_out || !d_k_pool || !d_v_pool || !d_k_scales_f16 || !d_v_scales_f16 || !d_page_slot || !d_page_start ||
        !d_scratch || !d_counters)
        return OJX_ERR_ARG;
    if (n_pages <= 0 || total_tokens <= 0 || batch <= 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads || page_size <= 0)
        return OJX_ERR_ARG;
    if (io_dtype != OJX_F32 && io_dtype != OJX_BF16) return OJX_ERR_ARG;
    if (head_dim != 64 && head_dim != 128 && head_dim != 256) return OJX_ERR_UNSUPPORTED;
    PagedDecodeProblem P{};
    P.q = d_q; P.out = d_out; P.k_pool = d_k_pool; P.v_pool = d_v_pool;
    P.ks_pool = static_cast<const __half*>(d_k_scales_f16); P.vs_pool = static_cast<const __half*>(d_v_scales_f16);
    P.page_slot = d_page_slot; P.page_start = d_page_start; P.partials = d_scratch; P.done = d_counters;
    P.n_pages = n_pages; P.B = batch; P.Hq = q_heads; P.Hkv = kv_heads; P.D = head_dim; P.page_size = page_size;
    P.io_dtype = io_dtype;
    P.scale = scale > 0.0f ? scale : 1.0f / sqrtf((float)head_dim);
    // context splits: about six CTAs per SM in all (the kernel is latency-bound per warp, so it wants the SMs
    // full of warps), ranges of at least 256 tokens
    const int heads = batch * q_heads, want = (6 * num_sms() + heads - 1) / heads;
    int chunk = round_up((total_tokens + want - 1) / want, 256);
    if (chunk < 256) chunk = 256;
    P.chunk = chunk;
    P.n_chunks = (total_tokens + chunk - 1) / chunk;
    const dim3 grid(P.n_chunks, q_heads, batch);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (head_dim) {
        case 64: paged_decode_kernel<2><<<grid, kPgThreads, 0, s>>>(P); break;
        case 128: paged_decode_kernel<4><<<grid, kPgThreads, 0, s>>>(P); break;
        default: paged_decode_kernel<8><<<grid, kPgThreads, 0, s>>>(P); break;
    }
    OJX_CUDA_TRY(cudaGetLastError());
    count_launch(1);
    return OJX_OK;
}

}  // extern "C"
