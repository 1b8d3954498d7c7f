// Residual-VQ layers in the package's bit-packed layout (ojasx_24x96/codec.py:176-214: code i of a
// stage sits in bits [(i mod per_byte)*bits, ...) of byte i / per_byte) for every supported width
// (1, 2, 4, 8 bits) and stage count.  Same computation as ojasx_rvq_fused_gemm
// (ojasx_24x96/native/leech24_cpu.cpp:372-483) and ojasx_rvq_fused_gemv_cuda_kernel
// (ojasx_24x96/native/vq_kernels_cuda.cu:83-147): per block, sum the stage codebook entries, dot
// with the activation block, accumulate over blocks, then scale and bias.
//
// 8-bit single-stage layers do not come here: they are the split-manifold layout and run on the
// table kernels of linear.cu.  Narrow widths (1, 2, 4 bits) with word-aligned rows run on the table
// kernel at the end of this file; rvq_generic_kernel is the compatibility path for everything else: one
// warp per (batch item, row), lanes stride over the row's blocks, fixed-shape shuffle reduction.
#include <cstdlib>

#include "common.cuh"
#include "launch.h"
#include "handles.h"

namespace ojx {

__global__ void __launch_bounds__(256) rvq_generic_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ codebooks,
                                                          const float* __restrict__ row_scales, const float* __restrict__ bias,
                                                          const float* __restrict__ x, int batch, int stages, int bits, int D,
                                                          int rows, int columns, int row_start, int row_stop,
                                                          float* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const long long item = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int row_count = row_stop - row_start;
    if (item >= (long long)batch * row_count) return;
    const int b = (int)(item / row_count), r = row_start + (int)(item - (long long)b * row_count);
    const int G = (columns + D - 1) / D;
    const size_t total_vectors = (size_t)rows * G;
    const size_t stage_stride = (total_vectors * bits + 7) / 8;
    const unsigned mask = (1u << bits) - 1u;
    const int Q = 1 << bits;
    const float* xb = x + (size_t)b * columns;
    float acc = 0.0f;
    for (int blk = lane; blk < G; blk += 32) {
        const size_t bit_pos = ((size_t)r * G + blk) * bits;
        const size_t byte_pos = bit_pos >> 3;
        const unsigned shift = (unsigned)(bit_pos & 7);
        const int c0 = blk * D, cn = min(D, columns - c0);
        float dot = 0.0f;
        for (int c = 0; c < cn; ++c) {
            float w = 0.0f;
            for (int s = 0; s < stages; ++s) {
                const unsigned code = (packed[(size_t)s * stage_stride + byte_pos] >> shift) & mask;
                w += codebooks[((size_t)s * Q + code) * D + c];
            }
            dot = fmaf(xb[c0 + c], w, dot);
        }
        acc += dot;
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0) out[(size_t)b * row_count + (r - row_start)] = acc * row_scales[r] + (bias ? bias[r] : 0.0f);
}

// Table form for the narrow widths (1, 2, 4 bits; the reference's default artefacts are 4 bits x 4 stages):
// T[s, g, q] = <x_g, C_s[q]> for every stage, group and codebook entry is tiny (stages * G * 2^bits floats,
// 80 KB for 4 x 320 x 16), so a CTA builds all of it and a row costs stages * G table reads, with no weight
// ever dequantised -- the computation of subspace_lut_rvq_gemm (ojasx_24x96/math_engine.py:172-203) rather than
// the dequantise-and-dot of the compatibility kernel above (the two differ in summation order only).
// A warp takes four rows, eight lanes each: lane t of a row reads the row's 32-bit code words t, t + 8, ...
// of every stage (coalesced across the eight lanes) and adds its table entries; a fixed xor tree joins the
// eight partial sums.  Needs word-aligned rows: G * bits a multiple of 32.
constexpr int kRvqLutThreads = 256;
constexpr int kRvqLutRows = kRvqLutThreads / 8;   // rows per CTA pass

template <int BITS>
__global__ void __launch_bounds__(kRvqLutThreads) rvq_lut_kernel(const uint8_t* __restrict__ packed,
                                                                 const float* __restrict__ codebooks,
                                                                 const float* __restrict__ row_scales,
                                                                 const float* __restrict__ bias, const float* __restrict__ x,
                                                                 int batch, int stages, int D, int rows, int columns,
                                                                 int row_start, int row_stop, float* __restrict__ out) {
    extern __shared__ __align__(16) float rvq_smem[];
    constexpr int Q = 1 << BITS, CPW = 32 / BITS;
    constexpr unsigned mask = Q - 1;
    const int G = (columns + D - 1) / D;
    float* lut = rvq_smem;                        // [stages][G][Q]
    float* xs = lut + (size_t)stages * G * Q;     // [G * D], zero beyond `columns`
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, t = lane & 7;
    const int row_count = row_stop - row_start;
    const int tiles = (row_count + kRvqLutRows - 1) / kRvqLutRows;
    const int wpr = G * BITS / 32;                // code words per row and stage
    const size_t stage_words = (size_t)rows * wpr;
    const unsigned* words = reinterpret_cast<const unsigned*>(packed);
    for (int b = 0; b < batch; ++b) {
        for (int i = tid; i < G * D; i += kRvqLutThreads) xs[i] = i < columns ? x[(size_t)b * columns + i] : 0.0f;
        __syncthreads();
        {   // thread = (codebook entry q, group slot): no runtime division, consecutive threads write consecutive cells
            const int q = tid & (Q - 1), gslot = tid >> BITS;
            constexpr int kSlots = kRvqLutThreads >> BITS;
            for (int s = 0; s < stages; ++s) {
                const float* c = codebooks + ((size_t)s * Q + q) * D;
                float* ls = lut + (size_t)s * G * Q;
                for (int g = gslot; g < G; g += kSlots) {
                    const float* xg = xs + g * D;
                    float dot = 0.0f;
                    for (int d = 0; d < D; d += 4) {   // block sizes are multiples of 4
                        const float4 xv = *reinterpret_cast<const float4*>(xg + d);
                        const float4 cv = *reinterpret_cast<const float4*>(c + d);
                        dot = fmaf(xv.x, cv.x, dot); dot = fmaf(xv.y, cv.y, dot);
                        dot = fmaf(xv.z, cv.z, dot); dot = fmaf(xv.w, cv.w, dot);
                    }
                    ls[g * Q + q] = dot;
                }
            }
        }
        __syncthreads();
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
            const int r = row_start + tile * kRvqLutRows + warp * 4 + (lane >> 3);
            float acc = 0.0f;
            if (r < row_stop) {
                for (int s = 0; s < stages; ++s) {
                    const unsigned* rw = words + (size_t)s * stage_words + (size_t)r * wpr;
                    const float* ls = lut + (size_t)s * G * Q;
                    for (int w0 = t; w0 < wpr; w0 += 8 * 4) {   // four words of this lane in flight
                        unsigned word[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) word[u] = w0 + 8 * u < wpr ? rw[w0 + 8 * u] : 0u;
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            if (w0 + 8 * u < wpr) {
                                const float* lw = ls + (size_t)(w0 + 8 * u) * CPW * Q;
#pragma unroll
                                for (int j = 0; j < CPW; ++j) acc += lw[j * Q + ((word[u] >> (j * BITS)) & mask)];
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int off = 1; off <= 4; off <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
            if (t == 0 && r < row_stop)
                out[(size_t)b * row_count + (r - row_start)] = acc * row_scales[r] + (bias ? bias[r] : 0.0f);
        }
        __syncthreads();   // the next batch row rebuilds the table
    }
}

// OJX_ERR_UNSUPPORTED: the caller uses the compatibility kernel.
static int launch_rvq_lut(const uint8_t* packed, const float* codebooks, const float* row_scales, const float* bias,
                          const float* x, int batch, int stages, int bits, int D, int rows, int columns, int row_start,
                          int row_stop, float* out, cudaStream_t s) {
    if (bits != 1 && bits != 2 && bits != 4) return OJX_ERR_UNSUPPORTED;
    const int G = (columns + D - 1) / D;
    if ((G * bits) % 32 != 0 || (reinterpret_cast<uintptr_t>(packed) & 3)) return OJX_ERR_UNSUPPORTED;
    const size_t smem = sizeof(float) * ((size_t)stages * G * (1 << bits) + (size_t)G * D);
    if (smem > 200 * 1024) return OJX_ERR_UNSUPPORTED;
    const int tiles = (row_stop - row_start + kRvqLutRows - 1) / kRvqLutRows;
    const int cap = 8 * num_sms();
    const int grid = tiles < cap ? tiles : cap;
    if (D % 4 != 0 || (reinterpret_cast<uintptr_t>(codebooks) & 15)) return OJX_ERR_UNSUPPORTED;
    auto go = [&](auto kern) -> int {
        static thread_local size_t opted[16][3] = {};   // largest opt-in so far, per device and width
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) dev = 0;
        size_t& have = opted[dev][bits == 1 ? 0 : bits == 2 ? 1 : 2];
        if (smem > 48 * 1024 && smem > have) {
            OJX_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            have = smem;
        }
        kern<<<grid, kRvqLutThreads, smem, s>>>(packed, codebooks, row_scales, bias, x, batch, stages, D, rows, columns,
                                                row_start, row_stop, out);
        OJX_CUDA_TRY(cudaGetLastError());
        count_launch(1);
        return OJX_OK;
    };
    switch (bits) {
        case 1: return go(rvq_lut_kernel<1>);
        case 2: return go(rvq_lut_kernel<2>);
        default: return go(rvq_lut_kernel<4>);
    }
}

int launch_rvq_generic(const uint8_t* packed, const float* codebooks, const float* row_scales, const float* bias,
                       const float* x, int batch, int stages, int bits, int D, int rows, int columns, int row_start,
                       int row_stop, float* out, cudaStream_t s) {
    if (!getenv("OJASX_B200_RVQ_COMPAT")) {   // set to force the compatibility kernel (tests compare the two)
        const int rc = launch_rvq_lut(packed, codebooks, row_scales, bias, x, batch, stages, bits, D, rows, columns, row_start,
                                      row_stop, out, s);
        if (rc != OJX_ERR_UNSUPPORTED) return rc;
    }
    const long long items = (long long)batch * (row_stop - row_start);
    const long long blocks = (items * 32 + 255) / 256;
    if (blocks > 0x7fffffffLL) return OJX_ERR_TOO_LARGE;
    rvq_generic_kernel<<<(unsigned)blocks, 256, 0, s>>>(packed, codebooks, row_scales, bias, x, batch, stages, bits, D, rows,
                                                         columns, row_start, row_stop, out);
    OJX_CUDA_TRY(cudaGetLastError());
    count_launch(1);
    return OJX_OK;
}

}  // namespace ojx
