// Residual-VQ layers in the package's bit-packed layout (ojasx_24x96/codec.py:176-214: code i of a
// stage sits in bits [(i mod per_byte)*bits, ...) of byte i / per_byte) for every supported width
// (1, 2, 4, 8 bits) and stage count.  Same computation as ojasx_rvq_fused_gemm
// (ojasx_24x96/native/leech24_cpu.cpp:372-483) and ojasx_rvq_fused_gemv_cuda_kernel
// (ojasx_24x96/native/vq_kernels_cuda.cu:83-147): per block, sum the stage codebook entries, dot
// with the activation block, accumulate over blocks, then scale and bias.
//
// 8-bit single-stage layers do not come here: they are the split-manifold layout and run on the
// table kernels of linear.cu.  This kernel is the compatibility path for the other widths: one
// warp per (batch item, row), lanes stride over the row's blocks, fixed-shape shuffle reduction.
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

int launch_rvq_generic(const uint8_t* packed, const float* codebooks, const float* row_scales, const float* bias,
                       const float* x, int batch, int stages, int bits, int D, int rows, int columns, int row_start,
                       int row_stop, float* out, cudaStream_t s) {
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
