// Small per-token operators around the VQ kernels of a decoder step, so that a whole step is a short,
// fixed sequence of launches that can be captured in a CUDA graph: RMSNorm, rotary embedding of q and k
// at per-sequence positions held on the device, and the position bump.  (The reference leaves these to
// the HuggingFace model classes it drives, ojasx_24x96/engine.py:176-199.)
#include "common.cuh"
#include "launch.h"
#include "handles.h"
#include "../../include/ojasx_lut_b200.h"

namespace ojx {

__device__ __forceinline__ float ld_io(const void* p, size_t i, int dt) {
    return dt == OJX_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]) : reinterpret_cast<const float*>(p)[i];
}
__device__ __forceinline__ void st_io(void* p, size_t i, int dt, float v) {
    if (dt == OJX_BF16) reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
    else reinterpret_cast<float*>(p)[i] = v;
}

// out[r, :] = x[r, :] * rsqrt(mean(x[r, :]^2) + eps) * w ; optionally x[r, :] += add[r, :] first
// (the residual add that precedes the norm), with the sum also written back to x.  A thread keeps its
// elements in registers between the two passes (up to kNormKeep of them; rows longer than
// 256 * kNormKeep re-read the rest), and the row sum is a shuffle tree per warp plus one exchange.
constexpr int kNormKeep = 16;

__global__ void __launch_bounds__(256) rmsnorm_kernel(void* __restrict__ x, const void* __restrict__ add,
                                                      const float* __restrict__ w, void* __restrict__ out, int H, float eps,
                                                      int io_dtype) {
    __shared__ float red[8];
    const size_t base = (size_t)blockIdx.x * H;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float keep[kNormKeep];
    float ss = 0.0f;
    auto element = [&](int i) {   // the (updated) value of x[r, i] as it is stored, i.e. rounded to the io dtype
        float v = ld_io(x, base + i, io_dtype);
        if (add) {
            v += ld_io(add, base + i, io_dtype);
            if (io_dtype == OJX_BF16) v = __bfloat162float(__float2bfloat16_rn(v));
            st_io(x, base + i, io_dtype, v);
        }
        return v;
    };
    float wk[kNormKeep];   // the weights do not depend on the row sum: asked for now, used after it
#pragma unroll
    for (int u = 0; u < kNormKeep; ++u) {
        const int i = tid + u * 256;
        keep[u] = i < H ? element(i) : 0.0f;
        wk[u] = i < H ? w[i] : 0.0f;
        ss += keep[u] * keep[u];
    }
    for (int i = tid + kNormKeep * 256; i < H; i += 256) {
        const float v = element(i);
        ss += v * v;
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) total += red[k];
    const float inv = rsqrtf(total / (float)H + eps);
#pragma unroll
    for (int u = 0; u < kNormKeep; ++u) {
        const int i = tid + u * 256;
        if (i < H) st_io(out, base + i, io_dtype, keep[u] * inv * wk[u]);
    }
    for (int i = tid + kNormKeep * 256; i < H; i += 256) st_io(out, base + i, io_dtype, ld_io(x, base + i, io_dtype) * inv * w[i]);
}

// Rotate-half rotary embedding in place on q [B, Hq, hd] and k [B, Hkv, hd] at positions pos[b].
// grid = (heads of q and k, batch): a block turns one head, a thread one pair, so that a single sequence still
// spreads over forty SMs instead of one block looping ten times over slow-path powf / sincosf.
__global__ void rope_qk_kernel(void* __restrict__ q, void* __restrict__ k, const int* __restrict__ pos, int Hq, int Hkv,
                               int hd, float theta, int io_dtype) {
    const int b = blockIdx.y, head = blockIdx.x, half = hd >> 1;
    const float p = (float)pos[b];
    void* buf = head < Hq ? q : k;
    const size_t base = head < Hq ? ((size_t)b * Hq + head) * hd : ((size_t)b * Hkv + (head - Hq)) * hd;
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        const float x1 = ld_io(buf, base + j, io_dtype), x2 = ld_io(buf, base + half + j, io_dtype);
        const float inv = 1.0f / powf(theta, (float)(2 * j) / (float)hd);
        float s, c;
        sincosf(p * inv, &s, &c);
        st_io(buf, base + j, io_dtype, x1 * c - x2 * s);
        st_io(buf, base + half + j, io_dtype, x2 * c + x1 * s);
    }
}

__global__ void add_int_kernel(int* p, int n, int delta) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] += delta;
}

}  // namespace ojx

using namespace ojx;

extern "C" {

int ojasx_b200_rmsnorm(void* d_x, const void* d_add, const float* d_weight, void* d_out, int rows, int hidden, float eps,
                       int io_dtype, void* stream) {
    if (!d_x || !d_weight || !d_out || rows <= 0 || hidden <= 0) return OJX_ERR_ARG;
    if (io_dtype != OJX_F32 && io_dtype != OJX_BF16) return OJX_ERR_ARG;
    rmsnorm_kernel<<<rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(d_x, d_add, d_weight, d_out, hidden, eps, io_dtype);
    OJX_CUDA_TRY(cudaGetLastError());
    count_launch(1);
    return OJX_OK;
}

int ojasx_b200_rope_qk(void* d_q, void* d_k, const int* d_positions, int batch, int q_heads, int kv_heads, int head_dim,
                       float theta, int io_dtype, void* stream) {
    if (!d_q || !d_k || !d_positions || batch <= 0 || q_heads <= 0 || kv_heads <= 0 || head_dim <= 0 || (head_dim & 1)) return OJX_ERR_ARG;
    if (io_dtype != OJX_F32 && io_dtype != OJX_BF16) return OJX_ERR_ARG;
    if (batch > 65535) return OJX_ERR_TOO_LARGE;   // a grid row per sequence
    rope_qk_kernel<<<dim3(q_heads + kv_heads, batch), (head_dim / 2 + 31) / 32 * 32 < 256 ? (head_dim / 2 + 31) / 32 * 32 : 256, 0, static_cast<cudaStream_t>(stream)>>>(d_q, d_k, d_positions, q_heads, kv_heads, head_dim, theta, io_dtype);
    OJX_CUDA_TRY(cudaGetLastError());
    count_launch(1);
    return OJX_OK;
}

int ojasx_b200_add_int(int* d_values, int count, int delta, void* stream) {
    if (!d_values || count <= 0) return OJX_ERR_ARG;
    add_int_kernel<<<(count + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(d_values, count, delta);
    OJX_CUDA_TRY(cudaGetLastError());
    count_launch(1);
    return OJX_OK;
}

}  // extern "C"
