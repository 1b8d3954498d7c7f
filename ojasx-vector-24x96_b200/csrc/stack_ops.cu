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
// (the residual add that precedes the norm), with the sum also written back to x.
__global__ void __launch_bounds__(256) rmsnorm_kernel(void* __restrict__ x, const void* __restrict__ add,
                                                      const float* __restrict__ w, void* __restrict__ out, int H, float eps,
                                                      int io_dtype) {
    __shared__ float red[256];
    const size_t base = (size_t)blockIdx.x * H;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = ld_io(x, base + i, io_dtype);
        if (add) { v += ld_io(add, base + i, io_dtype); st_io(x, base + i, io_dtype, v); v = ld_io(x, base + i, io_dtype); }
        ss += v * v;
    }
    red[threadIdx.x] = ss;
    __syncthreads();
    for (int s = blockDim.x / 2; s > 0; s >>= 1) {
        if (threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s];
        __syncthreads();
    }
    const float inv = rsqrtf(red[0] / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) st_io(out, base + i, io_dtype, ld_io(x, base + i, io_dtype) * inv * w[i]);
}

// Rotate-half rotary embedding in place on q [B, Hq, hd] and k [B, Hkv, hd] at positions pos[b].
__global__ void rope_qk_kernel(void* __restrict__ q, void* __restrict__ k, const int* __restrict__ pos, int Hq, int Hkv,
                               int hd, float theta, int io_dtype) {
    const int b = blockIdx.x, half = hd >> 1;
    const float p = (float)pos[b];
    const int total = (Hq + Hkv) * half;
    for (int i = threadIdx.x; i < total; i += blockDim.x) {
        const int head = i / half, j = i - head * half;
        void* buf = head < Hq ? q : k;
        const size_t base = head < Hq ? ((size_t)b * Hq + head) * hd : ((size_t)b * Hkv + (head - Hq)) * hd;
        const float inv = 1.0f / powf(theta, (float)(2 * j) / (float)hd);
        float s, c;
        sincosf(p * inv, &s, &c);
        const float x1 = ld_io(buf, base + j, io_dtype), x2 = ld_io(buf, base + half + j, io_dtype);
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
    rope_qk_kernel<<<batch, 256, 0, static_cast<cudaStream_t>(stream)>>>(d_q, d_k, d_positions, q_heads, kv_heads, head_dim, theta, io_dtype);
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
