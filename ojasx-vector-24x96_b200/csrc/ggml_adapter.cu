// GGML dispatch shim: the reference's ojasx_ggml_* entry points
// (split_manifold_lut_experiment/native/src/ojasx_ggml_adapter.cpp:17-92) forwarded to this library's
// handle API.  Host code only; the kernels are reached through ojasx_linear_forward, ojasx_moe_forward
// and ojasx_kv_cache_attention.
#include "../../include/ojasx_ggml_b200.h"

#include <cuda_runtime.h>

#include <atomic>

namespace {
std::atomic<bool> g_ready{false};
}

extern "C" {

int ojasx_ggml_init(void) {
    if (g_ready.load()) return 0;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n < 1) {
        (void)cudaGetLastError();
        return -3;
    }
    if (cudaFree(nullptr) != cudaSuccess) {   // creates the primary context so the first node pays no set-up
        (void)cudaGetLastError();
        return -3;
    }
    g_ready.store(true);
    return 0;
}

int ojasx_ggml_forward_linear(struct ojasx_ggml_tensor* dst, const struct ojasx_ggml_tensor* src0,
                              const struct ojasx_ggml_tensor* src1, int ith, int nth, void* userdata) {
    if (!dst || !src0 || !src1) return -1;
    OjasxLinearHandle h = src1->extra ? src1->extra : userdata;
    if (!h) return -2;
    const float* x = static_cast<const float*>(src0->data);
    float* y = static_cast<float*>(dst->data);
    if (!x || !y) return -3;
    if (nth > 1 && ith != 0) return 0;   // one launch per node, not one per worker
    const int batch = src0->ne[1] > 1 ? static_cast<int>(src0->ne[1]) : 1;
    return ojasx_linear_forward(h, x, y, batch, 0);
}

int ojasx_ggml_forward_moe(struct ojasx_ggml_tensor* dst, const struct ojasx_ggml_tensor* src0,
                           const int* top_k_indices, const float* top_k_weights, int top_k, void* moe_handle) {
    if (!dst || !src0 || !top_k_indices || !top_k_weights || !moe_handle) return -1;
    const float* x = static_cast<const float*>(src0->data);
    float* y = static_cast<float*>(dst->data);
    if (!x || !y) return -2;
    return ojasx_moe_forward(moe_handle, x, top_k_indices, top_k_weights, y, top_k);
}

int ojasx_ggml_forward_kv_attention(struct ojasx_ggml_tensor* dst, const struct ojasx_ggml_tensor* q_tensor,
                                    int head_idx, float scale_factor, void* kv_cache_handle) {
    if (!dst || !q_tensor || !kv_cache_handle) return -1;
    const float* q = static_cast<const float*>(q_tensor->data);
    float* out = static_cast<float*>(dst->data);
    if (!q || !out) return -2;
    return ojasx_kv_cache_attention(kv_cache_handle, head_idx, q, out, scale_factor);
}

}  // extern "C"
