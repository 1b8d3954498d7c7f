/*
 * ojasx_ggml_b200.h -- llama.cpp / GGML dispatch shim over libojasx_lut_b200.so.
 *
 * Same names, struct layout, argument lists and return codes as the reference's
 * split_manifold_lut_experiment/native/include/ojasx_ggml_adapter.h:28-97; each function forwards to
 * the handle API of ojasx_lut_b200.h (host pointers in, result in host memory on return), as
 * ojasx_ggml_adapter.cpp:29-92 forwards to the CPU kernels.  A llama.cpp build that links the
 * reference's adapter can link this library instead.
 *
 * Return codes as the reference: -1 null tensor (or null indices / weights / handle), -2 no handle
 * (linear) or null data pointer (MoE, KV), -3 null data pointer (linear); otherwise the code of
 * the forwarded call.
 */
#ifndef OJASX_GGML_B200_H
#define OJASX_GGML_B200_H

#include "ojasx_lut_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ojasx_ggml_adapter.h:28-29 */
#define GGML_TYPE_OJASX_LUT 100
#define GGML_TYPE_OJASX_MOE 101

/* ojasx_ggml_adapter.h:35-41: the fields of ggml_tensor that dispatch needs */
struct ojasx_ggml_tensor {
    int type;
    int64_t ne[4]; /* extents, innermost first */
    size_t nb[4];  /* strides in bytes */
    void* data;    /* host float buffer */
    void* extra;   /* OjasxLinearHandle or OjasxMoEHandle */
};

/* ojasx_ggml_adapter.h:47.  Idempotent; returns 0 once a CUDA device is usable, -3 otherwise. */
OJASX_API int ojasx_ggml_init(void);

/* ojasx_ggml_adapter.h:59-66.  dst [ne1 = batch, out], src0 = x [ne1 = batch, in] (batch 1 when
 * ne[1] <= 1), handle = src1->extra, else userdata.  GGML calls a node once per worker (ith of
 * nth); the reference computes the whole product in every worker (ojasx_ggml_adapter.cpp:54-57),
 * which on a GPU would repeat the launch nth times, so worker 0 computes and the others return
 * 0 at once: dst holds the same values when the node's barrier releases. */
OJASX_API int ojasx_ggml_forward_linear(struct ojasx_ggml_tensor* dst, const struct ojasx_ggml_tensor* src0,
                                        const struct ojasx_ggml_tensor* src1, int ith, int nth, void* userdata);

/* ojasx_ggml_adapter.h:79-86: one token; top_k_indices / top_k_weights are host arrays [top_k]. */
OJASX_API int ojasx_ggml_forward_moe(struct ojasx_ggml_tensor* dst, const struct ojasx_ggml_tensor* src0,
                                     const int* top_k_indices, const float* top_k_weights, int top_k,
                                     void* moe_handle);

/* ojasx_ggml_adapter.h:92-98: one head of the reference's int8 cache (ojasx_kv_cache_attention). */
OJASX_API int ojasx_ggml_forward_kv_attention(struct ojasx_ggml_tensor* dst, const struct ojasx_ggml_tensor* q_tensor,
                                              int head_idx, float scale_factor, void* kv_cache_handle);

#ifdef __cplusplus
}
#endif

#endif /* OJASX_GGML_B200_H */
