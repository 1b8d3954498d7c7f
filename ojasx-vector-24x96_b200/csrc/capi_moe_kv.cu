// C ABI, MoE and KV-cache part: the reference's ojasx_*moe* / ojasx_*kv_cache* handle API on
// host pointers (split_manifold_lut_experiment/native/src/ojasx_lut_c_api.cpp:131-287) and the
// ojasx_b200_moe_* / ojasx_b200_kvq_* device-pointer entry points.
#include "../../include/ojasx_lut_b200.h"
#include <mutex>

#include "handles.h"
#include "launch.h"
#include "peer.cuh"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <new>
#include <vector>

namespace ojx {

MoeHandle::~MoeHandle() {
    DeviceGuard g(dev);
    cudaFree(cb_in); cudaFree(cb_down); cudaFree(gu_codes); cudaFree(gu_scales); cudaFree(dn_codes); cudaFree(dn_scales);
    for (int i = 0; i < 2; ++i) { cudaFree(csr_rp[i]); cudaFree(csr_cols[i]); cudaFree(csr_vals[i]); }
    cudaFree(router); cudaFree(scratch); cudaFree(lut_scratch); cudaFree(route_scratch); cudaFree(stage);
    if (stream) cudaStreamDestroy(stream);
}

int MoeHandle::reserve(int n_tokens, int k) {
    const size_t pairs = (size_t)n_tokens * k;
    const size_t need = sizeof(float) * pairs * ((size_t)I + H) + sizeof(int) * (5 * pairs + 8);   // + work lists
    int rc = ensure_capacity(&scratch, &scratch_cap, need);
    if (rc != OJX_OK) return rc;
    // Token tables, shared by the k experts of a token (up to 1 GiB), in whichever layout the forward picks.
    const size_t lut_need = moe_table_bytes(n_tokens, H / D, D);
    if (lut_need <= ((size_t)1 << 30)) {
        if ((rc = ensure_capacity(&lut_scratch, &lut_cap, lut_need)) != OJX_OK) return rc;
    }
    if (router) {
        const size_t rneed = sizeof(float) * (size_t)n_tokens * 2 * E_total + pairs * (sizeof(int) + sizeof(float));
        rc = ensure_capacity(&route_scratch, &route_cap, rneed);
    }
    return rc;
}

MoeProblem MoeHandle::problem(const void* x, void* y, const int* idx, const float* w, int n_tokens, int k, int io) const {
    MoeProblem P{};
    P.x = x; P.y = y; P.topk_idx = idx; P.topk_w = w;
    P.cb_in = cb_in; P.cb_down = cb_down; P.gu_codes = gu_codes; P.gu_scales = gu_scales;
    P.dn_codes = dn_codes; P.dn_scales = dn_scales;
    P.gu_csr = CsrView{csr_rp[0], csr_cols[0], csr_vals[0], csr_nnz[0]};
    P.dn_csr = CsrView{csr_rp[1], csr_cols[1], csr_vals[1], csr_nnz[1]};
    const size_t lut_need = moe_table_bytes(n_tokens, H / D, D);
    P.lut_in = (lut_scratch && lut_cap >= lut_need) ? static_cast<const float*>(lut_scratch) : nullptr;
    P.inter = static_cast<float*>(scratch);
    P.expert_out = P.inter + (size_t)n_tokens * k * I;
    P.pair_list = reinterpret_cast<const int*>(P.expert_out + (size_t)n_tokens * k * H);
    P.plan = P.pair_list;   // the two expert paths keep their work lists in the same scratch
    P.chain_ctl = P.pair_list + (size_t)n_tokens * k + 4;   // behind the pair list (1 + pairs ints of the 5 * pairs + 8 reserved)
    P.E_total = E_total;
    P.n_tokens = n_tokens; P.k_active = k; P.E = E; P.expert_offset = expert_offset;
    P.H = H; P.I = I; P.G = H / D; P.Gi = I / D; P.D = D; P.Kcb = 256; P.io_dtype = io;
    P.gate_limit = gate_limit;
    return P;
}

KvqHandle::~KvqHandle() {
    DeviceGuard g(dev);
    cudaFree(k_codes); cudaFree(v_codes); cudaFree(k_cb); cudaFree(v_cb); cudaFree(seq_lens); cudaFree(error_flag); cudaFree(counters);
    cudaFree(partials);
}

LegacyKvHandle::~LegacyKvHandle() {
    DeviceGuard g(dev);
    for (auto& h : heads) { cudaFree(h.k_codes); cudaFree(h.v_codes); cudaFree(h.k_scales); cudaFree(h.v_scales); }
    cudaFree(stage); cudaFree(logits);
    if (stream) cudaStreamDestroy(stream);
}

static int grow_legacy_head(LegacyKvHandle* kv, LegacyKvHandle::Head& h, int new_cap) {
    // ojasx_lut_kv_cache.cpp:17-25: capacity doubles (at least 1024) when the head is full.
    uint8_t *kc = nullptr, *vc = nullptr;
    float *ks = nullptr, *vs = nullptr;
    const size_t G = kv->G;
    OJX_CUDA_TRY(cudaMalloc((void**)&kc, (size_t)new_cap * G));
    OJX_CUDA_TRY(cudaMalloc((void**)&vc, (size_t)new_cap * G));
    OJX_CUDA_TRY(cudaMalloc((void**)&ks, sizeof(float) * (size_t)new_cap));
    OJX_CUDA_TRY(cudaMalloc((void**)&vs, sizeof(float) * (size_t)new_cap));
    if (h.len > 0) {
        OJX_CUDA_TRY(cudaMemcpy(kc, h.k_codes, (size_t)h.len * G, cudaMemcpyDeviceToDevice));
        OJX_CUDA_TRY(cudaMemcpy(vc, h.v_codes, (size_t)h.len * G, cudaMemcpyDeviceToDevice));
        OJX_CUDA_TRY(cudaMemcpy(ks, h.k_scales, sizeof(float) * (size_t)h.len, cudaMemcpyDeviceToDevice));
        OJX_CUDA_TRY(cudaMemcpy(vs, h.v_scales, sizeof(float) * (size_t)h.len, cudaMemcpyDeviceToDevice));
    }
    cudaFree(h.k_codes); cudaFree(h.v_codes); cudaFree(h.k_scales); cudaFree(h.v_scales);
    h.k_codes = kc; h.v_codes = vc; h.k_scales = ks; h.v_scales = vs; h.cap = new_cap;
    return OJX_OK;
}

// The device-pointer MoE entry points allocate scratch on the current device and launch there, so the
// handle's device must be current (the caller's stream belongs to it anyway).
static int moe_check_device(const MoeHandle* h, const char* who) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev != h->dev) {
        char msg[160];
        std::snprintf(msg, sizeof(msg), "%s: the handle's device (%d) must be the current device (%d)", who, h->dev, dev);
        set_last_error_msg(msg);
        return OJX_ERR_ARG;
    }
    return OJX_OK;
}

}  // namespace ojx

using namespace ojx;

extern "C" {

/* ------------------------------------------------------------------------------------ MoE */
OjasxMoEHandle ojasx_create_moe(int num_experts, int hidden_dim, int intermediate_dim, int top_k, int block_dim,
                                const float* codebook_in, const float* codebook_down, const uint8_t* gate_up_codes,
                                const float* gate_up_scales, const uint8_t* down_codes, const float* down_scales) {
    if (num_experts <= 0 || hidden_dim <= 0 || intermediate_dim <= 0 || block_dim <= 0) return nullptr;
    auto* h = new (std::nothrow) MoeHandle();
    if (!h) return nullptr;
    h->E = num_experts; h->E_total = num_experts; h->H = hidden_dim; h->I = intermediate_dim; h->top_k = top_k;
    h->D = block_dim;
    const size_t G = hidden_dim / block_dim, Gi = intermediate_dim / block_dim;
    int rc = cudaGetDevice(&h->dev) == cudaSuccess ? OJX_OK : OJX_ERR_CUDA;
    const size_t cbb = sizeof(float) * 256 * (size_t)block_dim;
    if (rc == OJX_OK) rc = upload((void**)&h->cb_in, codebook_in, cbb);
    if (rc == OJX_OK) rc = upload((void**)&h->cb_down, codebook_down, cbb);
    if (rc == OJX_OK) rc = upload((void**)&h->gu_codes, gate_up_codes, (size_t)num_experts * 2 * intermediate_dim * G);
    if (rc == OJX_OK) rc = upload((void**)&h->dn_codes, down_codes, (size_t)num_experts * hidden_dim * Gi);
    // Null scale pointers keep the reference's default of 1.0 (ojasx_lut.h:196-199).
    if (rc == OJX_OK && gate_up_scales)
        rc = upload((void**)&h->gu_scales, gate_up_scales, sizeof(float) * (size_t)num_experts * 2 * intermediate_dim);
    if (rc == OJX_OK && down_scales)
        rc = upload((void**)&h->dn_scales, down_scales, sizeof(float) * (size_t)num_experts * hidden_dim);
    if (rc == OJX_OK && cudaStreamCreateWithFlags(&h->stream, cudaStreamNonBlocking) != cudaSuccess) rc = OJX_ERR_CUDA;
    if (rc != OJX_OK) { delete h; return nullptr; }
    return h;
}

int ojasx_b200_moe_set_outliers(OjasxMoEHandle handle, int which, int nnz, const int* row_ptrs, const int* col_indices,
                                const float* values) {
    if (!handle || which < 0 || which > 1 || nnz < 0 || !row_ptrs || (nnz > 0 && (!col_indices || !values))) return OJX_ERR_ARG;
    auto* h = static_cast<MoeHandle*>(handle);
    DeviceGuard g(h->dev);
    const size_t rows = which == 0 ? (size_t)h->E * 2 * h->I : (size_t)h->E * h->H;
    cudaFree(h->csr_rp[which]); cudaFree(h->csr_cols[which]); cudaFree(h->csr_vals[which]);
    h->csr_rp[which] = nullptr; h->csr_cols[which] = nullptr; h->csr_vals[which] = nullptr; h->csr_nnz[which] = 0;
    int rc;
    if ((rc = upload((void**)&h->csr_rp[which], row_ptrs, sizeof(int) * (rows + 1))) != OJX_OK) return rc;
    if ((rc = upload((void**)&h->csr_cols[which], col_indices, sizeof(int) * (size_t)nnz)) != OJX_OK) return rc;
    if ((rc = upload((void**)&h->csr_vals[which], values, sizeof(float) * (size_t)nnz)) != OJX_OK) return rc;
    h->csr_nnz[which] = nnz;
    return OJX_OK;
}

int ojasx_b200_moe_set_router(OjasxMoEHandle handle, const float* router_weight, int num_experts_total) {
    if (!handle || !router_weight || num_experts_total <= 0) return OJX_ERR_ARG;
    auto* h = static_cast<MoeHandle*>(handle);
    DeviceGuard g(h->dev);
    cudaFree(h->router);
    h->router = nullptr;
    h->E_total = num_experts_total;
    return upload((void**)&h->router, router_weight, sizeof(float) * (size_t)num_experts_total * h->H);
}

int ojasx_b200_moe_set_expert_offset(OjasxMoEHandle handle, int first_global_expert) {
    if (!handle) return OJX_ERR_ARG;
    static_cast<MoeHandle*>(handle)->expert_offset = first_global_expert;
    return OJX_OK;
}

int ojasx_b200_moe_set_gate_limit(OjasxMoEHandle handle, float limit) {
    if (!handle || !(limit == limit)) return OJX_ERR_ARG;
    static_cast<MoeHandle*>(handle)->gate_limit = limit > 0.0f ? limit : 0.0f;
    return OJX_OK;
}

int ojasx_b200_moe_reserve(OjasxMoEHandle handle, int max_tokens, int k_active) {
    if (!handle || max_tokens <= 0 || k_active <= 0) return OJX_ERR_ARG;
    auto* h = static_cast<MoeHandle*>(handle);
    DeviceGuard g(h->dev);
    return h->reserve(max_tokens, k_active);
}

int ojasx_b200_moe_forward(OjasxMoEHandle handle, const void* d_x, const int* d_topk_idx, const float* d_topk_w, void* d_y,
                           int n_tokens, int k_active, int io_dtype, void* stream) {
    if (!handle || !d_x || !d_topk_idx || !d_topk_w || !d_y) return OJX_ERR_ARG;
    if (n_tokens <= 0 || k_active <= 0 || (io_dtype != OJX_F32 && io_dtype != OJX_BF16)) return OJX_ERR_ARG;
    auto* h = static_cast<MoeHandle*>(handle);
    if (int drc = moe_check_device(h, "ojasx_b200_moe_forward")) return drc;
    int rc = h->reserve(n_tokens, k_active);
    if (rc != OJX_OK) return rc;
    return launch_moe_experts(h->problem(d_x, d_y, d_topk_idx, d_topk_w, n_tokens, k_active, io_dtype),
                              static_cast<cudaStream_t>(stream));
}

int ojasx_b200_moe_forward_gather(OjasxMoEHandle handle, const void* d_x, const int* d_topk_idx, const float* d_topk_w,
                                  void* d_y, int n_tokens, int k_active, int io_dtype, OjasxPeerLinkHandle link,
                                  float* d_expert_out_shared, void* stream) {
    if (!handle || !d_x || !d_topk_idx || !d_topk_w || !d_y || !link || !d_expert_out_shared) return OJX_ERR_ARG;
    if (n_tokens <= 0 || k_active <= 0 || (io_dtype != OJX_F32 && io_dtype != OJX_BF16)) return OJX_ERR_ARG;
    auto* h = static_cast<MoeHandle*>(handle);
    if (int drc = moe_check_device(h, "ojasx_b200_moe_forward_gather")) return drc;
    int rc = h->reserve(n_tokens, k_active);
    if (rc != OJX_OK) return rc;
    MoeProblem P = h->problem(d_x, d_y, d_topk_idx, d_topk_w, n_tokens, k_active, io_dtype);
    P.expert_out = d_expert_out_shared;
    return launch_moe_experts(P, static_cast<cudaStream_t>(stream), peer_link_of(link));
}

int ojasx_b200_moe_forward_routed_gather(OjasxMoEHandle handle, const void* d_x, void* d_y, int n_tokens, int top_k,
                                         int io_dtype, OjasxPeerLinkHandle link, float* d_expert_out_shared,
                                         float* d_logits_shared, void* stream) {
    if (!handle || !d_x || !d_y || n_tokens <= 0 || top_k <= 0 || !link || !d_expert_out_shared) return OJX_ERR_ARG;
    auto* h = static_cast<MoeHandle*>(handle);
    if (!h->router) { set_last_error_msg("moe_forward_routed_gather: no router weights set"); return OJX_ERR_ARG; }
    if (int drc = moe_check_device(h, "ojasx_b200_moe_forward_routed_gather")) return drc;
    int rc = h->reserve(n_tokens, top_k);
    if (rc != OJX_OK) return rc;
    float* logits = static_cast<float*>(h->route_scratch);
    float* probs = logits + (size_t)n_tokens * h->E_total;
    int* idx = reinterpret_cast<int*>(probs + (size_t)n_tokens * h->E_total);
    float* w = reinterpret_cast<float*>(idx + (size_t)n_tokens * top_k);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    MoeProblem P = h->problem(d_x, d_y, idx, w, n_tokens, top_k, io_dtype);
    P.expert_out = d_expert_out_shared;
    P.lut_blocks = moe_table_layout(P);
    // with a shared logits buffer every rank scores only the experts it holds (an exchange of its own on the link)
    rc = launch_moe_router(h->router, d_x, io_dtype, n_tokens, h->H, h->E_total, top_k, d_logits_shared ? d_logits_shared : logits,
                           probs, idx, w, s, P.cb_in, P.Kcb, P.D, const_cast<float*>(P.lut_in), P.lut_blocks,
                           d_logits_shared ? peer_link_of(link) : nullptr, h->expert_offset, h->expert_offset + h->E);
    if (rc != OJX_OK) return rc;
    P.lut_ready = P.lut_in != nullptr;
    return launch_moe_experts(P, s, peer_link_of(link));
}

int ojasx_b200_moe_route(OjasxMoEHandle handle, const void* d_x, int n_tokens, int top_k, int* d_idx_out, float* d_w_out,
                         int io_dtype, void* stream) {
    if (!handle || !d_x || !d_idx_out || !d_w_out || n_tokens <= 0 || top_k <= 0) return OJX_ERR_ARG;
    auto* h = static_cast<MoeHandle*>(handle);
    if (!h->router) { set_last_error_msg("moe_route: no router weights set"); return OJX_ERR_ARG; }
    if (int drc = moe_check_device(h, "ojasx_b200_moe_route")) return drc;
    int rc = h->reserve(n_tokens, top_k);
    if (rc != OJX_OK) return rc;
    float* logits = static_cast<float*>(h->route_scratch);
    float* probs = logits + (size_t)n_tokens * h->E_total;
    return launch_moe_router(h->router, d_x, io_dtype, n_tokens, h->H, h->E_total, top_k, logits, probs, d_idx_out, d_w_out,
                             static_cast<cudaStream_t>(stream));
}

int ojasx_b200_moe_forward_routed(OjasxMoEHandle handle, const void* d_x, void* d_y, int n_tokens, int top_k, int io_dtype,
                                  void* stream) {
    if (!handle || !d_x || !d_y || n_tokens <= 0 || top_k <= 0) return OJX_ERR_ARG;
    auto* h = static_cast<MoeHandle*>(handle);
    if (!h->router) { set_last_error_msg("moe_forward_routed: no router weights set"); return OJX_ERR_ARG; }
    if (int drc = moe_check_device(h, "ojasx_b200_moe_forward_routed")) return drc;
    int rc = h->reserve(n_tokens, top_k);
    if (rc != OJX_OK) return rc;
    float* logits = static_cast<float*>(h->route_scratch);
    float* probs = logits + (size_t)n_tokens * h->E_total;
    int* idx = reinterpret_cast<int*>(probs + (size_t)n_tokens * h->E_total);
    float* w = reinterpret_cast<float*>(idx + (size_t)n_tokens * top_k);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    MoeProblem P = h->problem(d_x, d_y, idx, w, n_tokens, top_k, io_dtype);
    P.lut_blocks = moe_table_layout(P);
    rc = launch_moe_router(h->router, d_x, io_dtype, n_tokens, h->H, h->E_total, top_k, logits, probs, idx, w, s,
                           P.cb_in, P.Kcb, P.D, const_cast<float*>(P.lut_in), P.lut_blocks);
    if (rc != OJX_OK) return rc;
    P.lut_ready = P.lut_in != nullptr;
    return launch_moe_experts(P, s);
}

int ojasx_b200_build_lut(const void* d_x, int n_vectors, int in_features, int block_dim, const float* d_codebook,
                         int codebook_size, float* d_lut, int io_dtype, void* stream) {
    if (io_dtype != OJX_F32 && io_dtype != OJX_BF16) return OJX_ERR_ARG;
    return launch_build_lut(d_x, io_dtype, n_vectors, in_features, block_dim, d_codebook, codebook_size, d_lut,
                            static_cast<cudaStream_t>(stream));
}

int ojasx_b200_silu_mul(const void* d_gate, const void* d_up, void* d_out, size_t count, int io_dtype, void* stream) {
    if (io_dtype != OJX_F32 && io_dtype != OJX_BF16) return OJX_ERR_ARG;
    return launch_silu_mul(d_gate, d_up, d_out, count, io_dtype, static_cast<cudaStream_t>(stream));
}

int ojasx_moe_forward(OjasxMoEHandle handle, const float* x, const int* top_k_indices, const float* top_k_weights,
                      float* y_out, int k_active) {
    if (!handle || !x || !top_k_indices || !top_k_weights || !y_out) return OJX_ERR_ARG;  // ojasx_lut_c_api.cpp:267
    if (k_active <= 0) return OJX_OK;                                                       // ojasx_lut_cpu.cpp:220
    auto* h = static_cast<MoeHandle*>(handle);
    std::lock_guard<std::mutex> lock(h->host_mu);
    DeviceGuard g(h->dev);
    const size_t xb = sizeof(float) * (size_t)h->H, kb = (size_t)k_active * 4;
    int rc = ensure_capacity(&h->stage, &h->stage_cap, 2 * xb + 2 * kb + 64);
    if (rc != OJX_OK) return rc;
    if ((rc = h->reserve(1, k_active)) != OJX_OK) return rc;
    char* base = static_cast<char*>(h->stage);
    float* dx = reinterpret_cast<float*>(base);
    float* dy = reinterpret_cast<float*>(base + xb);
    int* di = reinterpret_cast<int*>(base + 2 * xb);
    float* dw = reinterpret_cast<float*>(base + 2 * xb + kb);
    OJX_CUDA_TRY(cudaMemcpyAsync(dx, x, xb, cudaMemcpyHostToDevice, h->stream));
    OJX_CUDA_TRY(cudaMemcpyAsync(di, top_k_indices, kb, cudaMemcpyHostToDevice, h->stream));
    OJX_CUDA_TRY(cudaMemcpyAsync(dw, top_k_weights, kb, cudaMemcpyHostToDevice, h->stream));
    rc = launch_moe_experts(h->problem(dx, dy, di, dw, 1, k_active, OJX_F32), h->stream);
    if (rc != OJX_OK) return rc;
    OJX_CUDA_TRY(cudaMemcpyAsync(y_out, dy, xb, cudaMemcpyDeviceToHost, h->stream));
    OJX_CUDA_TRY(cudaStreamSynchronize(h->stream));
    return OJX_OK;
}

/* Size formulas of ojasx_lut.h:202-217 (scale vectors always counted). */
size_t ojasx_moe_get_compressed_size(OjasxMoEHandle handle) {
    if (!handle) return 0;
    auto* h = static_cast<MoeHandle*>(handle);
    const size_t G = h->H / h->D, Gi = h->I / h->D;
    const size_t gu = (size_t)h->E * 2 * h->I * G + sizeof(float) * (size_t)h->E * 2 * h->I;
    const size_t dn = (size_t)h->E * h->H * Gi + sizeof(float) * (size_t)h->E * h->H;
    return gu + dn + 2 * sizeof(float) * 256 * (size_t)h->D;
}
float ojasx_moe_get_compression_ratio(OjasxMoEHandle handle) {
    if (!handle) return 0.0f;
    auto* h = static_cast<MoeHandle*>(handle);
    const size_t dense = (size_t)h->E * 3 * h->H * h->I * sizeof(float);
    const size_t c = ojasx_moe_get_compressed_size(handle);
    return (float)dense / (float)(c ? c : 1);
}
void ojasx_destroy_moe(OjasxMoEHandle handle) {
    if (handle) delete static_cast<MoeHandle*>(handle);
}

/* ------------------------------------------------------------------------- codebook-VQ KV */
OjasxKvqHandle ojasx_b200_kvq_create(int batch, int kv_heads, int q_heads, int head_dim, int block_dim, int max_seq_len,
                                     const float* k_codebook, const float* v_codebook) {
    if (batch <= 0 || kv_heads <= 0 || q_heads <= 0 || q_heads % kv_heads || head_dim <= 0 || block_dim <= 0 ||
        head_dim % block_dim || max_seq_len <= 0 || !k_codebook || !v_codebook)
        return nullptr;
    auto* h = new (std::nothrow) KvqHandle();
    if (!h) return nullptr;
    h->B = batch; h->Hkv = kv_heads; h->Hq = q_heads; h->head_dim = head_dim; h->D = block_dim;
    h->G = head_dim / block_dim; h->max_seq = max_seq_len;
    int rc = cudaGetDevice(&h->dev) == cudaSuccess ? OJX_OK : OJX_ERR_CUDA;
    const size_t codes = (size_t)batch * kv_heads * max_seq_len * h->G;
    const size_t cbb = sizeof(float) * (size_t)kv_heads * 256 * block_dim;
    if (rc == OJX_OK) rc = upload((void**)&h->k_codes, nullptr, codes);
    if (rc == OJX_OK) rc = upload((void**)&h->v_codes, nullptr, codes);
    if (rc == OJX_OK) rc = upload((void**)&h->k_cb, k_codebook, cbb);
    if (rc == OJX_OK) rc = upload((void**)&h->v_cb, v_codebook, cbb);
    if (rc == OJX_OK) rc = upload((void**)&h->seq_lens, nullptr, sizeof(int) * (size_t)batch);
    if (rc == OJX_OK) rc = upload((void**)&h->error_flag, nullptr, sizeof(int));
    if (rc == OJX_OK) rc = upload((void**)&h->counters, nullptr, sizeof(int) * ((size_t)batch + (size_t)batch * kv_heads));
    if (rc != OJX_OK) { delete h; return nullptr; }
    return h;
}

int ojasx_b200_kvq_load(OjasxKvqHandle handle, const uint8_t* k_codes, const uint8_t* v_codes, int seq_len) {
    if (!handle || !k_codes || !v_codes) return OJX_ERR_ARG;
    auto* h = static_cast<KvqHandle*>(handle);
    if (seq_len < 0 || seq_len > h->max_seq) return OJX_ERR_RANGE;
    DeviceGuard g(h->dev);
    const size_t row = (size_t)seq_len * h->G, dst_row = (size_t)h->max_seq * h->G;
    if (seq_len > 0) {
        OJX_CUDA_TRY(cudaMemcpy2D(h->k_codes, dst_row, k_codes, row, row, (size_t)h->B * h->Hkv, cudaMemcpyHostToDevice));
        OJX_CUDA_TRY(cudaMemcpy2D(h->v_codes, dst_row, v_codes, row, row, (size_t)h->B * h->Hkv, cudaMemcpyHostToDevice));
    }
    std::vector<int> lens(h->B, seq_len);
    OJX_CUDA_TRY(cudaMemcpy(h->seq_lens, lens.data(), sizeof(int) * lens.size(), cudaMemcpyHostToDevice));
    h->host_len = seq_len;
    return OJX_OK;
}

int ojasx_b200_kvq_read(OjasxKvqHandle handle, uint8_t* k_codes, uint8_t* v_codes, int t_begin, int t_end) {
    if (!handle || !k_codes || !v_codes) return OJX_ERR_ARG;
    auto* h = static_cast<KvqHandle*>(handle);
    if (t_begin < 0 || t_end > h->max_seq || t_begin >= t_end) return OJX_ERR_RANGE;
    DeviceGuard g(h->dev);
    const size_t row = (size_t)(t_end - t_begin) * h->G, src_row = (size_t)h->max_seq * h->G;
    OJX_CUDA_TRY(cudaDeviceSynchronize());
    OJX_CUDA_TRY(cudaMemcpy2D(k_codes, row, h->k_codes + (size_t)t_begin * h->G, src_row, row, (size_t)h->B * h->Hkv,
                              cudaMemcpyDeviceToHost));
    OJX_CUDA_TRY(cudaMemcpy2D(v_codes, row, h->v_codes + (size_t)t_begin * h->G, src_row, row, (size_t)h->B * h->Hkv,
                              cudaMemcpyDeviceToHost));
    return OJX_OK;
}

int ojasx_b200_kvq_seq_len(OjasxKvqHandle handle) { return handle ? static_cast<KvqHandle*>(handle)->host_len : -1; }

int ojasx_b200_kvq_reset(OjasxKvqHandle handle) {
    if (!handle) return OJX_ERR_ARG;
    auto* h = static_cast<KvqHandle*>(handle);
    DeviceGuard g(h->dev);
    OJX_CUDA_TRY(cudaMemset(h->seq_lens, 0, sizeof(int) * (size_t)h->B));
    OJX_CUDA_TRY(cudaMemset(h->error_flag, 0, sizeof(int)));
    h->host_len = 0;
    return OJX_OK;
}

static KvqProblem kvq_problem(const KvqHandle* h, int io) {
    KvqProblem P{};
    P.k_codes = h->k_codes; P.v_codes = h->v_codes; P.k_cb = h->k_cb; P.v_cb = h->v_cb;
    P.seq_lens = h->seq_lens; P.error_flag = h->error_flag; P.partials = static_cast<float*>(h->partials);
    P.append_done = h->counters; P.split_done = h->counters + h->B;
    P.B = h->B; P.Hkv = h->Hkv; P.Hq = h->Hq; P.head_dim = h->head_dim; P.D = h->D; P.G = h->G; P.Kcb = 256;
    P.max_seq = h->max_seq; P.io_dtype = io;
    return P;
}

static int kvq_max_splits(int max_seq) { return std::min(kKvMaxSplits, (max_seq + 255) / 256); }

int ojasx_b200_kvq_append(OjasxKvqHandle handle, const void* d_k, const void* d_v, int io_dtype, void* stream) {
    if (!handle || !d_k || !d_v || (io_dtype != OJX_F32 && io_dtype != OJX_BF16)) return OJX_ERR_ARG;
    auto* h = static_cast<KvqHandle*>(handle);
    if (!h->static_plan && h->host_len >= h->max_seq) return OJX_ERR_RANGE;
    KvqProblem P = kvq_problem(h, io_dtype);
    P.new_k = d_k; P.new_v = d_v;
    int rc = launch_kvq_append(P, static_cast<cudaStream_t>(stream));
    if (rc == OJX_OK && !h->static_plan) h->host_len += 1;
    return rc;
}

static int kvq_decode_impl(OjasxKvqHandle handle, const void* d_q, void* d_out, float scale, int io_dtype, void* stream,
                           int out_heads, int out_head0, const PeerLink* link);

int ojasx_b200_kvq_decode(OjasxKvqHandle handle, const void* d_q, void* d_out, float scale, int io_dtype, void* stream) {
    return kvq_decode_impl(handle, d_q, d_out, scale, io_dtype, stream, 0, 0, nullptr);
}

int ojasx_b200_kvq_decode_gather(OjasxKvqHandle handle, const void* d_q, void* d_out_full, float scale, int io_dtype,
                                 int total_q_heads, int first_q_head, OjasxPeerLinkHandle link, void* stream) {
    if (!link || !handle) return OJX_ERR_ARG;
    auto* h = static_cast<KvqHandle*>(handle);
    if (first_q_head < 0 || first_q_head + h->Hq > total_q_heads) return OJX_ERR_RANGE;
    return kvq_decode_impl(handle, d_q, d_out_full, scale, io_dtype, stream, total_q_heads, first_q_head, peer_link_of(link));
}

static int kvq_decode_impl(OjasxKvqHandle handle, const void* d_q, void* d_out, float scale, int io_dtype, void* stream,
                           int out_heads, int out_head0, const PeerLink* link) {
    if (!handle || !d_q || !d_out || (io_dtype != OJX_F32 && io_dtype != OJX_BF16)) return OJX_ERR_ARG;
    auto* h = static_cast<KvqHandle*>(handle);
    if (!h->static_plan && h->host_len <= 0) return OJX_ERR_RANGE;
    KvqProblem P = kvq_problem(h, io_dtype);
    P.q = d_q; P.out = d_out;
    P.scale = scale > 0.0f ? scale : 1.0f / std::sqrt((float)h->head_dim);
    const int T = h->static_plan ? h->max_seq : h->host_len, heads = h->B * h->Hkv;
    plan_kvq_decode(P, T, num_sms());
    const int R = h->Hq / h->Hkv;
    // sized once for the largest split count, so a growing context never reallocates
    const size_t need = sizeof(float) * (size_t)heads * kvq_max_splits(h->max_seq) * R * (h->head_dim + 2);
    DeviceGuard g(h->dev);
    int rc = ensure_capacity(&h->partials, &h->partials_cap, need);
    if (rc != OJX_OK) return rc;
    P.partials = static_cast<float*>(h->partials);
    P.out_heads = out_heads;
    P.out_head0 = out_head0;
    return launch_kvq_decode(P, static_cast<cudaStream_t>(stream), link);
}

int ojasx_b200_kvq_set_static_plan(OjasxKvqHandle handle, int enabled) {
    if (!handle) return OJX_ERR_ARG;
    auto* h = static_cast<KvqHandle*>(handle);
    h->static_plan = enabled != 0;
    if (h->static_plan) {   // size the chunk scratch for the full capacity now, so that decode never allocates
        DeviceGuard g(h->dev);
        const int heads = h->B * h->Hkv, R = h->Hq / h->Hkv;
        const size_t need = sizeof(float) * (size_t)heads * kvq_max_splits(h->max_seq) * R * (h->head_dim + 2);
        return ensure_capacity(&h->partials, &h->partials_cap, need);
    }
    return OJX_OK;
}

int ojasx_b200_kvq_sync_len(OjasxKvqHandle handle) {
    if (!handle) return OJX_ERR_ARG;
    auto* h = static_cast<KvqHandle*>(handle);
    DeviceGuard g(h->dev);
    std::vector<int> lens(h->B);
    OJX_CUDA_TRY(cudaMemcpy(lens.data(), h->seq_lens, sizeof(int) * lens.size(), cudaMemcpyDeviceToHost));
    h->host_len = *std::max_element(lens.begin(), lens.end());
    // An append that found its sequence full (possible only under the static plan, where the host-side
    // capacity check is skipped) dropped the token and raised this flag: report it once and clear it.
    int overflow = 0;
    OJX_CUDA_TRY(cudaMemcpy(&overflow, h->error_flag, sizeof(int), cudaMemcpyDeviceToHost));
    if (overflow) {
        OJX_CUDA_TRY(cudaMemset(h->error_flag, 0, sizeof(int)));
        set_last_error_msg("kvq: an append ran past max_seq_len and its token was dropped");
        return OJX_ERR_RANGE;
    }
    return h->host_len;
}

int ojasx_b200_kvq_crop(OjasxKvqHandle handle, int max_len) {
    if (!handle) return OJX_ERR_ARG;
    auto* h = static_cast<KvqHandle*>(handle);
    if (max_len < 0) return OJX_ERR_RANGE;
    DeviceGuard g(h->dev);
    std::vector<int> lens(h->B);
    OJX_CUDA_TRY(cudaMemcpy(lens.data(), h->seq_lens, sizeof(int) * lens.size(), cudaMemcpyDeviceToHost));
    for (int& v : lens) v = std::min(v, max_len);
    OJX_CUDA_TRY(cudaMemcpy(h->seq_lens, lens.data(), sizeof(int) * lens.size(), cudaMemcpyHostToDevice));
    h->host_len = *std::max_element(lens.begin(), lens.end());
    return h->host_len;
}

size_t ojasx_b200_kvq_get_memory_size(OjasxKvqHandle handle) {
    if (!handle) return 0;
    auto* h = static_cast<KvqHandle*>(handle);
    return 2 * (size_t)h->B * h->Hkv * h->max_seq * h->G + 2 * sizeof(float) * (size_t)h->Hkv * 256 * h->D;
}

void ojasx_b200_kvq_destroy(OjasxKvqHandle handle) {
    if (handle) delete static_cast<KvqHandle*>(handle);
}

/* ------------------------------------------------------------- reference KV cache as shipped */
OjasxKVHandle ojasx_create_kv_cache(int num_heads, int head_dim, int max_seq_len, int block_dim) {
    if (num_heads <= 0 || head_dim <= 0 || block_dim <= 0 || max_seq_len < 0) return nullptr;
    auto* kv = new (std::nothrow) LegacyKvHandle();
    if (!kv) return nullptr;
    kv->num_heads = num_heads; kv->head_dim = head_dim; kv->D = block_dim; kv->G = head_dim / block_dim;
    kv->initial_cap = max_seq_len;
    kv->heads.resize(num_heads);
    int rc = cudaGetDevice(&kv->dev) == cudaSuccess ? OJX_OK : OJX_ERR_CUDA;
    for (auto& h : kv->heads)
        if (rc == OJX_OK && max_seq_len > 0) rc = grow_legacy_head(kv, h, max_seq_len);
    if (rc == OJX_OK) rc = ensure_capacity(&kv->stage, &kv->stage_cap, sizeof(float) * 3 * (size_t)head_dim);
    if (rc == OJX_OK && cudaStreamCreateWithFlags(&kv->stream, cudaStreamNonBlocking) != cudaSuccess) rc = OJX_ERR_CUDA;
    if (rc != OJX_OK) { delete kv; return nullptr; }
    return kv;
}

int ojasx_kv_cache_append(OjasxKVHandle handle, int head_idx, const float* k, const float* v) {
    if (!handle || !k || !v) return OJX_ERR_ARG;
    auto* kv = static_cast<LegacyKvHandle*>(handle);
    if (head_idx < 0 || head_idx >= kv->num_heads) return OJX_ERR_RANGE;
    std::lock_guard<std::mutex> lock(kv->host_mu);
    DeviceGuard g(kv->dev);
    auto& h = kv->heads[head_idx];
    if (h.len >= h.cap) {
        OJX_CUDA_TRY(cudaStreamSynchronize(kv->stream));
        int rc = grow_legacy_head(kv, h, std::max(1024, h.cap * 2));
        if (rc != OJX_OK) return rc;
    }
    float* dk = static_cast<float*>(kv->stage);
    float* dv = dk + kv->head_dim;
    const size_t vb = sizeof(float) * (size_t)kv->head_dim;
    OJX_CUDA_TRY(cudaMemcpyAsync(dk, k, vb, cudaMemcpyHostToDevice, kv->stream));
    OJX_CUDA_TRY(cudaMemcpyAsync(dv, v, vb, cudaMemcpyHostToDevice, kv->stream));
    int rc = launch_legacy_append(dk, dv, kv->head_dim, kv->D, h.k_codes + (size_t)h.len * kv->G,
                                  h.v_codes + (size_t)h.len * kv->G, h.k_scales + h.len, h.v_scales + h.len, kv->stream);
    if (rc != OJX_OK) return rc;
    OJX_CUDA_TRY(cudaStreamSynchronize(kv->stream));  // k and v may be reused by the caller on return
    h.len += 1;
    return OJX_OK;
}

int ojasx_kv_cache_attention(OjasxKVHandle handle, int head_idx, const float* q, float* out_context, float scale_factor) {
    if (!handle || !q || !out_context) return OJX_ERR_ARG;
    auto* kv = static_cast<LegacyKvHandle*>(handle);
    if (head_idx < 0 || head_idx >= kv->num_heads) return OJX_ERR_RANGE;
    std::lock_guard<std::mutex> lock(kv->host_mu);
    auto& h = kv->heads[head_idx];
    if (h.len == 0) return OJX_OK;  // ojasx_lut_c_api.cpp:173: out_context is left untouched
    DeviceGuard g(kv->dev);
    int rc = ensure_capacity(&kv->logits, &kv->logits_cap, sizeof(float) * (size_t)h.len);
    if (rc != OJX_OK) return rc;
    float* dq = static_cast<float*>(kv->stage);
    float* dout = dq + 2 * kv->head_dim;
    const size_t vb = sizeof(float) * (size_t)kv->head_dim;
    OJX_CUDA_TRY(cudaMemcpyAsync(dq, q, vb, cudaMemcpyHostToDevice, kv->stream));
    rc = launch_legacy_attention(dq, kv->head_dim, kv->D, h.len, h.k_codes, h.v_codes, h.k_scales, h.v_scales, scale_factor,
                                 static_cast<float*>(kv->logits), dout, kv->stream);
    if (rc != OJX_OK) return rc;
    OJX_CUDA_TRY(cudaMemcpyAsync(out_context, dout, vb, cudaMemcpyDeviceToHost, kv->stream));
    OJX_CUDA_TRY(cudaStreamSynchronize(kv->stream));
    return OJX_OK;
}

/* ojasx_lut_kv_cache.h:64-79, 127-133 */
size_t ojasx_kv_cache_get_memory_size(OjasxKVHandle handle) {
    if (!handle) return 0;
    auto* kv = static_cast<LegacyKvHandle*>(handle);
    size_t total = 0;
    for (auto& h : kv->heads)
        total += 2 * (size_t)h.cap * kv->G + 2 * sizeof(float) * (size_t)h.cap + 2 * sizeof(float) * 256 * (size_t)kv->D;
    return total;
}
float ojasx_kv_cache_get_compression_ratio(OjasxKVHandle handle) {
    if (!handle) return 0.0f;
    auto* kv = static_cast<LegacyKvHandle*>(handle);
    if (kv->num_heads == 0) return 0.0f;
    const size_t len = kv->heads[0].len;
    const size_t dense = (size_t)2 * kv->head_dim * len * sizeof(float);
    const size_t comp = len * ((size_t)kv->G * 2 + 2 * sizeof(float));
    return (float)dense / (float)std::max((size_t)1, comp);
}
void ojasx_destroy_kv_cache(OjasxKVHandle handle) {
    if (handle) delete static_cast<LegacyKvHandle*>(handle);
}

}  // extern "C"
