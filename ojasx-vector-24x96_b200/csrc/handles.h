// Host-side objects behind the opaque C handles.
#pragma once
#include "common.cuh"
#include "launch.h"
#include <mutex>
#include <vector>

namespace ojx {

void count_launch(int n);
int upload(void** dptr, const void* host, size_t bytes);          // cudaMalloc + copy (zero-fill when host == null)
int ensure_capacity(void** dptr, size_t* cap, size_t bytes);      // grow-only device staging buffer
int wait_stream(cudaStream_t s);                                  // low-latency stream wait
int ensure_pinned(void** hptr, size_t* cap, size_t bytes);        // grow-only pinned, device-mapped host buffer

// Makes `dev` current for the lifetime of the guard.
class DeviceGuard {
public:
    explicit DeviceGuard(int dev);
    ~DeviceGuard();
private:
    int prev_;
};

struct LinearHandle {
    int dev = 0;
    int in = 0, out = 0, D = 0, Kcb = 256, G = 0;
    uint8_t* codes = nullptr;
    float* codebook = nullptr;
    float* scales = nullptr;   // null = ones
    float* bias = nullptr;     // null = none
    int nnz = 0;
    bool has_outlier_arrays = false;
    bool csr_sorted = true;    // column indices ascending inside every row (needed by the tensor-core path)
    int* row_ptrs = nullptr;
    int* cols = nullptr;
    float* vals = nullptr;
    // staging for the host-pointer forward
    void* d_x = nullptr;
    void* d_y = nullptr;
    size_t cap_x = 0, cap_y = 0;
    void* pin_x = nullptr;     // pinned host staging for x (source of an asynchronous copy)
    void* pin_y = nullptr;     // pinned, device-mapped host staging for y (written by the kernel itself)
    size_t cap_pin_x = 0, cap_pin_y = 0;
    void* pin_y_dev = nullptr;     // device alias of pin_y (cached)
    void* pin_y_dev_of = nullptr;  // the pin_y it was taken from
    cudaStream_t stream = nullptr;
    std::mutex host_mu;            // the host-pointer entry points use this handle's staging buffers one call at a time
    DqLists dq_lists;              // tensor-core path: outliers listed per weight tile (freed by its own destructor)
    // host-pointer forward: the copy of x and the kernel as one instantiated graph (one launch call per forward)
    cudaGraphExec_t host_graph = nullptr;
    int host_graph_batch = 0;
    const void* host_graph_key[3] = {nullptr, nullptr, nullptr};   // pin_x, d_x, pin_y_dev it was captured with
    // Bumped whenever the arrays a captured launch or a problem snapshot points at are replaced
    // (ojasx_set_linear_outliers); graphs and groups built from an older generation are rebuilt.
    unsigned generation = 0;

    ~LinearHandle();
    LinearProblem problem(const void* x, void* y, int batch, int io_dtype, int row_start, int row_stop) const;
};

struct LinearGroup {
    int dev = 0;
    int D = 0;
    int total_items = 0;
    std::vector<LinearProblem> host;
    std::vector<const LinearHandle*> members;   // borrowed: the layers must outlive the group
    std::vector<unsigned> member_generation;    // generation of each layer when host[i] was taken
    LinearProblem* dev_probs = nullptr;
    const void* bound_x = nullptr;
    void* bound_y = nullptr;
    size_t bound_xs = 0, bound_ys = 0;
    int bound_dtype = -1;
    int bound_full = 0;   // the table on the device was written for the gathered output layout
};

struct MoeHandle {
    int dev = 0;
    int E = 0;            // experts held here
    int E_total = 0;      // experts the router scores (== E unless sharded)
    int expert_offset = 0;
    int H = 0, I = 0, top_k = 0, D = 0;
    float gate_limit = 0.0f;   // <= 0: none
    float* cb_in = nullptr;
    float* cb_down = nullptr;
    uint8_t* gu_codes = nullptr;
    float* gu_scales = nullptr;
    uint8_t* dn_codes = nullptr;
    float* dn_scales = nullptr;
    int* csr_rp[2] = {nullptr, nullptr};     // 0 gate_up, 1 down
    int* csr_cols[2] = {nullptr, nullptr};
    float* csr_vals[2] = {nullptr, nullptr};
    int csr_nnz[2] = {0, 0};
    float* router = nullptr;                 // [E_total, H]
    void* scratch = nullptr;                 // inter [pairs, I] + expert_out [pairs, H]
    size_t scratch_cap = 0;
    void* lut_scratch = nullptr;             // token tables [tokens, G, 256]
    size_t lut_cap = 0;
    void* route_scratch = nullptr;           // logits, probs [tokens, E_total], idx, w [pairs]
    size_t route_cap = 0;
    void* stage = nullptr;                   // host-pointer forward staging
    size_t stage_cap = 0;
    cudaStream_t stream = nullptr;
    std::mutex host_mu;                      // host-pointer forwards of one handle run one at a time

    ~MoeHandle();
    int reserve(int n_tokens, int k);
    MoeProblem problem(const void* x, void* y, const int* idx, const float* w, int n_tokens, int k, int io) const;
};

struct KvqHandle {
    int dev = 0;
    int B = 0, Hkv = 0, Hq = 0, head_dim = 0, D = 0, G = 0, max_seq = 0;
    int host_len = 0;                        // host mirror of the (uniform) cached length
    bool static_plan = false;                // plan launches for max_seq; only the device-side lengths are consulted
    uint8_t* k_codes = nullptr;
    uint8_t* v_codes = nullptr;
    float* k_cb = nullptr;
    float* v_cb = nullptr;
    int* seq_lens = nullptr;
    int* error_flag = nullptr;
    int* counters = nullptr;                 // [B] append + [B*Hkv] decode completion counters (zero between launches)
    void* partials = nullptr;
    size_t partials_cap = 0;
    ~KvqHandle();
};

struct LegacyKvHandle {
    struct Head {
        uint8_t* k_codes = nullptr;
        uint8_t* v_codes = nullptr;
        float* k_scales = nullptr;
        float* v_scales = nullptr;
        int len = 0, cap = 0;
    };
    int dev = 0;
    int num_heads = 0, head_dim = 0, D = 0, G = 0, initial_cap = 0;
    std::vector<Head> heads;
    void* stage = nullptr;    // q | k,v | out
    size_t stage_cap = 0;
    void* logits = nullptr;
    size_t logits_cap = 0;
    cudaStream_t stream = nullptr;
    std::mutex host_mu;       // append / attention of one cache run one at a time
    ~LegacyKvHandle();
};

}  // namespace ojx
