// Shared declarations for the sm_100a split-manifold LUT kernels.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stddef.h>

namespace ojx {

// Status codes returned through the C ABI (same numbering as the reference's handle API:
// 0 ok, -1 null/invalid argument, -2 index out of range; -3.. are CUDA-side additions).
enum : int {
    OJX_OK = 0,
    OJX_ERR_ARG = -1,
    OJX_ERR_RANGE = -2,
    OJX_ERR_CUDA = -3,
    OJX_ERR_UNSUPPORTED = -4,
    OJX_ERR_TOO_LARGE = -5,
};

enum : int { OJX_F32 = 0, OJX_BF16 = 1 };

constexpr int kNumSMsDefault = 148;

// CSR outliers over a row range of a (possibly flattened) matrix.  Pointers are device pointers.
struct CsrView {
    const int* row_ptrs;    // indexed by absolute row
    const int* cols;
    const float* vals;
    int nnz;                // 0 = no outliers (row_ptrs may be null)
};

// One VQ linear problem: y[b, m - row_start] for m in [row_start, row_stop).
struct LinearProblem {
    const uint8_t* codes;     // [M, G] row-major
    const float* codebook;    // [Kcb, D]
    const float* scales;      // [M] or null (= 1)
    const float* bias;        // [M] or null
    CsrView csr;
    const void* x;            // [batch, K]  io dtype
    void* y;                  // [batch, row_stop-row_start] io dtype
    int K;                    // input features (x row length)
    int G;                    // groups per row (code bytes per row)
    int D;                    // block_dim
    int Kcb;                  // codebook entries (<= 256)
    int row_start, row_stop;
    int batch;
    int io_dtype;             // OJX_F32 / OJX_BF16
    int tile_rows;            // rows per work item (multiple of 32, <= kAccRows)
    int tiles;                // ceil((row_stop-row_start)/tile_rows)
    int item_begin;           // first global work item of this problem (grouped launches)
    int y_full;               // 0: y is [batch, row_stop - row_start]; 1: y is [batch, y_ld] and row m goes to column m
    int y_ld;                 //    (the gathered layout of a row-split layer: every rank fills its own columns)
};

// Top-k MoE over VQ experts (layout of SplitManifoldMoE, ojasx_lut.h:156-242).  Device pointers.
struct MoeProblem {
    const void* x;            // [n_tokens, H] io dtype
    void* y;                  // [n_tokens, H] io dtype
    const int* topk_idx;      // [n_tokens, k_active] global expert ids
    const float* topk_w;      // [n_tokens, k_active]
    const float* cb_in;       // [Kcb, D] shared by every expert's gate/up
    const float* cb_down;     // [Kcb, D]
    const uint8_t* gu_codes;  // [E, 2I, G]  gate rows [0,I) then up rows [I,2I)
    const float* gu_scales;   // [E, 2I] or null
    const uint8_t* dn_codes;  // [E, H, Gi]
    const float* dn_scales;   // [E, H] or null
    CsrView gu_csr;           // rows of the flattened [E*2I, H] matrix
    CsrView dn_csr;           // rows of the flattened [E*H, I] matrix
    const float* lut_in;      // optional scratch [n_tokens, G, 256]: tables of the tokens, built once per token
    int lut_ready;            // lut_in was filled by the router launch: the expert launch does not rebuild it
    const int* pair_list;     // optional scratch [pairs + 1]: [0] = number of pairs this handle evaluates, then
                              // their ids grouped by expert; null = every pair is visited and skipped if not local
    float* inter;             // scratch [pairs, I]
    float* expert_out;        // scratch [pairs, H]
    int n_tokens, k_active;
    int E;                    // experts held by this handle
    int E_total;              // experts the router scores (>= E)
    int expert_offset;        // global id of local expert 0 (expert-parallel shards)
    int H, I, G, Gi, D, Kcb;
    int io_dtype;
    int gu_tile, gu_tiles, dn_tile, dn_tiles;
    // fused expert kernel (moe_fused.cu): work-list scratch [4 + 5 * pairs] ints, largest chunk, floats per
    // token in the parked sums; lut_blocks: lut_in is laid out in 16-group blocks (moe_prebuild_kernel)
    const int* plan;
    int mc_cmax, mc_nacc;
    int mc_debug;
    int combine_all;          // 1: the combine adds every routed pair with a valid id (outputs of other ranks' experts were
                              // gathered into expert_out); 0: only the pairs this handle evaluated
    float gate_limit;         // > 0: gate is clamped from above and up to [-limit, limit] before silu(gate) * up
                              // (ResidualVQFusedExperts._apply_gate, ojasx_24x96/module.py:646-651); <= 0: no clamp
    const int* chain_ctl;     // [1 + pairs] claim counter and per-slot flags of moe_experts_chain_kernel (zeroed by the plan kernel), or null
    int lut_blocks;           // layout of lut_in: 0 = [token][group][256]; 1 = 16-group blocks (moe_prebuild_kernel);
                              // 2 = per-slice images of the chain walk's table area (moe_chain_prebuild_kernel)
};

// Codebook-VQ KV cache of one layer.  Device pointers.
struct KvqProblem {
    const void* q;          // [B, Hq, head_dim] io dtype (decode)
    void* out;              // [B, Hq, head_dim] io dtype (decode)
    const void* new_k;      // [B, Hkv, head_dim] io dtype (append)
    const void* new_v;
    uint8_t* k_codes;       // [B, Hkv, max_seq, G]
    uint8_t* v_codes;
    const float* k_cb;      // [Hkv, Kcb, D]
    const float* v_cb;
    int* seq_lens;          // [B] tokens cached per sequence
    int* error_flag;        // set to 1 when an append found the cache full
    float* partials;        // scratch [B, Hkv, n_chunks, R, head_dim + 2]
    int* append_done;       // [B] CTAs of the running append that have finished (returns to 0)
    int* split_done;        // [B, Hkv] decode CTAs of a (sequence, head) that have written their partial (returns to 0)
    int B, Hkv, Hq, head_dim, D, G, Kcb, max_seq;
    int chunk, n_chunks;
    int v_copies;           // copies of the value codebook in the decode kernel's shared memory (1 or 8)
    int io_dtype;
    float scale;
    int out_heads;          // query heads of a row of `out` (0: Hq); > Hq when this cache holds a KV-head shard and
    int out_head0;          // writes its heads at [out_head0, out_head0 + Hq) of the gathered output
};

inline int round_up(int a, int b) { return (a + b - 1) / b * b; }

#define OJX_CUDA_TRY(expr)                                   \
    do {                                                     \
        cudaError_t _e = (expr);                             \
        if (_e != cudaSuccess) {                             \
            ojx::set_last_error(#expr, _e);                  \
            return ojx::OJX_ERR_CUDA;                        \
        }                                                    \
    } while (0)

void set_last_error(const char* what, cudaError_t e);
void set_last_error_msg(const char* what);
int num_sms();

}  // namespace ojx
