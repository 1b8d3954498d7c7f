// Host-side launch entry points shared by the C ABI translation unit.
#pragma once
#include "common.cuh"

namespace ojx {

struct PeerLink;   // peer.cuh: exchange over peer memory fused into a kernel's epilogue (null / n == 0: none)
const PeerLink* peer_link_of(void* peer_link_handle);

// --- linear.cu
int plan_tile_rows(int rows, int parallel_items);
int validate_linear(const LinearProblem& P);
int launch_linear(LinearProblem P, cudaStream_t stream, const PeerLink* link = nullptr);
int launch_linear_group(const LinearProblem* d_probs, int nprobs, int total_items, int D, cudaStream_t stream,
                        const PeerLink* link = nullptr);

// --- linear_cluster.cu: OJX_ERR_UNSUPPORTED means "use the persistent kernel"
int try_launch_linear_cluster(const LinearProblem& P, cudaStream_t stream, const PeerLink* link = nullptr);
// Up to 8 host-side problems with the same K, G, block_dim, batch and io dtype in one cluster launch.
int try_launch_linear_cluster_group(const LinearProblem* probs, int count, cudaStream_t stream, const PeerLink* link = nullptr);
// True when OJASX_B200_LINEAR_KERNEL=persistent asks for the streaming kernel only.
bool linear_cluster_disabled();

// --- rvq_generic.cu
int launch_rvq_generic(const uint8_t* packed, const float* codebooks, const float* row_scales, const float* bias,
                       const float* x, int batch, int stages, int bits, int D, int rows, int columns, int row_start,
                       int row_stop, float* out, cudaStream_t stream);

// --- dequant_gemm.cu (tcgen05 path for bf16 batches)
bool dequant_gemm_supported(const LinearProblem& P, bool csr_sorted);
// scratch / scratch_cap: a grow-only device buffer of the caller (per layer handle) for the split-K partial
// sums and tile counters; null = never split.  Calls that share the buffer must not overlap in time.
// Outliers of a layer listed per (128-row, 64-column) weight tile for the tensor-core path; built on the device the
// first time a layer and row range take that path, kept by the layer's handle.
struct DqLists {
    int* off = nullptr;        // [row_tiles * (K / 64 + 1) + 1] tile offsets, followed by the scatter cursors
    int2* ent = nullptr;       // [nnz] (row in tile << 8 | column in tile, value / row scale)
    size_t off_cap = 0, ent_cap = 0;
    int row_start = -1, row_stop = -1;
    unsigned generation = 0;
    const float* csr_vals = nullptr;
    bool valid = false;
    ~DqLists();
};
int launch_dequant_gemm(const LinearProblem& P, cudaStream_t stream, DqLists* lists = nullptr, unsigned generation = 0);
int take_dequant_gemm_error(int* out);

// --- moe.cu
// link: expert-parallel ranks gather every pair's expert output over peer memory before the combine (null: one rank)
int launch_moe_experts(MoeProblem P, cudaStream_t stream, const PeerLink* link = nullptr);
int launch_build_lut(const void* x, int io_dtype, int n_vectors, int K, int D, const float* codebook, int Kcb, float* out,
                     cudaStream_t stream);
int launch_silu_mul(const void* gate, const void* up, void* out, size_t n, int io_dtype, cudaStream_t stream);
// codebook .. lut_out: when lut_out is not null the gate/up tables of the tokens ([n_tokens, H/D, 256]) are
// built by the same launch as the logits.
int launch_moe_router(const float* Wr, const void* x, int io_dtype, int n_tokens, int H, int E, int k,
                      float* logits, float* probs, int* idx_out, float* w_out, cudaStream_t stream,
                      const float* codebook = nullptr, int Kcb = 0, int D = 0, float* lut_out = nullptr,
                      int lut_blocks = 0, const PeerLink* link = nullptr, int e_begin = 0, int e_end = 0);

// --- moe_fused.cu: whole-expert work items (gate/up, SiLU gate and down fused) for batches of tokens
bool moe_chain_wanted(const MoeProblem& P);   // gate/up by the chain walk: whole experts per work item and a fitting shape
int moe_table_layout(const MoeProblem& P);    // MoeProblem::lut_blocks this forward wants
size_t moe_table_bytes(int n_tokens, int G, int D);   // table scratch that fits every layout
int launch_moe_chain_images(const void* x, int io_dtype, int n_tokens, int H, int D, const float* cb, int Kcb, float* out, cudaStream_t s);
bool moe_fused_wanted(const MoeProblem& P);   // shape fits and enough routed pairs are expected here
int launch_moe_fused(MoeProblem P, cudaStream_t stream, const PeerLink* link = nullptr);   // work list, token tables (unless lut_ready), experts
int launch_moe_prebuild_blocks(const void* x, int io_dtype, int n_tokens, int H, int D, const float* codebook, int Kcb,
                               float* out, cudaStream_t stream);
int take_moe_fused_error(int* out);
int take_moe_bulk_copy_error(int* out);   // moe.cu: a bounded wait for a bulk table copy ran out

// --- kv.cu
constexpr int kKvMaxSplits = 256;   // context splits of one (sequence, KV head) in kvq decode
size_t kvq_decode_smem(const KvqProblem& P, int R);
// Fills P.chunk (tokens per CTA) and P.n_chunks (<= kKvMaxSplits) for a context of T tokens.
void plan_kvq_decode(KvqProblem& P, int T, int sms);
int launch_kvq_append(const KvqProblem& P, cudaStream_t stream);
int launch_kvq_decode(const KvqProblem& P, cudaStream_t stream, const PeerLink* link = nullptr);
int launch_legacy_append(const float* k, const float* v, int head_dim, int block_dim, uint8_t* k_row, uint8_t* v_row,
                         float* k_scale, float* v_scale, cudaStream_t stream);
int launch_legacy_attention(const float* q, int head_dim, int block_dim, int T, const uint8_t* k_codes,
                            const uint8_t* v_codes, const float* k_scales, const float* v_scales, float scale_factor,
                            float* logits, float* out, cudaStream_t stream);

}  // namespace ojx
