/*
 * ojasx_lut_b200.h -- C ABI of libojasx_lut_b200.so, the sm_100a (B200) implementation of the
 * split-manifold LUT execution path.
 *
 * Two groups of entry points:
 *
 *  1. The reference's handle API, same names, argument lists and return codes as
 *     split_manifold_lut_experiment/native/include/ojasx_lut_c_api.h:35-150.  All data
 *     pointers are HOST pointers; create_* deep-copies the arrays into device memory (the
 *     reference deep-copies into std::vector, ojasx_lut_c_api.cpp:44-58, 230-251); *_forward
 *     copies x to the device, runs the CUDA kernels on the handle's stream, copies y back and
 *     returns after the result is in host memory.  A program or binding written against the
 *     reference's libojasx_lut.so can load this library instead without changes.
 *
 *  2. ojasx_b200_* entry points that take DEVICE pointers and a CUDA stream (passed as void*,
 *     like ojasx_cuda_rvq_fused_gemm in ojasx_24x96/native/vq_kernels_cuda.cu:230-245).  They
 *     enqueue work and return without synchronising.
 *
 * Return codes: 0 ok, -1 null or invalid argument, -2 index out of range (both as the
 * reference), -3 CUDA runtime error (text via ojasx_b200_last_error), -4 unsupported
 * configuration, -5 size beyond a stated limit.
 *
 * There is no CPU fallback: every forward needs a CUDA device.
 */
#ifndef OJASX_LUT_B200_H
#define OJASX_LUT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OJASX_API __attribute__((visibility("default")))

typedef void* OjasxLinearHandle;
typedef void* OjasxKVHandle;
typedef void* OjasxMoEHandle;

#define OJASX_B200_F32 0
#define OJASX_B200_BF16 1

/* ------------------------------------------------------------------ 1. reference handle API */

/* ojasx_lut_c_api.h:40-41 */
OJASX_API const char* ojasx_get_version(void);
OJASX_API const char* ojasx_get_backend_name(void);

/* ojasx_lut_c_api.h:46-55.  codebook [codebook_size, block_dim] f32, codes [out, in/block_dim]
 * u8, scales [out] f32 (NULL = ones), bias [out] f32 (NULL = none). */
OJASX_API OjasxLinearHandle ojasx_create_linear(int in_features, int out_features, int block_dim,
                                                int codebook_size, const float* codebook_data,
                                                const uint8_t* codes_data, const float* scales_data,
                                                const float* bias_data);
/* ojasx_lut_c_api.h:60-66.  row_ptrs has out_features+1 entries. */
OJASX_API int ojasx_set_linear_outliers(OjasxLinearHandle handle, int nnz, const int* row_ptrs,
                                        const int* col_indices, const float* values);
/* ojasx_lut_c_api.h:72-78.  x [batch, in] f32 host, y [batch, out] f32 host.  num_threads is
 * accepted and ignored (the work runs on the GPU). */
OJASX_API int ojasx_linear_forward(OjasxLinearHandle handle, const float* x, float* y, int batch_size,
                                   int num_threads);
/* ojasx_lut_c_api.h:83-86 */
OJASX_API size_t ojasx_get_compressed_size(OjasxLinearHandle handle);
OJASX_API size_t ojasx_get_dense_size(OjasxLinearHandle handle);
OJASX_API size_t ojasx_get_lut_sram_size(OjasxLinearHandle handle);
OJASX_API float ojasx_get_compression_ratio(OjasxLinearHandle handle);
/* ojasx_lut_c_api.h:91 */
OJASX_API void ojasx_destroy_linear(OjasxLinearHandle handle);

/* ojasx_lut_c_api.h:96-121.  The reference's cache as shipped: per token and per block_dim-wide
 * block, the block's first coordinate as int8 with a per-token abs-max scale
 * (ojasx_lut_kv_cache.cpp:16-65).  Grows by doubling like the reference. */
OJASX_API OjasxKVHandle ojasx_create_kv_cache(int num_heads, int head_dim, int max_seq_len, int block_dim);
OJASX_API int ojasx_kv_cache_append(OjasxKVHandle handle, int head_idx, const float* k, const float* v);
OJASX_API int ojasx_kv_cache_attention(OjasxKVHandle handle, int head_idx, const float* q,
                                       float* out_context, float scale_factor);
OJASX_API size_t ojasx_kv_cache_get_memory_size(OjasxKVHandle handle);
OJASX_API float ojasx_kv_cache_get_compression_ratio(OjasxKVHandle handle);
OJASX_API void ojasx_destroy_kv_cache(OjasxKVHandle handle);

/* ojasx_lut_c_api.h:126-150 */
OJASX_API OjasxMoEHandle ojasx_create_moe(int num_experts, int hidden_dim, int intermediate_dim, int top_k,
                                          int block_dim, const float* codebook_in, const float* codebook_down,
                                          const uint8_t* gate_up_codes, const float* gate_up_scales,
                                          const uint8_t* down_codes, const float* down_scales);
OJASX_API int ojasx_moe_forward(OjasxMoEHandle handle, const float* x, const int* top_k_indices,
                                const float* top_k_weights, float* y_out, int k_active);
OJASX_API size_t ojasx_moe_get_compressed_size(OjasxMoEHandle handle);
OJASX_API float ojasx_moe_get_compression_ratio(OjasxMoEHandle handle);
OJASX_API void ojasx_destroy_moe(OjasxMoEHandle handle);

/* ------------------------------------------------------------------ 2. device-pointer API */

/* Text of the last error raised on the calling thread ("" if none). */
OJASX_API const char* ojasx_b200_last_error(void);
/* Number of kernels this library has launched since it was loaded (all threads). */
OJASX_API unsigned long long ojasx_b200_launch_count(void);

/* Forward of a linear handle on device buffers; replaces ojasx_linear_forward
 * (ojasx_lut_c_api.h:72-78) for callers whose activations already live on the GPU.
 * d_x [batch, in] and d_y [batch, row_stop-row_start] are of io_dtype (OJASX_B200_F32 / _BF16;
 * bf16 follows ojasx_24x96/math_engine.py:161,208: widen x to fp32, compute in fp32, round y).
 * Rows [row_start,row_stop) follow the row-slice contract of rvq_fused_gemm
 * (ojasx_24x96/native/ojasx_backend_abi.h:97-111); pass 0, out_features for the whole layer. */
OJASX_API int ojasx_b200_linear_forward(OjasxLinearHandle handle, const void* d_x, void* d_y, int batch_size,
                                        int io_dtype, int row_start, int row_stop, void* stream);

/* The same layer on the tensor cores (tcgen05): bf16 d_x [batch, in] and d_y [batch, row_stop-row_start],
 * weights dequantised tile by tile into shared memory (rounded to bf16), fp32 accumulation.  No
 * counterpart in the reference (its GPU kernels are CUDA-core GEMVs, ojasx_lut_cuda.cu:59-87).
 * Results follow the bf16-activation tolerance (rel 2e-2), not the bit-exact order of the table
 * kernels.  ojasx_b200_linear_forward picks this path by itself for bf16 batches >= 32
 * (OJASX_B200_TENSOR_MIN_BATCH overrides; 0 disables).  Needs block_dim 8, 256 centroids,
 * in_features % 64 == 0 and CSR columns ascending inside each row; otherwise -4. */
OJASX_API int ojasx_b200_linear_forward_tensor(OjasxLinearHandle handle, const void* d_x, void* d_y, int batch_size,
                                               int row_start, int row_stop, void* stream);
/* Device-side error flags raised since the last call (the outputs of the launch that raised one are
 * invalid), 0 if none; synchronises the device.  Bit 0: a tensor-core launch gave up on a bounded
 * barrier wait.  Bit 1: the batched MoE expert kernel found its shared memory at an unexpected address
 * and did nothing.  Bit 2: a bounded wait for a bulk copy of a lookup table ran out, or a whole-expert
 * MoE kernel of the chain walk found the same placement and did nothing.  Negative = CUDA error. */
OJASX_API int ojasx_b200_take_device_error(void);

/* Same computation on borrowed device arrays, no handle: the device twin of
 * ojasx_cuda_rvq_fused_gemm (ojasx_24x96/native/vq_kernels_cuda.cu:230-258) for the
 * 8-bit single-stage layout, plus the CSR outliers of ojasx_set_linear_outliers. */
OJASX_API int ojasx_b200_linear_forward_raw(const uint8_t* d_codes, const float* d_codebook,
                                            const float* d_scales, const float* d_bias, int nnz,
                                            const int* d_row_ptrs, const int* d_col_indices,
                                            const float* d_values, const void* d_x, void* d_y,
                                            int batch_size, int io_dtype, int block_dim, int codebook_size,
                                            int rows, int columns, int row_start, int row_stop, void* stream);

/* Device twin of the vtable entry rvq_fused_gemm (ojasx_24x96/native/ojasx_backend_abi.h:97-111)
 * with the argument list of ojasx_cuda_rvq_fused_gemm (ojasx_24x96/native/vq_kernels_cuda.cu:230-245):
 * bit-packed residual-VQ codes of any supported width (1, 2, 4, 8) and stage count, fp32 in and
 * out, output [batch, row_stop-row_start].  8-bit single-stage layers run on the table kernels;
 * other layouts run on a compatibility kernel.  Returns -1 for invalid arguments and -2 for an
 * unsupported bit width, as ojasx_rvq_fused_gemm does (leech24_cpu.cpp:386-397). */
OJASX_API int ojasx_b200_rvq_fused_gemm(const uint8_t* packed_codes, const float* codebooks, const float* row_scales,
                                        const float* bias, const float* inputs, int batch_size, int stages,
                                        int bits_per_stage, int block_size, int rows, int columns, int row_start,
                                        int row_stop, float* output, void* stream);

/* One launch over many independent linear handles (no counterpart in the reference, which
 * runs one layer per call): problem p reads d_x + p*x_stride_bytes and writes
 * d_y + p*y_stride_bytes.  x_stride_bytes == 0 feeds every layer the same activations
 * (q/k/v, gate/up).  All handles must share block_dim and must outlive the group (the group
 * borrows them; outliers set on a member after the group was made are picked up by the next
 * forward). */
typedef void* OjasxLinearGroupHandle;
OJASX_API OjasxLinearGroupHandle ojasx_b200_create_linear_group(const OjasxLinearHandle* handles, int count);
OJASX_API int ojasx_b200_linear_group_forward(OjasxLinearGroupHandle group, const void* d_x,
                                              size_t x_stride_bytes, void* d_y, size_t y_stride_bytes,
                                              int io_dtype, void* stream);
OJASX_API void ojasx_b200_destroy_linear_group(OjasxLinearGroupHandle group);

/* ---- MoE on device buffers; replaces ojasx_moe_forward (ojasx_lut_c_api.h:139-146) for any
 * number of tokens.  d_x, d_y [n_tokens, hidden] of io_dtype; d_topk_idx i32 and d_topk_w f32
 * are [n_tokens, k_active] with GLOBAL expert ids; ids outside this handle's experts and
 * weights with |w| < 1e-8 are skipped (ojasx_lut_cpu.cpp:284-286).  The first call with a
 * larger n_tokens*k_active grows the handle's scratch (cudaMalloc); ojasx_b200_moe_reserve
 * does that ahead of time.  The handle's device must be the current device (-1 otherwise), and a
 * handle serves one stream at a time: its scratch is shared by every call on it, so calls on
 * different streams must be ordered by the caller. */
OJASX_API int ojasx_b200_moe_forward(OjasxMoEHandle handle, const void* d_x, const int* d_topk_idx,
                                     const float* d_topk_w, void* d_y, int n_tokens, int k_active, int io_dtype,
                                     void* stream);
OJASX_API int ojasx_b200_moe_reserve(OjasxMoEHandle handle, int max_tokens, int k_active);
/* Clamp of the fused-experts operator (ResidualVQFusedExperts._apply_gate, ojasx_24x96/module.py:646-651):
 * with limit > 0 the gate value is clamped from above to limit and the up value to [-limit, limit] before
 * silu(gate) * up; limit <= 0 (the default) applies none, which is the reference library's MoE
 * (ojasx_lut_cpu.cpp:325). */
OJASX_API int ojasx_b200_moe_set_gate_limit(OjasxMoEHandle handle, float limit);
/* CSR outliers on the expert matrices (host arrays; no counterpart in the reference MoE, which
 * has none: composed like ojasx_set_linear_outliers, ojasx_lut_c_api.h:60-66).  which = 0: the
 * flattened gate_up matrix [E*2I, hidden]; which = 1: the flattened down matrix [E*hidden, I]. */
OJASX_API int ojasx_b200_moe_set_outliers(OjasxMoEHandle handle, int which, int nnz, const int* row_ptrs,
                                          const int* col_indices, const float* values);
/* Router weights f32 [num_experts_total, hidden] (host).  Formula of
 * split_manifold_lut_experiment/tools/run_full_48_layers_and_generate.py:172-175:
 * softmax(x W^T) -> top-k -> renormalise. */
OJASX_API int ojasx_b200_moe_set_router(OjasxMoEHandle handle, const float* router_weight, int num_experts_total);
/* Expert-parallel shard: this handle holds global experts [first, first + num_experts). */
OJASX_API int ojasx_b200_moe_set_expert_offset(OjasxMoEHandle handle, int first_global_expert);
OJASX_API int ojasx_b200_moe_route(OjasxMoEHandle handle, const void* d_x, int n_tokens, int top_k, int* d_idx_out,
                                   float* d_w_out, int io_dtype, void* stream);
/* Router followed by the experts, one stream, no host round trip. */
OJASX_API int ojasx_b200_moe_forward_routed(OjasxMoEHandle handle, const void* d_x, void* d_y, int n_tokens, int top_k,
                                            int io_dtype, void* stream);

/* The lookup table on its own: d_lut[t, g, k] = sum_d x[t, g*block_dim + d] * codebook[k, d], d ascending, fp32,
 * separate multiply and add -- SplitManifoldLinear::build_lut (ojasx_lut_cpu.cpp:18-102; the Python twin is
 * SplitManifoldLUTLinear.build_lut, split_manifold_engine.py:185-199).  d_x [n_vectors, in_features] of io_dtype
 * (features beyond in_features read as zero), d_lut f32 [n_vectors, ceil(in_features / block_dim), 256] with
 * entries k >= codebook_size set to zero.  The forward kernels build their tables in shared memory and never
 * call this; it exists for callers (and tests) that want kernel (a)'s result itself. */
OJASX_API int ojasx_b200_build_lut(const void* d_x, int n_vectors, int in_features, int block_dim,
                                   const float* d_codebook, int codebook_size, float* d_lut, int io_dtype, void* stream);

/* out[i] = silu(gate[i]) * up[i] on device arrays of io_dtype: the SwiGLU step between the gate/up and
 * down linears of a dense VQ MLP block, with the silu of the expert kernels
 * (v / (1 + exp(-v)), ojasx_lut_cpu.cpp:209-211; :325 for the product). */
OJASX_API int ojasx_b200_silu_mul(const void* d_gate, const void* d_up, void* d_out, size_t count, int io_dtype,
                                  void* stream);

/* MoE forward that obtains no memory.  It has no counterpart in the reference.
 *
 * Who it is for: code that runs where asking the CUDA runtime for memory is not possible or not
 * allowed -- a serving loop whose device memory was handed out in full at start-up to a pool
 * owned by someone else, a plugin called from inside another framework's step where an
 * allocation would synchronise the device and stall that framework's streams, or a host thread
 * with a hard latency budget.  ojasx_b200_moe_forward grows a per-handle scratch buffer with
 * cudaMalloc whenever n_tokens*k_active rises; this variant instead keeps its scratch (the
 * per-pair intermediate activations and per-pair expert outputs) in a fixed array inside the
 * library's device image and calls no cudaMalloc, cudaFree or other allocating routine.
 *
 * Same arguments, same results, same skipping rules as ojasx_b200_moe_forward.  Limits and rules:
 *  - n_tokens * k_active * (intermediate_dim + hidden_dim) must not exceed
 *    OJASX_B200_NOALLOC_SCRATCH_FLOATS (1 MiB of fp32; 81 routed pairs at hidden 2560 /
 *    intermediate 640, i.e. 8 tokens at top-10).  Larger requests return -5 and do nothing.
 *  - Every GPU that loads the library holds that 1 MiB until the process exits.
 *  - The handle's device must be the current device (-1 otherwise).
 *  - The first call on each device looks up the array's device address; make that first call
 *    outside of any stream capture.
 *  - All calls, from every handle and stream, share the one array.  The array keeps whatever the
 *    last call left in it (nothing needs clearing: each call writes every slot before reading it),
 *    and two calls that overlap in time on the same GPU race on it.  Keep calls on one stream, or
 *    order them with events. */
#define OJASX_B200_NOALLOC_SCRATCH_FLOATS 262144
OJASX_API int ojasx_b200_moe_forward_noalloc(OjasxMoEHandle handle, const void* d_x, const int* d_topk_idx,
                                             const float* d_topk_w, void* d_y, int n_tokens, int k_active,
                                             int io_dtype, void* stream);

/* ---- Exchange between the GPUs of one box over peer memory, fused into the producing kernel (no counterpart
 * in the reference, which has no multi-device code; the row contract it serves is row_start / row_stop of
 * rvq_fused_gemm, ojasx_24x96/native/ojasx_backend_abi.h:97-111).  Every rank allocates one segment of the same
 * size, exports it, opens the others' (CUDA IPC: one process per GPU on one machine) and makes a link from the
 * n mappings.  Buffers that take part in an exchange live at the same offset in every rank's segment; n ints at
 * flags_offset are the link's flags.  A "gather" entry point stores its shard into every rank's segment and then
 * raises this rank's flag everywhere; ojasx_b200_peer_wait (or the consumer kernel of this library) polls all
 * flags before the gathered buffer is read.  Waits are bounded (a few seconds): a rank that never signals
 * raises ojasx_b200_peer_take_status instead of hanging.  A buffer may be written again two exchanges later;
 * repeat one exchange on two alternating buffers.  Plain loads and stores only: no multicast of any kind. */
#define OJASX_B200_PEER_HANDLE_BYTES 64
typedef void* OjasxPeerLinkHandle;
OJASX_API void* ojasx_b200_peer_alloc(size_t bytes);                                  /* zero-filled device segment */
OJASX_API int ojasx_b200_peer_free(void* d_segment);
OJASX_API int ojasx_b200_peer_export(void* d_segment, unsigned char* handle_out);    /* 64 bytes to send to the others */
OJASX_API void* ojasx_b200_peer_open(const unsigned char* handle);                   /* mapping of another rank's segment */
OJASX_API int ojasx_b200_peer_close(void* d_mapped);
OJASX_API OjasxPeerLinkHandle ojasx_b200_peer_link_create(void* const* d_segments, int n_ranks, int self,
                                                          size_t flags_offset);
OJASX_API void ojasx_b200_peer_link_destroy(OjasxPeerLinkHandle link);
OJASX_API int ojasx_b200_peer_signal(OjasxPeerLinkHandle link, void* stream);       /* for producers outside this library */
OJASX_API int ojasx_b200_peer_wait(OjasxPeerLinkHandle link, void* stream);
/* d_src [bytes] (a multiple of 4) to d_dst_shared in every rank's segment, then the flag: the gather of small
 * per-rank records (each rank puts into its own slot), e.g. the (max, index) pairs of a vocabulary-split arg-max. */
OJASX_API int ojasx_b200_peer_put(OjasxPeerLinkHandle link, void* d_dst_shared, const void* d_src, size_t bytes, void* stream);
OJASX_API int ojasx_b200_peer_take_status(OjasxPeerLinkHandle link);                 /* 1: a wait ran out since the last call */
/* Rows [row_start, row_stop) of the layer into columns [row_start, row_stop) of d_y_full [batch, out_features]
 * on every rank (d_y_full inside the link's segment), then the flag: the row-split linear with its all-gather.
 * An empty row range only raises the flag. */
OJASX_API int ojasx_b200_linear_forward_gather(OjasxLinearHandle handle, const void* d_x, void* d_y_full, int batch_size,
                                               int io_dtype, int row_start, int row_stop, OjasxPeerLinkHandle link,
                                               void* stream);
/* The same for a group: set_rows restricts every member to rows [row_start, row_stop) (clipped to its size);
 * forward_gather writes the gathered layout ([.., out_features] per problem at y_stride_bytes) on every rank. */
OJASX_API int ojasx_b200_linear_group_set_rows(OjasxLinearGroupHandle group, int row_start, int row_stop);
OJASX_API int ojasx_b200_linear_group_forward_gather(OjasxLinearGroupHandle group, const void* d_x, size_t x_stride_bytes,
                                                     void* d_y_full, size_t y_stride_bytes, int io_dtype,
                                                     OjasxPeerLinkHandle link, void* stream);
/* Expert-parallel MoE: this handle's experts are evaluated, every (token, expert) output row goes to
 * d_expert_out_shared [n_tokens * k, hidden] (inside the segment) on every rank, and the combine -- which waits for
 * all flags -- adds a token's k rows in caller order on every rank: d_y is the full layer output everywhere, with
 * the bits a single device produces. */
OJASX_API int ojasx_b200_moe_forward_gather(OjasxMoEHandle handle, const void* d_x, const int* d_topk_idx,
                                            const float* d_topk_w, void* d_y, int n_tokens, int k_active, int io_dtype,
                                            OjasxPeerLinkHandle link, float* d_expert_out_shared, void* stream);
/* Routed form.  d_logits_shared [n_tokens, num_experts_total] (inside the segment) or NULL: with it every rank scores
 * only the experts it holds and stores their logits into every rank's buffer (one more exchange on the link, before
 * the top-k pass); without it every rank scores all experts itself.  Same routing either way. */
OJASX_API int ojasx_b200_moe_forward_routed_gather(OjasxMoEHandle handle, const void* d_x, void* d_y, int n_tokens,
                                                   int top_k, int io_dtype, OjasxPeerLinkHandle link,
                                                   float* d_expert_out_shared, float* d_logits_shared, void* stream);

/* ---- Codebook-VQ KV cache of one layer (no counterpart in the reference, whose HeadKVCache
 * allocates k_codebook / v_codebook but never reads them, ojasx_lut_kv_cache.h:33-35): every
 * head vector is head_dim/block_dim uint8 codes into a per-KV-head codebook
 * f32 [kv_heads, 256, block_dim] (host arrays at create).  Codes live on the device as
 * [batch, kv_heads, max_seq_len, groups]. */
typedef void* OjasxKvqHandle;
OJASX_API OjasxKvqHandle ojasx_b200_kvq_create(int batch, int kv_heads, int q_heads, int head_dim, int block_dim,
                                               int max_seq_len, const float* k_codebook, const float* v_codebook);
/* Fill the cache from host codes [batch, kv_heads, seq_len, groups] and set every length to seq_len. */
OJASX_API int ojasx_b200_kvq_load(OjasxKvqHandle handle, const uint8_t* k_codes, const uint8_t* v_codes, int seq_len);
/* Copy tokens [t_begin, t_end) of every head back to host arrays [batch, kv_heads, t_end-t_begin, groups]. */
OJASX_API int ojasx_b200_kvq_read(OjasxKvqHandle handle, uint8_t* k_codes, uint8_t* v_codes, int t_begin, int t_end);
OJASX_API int ojasx_b200_kvq_seq_len(OjasxKvqHandle handle);
OJASX_API int ojasx_b200_kvq_reset(OjasxKvqHandle handle);
/* Append one token per sequence: d_k, d_v [batch, kv_heads, head_dim] of io_dtype; nearest
 * centroid per sub-vector, rule of ojasx_24x96/codec.py:217-224.  -2 when the cache is full. */
OJASX_API int ojasx_b200_kvq_append(OjasxKvqHandle handle, const void* d_k, const void* d_v, int io_dtype, void* stream);
/* One decode query per sequence: d_q, d_out [batch, q_heads, head_dim] of io_dtype; softmax over
 * every cached token; scale <= 0 means 1/sqrt(head_dim) (ojasx_lut_kv_cache.cpp:74-76). */
OJASX_API int ojasx_b200_kvq_decode(OjasxKvqHandle handle, const void* d_q, void* d_out, float scale, int io_dtype,
                                    void* stream);
OJASX_API void ojasx_b200_kvq_destroy(OjasxKvqHandle handle);

/* ---- Per-token operators of a decoder step (no counterpart in the reference, which leaves them to the
 * HuggingFace model it drives, ojasx_24x96/engine.py:176-199); they exist so that one decode step is a
 * fixed sequence of launches of this library and can be captured in a CUDA graph.
 * rmsnorm: if d_add is not NULL, d_x += d_add first (residual), then d_out = d_x * rsqrt(mean(d_x^2)+eps) * w.
 * rope_qk: rotate-half rotary embedding in place on q [batch, q_heads, head_dim] and k [batch, kv_heads,
 * head_dim] at the per-sequence positions d_positions (int32, device).  add_int: d_values[i] += delta. */
OJASX_API int ojasx_b200_rmsnorm(void* d_x, const void* d_add, const float* d_weight, void* d_out, int rows, int hidden,
                                 float eps, int io_dtype, void* stream);
OJASX_API int ojasx_b200_rope_qk(void* d_q, void* d_k, const int* d_positions, int batch, int q_heads, int kv_heads,
                                 int head_dim, float theta, int io_dtype, void* stream);
OJASX_API int ojasx_b200_add_int(int* d_values, int count, int delta, void* stream);
/* KV-head shard: this cache holds some of the layer's KV heads (with their query heads); its attention outputs go
 * to heads [first_q_head, first_q_head + q_heads) of d_out_full [batch, total_q_heads, head_dim] on every rank of the
 * link (d_out_full inside the link's segment), then the flag is raised: the all-gather of head-sharded attention,
 * fused into the decode kernel.  Wait with ojasx_b200_peer_wait before reading d_out_full. */
OJASX_API int ojasx_b200_kvq_decode_gather(OjasxKvqHandle handle, const void* d_q, void* d_out_full, float scale,
                                           int io_dtype, int total_q_heads, int first_q_head, OjasxPeerLinkHandle link,
                                           void* stream);
/* Plan decode launches for the cache's capacity instead of its current length, and let the device-side
 * length be the only one consulted: the launch sequence of append/decode then never changes as the
 * context grows, so it can be replayed from a CUDA graph.  ojasx_b200_kvq_seq_len stays at the value of
 * the last eager call until ojasx_b200_kvq_sync_len reads the device length back (synchronises).
 * Under the static plan the host cannot refuse an append to a full cache: the kernel drops that
 * token and raises a device flag; ojasx_b200_kvq_sync_len then returns -2 once (and clears the
 * flag) instead of the length, so poll it whenever the context may have reached max_seq_len. */
OJASX_API int ojasx_b200_kvq_set_static_plan(OjasxKvqHandle handle, int enabled);
/* Drops the cached tokens beyond max_len of every sequence (the crop of OjasXKVCacheManager,
 * ojasx_24x96/kv_cache.py:196-256, for this cache); returns the new length, -2 for a negative max_len.
 * Synchronises.  ojasx_b200_kvq_get_memory_size: bytes of code storage and codebooks the cache holds
 * (the figure ojasx_kv_cache_get_memory_size reports for the reference's cache, ojasx_lut_c_api.h:122). */
OJASX_API int ojasx_b200_kvq_crop(OjasxKvqHandle handle, int max_len);
OJASX_API size_t ojasx_b200_kvq_get_memory_size(OjasxKvqHandle handle);
OJASX_API int ojasx_b200_kvq_sync_len(OjasxKvqHandle handle);

/* ---- offline encoder: nearest-centroid assignment of n block vectors [n, block_dim] (fp32, 16-byte aligned)
 * to a codebook [codebook_size <= 256, block_dim]: codes[i] = arg-min_k |v_i - c_k|^2, first minimum.  With
 * d_sums (f64 [codebook_size, block_dim]) and d_counts (u64 [codebook_size]) not null, the per-cluster sums
 * and sizes of a k-means update are ADDED to them (zero them first).  Device pointers; the hot step of
 * SplitManifoldLUTLinear.from_dense (split_manifold_lut_experiment/engine/split_manifold_engine.py:140-160,
 * torch.cdist + argmin + index_add_ there). */
OJASX_API int ojasx_b200_vq_assign(const float* d_vectors, size_t n_vectors, int block_dim, const float* d_centroids,
                                   int codebook_size, uint8_t* d_codes, double* d_sums, unsigned long long* d_counts,
                                   void* stream);

/* ---- paged int8 KV cache: device side of PagedCompressedKVCache (ojasx_24x96/long_context.py:212-279).
 * quantize: n_vectors rows [head_dim] of io_dtype -> int8 rows and one fp16 scale per row, the arithmetic of
 * _quantize_int8 (:236-241: abs-max clamped at 1e-8, / 127, round half to even, clamp to +-127).
 * decode: softmax(q K^T * scale) V of one query per (sequence, head) over the resident pages, read as int8.
 * Pools are [slots, batch, kv_heads, page_size, head_dim] int8 and [slots, batch, kv_heads, page_size] fp16;
 * d_page_slot[i] is the pool slot of the i-th resident page (oldest first) and d_page_start the prefix sums
 * of the pages' token counts (n_pages + 1 entries, total_tokens last).  d_scratch: at least
 * ojasx_b200_paged_kv_scratch_floats(batch, q_heads, head_dim, total_tokens) floats; d_counters: batch * q_heads
 * ints, zero before the first call (they return to zero).  head_dim 64, 128 or 256; scale <= 0 = 1/sqrt(head_dim). */
OJASX_API int ojasx_b200_paged_kv_quantize(const void* d_src, int io_dtype, size_t n_vectors, int head_dim, int8_t* d_q8,
                                           void* d_scales_f16, void* stream);
OJASX_API int ojasx_b200_paged_kv_scratch_floats(int batch, int q_heads, int head_dim, int max_tokens);
OJASX_API int ojasx_b200_paged_kv_decode(const void* d_q, void* d_out, const int8_t* d_k_pool, const int8_t* d_v_pool,
                                         const void* d_k_scales_f16, const void* d_v_scales_f16, const int* d_page_slot,
                                         const int* d_page_start, int n_pages, int total_tokens, int batch, int q_heads,
                                         int kv_heads, int head_dim, int page_size, float scale, int io_dtype,
                                         float* d_scratch, int* d_counters, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* OJASX_LUT_B200_H */
