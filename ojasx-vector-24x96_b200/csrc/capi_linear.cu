// C ABI, linear-layer part: the reference's ojasx_*linear* handle API on host pointers
// (split_manifold_lut_experiment/native/src/ojasx_lut_c_api.cpp:31-129) and the ojasx_b200_*
// device-pointer entry points.  Handles own device copies of every array.
#include "../../include/ojasx_lut_b200.h"
#include "handles.h"
#include "launch.h"
#include "peer.cuh"

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

namespace ojx {

static thread_local char g_err[512] = "";
static std::atomic<unsigned long long> g_launches{0};

void set_last_error(const char* what, cudaError_t e) {
    std::snprintf(g_err, sizeof(g_err), "%s: %s", what, cudaGetErrorString(e));
}
void set_last_error_msg(const char* what) { std::snprintf(g_err, sizeof(g_err), "%s", what); }
void count_launch(int n) { g_launches.fetch_add((unsigned long long)n, std::memory_order_relaxed); }

int num_sms() {
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return kNumSMsDefault;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = kNumSMsDefault;
        cached[dev] = n;
    }
    return cached[dev];
}

int upload(void** dptr, const void* host, size_t bytes) {
    *dptr = nullptr;
    if (bytes == 0) return OJX_OK;
    OJX_CUDA_TRY(cudaMalloc(dptr, bytes));
    if (host) OJX_CUDA_TRY(cudaMemcpy(*dptr, host, bytes, cudaMemcpyHostToDevice));
    else OJX_CUDA_TRY(cudaMemset(*dptr, 0, bytes));
    return OJX_OK;
}

int ensure_capacity(void** dptr, size_t* cap, size_t bytes) {
    if (*cap >= bytes && *dptr) return OJX_OK;
    if (*dptr) OJX_CUDA_TRY(cudaFree(*dptr));
    *dptr = nullptr;
    *cap = 0;
    size_t want = bytes < 4096 ? 4096 : bytes;
    OJX_CUDA_TRY(cudaMalloc(dptr, want));
    *cap = want;
    return OJX_OK;
}

int ensure_pinned(void** hptr, size_t* cap, size_t bytes) {
    if (*cap >= bytes && *hptr) return OJX_OK;
    if (*hptr) OJX_CUDA_TRY(cudaFreeHost(*hptr));
    *hptr = nullptr;
    *cap = 0;
    size_t want = bytes < 65536 ? 65536 : bytes;
    OJX_CUDA_TRY(cudaHostAlloc(hptr, want, cudaHostAllocMapped));
    *cap = want;
    return OJX_OK;
}

// Waits for a stream by polling: the host-pointer entry points are latency-bound (one small
// kernel per call) and a polled query returns a few microseconds sooner than a blocking
// synchronise.  Falls back to the blocking call after ~2 ms of polling.
int wait_stream(cudaStream_t s) {
    for (int i = 0; i < 20000; ++i) {
        cudaError_t e = cudaStreamQuery(s);
        if (e == cudaSuccess) return OJX_OK;
        if (e != cudaErrorNotReady) { set_last_error("cudaStreamQuery", e); return OJX_ERR_CUDA; }
    }
    OJX_CUDA_TRY(cudaStreamSynchronize(s));
    return OJX_OK;
}

DeviceGuard::DeviceGuard(int dev) : prev_(-1) {
    if (cudaGetDevice(&prev_) != cudaSuccess) prev_ = -1;
    if (prev_ != dev) cudaSetDevice(dev); else prev_ = -1;
}
DeviceGuard::~DeviceGuard() { if (prev_ >= 0) cudaSetDevice(prev_); }

LinearHandle::~LinearHandle() {
    DeviceGuard g(dev);
    cudaFree(codes); cudaFree(codebook); cudaFree(scales); cudaFree(bias);
    cudaFree(row_ptrs); cudaFree(cols); cudaFree(vals); cudaFree(d_x); cudaFree(d_y);
    if (host_graph) cudaGraphExecDestroy(host_graph);
    if (pin_x) cudaFreeHost(pin_x);
    if (pin_y) cudaFreeHost(pin_y);
    if (stream) cudaStreamDestroy(stream);
}

LinearProblem LinearHandle::problem(const void* x, void* y, int batch, int io_dtype, int row_start, int row_stop) const {
    LinearProblem P{};
    P.codes = codes; P.codebook = codebook; P.scales = scales; P.bias = bias;
    P.csr = CsrView{row_ptrs, cols, vals, nnz};
    P.x = x; P.y = y; P.K = in; P.G = G; P.D = D; P.Kcb = Kcb;
    P.row_start = row_start; P.row_stop = row_stop; P.batch = batch; P.io_dtype = io_dtype;
    return P;
}

}  // namespace ojx

using namespace ojx;

// Batch from which a bf16 linear runs on the tensor cores instead of the table kernels (measured on
// B200, 2560->6912: table path 61 us vs tensor path 53 us at batch 32, 98 vs 55 at 64).
static constexpr int kTensorMinBatch = 32;

extern "C" {

const char* ojasx_get_version(void) { return "OjasX-LUT-Engine-v1.0.0-B200"; }
const char* ojasx_get_backend_name(void) { return "NVIDIA_CUDA_sm_100a"; }
const char* ojasx_b200_last_error(void) { return g_err; }
unsigned long long ojasx_b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

OjasxLinearHandle ojasx_create_linear(int in_features, int out_features, int block_dim, int codebook_size,
                                      const float* codebook_data, const uint8_t* codes_data,
                                      const float* scales_data, const float* bias_data) {
    if (in_features <= 0 || out_features <= 0 || block_dim <= 0 || codebook_size <= 0 || codebook_size > 256) {
        set_last_error_msg("ojasx_create_linear: invalid dimensions");
        return nullptr;
    }
    auto* h = new (std::nothrow) LinearHandle();
    if (!h) return nullptr;
    h->in = in_features; h->out = out_features; h->D = block_dim; h->Kcb = codebook_size;
    h->G = in_features / block_dim;  // ojasx_lut.h:92
    if (cudaGetDevice(&h->dev) != cudaSuccess) { set_last_error_msg("no CUDA device"); delete h; return nullptr; }
    int rc = OJX_OK;
    // Null data pointers leave the array zero-filled (codes, codebook) or at its default
    // (scales = 1, no bias), as the reference constructor does (ojasx_lut.h:95-98).
    if ((rc = upload((void**)&h->codebook, codebook_data, sizeof(float) * (size_t)codebook_size * block_dim)) == OJX_OK &&
        (rc = upload((void**)&h->codes, codes_data, (size_t)out_features * h->G)) == OJX_OK) {
        if (scales_data) rc = upload((void**)&h->scales, scales_data, sizeof(float) * (size_t)out_features);
        if (rc == OJX_OK && bias_data) rc = upload((void**)&h->bias, bias_data, sizeof(float) * (size_t)out_features);
    }
    if (rc == OJX_OK && cudaStreamCreateWithFlags(&h->stream, cudaStreamNonBlocking) != cudaSuccess) rc = OJX_ERR_CUDA;
    if (rc != OJX_OK) { delete h; return nullptr; }
    return h;
}

int ojasx_set_linear_outliers(OjasxLinearHandle handle, int nnz, const int* row_ptrs, const int* col_indices,
                              const float* values) {
    if (!handle) return OJX_ERR_ARG;
    auto* h = static_cast<LinearHandle*>(handle);
    if (nnz < 0 || !row_ptrs || (nnz > 0 && (!col_indices || !values))) return OJX_ERR_ARG;
    // The reference accepts new outliers at any time (ojasx_lut_c_api.cpp:67-91).  A recorded host-pointer
    // launch and any group snapshot still point at the arrays freed below, so both are invalidated.
    std::lock_guard<std::mutex> lock(h->host_mu);
    DeviceGuard g(h->dev);
    if (h->host_graph) { cudaGraphExecDestroy(h->host_graph); h->host_graph = nullptr; }
    ++h->generation;
    cudaFree(h->row_ptrs); cudaFree(h->cols); cudaFree(h->vals);
    h->row_ptrs = nullptr; h->cols = nullptr; h->vals = nullptr; h->nnz = 0;
    int rc;
    if ((rc = upload((void**)&h->row_ptrs, row_ptrs, sizeof(int) * (size_t)(h->out + 1))) != OJX_OK) return rc;
    if ((rc = upload((void**)&h->cols, col_indices, sizeof(int) * (size_t)nnz)) != OJX_OK) return rc;
    if ((rc = upload((void**)&h->vals, values, sizeof(float) * (size_t)nnz)) != OJX_OK) return rc;
    h->nnz = nnz;
    h->has_outlier_arrays = true;
    h->csr_sorted = true;
    for (int m = 0; m < h->out && h->csr_sorted; ++m)
        for (int j = row_ptrs[m] + 1; j < row_ptrs[m + 1]; ++j)
            if (col_indices[j] <= col_indices[j - 1]) { h->csr_sorted = false; break; }
    return OJX_OK;
}

int ojasx_b200_linear_forward(OjasxLinearHandle handle, const void* d_x, void* d_y, int batch_size, int io_dtype,
                              int row_start, int row_stop, void* stream) {
    if (!handle || !d_x || !d_y) return OJX_ERR_ARG;
    auto* h = static_cast<LinearHandle*>(handle);
    if (batch_size <= 0 || row_start < 0 || row_stop > h->out || row_start >= row_stop) return OJX_ERR_ARG;
    if (io_dtype != OJX_F32 && io_dtype != OJX_BF16) return OJX_ERR_ARG;
    LinearProblem P = h->problem(d_x, d_y, batch_size, io_dtype, row_start, row_stop);
    // bf16 batches at or above the measured switch-over run on the tensor cores (dequant_gemm.cu);
    // OJASX_B200_TENSOR_MIN_BATCH overrides the threshold (0 = never).
    if (io_dtype == OJX_BF16 && dequant_gemm_supported(P, h->csr_sorted)) {
        const char* e = getenv("OJASX_B200_TENSOR_MIN_BATCH");   // read per call: a process can time both paths
        const int min_batch = e ? atoi(e) : kTensorMinBatch;
        if (min_batch > 0 && batch_size >= min_batch) return launch_dequant_gemm(P, static_cast<cudaStream_t>(stream), &h->dq_lists, h->generation);
    }
    return launch_linear(P, static_cast<cudaStream_t>(stream));
}

int ojasx_b200_linear_forward_gather(OjasxLinearHandle handle, const void* d_x, void* d_y_full, int batch_size, int io_dtype,
                                     int row_start, int row_stop, OjasxPeerLinkHandle link, void* stream) {
    if (!handle || !d_x || !d_y_full || !link) return OJX_ERR_ARG;
    auto* h = static_cast<LinearHandle*>(handle);
    if (batch_size <= 0 || row_start < 0 || row_stop > h->out || row_start > row_stop) return OJX_ERR_ARG;
    if (io_dtype != OJX_F32 && io_dtype != OJX_BF16) return OJX_ERR_ARG;
    if (row_start == row_stop) return ojasx_b200_peer_signal(link, stream);   // a rank without rows still takes part
    LinearProblem P = h->problem(d_x, d_y_full, batch_size, io_dtype, row_start, row_stop);
    P.y_full = 1;
    P.y_ld = h->out;
    return launch_linear(P, static_cast<cudaStream_t>(stream), peer_link_of(link));
}

int ojasx_b200_linear_forward_raw(const uint8_t* d_codes, const float* d_codebook, const float* d_scales,
                                  const float* d_bias, int nnz, const int* d_row_ptrs, const int* d_col_indices,
                                  const float* d_values, const void* d_x, void* d_y, int batch_size, int io_dtype,
                                  int block_dim, int codebook_size, int rows, int columns, int row_start,
                                  int row_stop, void* stream) {
    if (!d_codes || !d_codebook || !d_x || !d_y) return OJX_ERR_ARG;
    if (batch_size <= 0 || rows <= 0 || columns <= 0 || block_dim <= 0 || row_start < 0 || row_stop > rows ||
        row_start >= row_stop)
        return OJX_ERR_ARG;
    if (io_dtype != OJX_F32 && io_dtype != OJX_BF16) return OJX_ERR_ARG;
    LinearProblem P{};
    P.codes = d_codes; P.codebook = d_codebook; P.scales = d_scales; P.bias = d_bias;
    P.csr = CsrView{d_row_ptrs, d_col_indices, d_values, nnz};
    P.x = d_x; P.y = d_y; P.K = columns;
    P.G = (columns + block_dim - 1) / block_dim;  // blocks_per_row of the packed layout (codec.py:108)
    P.D = block_dim; P.Kcb = codebook_size;
    P.row_start = row_start; P.row_stop = row_stop; P.batch = batch_size; P.io_dtype = io_dtype;
    return launch_linear(P, static_cast<cudaStream_t>(stream));
}

int ojasx_b200_rvq_fused_gemm(const uint8_t* packed_codes, const float* codebooks, const float* row_scales,
                              const float* bias, const float* inputs, int batch_size, int stages, int bits_per_stage,
                              int block_size, int rows, int columns, int row_start, int row_stop, float* output,
                              void* stream) {
    // Argument checks and codes of ojasx_rvq_fused_gemm (leech24_cpu.cpp:386-397).
    if (stages <= 0 || bits_per_stage <= 0 || block_size <= 0 || rows <= 0 || columns <= 0 || row_start < 0 ||
        row_stop <= row_start || row_stop > rows || batch_size <= 0 || !packed_codes || !codebooks || !row_scales ||
        !inputs || !output)
        return OJX_ERR_ARG;
    if (bits_per_stage != 1 && bits_per_stage != 2 && bits_per_stage != 4 && bits_per_stage != 8) return OJX_ERR_RANGE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool table_path = bits_per_stage == 8 && stages == 1 &&
                            (block_size == 4 || block_size == 8 || block_size == 16 || block_size == 32);
    if (table_path)
        return ojasx_b200_linear_forward_raw(packed_codes, codebooks, row_scales, bias, 0, nullptr, nullptr, nullptr, inputs,
                                             output, batch_size, OJX_F32, block_size, 256, rows, columns, row_start,
                                             row_stop, stream);
    if (stages > 8) return OJX_ERR_ARG;
    return launch_rvq_generic(packed_codes, codebooks, row_scales, bias, inputs, batch_size, stages, bits_per_stage,
                              block_size, rows, columns, row_start, row_stop, output, s);
}

int ojasx_b200_linear_forward_tensor(OjasxLinearHandle handle, const void* d_x, void* d_y, int batch_size, int row_start,
                                     int row_stop, void* stream) {
    if (!handle || !d_x || !d_y) return OJX_ERR_ARG;
    auto* h = static_cast<LinearHandle*>(handle);
    if (batch_size <= 0 || row_start < 0 || row_stop > h->out || row_start >= row_stop) return OJX_ERR_ARG;
    LinearProblem P = h->problem(d_x, d_y, batch_size, OJX_BF16, row_start, row_stop);
    if (!dequant_gemm_supported(P, h->csr_sorted)) return OJX_ERR_UNSUPPORTED;
    return launch_dequant_gemm(P, static_cast<cudaStream_t>(stream), &h->dq_lists, h->generation);
}

int ojasx_b200_take_device_error(void) {
    int v = 0, m = 0, c = 0;
    int rc = take_dequant_gemm_error(&v);
    if (rc == OJX_OK) rc = take_moe_fused_error(&m);
    if (rc == OJX_OK) rc = take_moe_bulk_copy_error(&c);
    return rc != OJX_OK ? rc : (v | (m ? 2 : 0) | (c ? 4 : 0));
}

int ojasx_linear_forward(OjasxLinearHandle handle, const float* x, float* y, int batch_size, int num_threads) {
    (void)num_threads;
    if (!handle || !x || !y) return OJX_ERR_ARG;  // ojasx_lut_c_api.cpp:100
    auto* h = static_cast<LinearHandle*>(handle);
    if (batch_size <= 0) return OJX_OK;           // the reference's batch loop simply does not run
    std::lock_guard<std::mutex> lock(h->host_mu);   // concurrent callers of one layer take turns (as safe as the const CPU method)
    DeviceGuard g(h->dev);
    const size_t xb = sizeof(float) * (size_t)batch_size * h->in, yb = sizeof(float) * (size_t)batch_size * h->out;
    int rc;
    if ((rc = ensure_capacity(&h->d_x, &h->cap_x, xb)) != OJX_OK) return rc;
    if ((rc = ensure_pinned(&h->pin_x, &h->cap_pin_x, xb)) != OJX_OK) return rc;
    if ((rc = ensure_pinned(&h->pin_y, &h->cap_pin_y, yb)) != OJX_OK) return rc;
    // x: host copy into pinned staging, then one asynchronous H2D copy.  y: the kernel stores its
    // results straight into device-mapped pinned memory, so no D2H copy is enqueued; after the
    // stream synchronises the results are in host memory and are copied to the caller's buffer.
    if (h->pin_y_dev == nullptr || h->pin_y_dev_of != h->pin_y) {
        OJX_CUDA_TRY(cudaHostGetDevicePointer(&h->pin_y_dev, h->pin_y, 0));
        h->pin_y_dev_of = h->pin_y;
    }
    void* y_dev = h->pin_y_dev;
    std::memcpy(h->pin_x, x, xb);
    // The copy and the kernel have the same arguments on every call of a given batch size, so they are
    // recorded once as a graph and replayed with one launch call (OJASX_B200_HOST_GRAPH=0 disables).
    static const bool use_graph = [] { const char* e = getenv("OJASX_B200_HOST_GRAPH"); return !(e && e[0] == '0'); }();
    const bool graph_ok = use_graph && h->host_graph && h->host_graph_batch == batch_size && h->host_graph_key[0] == h->pin_x &&
                          h->host_graph_key[1] == h->d_x && h->host_graph_key[2] == y_dev;
    if (graph_ok) {
        OJX_CUDA_TRY(cudaGraphLaunch(h->host_graph, h->stream));
        count_launch(1);   // the graph's one kernel
    } else if (use_graph) {
        if (h->host_graph) { cudaGraphExecDestroy(h->host_graph); h->host_graph = nullptr; }
        cudaGraph_t g = nullptr;
        OJX_CUDA_TRY(cudaStreamBeginCapture(h->stream, cudaStreamCaptureModeThreadLocal));
        cudaError_t ce = cudaMemcpyAsync(h->d_x, h->pin_x, xb, cudaMemcpyHostToDevice, h->stream);
        rc = ce == cudaSuccess ? launch_linear(h->problem(h->d_x, y_dev, batch_size, OJX_F32, 0, h->out), h->stream) : OJX_ERR_CUDA;
        const cudaError_t ee = cudaStreamEndCapture(h->stream, &g);
        if (rc != OJX_OK || ee != cudaSuccess || !g) {
            if (g) cudaGraphDestroy(g);
            (void)cudaGetLastError();
            if (rc != OJX_OK) return rc;
            set_last_error("cudaStreamEndCapture", ee);
            return OJX_ERR_CUDA;
        }
        ce = cudaGraphInstantiate(&h->host_graph, g, 0);
        cudaGraphDestroy(g);
        if (ce != cudaSuccess) { h->host_graph = nullptr; set_last_error("cudaGraphInstantiate", ce); return OJX_ERR_CUDA; }
        h->host_graph_batch = batch_size;
        h->host_graph_key[0] = h->pin_x; h->host_graph_key[1] = h->d_x; h->host_graph_key[2] = y_dev;
        OJX_CUDA_TRY(cudaGraphLaunch(h->host_graph, h->stream));
    } else {
        OJX_CUDA_TRY(cudaMemcpyAsync(h->d_x, h->pin_x, xb, cudaMemcpyHostToDevice, h->stream));
        rc = launch_linear(h->problem(h->d_x, y_dev, batch_size, OJX_F32, 0, h->out), h->stream);
        if (rc != OJX_OK) return rc;
    }
    if ((rc = wait_stream(h->stream)) != OJX_OK) return rc;
    std::memcpy(y, h->pin_y, yb);
    return OJX_OK;
}

/* Size queries: formulas of ojasx_lut.h:101-124 (the scales vector always exists in the
 * reference object, so its bytes are always counted). */
size_t ojasx_get_compressed_size(OjasxLinearHandle handle) {
    if (!handle) return 0;
    auto* h = static_cast<LinearHandle*>(handle);
    size_t n = (size_t)h->out * h->G + sizeof(float) * (size_t)h->Kcb * h->D + sizeof(float) * (size_t)h->out;
    if (h->bias) n += sizeof(float) * (size_t)h->out;
    if (h->has_outlier_arrays) n += (size_t)h->nnz * 8 + sizeof(int) * (size_t)(h->out + 1);
    return n;
}
size_t ojasx_get_dense_size(OjasxLinearHandle handle) {
    if (!handle) return 0;
    auto* h = static_cast<LinearHandle*>(handle);
    return (size_t)h->out * h->in * sizeof(float);
}
size_t ojasx_get_lut_sram_size(OjasxLinearHandle handle) {
    if (!handle) return 0;
    auto* h = static_cast<LinearHandle*>(handle);
    return (size_t)h->G * h->Kcb * sizeof(float);
}
float ojasx_get_compression_ratio(OjasxLinearHandle handle) {
    if (!handle) return 0.0f;
    size_t c = ojasx_get_compressed_size(handle);
    return (float)ojasx_get_dense_size(handle) / (float)(c ? c : 1);
}
void ojasx_destroy_linear(OjasxLinearHandle handle) {
    if (handle) delete static_cast<LinearHandle*>(handle);
}

/* ---- grouped launch */
OjasxLinearGroupHandle ojasx_b200_create_linear_group(const OjasxLinearHandle* handles, int count) {
    if (!handles || count <= 0) return nullptr;
    auto* g = new (std::nothrow) LinearGroup();
    if (!g) return nullptr;
    g->host.resize(count);
    g->members.resize(count);
    g->member_generation.resize(count);
    int item = 0;
    for (int i = 0; i < count; ++i) {
        auto* h = static_cast<LinearHandle*>(handles[i]);
        if (!h || (i > 0 && h->D != g->D)) { set_last_error_msg("linear group: null handle or mixed block_dim"); delete g; return nullptr; }
        if (i == 0) { g->D = h->D; g->dev = h->dev; }
        LinearProblem P = h->problem(nullptr, nullptr, 1, OJX_F32, 0, h->out);
        P.tile_rows = plan_tile_rows(h->out, count);
        P.tiles = (h->out + P.tile_rows - 1) / P.tile_rows;
        P.item_begin = item;
        item += P.tiles;
        g->host[i] = P;
        g->members[i] = h;
        g->member_generation[i] = h->generation;
    }
    g->total_items = item;
    if (cudaMalloc((void**)&g->dev_probs, sizeof(LinearProblem) * (size_t)count) != cudaSuccess) { delete g; return nullptr; }
    return g;
}

static int linear_group_forward(OjasxLinearGroupHandle group, const void* d_x, size_t x_stride_bytes, void* d_y,
                                size_t y_stride_bytes, int io_dtype, void* stream, const PeerLink* link) {
    if (!group || !d_x || !d_y) return OJX_ERR_ARG;
    if (io_dtype != OJX_F32 && io_dtype != OJX_BF16) return OJX_ERR_ARG;
    auto* g = static_cast<LinearGroup*>(group);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int y_full = link ? 1 : 0;
    if (g->bound_full != y_full) { g->bound_full = y_full; g->bound_x = nullptr; }
    // A layer whose outliers were replaced since the snapshot: take its arrays again and rewrite the table.
    for (size_t i = 0; i < g->host.size(); ++i) {
        const LinearHandle* h = g->members[i];
        if (h->generation == g->member_generation[i]) continue;
        const LinearProblem old = g->host[i];
        LinearProblem P = h->problem(old.x, old.y, 1, old.io_dtype, old.row_start, old.row_stop);
        P.tile_rows = old.tile_rows; P.tiles = old.tiles; P.item_begin = old.item_begin;
        g->host[i] = P;
        g->member_generation[i] = h->generation;
        g->bound_x = nullptr;
    }
    // A few problems of one shape (q/k/v, gate/up): one cluster launch, the problems travel as kernel
    // arguments, so nothing is copied or synchronised (safe inside a stream capture).
    if (g->host.size() <= 8 && !linear_cluster_disabled()) {
        LinearProblem tmp[8];
        for (size_t i = 0; i < g->host.size(); ++i) {
            tmp[i] = g->host[i];
            tmp[i].x = static_cast<const char*>(d_x) + i * x_stride_bytes;
            tmp[i].y = static_cast<char*>(d_y) + i * y_stride_bytes;
            tmp[i].io_dtype = io_dtype;
            tmp[i].y_full = y_full;
            tmp[i].y_ld = g->members[i]->out;
        }
        const int rc = try_launch_linear_cluster_group(tmp, (int)g->host.size(), s, link);
        if (rc != OJX_ERR_UNSUPPORTED) return rc;
    }
    // The problem table is rewritten only when the I/O binding changes, so steady-state calls
    // enqueue exactly one kernel.
    if (g->bound_x != d_x || g->bound_y != d_y || g->bound_xs != x_stride_bytes || g->bound_ys != y_stride_bytes ||
        g->bound_dtype != io_dtype) {
        for (size_t i = 0; i < g->host.size(); ++i) {
            g->host[i].x = static_cast<const char*>(d_x) + i * x_stride_bytes;
            g->host[i].y = static_cast<char*>(d_y) + i * y_stride_bytes;
            g->host[i].io_dtype = io_dtype;
            g->host[i].y_full = y_full;
            g->host[i].y_ld = g->members[i]->out;
        }
        OJX_CUDA_TRY(cudaMemcpyAsync(g->dev_probs, g->host.data(), sizeof(LinearProblem) * g->host.size(),
                                     cudaMemcpyHostToDevice, s));
        OJX_CUDA_TRY(cudaStreamSynchronize(s));
        g->bound_x = d_x; g->bound_y = d_y; g->bound_xs = x_stride_bytes; g->bound_ys = y_stride_bytes;
        g->bound_dtype = io_dtype;
    }
    return launch_linear_group(g->dev_probs, (int)g->host.size(), g->total_items, g->D, s, link);
}

int ojasx_b200_linear_group_forward(OjasxLinearGroupHandle group, const void* d_x, size_t x_stride_bytes, void* d_y,
                                    size_t y_stride_bytes, int io_dtype, void* stream) {
    return linear_group_forward(group, d_x, x_stride_bytes, d_y, y_stride_bytes, io_dtype, stream, nullptr);
}

int ojasx_b200_linear_group_forward_gather(OjasxLinearGroupHandle group, const void* d_x, size_t x_stride_bytes,
                                           void* d_y_full, size_t y_stride_bytes, int io_dtype, OjasxPeerLinkHandle link,
                                           void* stream) {
    if (!link) return OJX_ERR_ARG;
    return linear_group_forward(group, d_x, x_stride_bytes, d_y_full, y_stride_bytes, io_dtype, stream, peer_link_of(link));
}

int ojasx_b200_linear_group_set_rows(OjasxLinearGroupHandle group, int row_start, int row_stop) {
    if (!group) return OJX_ERR_ARG;
    auto* g = static_cast<LinearGroup*>(group);
    int item = 0;
    for (size_t i = 0; i < g->host.size(); ++i) {
        const LinearHandle* h = g->members[i];
        const int a = row_start < 0 ? 0 : row_start, b = row_stop > h->out ? h->out : row_stop;
        if (a >= b) return OJX_ERR_ARG;
        LinearProblem& P = g->host[i];
        P.row_start = a; P.row_stop = b;
        P.tile_rows = plan_tile_rows(b - a, (int)g->host.size());
        P.tiles = (b - a + P.tile_rows - 1) / P.tile_rows;
        P.item_begin = item;
        item += P.tiles;
    }
    g->total_items = item;
    g->bound_x = nullptr;   // the device table is rewritten by the next forward
    return OJX_OK;
}

void ojasx_b200_destroy_linear_group(OjasxLinearGroupHandle group) {
    if (!group) return;
    auto* g = static_cast<LinearGroup*>(group);
    cudaFree(g->dev_probs);
    delete g;
}

}  // extern "C"
