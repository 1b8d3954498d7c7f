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
