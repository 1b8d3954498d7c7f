// Host-side objects behind the opaque C handles.
#pragma once
#include "common.cuh"
#include <vector>

namespace ojx {

void count_launch(int n);
int upload(void** dptr, const void* host, size_t bytes);          // cudaMalloc + copy (zero-fill when host == null)
int ensure_capacity(void** dptr, size_t* cap, size_t bytes);      // grow-only device staging buffer

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
    int* row_ptrs = nullptr;
    int* cols = nullptr;
    float* vals = nullptr;
    // staging for the host-pointer forward
    void* d_x = nullptr;
    void* d_y = nullptr;
    size_t cap_x = 0, cap_y = 0;
    cudaStream_t stream = nullptr;

    ~LinearHandle();
    LinearProblem problem(const void* x, void* y, int batch, int io_dtype, int row_start, int row_stop) const;
};

struct LinearGroup {
    int dev = 0;
    int D = 0;
    int total_items = 0;
    std::vector<LinearProblem> host;
    LinearProblem* dev_probs = nullptr;
    const void* bound_x = nullptr;
    void* bound_y = nullptr;
    size_t bound_xs = 0, bound_ys = 0;
    int bound_dtype = -1;
};

}  // namespace ojx
