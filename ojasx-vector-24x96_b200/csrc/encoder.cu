// Offline encoder hot step: nearest-centroid assignment of block vectors, with the sums that a k-means
// update needs (the reference fits split-manifold layers with torch.cdist + argmin + index_add_ on the
// host, split_manifold_lut_experiment/engine/split_manifold_engine.py:140-160).
//
// One thread per vector: the D coordinates stay in registers, the codebook sits in shared memory and is
// read by broadcast (every lane of a warp reads the same centroid), distance = sum_d (v_d - c_d)^2 in
// fp32, arg-min keeps the first minimum (lowest index).  The [n, 256] distance matrix of the reference
// is never materialised.  Cluster sums are accumulated in double precision (shared memory per CTA, then
// one global atomic per cell), so that the order in which vectors arrive does not show in the fp32 means.
#include "common.cuh"
#include "launch.h"
#include "handles.h"
#include "../../include/ojasx_lut_b200.h"

namespace ojx {

constexpr int kEncThreads = 256;

template <int D>
__global__ void __launch_bounds__(kEncThreads) vq_assign_kernel(const float* __restrict__ vectors, size_t n,
                                                                const float* __restrict__ centroids, int Kcb,
                                                                uint8_t* __restrict__ codes, double* __restrict__ sums,
                                                                unsigned long long* __restrict__ counts) {
    extern __shared__ __align__(16) unsigned char enc_smem[];
    float* cb = reinterpret_cast<float*>(enc_smem);                       // [Kcb][D]
    double* ssum = reinterpret_cast<double*>(cb + ((Kcb * D + 1) & ~1));  // [Kcb][D] when sums are wanted
    unsigned* scnt = reinterpret_cast<unsigned*>(ssum + (sums ? Kcb * D : 0));   // [Kcb]
    for (int i = threadIdx.x; i < Kcb * D; i += kEncThreads) cb[i] = centroids[i];
    if (sums) {
        for (int i = threadIdx.x; i < Kcb * D; i += kEncThreads) ssum[i] = 0.0;
        for (int i = threadIdx.x; i < Kcb; i += kEncThreads) scnt[i] = 0u;
    }
    __syncthreads();
    for (size_t v0 = (size_t)blockIdx.x * kEncThreads; v0 < n; v0 += (size_t)gridDim.x * kEncThreads) {
        const size_t vi = v0 + threadIdx.x;
        if (vi < n) {
            float v[D];
#pragma unroll
            for (int q = 0; q < D / 4; ++q) {
                const float4 f = reinterpret_cast<const float4*>(vectors + vi * D)[q];
                v[4 * q] = f.x; v[4 * q + 1] = f.y; v[4 * q + 2] = f.z; v[4 * q + 3] = f.w;
            }
            float best = INFINITY;
            int bi = 0;
            for (int c = 0; c < Kcb; ++c) {
                float dist = 0.0f;
#pragma unroll
                for (int d = 0; d < D; ++d) {
                    const float t = v[d] - cb[c * D + d];
                    dist = fmaf(t, t, dist);
                }
                if (dist < best) { best = dist; bi = c; }
            }
            codes[vi] = (uint8_t)bi;
            if (sums) {
#pragma unroll
                for (int d = 0; d < D; ++d) atomicAdd(&ssum[bi * D + d], (double)v[d]);
                atomicAdd(&scnt[bi], 1u);
            }
        }
    }
    if (sums) {
        __syncthreads();
        for (int i = threadIdx.x; i < Kcb * D; i += kEncThreads)
            if (ssum[i] != 0.0) atomicAdd(&sums[i], ssum[i]);
        for (int i = threadIdx.x; i < Kcb; i += kEncThreads)
            if (scnt[i]) atomicAdd(&counts[i], (unsigned long long)scnt[i]);
    }
}

template <int D>
static int launch_assign_t(const float* vectors, size_t n, const float* centroids, int Kcb, uint8_t* codes, double* sums,
                           unsigned long long* counts, cudaStream_t s) {
    const size_t smem = sizeof(float) * ((size_t)(Kcb * D + 1) & ~(size_t)1) + (sums ? sizeof(double) * Kcb * D + sizeof(unsigned) * Kcb : 0);
    if (smem > 200 * 1024) return OJX_ERR_TOO_LARGE;
    if (smem > 48 * 1024) OJX_CUDA_TRY(cudaFuncSetAttribute(vq_assign_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const size_t want = (n + kEncThreads - 1) / kEncThreads;
    const size_t cap = (size_t)num_sms() * 8;
    const int grid = (int)(want < cap ? want : cap);
    vq_assign_kernel<D><<<grid, kEncThreads, smem, s>>>(vectors, n, centroids, Kcb, codes, sums, counts);
    OJX_CUDA_TRY(cudaGetLastError());
    count_launch(1);
    return OJX_OK;
}

}  // namespace ojx

using namespace ojx;

extern "C" int ojasx_b200_vq_assign(const float* d_vectors, size_t n_vectors, int block_dim, const float* d_centroids,
                                    int codebook_size, uint8_t* d_codes, double* d_sums, unsigned long long* d_counts,
                                    void* stream) {
    if (!d_vectors || !d_centroids || !d_codes || (d_sums != nullptr) != (d_counts != nullptr)) return OJX_ERR_ARG;
    if (codebook_size <= 0 || codebook_size > 256) return OJX_ERR_ARG;
    if (n_vectors == 0) return OJX_OK;
    if (reinterpret_cast<uintptr_t>(d_vectors) & 15) return OJX_ERR_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (block_dim) {
        case 4: return launch_assign_t<4>(d_vectors, n_vectors, d_centroids, codebook_size, d_codes, d_sums, d_counts, s);
        case 8: return launch_assign_t<8>(d_vectors, n_vectors, d_centroids, codebook_size, d_codes, d_sums, d_counts, s);
        case 16: return launch_assign_t<16>(d_vectors, n_vectors, d_centroids, codebook_size, d_codes, d_sums, d_counts, s);
        case 32: return launch_assign_t<32>(d_vectors, n_vectors, d_centroids, codebook_size, d_codes, d_sums, d_counts, s);
        default: return OJX_ERR_UNSUPPORTED;
    }
}
