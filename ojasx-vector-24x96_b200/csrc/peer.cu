// Host side of the exchange over peer memory (peer.cuh): shared segments (cudaMalloc + CUDA IPC),
// links, and the stand-alone signal / wait launches for producers and consumers that are not
// kernels of this library.
#include "../../include/ojasx_lut_b200.h"
#include "handles.h"
#include "launch.h"
#include "peer.cuh"

#include <cstring>
#include <new>

namespace ojx {

struct PeerLinkHandle {
    int dev = 0;
    PeerLink link{};
    int* counters = nullptr;   // epoch, done, status (device)
    ~PeerLinkHandle() {
        DeviceGuard g(dev);
        cudaFree(counters);
    }
};

__global__ void peer_signal_kernel(const __grid_constant__ PeerLink L) { peer_signal_when_last(L, 1u); }
__global__ void peer_wait_kernel(const __grid_constant__ PeerLink L) { peer_wait_warp(L); }

// dst (same offset in every rank's segment) <- src, 4 bytes per thread and step, then the flag.
__global__ void __launch_bounds__(256) peer_put_kernel(const __grid_constant__ PeerLink L, unsigned* __restrict__ dst,
                                                       const unsigned* __restrict__ src, size_t words) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < words; i += (size_t)gridDim.x * blockDim.x)
        peer_store(L, dst + i, src[i]);
    peer_signal_when_last(L, gridDim.x);
}

const PeerLink* peer_link_of(void* handle) { return handle ? &static_cast<PeerLinkHandle*>(handle)->link : nullptr; }

}  // namespace ojx

using namespace ojx;

extern "C" {

void* ojasx_b200_peer_alloc(size_t bytes) {
    void* p = nullptr;
    if (bytes == 0 || cudaMalloc(&p, bytes) != cudaSuccess) { set_last_error_msg("peer_alloc: cudaMalloc failed"); return nullptr; }
    if (cudaMemset(p, 0, bytes) != cudaSuccess) { cudaFree(p); return nullptr; }
    return p;
}

int ojasx_b200_peer_free(void* d_segment) {
    if (!d_segment) return OJX_ERR_ARG;
    OJX_CUDA_TRY(cudaFree(d_segment));
    return OJX_OK;
}

int ojasx_b200_peer_export(void* d_segment, unsigned char* handle_out) {
    if (!d_segment || !handle_out) return OJX_ERR_ARG;
    cudaIpcMemHandle_t h;
    static_assert(sizeof(h) == OJASX_B200_PEER_HANDLE_BYTES, "IPC handle size");
    OJX_CUDA_TRY(cudaIpcGetMemHandle(&h, d_segment));
    std::memcpy(handle_out, &h, sizeof(h));
    return OJX_OK;
}

void* ojasx_b200_peer_open(const unsigned char* handle) {
    if (!handle) return nullptr;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, sizeof(h));
    void* p = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) { set_last_error("cudaIpcOpenMemHandle", e); return nullptr; }
    return p;
}

int ojasx_b200_peer_close(void* d_mapped) {
    if (!d_mapped) return OJX_ERR_ARG;
    OJX_CUDA_TRY(cudaIpcCloseMemHandle(d_mapped));
    return OJX_OK;
}

OjasxPeerLinkHandle ojasx_b200_peer_link_create(void* const* d_segments, int n_ranks, int self, size_t flags_offset) {
    if (!d_segments || n_ranks < 1 || n_ranks > kMaxPeers || self < 0 || self >= n_ranks || (flags_offset & 3)) {
        set_last_error_msg("peer_link_create: 1..8 ranks, self inside, 4-byte aligned flags offset");
        return nullptr;
    }
    auto* h = new (std::nothrow) PeerLinkHandle();
    if (!h) return nullptr;
    if (cudaGetDevice(&h->dev) != cudaSuccess || upload((void**)&h->counters, nullptr, 4 * sizeof(int)) != OJX_OK) { delete h; return nullptr; }
    PeerLink& L = h->link;
    L.n = n_ranks;
    L.self = self;
    for (int p = 0; p < n_ranks; ++p) {
        if (!d_segments[p]) { delete h; return nullptr; }
        L.delta[p] = static_cast<const char*>(d_segments[p]) - static_cast<const char*>(d_segments[self]);
    }
    L.flags = reinterpret_cast<int*>(static_cast<char*>(d_segments[self]) + flags_offset);
    L.epoch = h->counters;
    L.done = reinterpret_cast<unsigned*>(h->counters + 1);
    L.status = h->counters + 2;
    return h;
}

void ojasx_b200_peer_link_destroy(OjasxPeerLinkHandle link) {
    if (link) delete static_cast<PeerLinkHandle*>(link);
}

int ojasx_b200_peer_signal(OjasxPeerLinkHandle link, void* stream) {
    if (!link) return OJX_ERR_ARG;
    peer_signal_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<PeerLinkHandle*>(link)->link);
    OJX_CUDA_TRY(cudaGetLastError());
    count_launch(1);
    return OJX_OK;
}

int ojasx_b200_peer_put(OjasxPeerLinkHandle link, void* d_dst_shared, const void* d_src, size_t bytes, void* stream) {
    if (!link || !d_dst_shared || !d_src || bytes == 0 || (bytes & 3)) return OJX_ERR_ARG;
    const size_t words = bytes / 4;
    const unsigned grid = (unsigned)((words + 255) / 256 < 148 ? (words + 255) / 256 : 148);
    peer_put_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<PeerLinkHandle*>(link)->link,
                                                                      static_cast<unsigned*>(d_dst_shared),
                                                                      static_cast<const unsigned*>(d_src), words);
    OJX_CUDA_TRY(cudaGetLastError());
    count_launch(1);
    return OJX_OK;
}

int ojasx_b200_peer_wait(OjasxPeerLinkHandle link, void* stream) {
    if (!link) return OJX_ERR_ARG;
    peer_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<PeerLinkHandle*>(link)->link);
    OJX_CUDA_TRY(cudaGetLastError());
    count_launch(1);
    return OJX_OK;
}

int ojasx_b200_peer_take_status(OjasxPeerLinkHandle link) {
    if (!link) return OJX_ERR_ARG;
    auto* h = static_cast<PeerLinkHandle*>(link);
    DeviceGuard g(h->dev);
    int v = 0;
    OJX_CUDA_TRY(cudaMemcpy(&v, h->link.status, sizeof(int), cudaMemcpyDeviceToHost));
    if (v) OJX_CUDA_TRY(cudaMemset(h->link.status, 0, sizeof(int)));
    return v;
}

}  // extern "C"
