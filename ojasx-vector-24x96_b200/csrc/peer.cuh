// Exchange between the GPUs of one box without a collective library: every rank owns one "shared
// segment" of device memory that all other ranks have mapped (CUDA IPC), laid out identically on
// every rank.  A kernel that produces a shard of a result stores it at the same offset in every
// rank's segment (plain st.global over NVLink, no multicast), and when the last CTA of the launch
// is done it raises this rank's flag on every rank; the consumer of the gathered result polls the
// flags of all ranks (bounded) before it reads.  This is the all-gather that follows a row-split
// linear (contract of row_start / row_stop, ojasx_24x96/native/ojasx_backend_abi.h:97-111), the
// gather of the expert outputs of an expert-parallel MoE, and the gather of KV-head-sharded
// attention outputs, fused into the epilogue of the kernel that produces the shard.
//
// Flags are epoch counters that only grow: flags[p] = number of exchanges rank p has signalled on
// this link.  Every rank runs the same sequence of exchanges, so "rank p has signalled at least as
// many exchanges as I have" means its shard of the current one has arrived.  A rank can run at most
// one exchange ahead of the slowest (it needs everybody's flag to get past its own wait), so a
// buffer may be written again two exchanges later; callers that repeat one exchange alternate
// between two buffers.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace ojx {

constexpr int kMaxPeers = 8;
constexpr int kPeerSpin = 1 << 23;      // bounded polling: about two seconds with the back-off below

struct PeerLink {
    long long delta[kMaxPeers];   // bytes from this rank's segment to rank p's mapping of its segment (0 for self)
    int n;                        // ranks (0: no exchange, plain local stores)
    int self;
    int* flags;                   // [n] inside this rank's segment: flags[p] written by rank p
    int* epoch;                   // local: exchanges this rank has signalled
    unsigned* done;               // local: CTAs of the running launch that have finished (returns to 0)
    int* status;                  // local: set to 1 when a wait ran out
};

template <class T>
__device__ __forceinline__ void peer_store(const PeerLink& L, T* local, T v) {
    *local = v;
    for (int p = 0; p < L.n; ++p)
        if (p != L.self) *reinterpret_cast<T*>(reinterpret_cast<char*>(local) + L.delta[p]) = v;
}

// Every CTA of a launch calls this once, after its last peer_store; `total` = CTAs of the launch.
__device__ __forceinline__ void peer_signal_when_last(const PeerLink& L, unsigned total) {
    if (L.n <= 0) return;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        const unsigned prev = atomicAdd(L.done, 1u);
        if (prev == total - 1) {
            *L.done = 0;
            __threadfence_system();
            const int e = *L.epoch + 1;
            *L.epoch = e;
            for (int p = 0; p < L.n; ++p) {
                int* f = reinterpret_cast<int*>(reinterpret_cast<char*>(L.flags + L.self) + L.delta[p]);
                asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(f), "r"(e) : "memory");
            }
        }
    }
}

// One warp (all 32 lanes): returns when every rank has signalled the exchange this rank signalled last,
// or when the polling budget is spent (status is raised then).  Other threads of the CTA wait at the
// caller's barrier.
__device__ __forceinline__ void peer_wait_warp(const PeerLink& L) {
    if (L.n <= 0) return;
    const int lane = threadIdx.x & 31;
    // Once a wait has run out the ranks are out of step and every later wait would run out too: give up at once
    // (the host reads and clears the status), so that a broken run ends quickly instead of spinning for hours.
    if (*reinterpret_cast<volatile int*>(L.status) != 0) return;
    const int e = *reinterpret_cast<volatile int*>(L.epoch);
    if (lane < L.n) {
        bool ok = false;
        for (int i = 0; i < kPeerSpin; ++i) {
            int v;
            asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(L.flags + lane) : "memory");
            if (v - e >= 0) { ok = true; break; }
            if (i > 1024) __nanosleep(256);
        }
        if (!ok) atomicExch(L.status, 1);
    }
    __syncwarp();
}

}  // namespace ojx
