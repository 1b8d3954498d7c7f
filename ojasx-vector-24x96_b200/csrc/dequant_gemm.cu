// Batched VQ linear on the 5th-generation tensor cores (tcgen05 + TMEM), for bf16 activations and
// batches large enough that the operation is a dense contraction:
//     Y[b, m] = scale[m] * sum_k X[b, k] * W[m, k] (+ bias[m]),   W[m, 8g + d] = codebook[code[m, g]][d] (+ outlier)
// The weights are never materialised in global memory: per 128-row x 64-column tile a group of
// two producer warps turns code bytes into bf16 (one 16-byte shared-memory gather from a bf16 copy
// of the codebook per code byte), adds the rows' CSR outliers that fall in the tile, and stores the
// tile in the 128-byte-swizzled K-major layout that tcgen05.mma reads; the matching X tile (batch rows x 64
// columns, up to 32 KB) is one tiled bulk-tensor copy of the copy engine (cp.async.bulk.tensor.2d with the same
// swizzle; rows past the batch are zero-filled), issued by one thread of the group -- per-thread 16-byte copies
// kept too few bytes in flight and made the X tile the slowest part of a stage.  Four such groups work on four consecutive K tiles at the same time, so the
// latencies of one tile's hand-over overlap with the others.  One thread of a ninth warp issues the MMAs (M = 128, N = padded batch, K = 16
// per instruction, fp32 accumulation in tensor memory) and signals stage reuse with
// tcgen05.commit.  After the last K tile the producer warps become the epilogue: tcgen05.ld the
// accumulator rows, scale, bias, store bf16.
//
// A layer has few 128-row tiles (54 for 6912 rows), so the K axis is split over up to four CTAs per
// tile until the GPU is full.  The CTAs of a tile form a thread-block cluster: each leaves its raw fp32
// partial sums in its own shared memory (the stage buffers are idle by then), and after a cluster barrier
// every CTA adds the partials of its share of the batch columns in split order, reading the other CTAs'
// copies through distributed shared memory, and applies scale and bias.  (Partial sums through global
// memory with the last CTA to arrive adding them cost 20 of the kernel's 40 microseconds at batch 256.)
//
// This path trades the bit-exactness of the table kernels for throughput (weights are rounded to
// bf16), so it is used only for bf16 I/O, inside the rel 2e-2 tolerance of the bf16 activation path.
// Every wait on an mbarrier is bounded; on a timeout the kernel raises a flag that the host reads.
#include <algorithm>
#include <cstdlib>

#include <cuda.h>   // CUtensorMap and the types of cuTensorMapEncodeTiled (the entry point is looked up at run time)

#include "common.cuh"
#include "launch.h"
#include "handles.h"

namespace ojx {

constexpr int kDqProducers = 256;    // 8 producer/epilogue warps
constexpr int kDqGroups = 4;         // producer groups; each builds every fourth K tile
constexpr int kDqGroupThreads = kDqProducers / kDqGroups;
constexpr int kDqMaxTiles = 254;     // K tiles of one CTA whose outliers can be listed per tile (else rows are walked)
constexpr int kDqThreads = kDqProducers + 32;   // + 1 MMA warp
constexpr int kDqBlockM = 128;
constexpr int kDqBlockK = 64;        // bf16 elements per K tile = one 128-byte swizzle row
constexpr int kDqStages = 8;        // most stage buffers; as many as fit next to the batch tile are used (3 at N = 256)
constexpr int kDqSpin = 1 << 22;     // bounded mbarrier polling



__device__ __forceinline__ void cp_async16_zfill(void* smem_dst, const void* gsrc, int src_bytes) {
    unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(src_bytes) : "memory");
}

__device__ __forceinline__ unsigned smem_u32(const void* p) { return static_cast<unsigned>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Returns false if the phase did not complete within the polling budget.
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity) {
    for (int i = 0; i < kDqSpin; ++i) {
        unsigned done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}

__device__ __forceinline__ void dq_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float dq_ld_cluster(unsigned local_addr, unsigned rank) {
    unsigned remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

// Shared-memory matrix descriptor of a K-major tile stored with the 128-byte swizzle: rows of 128
// bytes, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ unsigned long long make_desc_sw128(unsigned smem_addr) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_addr >> 4) & 0x3fff);        // start address
    d |= (unsigned long long)1 << 16;                            // leading byte offset (unused with swizzle)
    d |= (unsigned long long)(1024 >> 4) << 32;                  // stride byte offset: 8 rows
    d |= (unsigned long long)1 << 46;                            // descriptor version of sm_100
    d |= (unsigned long long)2 << 61;                            // SWIZZLE_128B
    return d;
}

struct DequantGemmProblem {
    const uint8_t* codes;       // [M, G]
    const float* codebook;      // [256, 8] fp32 (rounded to bf16 inside the kernel)
    const float* scales;        // [M] or null
    const float* bias;          // [M] or null
    CsrView csr;                // column indices ascending inside each row, or nnz == 0
    const __nv_bfloat16* x;     // [B, K]
    __nv_bfloat16* y;           // [B, row_stop - row_start]
    int* error_flag;
    int K, G, row_start, row_stop, batch;
    int n_pad;                  // MMA N: batch tile rounded up to 16 (<= 256)
    int tmem_cols;              // power of two >= n_pad, >= 32
    int stages;                 // stage buffers (3..8)
    int csr_cap;                // outlier entries of the CTA's rows that fit in shared memory
    int ksplit;                 // CTAs per tile along K (gridDim.z = the cluster's size)
    int tiles_per_split;        // K tiles per split (even, so that a split's code bytes start 16-byte aligned)
    // Outliers listed per (128-row tile, 64-column tile) once per layer (dq_list_* kernels), or null: the lists are
    // then made in shared memory by every CTA.  tile_off[rt * (KT_all + 1) + kt] .. [+ 1] = the tile's entries.
    const int* tile_off;
    const int2* tile_ent;       // (row in tile << 8 | column in tile, value / row scale)
    int use_tma;                // X tiles by the copy engine (xmap); 0 = 16-byte cp.async pieces
};

__global__ void __launch_bounds__(kDqThreads, 1) vq_dequant_gemm_kernel(const __grid_constant__ DequantGemmProblem P,
                                                                        const __grid_constant__ CUtensorMap xmap) {
    extern __shared__ unsigned char dq_smem_raw[];
    // swizzled tiles need 1024-byte alignment; the dynamic segment only promises 16
    unsigned char* dq_smem = dq_smem_raw + ((1024u - (smem_u32(dq_smem_raw) & 1023u)) & 1023u);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int N = P.n_pad;
    const int S = P.stages;
    const int a_bytes = kDqBlockM * 128, b_bytes = N * 128, stage_bytes = a_bytes + b_bytes;
    unsigned char* tiles = dq_smem;                                   // [stages][A | B], 1024-byte aligned
    uint4* cb16 = reinterpret_cast<uint4*>(tiles + S * stage_bytes);   // [256] centroids as 8 bf16
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(cb16 + 256);
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 2 * kDqStages + 1);
    int* rp_s = reinterpret_cast<int*>(tmem_slot + 2);                        // [129] row pointers of the CTA's rows
    int* tstart = rp_s + 130;                                                 // [kDqMaxTiles + 1] first entry of each K tile's outlier list
    int* tfill = tstart + kDqMaxTiles + 2;                                    // [kDqMaxTiles + 1] fill cursors
    int2* csr_s = reinterpret_cast<int2*>(tfill + kDqMaxTiles + 2);           // [csr_cap], 8-byte aligned
    const unsigned full0 = smem_u32(bars), empty0 = full0 + 8 * kDqStages, accum = empty0 + 8 * kDqStages;

    const int m0 = P.row_start + blockIdx.x * kDqBlockM;
    const int b0 = blockIdx.y * 256;
    const int nb = min(256, P.batch - b0);
    const int rows_out = P.row_stop - P.row_start;
    const int KT_all = P.K / kDqBlockK;
    const int kt0 = blockIdx.z * P.tiles_per_split;                  // this CTA's K tiles: [kt0, kt0 + KT)
    const int KT = min(P.tiles_per_split, KT_all - kt0);
    const bool split = P.ksplit > 1;

    // codebook -> bf16, one 16-byte entry per centroid
    for (int c = tid; c < 256; c += kDqThreads) {
        __nv_bfloat162 h[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) h[q] = __floats2bfloat162_rn(P.codebook[c * 8 + 2 * q], P.codebook[c * 8 + 2 * q + 1]);
        cb16[c] = *reinterpret_cast<uint4*>(h);
    }
    // Outliers of this CTA's rows and K range.  Normally they are listed per K tile in shared memory
    // (counting sort: count, prefix, scatter; entry = row << 8 | column in tile, value / row scale), so
    // that the group that builds a tile applies that tile's ~30 entries with one thread each.  If the
    // lists would not fit, the row-ordered entries are staged instead and every thread walks its rows.
    int csr_base = 0, csr_staged = 0;
    bool listed = false;
    const bool glists = P.tile_off != nullptr && P.csr.nnz > 0 && KT <= kDqMaxTiles;
    if (glists) {
        const int* off = P.tile_off + (size_t)blockIdx.x * (KT_all + 1) + kt0;
        for (int i = tid; i <= KT; i += kDqThreads) tstart[i] = off[i];
    } else if (P.csr.nnz > 0 && m0 < P.row_stop) {
        const int n_rows = min(kDqBlockM, P.row_stop - m0);
        for (int i = tid; i <= n_rows; i += kDqThreads) rp_s[i] = P.csr.row_ptrs[m0 + i];
        for (int i = tid; i <= kDqMaxTiles + 1; i += kDqThreads) tstart[i] = 0;
        __syncthreads();
        csr_base = rp_s[0];
        const int total = rp_s[n_rows] - csr_base;
        if (KT <= kDqMaxTiles) {
            for (int j = tid; j < total; j += kDqThreads) {
                const int t = P.csr.cols[csr_base + j] / kDqBlockK - kt0;
                if (t >= 0 && t < KT) atomicAdd(&tstart[t + 1], 1);
            }
            __syncthreads();
            if (tid == 0) {
                int run = 0;
                for (int t = 0; t <= KT; ++t) { run += tstart[t]; tstart[t] = run; tfill[t] = run; }
            }
            __syncthreads();
            listed = tstart[KT] <= P.csr_cap;
        }
        if (listed) {
            for (int j = tid; j < total; j += kDqThreads) {
                const int col = P.csr.cols[csr_base + j];
                const int t = col / kDqBlockK - kt0;
                if (t < 0 || t >= KT) continue;
                int lo = 0, hi = n_rows;   // row of entry csr_base + j: last row whose pointer is <= it
                while (hi - lo > 1) {
                    const int mid = (lo + hi) >> 1;
                    if (rp_s[mid] <= csr_base + j) lo = mid; else hi = mid;
                }
                // The reference adds the outlier row sum AFTER the row scale (ojasx_lut_cpu.cpp:178-182, 127), so an
                // outlier folded into the weight tile is pre-divided by the scale that the epilogue applies.
                const float sc = P.scales ? P.scales[m0 + lo] : 1.0f;
                const float v = sc != 0.0f ? P.csr.vals[csr_base + j] / sc : 0.0f;
                csr_s[atomicAdd(&tfill[t], 1)] = make_int2((lo << 8) | (col & (kDqBlockK - 1)), __float_as_int(v));
            }
        } else {
            csr_staged = min(P.csr_cap, total);
            for (int i = tid; i < csr_staged; i += kDqThreads)
                csr_s[i] = make_int2(P.csr.cols[csr_base + i], __float_as_int(P.csr.vals[csr_base + i]));
        }
    }
    if (tid == 0) {
        for (int s = 0; s < S; ++s) { mbar_init(full0 + 8 * s, kDqGroupThreads); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(accum, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kDqProducers / 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((unsigned)P.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = *tmem_slot;
    bool ok = true;

    if (warp < kDqProducers / 32) {
        // ---------------- producers: kDqGroups groups of 64 threads; group q builds K tiles q, q + 4, ... on its
        // own, so four tiles are in production at any time and the round trips of one tile (stage free ->
        // copies -> gathers -> arrival -> MMA) overlap with those of the others.  Thread t of a group owns
        // tile rows t and t + 64 (all eight code bytes of the tile each).
        const int gq = tid / kDqGroupThreads, gt = tid - gq * kDqGroupThreads;
        const int total_x = N * 8;
        int rm[2], cur[2], cend[2], col_next[2];
        float inv_scale[2], val_next[2];
        bool rok[2];
        const uint8_t* crow[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            rm[u] = m0 + gt + u * kDqGroupThreads;
            rok[u] = rm[u] < P.row_stop;
            crow[u] = P.codes + (size_t)(rok[u] ? rm[u] : P.row_start) * P.G;
            cur[u] = cend[u] = 0;
            if (rok[u] && P.csr.nnz > 0 && !glists) { cur[u] = P.csr.row_ptrs[rm[u]]; cend[u] = P.csr.row_ptrs[rm[u] + 1]; }
            // The reference adds the outlier row sum AFTER the row scale (ojasx_lut_cpu.cpp:178-182, 127), so an
            // outlier folded into the weight tile is pre-divided by the scale that the epilogue applies.
            const float sc = (rok[u] && P.scales) ? P.scales[rm[u]] : 1.0f;
            inv_scale[u] = sc != 0.0f ? 1.0f / sc : 0.0f;
            col_next[u] = 0x7fffffff;
            val_next[u] = 0.0f;
        }
        auto fetch_outlier = [&](int u) {   // entry cur[u] of row u: from shared memory when it was staged
            if (cur[u] >= cend[u]) { col_next[u] = 0x7fffffff; return; }
            const int i = cur[u] - csr_base;
            if (i < csr_staged) { const int2 e = csr_s[i]; col_next[u] = e.x; val_next[u] = __int_as_float(e.y) * inv_scale[u]; }
            else { col_next[u] = P.csr.cols[cur[u]]; val_next[u] = P.csr.vals[cur[u]] * inv_scale[u]; }
        };
        if (!listed && !glists) {
            fetch_outlier(0);
            fetch_outlier(1);
            while (col_next[0] < kt0 * kDqBlockK) { ++cur[0]; fetch_outlier(0); }   // outliers of the splits before this one
            while (col_next[1] < kt0 * kDqBlockK) { ++cur[1]; fetch_outlier(1); }
        }
        auto load_codes = [&](int kt, uint2 (&c)[2]) {   // the eight code bytes of both rows for K tile kt (8-byte aligned)
#pragma unroll
            for (int u = 0; u < 2; ++u)
                c[u] = kt < KT ? *reinterpret_cast<const uint2*>(crow[u] + (size_t)(kt0 + kt) * 8) : make_uint2(0u, 0u);
        };
        // listed outliers of a tile in global memory: thread gt takes entry gt of the tile (read one tile ahead)
        auto load_entry = [&](int kt) {
            int2 e = make_int2(-1, 0);
            if (glists && kt < KT && tstart[kt] + gt < tstart[kt + 1]) e = P.tile_ent[tstart[kt] + gt];
            return e;
        };
        auto apply_entry = [&](unsigned char* A, const int2 e) {
            const int row = e.x >> 8, kk = e.x & (kDqBlockK - 1), r7 = row & 7;
            __nv_bfloat16* w = reinterpret_cast<__nv_bfloat16*>(A + (row >> 3) * 1024 + r7 * 128 + (((kk >> 3) ^ r7) << 4)) + (kk & 7);
            *w = __float2bfloat16_rn(__bfloat162float(*w) + __int_as_float(e.y));
        };
        uint2 codes_now[2], codes_next[2];
        load_codes(gq, codes_now);
        int2 ent_now = load_entry(gq), ent_next;
        for (int kt = gq; kt < KT && ok; kt += kDqGroups) {
            const int s = kt % S;
            load_codes(kt + kDqGroups, codes_next);   // in flight while this tile is built
            ent_next = load_entry(kt + kDqGroups);
            // the MMAs that read this stage's previous contents must be done
            if (kt >= S) ok = mbar_wait(empty0 + 8 * s, ((kt / S) - 1) & 1);
            if (!ok) break;
            unsigned char* A = tiles + s * stage_bytes;
            unsigned char* B = A + a_bytes;
            if (P.use_tma) {
                if (gt == 0) {   // X tile: one tiled copy; its bytes complete the stage's full barrier together with the arrivals
                    const unsigned bar = full0 + 8 * s;
                    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"((unsigned)b_bytes) : "memory");
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                        ::"r"(smem_u32(B)), "l"(reinterpret_cast<unsigned long long>(&xmap)), "r"((kt0 + kt) * kDqBlockK), "r"(b0), "r"(bar)
                        : "memory");
                }
            } else {
                for (int i = gt; i < total_x; i += kDqGroupThreads) {   // X tile: 16-byte chunks straight into their swizzled place
                    const int r = i >> 3, c = i & 7;
                    const bool in = r < nb;
                    cp_async16_zfill(B + (r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4),
                                     P.x + (size_t)(b0 + (in ? r : 0)) * P.K + (kt0 + kt) * kDqBlockK + c * 8, in ? 16 : 0);
                }
                asm volatile("cp.async.commit_group;" ::: "memory");
            }
            const int kbeg = (kt0 + kt) * kDqBlockK, kend = kbeg + kDqBlockK;
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                // A: eight codes of the row -> eight 16-byte chunks, chunk index XOR (row % 8)
                const int trow = gt + u * kDqGroupThreads, r7 = trow & 7;
                unsigned char* arow = A + (trow >> 3) * 1024 + r7 * 128;
                const unsigned cw[2] = {codes_now[u].x, codes_now[u].y};
                uint4 wv[8];   // all gathers first, then the stores
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const unsigned code = (cw[q >> 2] >> ((q & 3) * 8)) & 0xffu;
                    wv[q] = rok[u] ? cb16[code] : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int q = 0; q < 8; ++q) *reinterpret_cast<uint4*>(arow + ((q ^ r7) << 4)) = wv[q];
                // row-walk fallback: CSR outliers of the row inside this tile (columns ascending): w += value / scale;
                // entries of the tiles that other groups build are passed over
                while (!listed && !glists && col_next[u] < kend) {
                    const int kk = col_next[u] - kbeg;
                    if (kk >= 0) {
                        __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(arow + (((kk >> 3) ^ r7) << 4)) + (kk & 7);
                        *e = __float2bfloat16_rn(__bfloat162float(*e) + val_next[u]);
                    }
                    ++cur[u];
                    fetch_outlier(u);
                }
            }
            if ((listed || glists) && tstart[kt + 1] > tstart[kt]) {   // uniform over the group
                asm volatile("bar.sync %0, %1;" ::"r"(1 + gq), "n"(kDqGroupThreads) : "memory");   // the group's rows are stored
                if (glists) {
                    if (ent_now.x >= 0) apply_entry(A, ent_now);
                    for (int i = tstart[kt] + gt + kDqGroupThreads; i < tstart[kt + 1]; i += kDqGroupThreads) apply_entry(A, P.tile_ent[i]);
                } else {
                    for (int i = tstart[kt] + gt; i < tstart[kt + 1]; i += kDqGroupThreads) apply_entry(A, csr_s[i]);
                }
            }
            if (!P.use_tma) asm volatile("cp.async.wait_group 0;" ::: "memory");   // this thread's share of the X tile has landed
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic and cp.async stores -> visible to the tensor core
            mbar_arrive(full0 + 8 * s);
            codes_now[0] = codes_next[0];
            codes_now[1] = codes_next[1];
            ent_now = ent_next;
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        // the epilogue and the split reduction address rows as (tid & 127, tid >> 7)
        const int trow = tid & 127, half = tid >> 7;
        const int m = m0 + trow;
        const bool row_ok = m < P.row_stop;
        const float row_scale = (row_ok && P.scales) ? P.scales[m] : 1.0f;
        int csr_begin = 0, cend_row = 0;
        if (row_ok && P.csr.nnz > 0) { csr_begin = P.csr.row_ptrs[m]; cend_row = P.csr.row_ptrs[m + 1]; }
        // ---------------- epilogue: accumulator row trow; the two threads of a row split the batch columns
        if (ok) ok = mbar_wait(accum, 0);
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float sc = row_scale;
            const float bi = (row_ok && P.bias) ? P.bias[m] : 0.0f;
            const int cbeg = half * (N >> 1), cstop = cbeg + (N >> 1);
            float* part = reinterpret_cast<float*>(tiles);   // split: [column][row] fp32, read by the whole cluster
            for (int c0 = cbeg; c0 < cstop; c0 += 16) {
                unsigned v[16];
                const unsigned taddr = tmem_base + ((unsigned)((warp & 3) * 32) << 16) + (unsigned)c0;
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                      "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                    : "r"(taddr));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (split) {   // raw partial sums, rows contiguous
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (c0 + j < cstop) part[(c0 + j) * kDqBlockM + trow] = __uint_as_float(v[j]);
                } else if (row_ok) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int b = c0 + j;
                        if (b < nb && b < cstop) {
                            float r = fmaf(__uint_as_float(v[j]), sc, bi);
                            if (sc == 0.0f)  // a zero row scale cannot carry the folded outliers: add them here
                                for (int q = csr_begin; q < cend_row; ++q)
                                    r += P.csr.vals[q] * __bfloat162float(P.x[(size_t)(b0 + b) * P.K + P.csr.cols[q]]);
                            P.y[(size_t)(b0 + b) * rows_out + (m - P.row_start)] = __float2bfloat16_rn(r);
                        }
                    }
                }
            }
        }
    } else if (lane == 0) {
        // ---------------- MMA issuer
        const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(N >> 3) << 17) | ((unsigned)(kDqBlockM >> 4) << 24);
        for (int kt = 0; kt < KT && ok; ++kt) {
            const int s = kt % S;
            ok = mbar_wait(full0 + 8 * s, (kt / S) & 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const unsigned a_addr = smem_u32(tiles + s * stage_bytes), b_addr = a_addr + a_bytes;
#pragma unroll
            for (int j = 0; j < kDqBlockK / 16; ++j) {
                const unsigned long long da = make_desc_sw128(a_addr + j * 32), db = make_desc_sw128(b_addr + j * 32);
                const unsigned acc = (kt > 0 || j > 0) ? 1u : 0u;
                asm volatile(
                    "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                    "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                    ::"r"(tmem_base), "l"(da), "l"(db), "r"(idesc), "r"(acc)
                    : "memory");
            }
            // frees the stage when the MMAs that read it have completed
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(empty0 + 8 * s) : "memory");
        }
        if (ok) asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(accum) : "memory");
    }
    if (!ok && P.error_flag) atomicExch(P.error_flag, 1);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == kDqProducers / 32) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((unsigned)P.tmem_cols) : "memory");
    }
    if (split) {
        // Every CTA of the cluster adds the partial sums of its share of the batch columns, in split order (the result
        // does not depend on timing), and finishes those outputs.  All threads take part in the two cluster barriers;
        // a CTA whose waits ran out still arrives, so the others are not left waiting.
        dq_cluster_sync();   // the partial sums of every split are in place
        if (warp < kDqProducers / 32) {
            unsigned rank;
            asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
            const int per = (N + P.ksplit - 1) / P.ksplit;
            const int cfirst = (int)rank * per, clast = min(min(N, nb), cfirst + per);
            const int trow = tid & 127, half = tid >> 7, m = m0 + trow;
            if (m < P.row_stop) {
                const float sc = P.scales ? P.scales[m] : 1.0f, bi = P.bias ? P.bias[m] : 0.0f;
                const unsigned part0 = smem_u32(tiles);
                for (int bb = cfirst + half; bb < clast; bb += 8) {   // four columns at a time: all loads first
                    float pv[4][4];
#pragma unroll
                    for (int j = 0; j < 4; ++j)
#pragma unroll
                        for (int z = 0; z < 4; ++z)
                            pv[j][z] = (bb + 2 * j < clast && z < P.ksplit)
                                           ? dq_ld_cluster(part0 + (unsigned)((bb + 2 * j) * kDqBlockM + trow) * 4u, (unsigned)z) : 0.0f;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int b = bb + 2 * j;
                        if (b >= clast) break;
                        float acc = 0.0f;
#pragma unroll
                        for (int z = 0; z < 4; ++z) if (z < P.ksplit) acc += pv[j][z];
                        float r = fmaf(acc, sc, bi);
                        if (sc == 0.0f && P.csr.nnz > 0)  // a zero row scale cannot carry the folded outliers: add them here
                            for (int q = P.csr.row_ptrs[m]; q < P.csr.row_ptrs[m + 1]; ++q)
                                r += P.csr.vals[q] * __bfloat162float(P.x[(size_t)(b0 + b) * P.K + P.csr.cols[q]]);
                        P.y[(size_t)(b0 + b) * rows_out + (m - P.row_start)] = __float2bfloat16_rn(r);
                    }
                }
            }
        }
        dq_cluster_sync();   // nobody leaves while its partial sums may still be read
    }
}

// ---------------------------------------------------------------------------------------------------------------
// 256-row variant, for batches of several 256-column tiles.  Every row tile streams all of X from L2 (an X tile is
// twice the size of a 128-row weight tile at batch 256), and L2 delivers about 25 bytes per clock and SM, which is
// what bounds the 128-row kernel at wide batches.  Here a CTA owns two adjacent 128-row tiles: a stage holds both
// weight tiles and ONE X tile, every K step issues two MMAs that share the B operand, and the two accumulators sit
// side by side in tensor memory (2 x N <= 512 columns).  Three producer groups of 128 threads each own one of three
// stages (thread t builds row t of both weight tiles), so a group can never be two phases ahead of a stage.
// It is used when (row pairs x batch tiles) fill the GPU without a split along K: with a split, the fp32 partial sums
// of a 256 x 256 tile (256 KB per CTA, whatever the split) cost as much traffic between the SMs as the X tiles they
// save -- measured at batch 256 with a cluster of five: 56 against 29 microseconds for the 128-row kernel; at batch
// 1024 (no split) 66 against 73.  Needs the X tiles by the copy engine and the outlier lists of the layer (or no
// outliers); other cases take the 128-row kernel.
constexpr int kDq2Groups = 3;
constexpr int kDq2GroupThreads = 128;
constexpr int kDq2Producers = kDq2Groups * kDq2GroupThreads;
constexpr int kDq2Threads = kDq2Producers + 32;
constexpr int kDq2Stages = kDq2Groups;

__global__ void __launch_bounds__(kDq2Threads, 1) vq_dequant_gemm256_kernel(const __grid_constant__ DequantGemmProblem P,
                                                                           const __grid_constant__ CUtensorMap xmap) {
    extern __shared__ unsigned char dq_smem_raw[];
    unsigned char* dq_smem = dq_smem_raw + ((1024u - (smem_u32(dq_smem_raw) & 1023u)) & 1023u);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int N = P.n_pad;
    constexpr int S = kDq2Stages;
    const int a_bytes = 2 * kDqBlockM * 128, b_bytes = N * 128, stage_bytes = a_bytes + b_bytes;
    unsigned char* tiles = dq_smem;                                    // [3][A0 | A1 | B], 1024-byte aligned
    uint4* cb16 = reinterpret_cast<uint4*>(tiles + S * stage_bytes);    // [256] centroids as 8 bf16
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(cb16 + 256);
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 2 * S + 1);
    int* toff = reinterpret_cast<int*>(tmem_slot + 2);                  // [2][kDqMaxTiles + 2] outlier list offsets of both row tiles
    const unsigned full0 = smem_u32(bars), empty0 = full0 + 8 * S, accum = empty0 + 8 * S;

    const int m0 = P.row_start + blockIdx.x * 2 * kDqBlockM;
    const int b0 = blockIdx.y * 256;
    const int nb = min(256, P.batch - b0);
    const int rows_out = P.row_stop - P.row_start;
    const int KT_all = P.K / kDqBlockK;
    const int kt0 = blockIdx.z * P.tiles_per_split;
    const int KT = min(P.tiles_per_split, KT_all - kt0);
    const bool split = P.ksplit > 1;
    const bool glists = P.tile_off != nullptr && P.csr.nnz > 0;
    const int row_tiles = (rows_out + kDqBlockM - 1) / kDqBlockM;

    for (int c = tid; c < 256; c += kDq2Threads) {
        __nv_bfloat162 h[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) h[q] = __floats2bfloat162_rn(P.codebook[c * 8 + 2 * q], P.codebook[c * 8 + 2 * q + 1]);
        cb16[c] = *reinterpret_cast<uint4*>(h);
    }
    for (int i = tid; i < 2 * (kDqMaxTiles + 2); i += kDq2Threads) {
        const int a = i / (kDqMaxTiles + 2), k = i - a * (kDqMaxTiles + 2), rt = 2 * (int)blockIdx.x + a;
        toff[i] = (glists && rt < row_tiles && k <= KT) ? P.tile_off[(size_t)rt * (KT_all + 1) + kt0 + k] : 0;
    }
    if (tid == 0) {
        for (int s = 0; s < S; ++s) { mbar_init(full0 + 8 * s, kDq2GroupThreads); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(accum, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kDq2Producers / 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((unsigned)P.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = *tmem_slot;
    bool ok = true;

    // accumulator rows of this thread in the epilogue: row (warp & 3) * 32 + lane of both tiles (tensor-memory lanes are
    // tied to warp % 4); the three warps of a lane quarter share the columns
    const int erow = (warp & 3) * 32 + lane, esib = warp >> 2;
    auto ld16 = [&](int a, int c0, unsigned (&v)[16]) {
        const unsigned taddr = tmem_base + ((unsigned)((warp & 3) * 32) << 16) + (unsigned)(a * N + c0);
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
              "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
            : "r"(taddr));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    };
    auto finish = [&](int m, int b, float acc, float sc, float bi) {   // scale, bias, store (zero scales: outliers added here)
        float r = fmaf(acc, sc, bi);
        if (sc == 0.0f && P.csr.nnz > 0)
            for (int q = P.csr.row_ptrs[m]; q < P.csr.row_ptrs[m + 1]; ++q)
                r += P.csr.vals[q] * __bfloat162float(P.x[(size_t)(b0 + b) * P.K + P.csr.cols[q]]);
        P.y[(size_t)(b0 + b) * rows_out + (m - P.row_start)] = __float2bfloat16_rn(r);
    };

    if (warp < kDq2Producers / 32) {
        const int gq = tid / kDq2GroupThreads, gt = tid - gq * kDq2GroupThreads;
        bool rok[2];
        const uint8_t* crow[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int m = m0 + u * kDqBlockM + gt;
            rok[u] = m < P.row_stop;
            crow[u] = P.codes + (size_t)(rok[u] ? m : P.row_start) * P.G;
        }
        auto load_codes = [&](int kt, uint2 (&c)[2]) {
#pragma unroll
            for (int u = 0; u < 2; ++u)
                c[u] = kt < KT ? *reinterpret_cast<const uint2*>(crow[u] + (size_t)(kt0 + kt) * 8) : make_uint2(0u, 0u);
        };
        auto load_entries = [&](int kt, int2 (&e)[2]) {   // entry gt of the K tile's list of each row tile (read one tile ahead)
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int* o = toff + u * (kDqMaxTiles + 2);
                e[u] = make_int2(-1, 0);
                if (glists && kt < KT && o[kt] + gt < o[kt + 1]) e[u] = P.tile_ent[o[kt] + gt];
            }
        };
        auto apply_entry = [&](unsigned char* A, const int2 e) {
            const int row = e.x >> 8, kk = e.x & (kDqBlockK - 1), r7 = row & 7;
            __nv_bfloat16* w = reinterpret_cast<__nv_bfloat16*>(A + (row >> 3) * 1024 + r7 * 128 + (((kk >> 3) ^ r7) << 4)) + (kk & 7);
            *w = __float2bfloat16_rn(__bfloat162float(*w) + __int_as_float(e.y));
        };
        uint2 codes_now[2], codes_next[2];
        int2 ent_now[2], ent_next[2];
        load_codes(gq, codes_now);
        load_entries(gq, ent_now);
        for (int kt = gq; kt < KT && ok; kt += kDq2Groups) {
            const int s = gq;   // == kt % 3: every group owns one stage
            load_codes(kt + kDq2Groups, codes_next);
            load_entries(kt + kDq2Groups, ent_next);
            if (kt >= S) ok = mbar_wait(empty0 + 8 * s, ((kt / S) - 1) & 1);
            if (!ok) break;
            unsigned char* A = tiles + s * stage_bytes;
            unsigned char* B = A + a_bytes;
            if (gt == 0) {   // the X tile of this K step, once for both weight tiles
                const unsigned bar = full0 + 8 * s;
                asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"((unsigned)b_bytes) : "memory");
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                    ::"r"(smem_u32(B)), "l"(reinterpret_cast<unsigned long long>(&xmap)), "r"((kt0 + kt) * kDqBlockK), "r"(b0), "r"(bar)
                    : "memory");
            }
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int r7 = gt & 7;
                unsigned char* arow = A + u * (kDqBlockM * 128) + (gt >> 3) * 1024 + r7 * 128;
                const unsigned cw[2] = {codes_now[u].x, codes_now[u].y};
                uint4 wv[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const unsigned code = (cw[q >> 2] >> ((q & 3) * 8)) & 0xffu;
                    wv[q] = rok[u] ? cb16[code] : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int q = 0; q < 8; ++q) *reinterpret_cast<uint4*>(arow + ((q ^ r7) << 4)) = wv[q];
            }
            const int* o0 = toff;
            const int* o1 = toff + (kDqMaxTiles + 2);
            if (o0[kt + 1] > o0[kt] || o1[kt + 1] > o1[kt]) {   // uniform over the group
                asm volatile("bar.sync %0, %1;" ::"r"(1 + gq), "n"(kDq2GroupThreads) : "memory");   // the group's rows are stored
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const int* o = u ? o1 : o0;
                    unsigned char* Au = A + u * (kDqBlockM * 128);
                    if (ent_now[u].x >= 0) apply_entry(Au, ent_now[u]);
                    for (int i = o[kt] + gt + kDq2GroupThreads; i < o[kt + 1]; i += kDq2GroupThreads) apply_entry(Au, P.tile_ent[i]);
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(full0 + 8 * s);
            codes_now[0] = codes_next[0];
            codes_now[1] = codes_next[1];
            ent_now[0] = ent_next[0];
            ent_now[1] = ent_next[1];
        }
        if (ok) ok = mbar_wait(accum, 0);
        if (__all_sync(0xffffffffu, ok) && !split) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            for (int ci = esib; ci < 2 * N / 16; ci += kDq2Groups) {
                const int a = (ci * 16) / N, c0 = ci * 16 - a * N, m = m0 + a * kDqBlockM + erow;
                unsigned v[16];
                ld16(a, c0, v);   // every lane of the warp takes part in the load
                if (m < P.row_stop) {
                    const float sc = P.scales ? P.scales[m] : 1.0f, bi = P.bias ? P.bias[m] : 0.0f;
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (c0 + j < nb) finish(m, c0 + j, __uint_as_float(v[j]), sc, bi);
                }
            }
        }
    } else if (lane == 0) {
        const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(N >> 3) << 17) | ((unsigned)(kDqBlockM >> 4) << 24);
        for (int kt = 0; kt < KT && ok; ++kt) {
            const int s = kt % S;
            ok = mbar_wait(full0 + 8 * s, (kt / S) & 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const unsigned a_addr = smem_u32(tiles + s * stage_bytes), b_addr = a_addr + a_bytes;
#pragma unroll
            for (int j = 0; j < kDqBlockK / 16; ++j) {
                const unsigned long long db = make_desc_sw128(b_addr + j * 32);
                const unsigned acc = (kt > 0 || j > 0) ? 1u : 0u;
#pragma unroll
                for (int a = 0; a < 2; ++a) {
                    const unsigned long long da = make_desc_sw128(a_addr + a * (kDqBlockM * 128) + j * 32);
                    asm volatile(
                        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                        ::"r"(tmem_base + (unsigned)(a * N)), "l"(da), "l"(db), "r"(idesc), "r"(acc)
                        : "memory");
                }
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(empty0 + 8 * s) : "memory");
        }
        if (ok) asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(accum) : "memory");
    }
    if (!ok && P.error_flag) atomicExch(P.error_flag, 1);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (split) {
        // One accumulator at a time (both do not fit in shared memory): every CTA of the cluster leaves its partial sums
        // in its stage buffers, then adds its share of the batch columns over all splits, in split order.
        unsigned rank;
        asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
        const int per = (N + P.ksplit - 1) / P.ksplit;
        const int cfirst = (int)rank * per, clast = min(min(N, nb), cfirst + per);
        float* part = reinterpret_cast<float*>(tiles);   // [column][row] fp32
        const unsigned part0 = smem_u32(tiles);
        for (int a = 0; a < 2; ++a) {
            if (warp < kDq2Producers / 32 && __all_sync(0xffffffffu, ok)) {   // (a warp whose waits ran out leaves its part undefined; the flag is up)
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int ci = esib; ci < N / 16; ci += kDq2Groups) {
                    unsigned v[16];
                    ld16(a, ci * 16, v);
#pragma unroll
                    for (int j = 0; j < 16; ++j) part[(ci * 16 + j) * kDqBlockM + erow] = __uint_as_float(v[j]);
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            }
            dq_cluster_sync();   // the partial sums of every split are in place
            const int m = m0 + a * kDqBlockM + erow;
            if (warp < kDq2Producers / 32 && m < P.row_stop) {
                const float sc = P.scales ? P.scales[m] : 1.0f, bi = P.bias ? P.bias[m] : 0.0f;
                for (int bb = cfirst + esib; bb < clast; bb += 4 * kDq2Groups) {   // four columns at a time: all loads first
                    float pv[4][8];
#pragma unroll
                    for (int j = 0; j < 4; ++j)
#pragma unroll
                        for (int z = 0; z < 8; ++z)
                            pv[j][z] = (bb + kDq2Groups * j < clast && z < P.ksplit)
                                           ? dq_ld_cluster(part0 + (unsigned)((bb + kDq2Groups * j) * kDqBlockM + erow) * 4u, (unsigned)z) : 0.0f;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int b = bb + kDq2Groups * j;
                        if (b >= clast) break;
                        float acc = 0.0f;
#pragma unroll
                        for (int z = 0; z < 8; ++z) if (z < P.ksplit) acc += pv[j][z];
                        finish(m, b, acc, sc, bi);
                    }
                }
            }
            dq_cluster_sync();   // nobody overwrites or leaves while its partial sums may still be read
        }
    }
    if (warp == kDq2Producers / 32) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((unsigned)P.tmem_cols) : "memory");
    }
}

size_t dequant_gemm256_smem(int n_pad) {
    return (size_t)kDq2Stages * (2 * kDqBlockM * 128 + (size_t)n_pad * 128) + 256 * 16 + (2 * kDq2Stages + 1) * 8 + 16 +
           sizeof(int) * 2 * (kDqMaxTiles + 2) + 1024;
}

constexpr size_t kDqSmemBudget = 226 * 1024;   // dynamic shared memory; the kernel also has a few static bytes

size_t dequant_gemm_smem(int n_pad, int stages, int csr_cap) {
    return (size_t)stages * (kDqBlockM * 128 + (size_t)n_pad * 128) + 256 * 16 + (2 * kDqStages + 1) * 8 + 16 +
           sizeof(int) * (130 + 2 * (kDqMaxTiles + 2)) + (size_t)csr_cap * 8 + 1024;
}

static __device__ int g_dq_error;  // raised when a bounded wait inside the kernel ran out

// Reads and clears the flag (synchronises the device).  1 = some dequant-GEMM launch since the last
// call gave up waiting on a barrier and its output must not be trusted.
int take_dequant_gemm_error(int* out) {
    int v = 0, zero = 0;
    OJX_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_dq_error, sizeof(int)));
    if (v) OJX_CUDA_TRY(cudaMemcpyToSymbol(g_dq_error, &zero, sizeof(int)));
    *out = v;
    return OJX_OK;
}

// Conditions under which the tensor-core path may stand in for the table kernels.
bool dequant_gemm_supported(const LinearProblem& P, bool csr_sorted) {
    return P.io_dtype == OJX_BF16 && P.D == 8 && P.Kcb == 256 && P.K == P.G * 8 && (P.K % kDqBlockK) == 0 &&
           (P.csr.nnz == 0 || csr_sorted) && (reinterpret_cast<uintptr_t>(P.codes) & 15) == 0 && (P.G & 15) == 0 &&
           (reinterpret_cast<uintptr_t>(P.x) & 15) == 0;
}

// Splits along K for `ctas` (row tile, batch tile) pairs and KT tiles of 64 columns: fill the SMs, at most
// four splits (one thread-block cluster), at least eight tiles per split, an even number of tiles per split.
static void plan_ksplit(int ctas, int KT, int sms, int zmax, int* ksplit, int* per) {
    int z = sms / (ctas > 0 ? ctas : 1);
    z = z < 1 ? 1 : z > zmax ? zmax : z;
    while (z > 1 && KT / z < 8) --z;
    int p = (KT + z - 1) / z;
    p += p & 1;
    *per = z > 1 ? p : KT;
    *ksplit = z > 1 ? (KT + p - 1) / p : 1;
}

// ---- outliers listed per (128-row tile, 64-column tile), once per layer and row range
// counts[rt * (KT + 1) + kt + 1] = entries of tile (rt, kt); after the scan the same array holds the offsets.
__global__ void dq_list_count_kernel(CsrView csr, int row_start, int row_stop, int KT, int* counts) {
    const int m = row_start + blockIdx.x * blockDim.x + threadIdx.x;
    if (m >= row_stop) return;
    const int rt = (m - row_start) / kDqBlockM;
    for (int j = csr.row_ptrs[m]; j < csr.row_ptrs[m + 1]; ++j) {
        const int kt = csr.cols[j] / kDqBlockK;
        if (kt < KT) atomicAdd(&counts[(size_t)rt * (KT + 1) + kt + 1], 1);
    }
}
// One block: inclusive scan of counts[0, n) in place (counts[0] and every tile row's first slot are zero, so
// slot rt * (KT + 1) + kt ends up as the first entry of tile (rt, kt)); `fill` gets a copy for the scatter.
__global__ void dq_list_scan_kernel(int* counts, int* fill, int n, int base) {
    __shared__ int warp_sum[32];
    __shared__ int carry;
    if (threadIdx.x == 0) carry = base;
    __syncthreads();
    for (int i0 = 0; i0 < n; i0 += blockDim.x) {
        const int i = i0 + threadIdx.x;
        int v = i < n ? counts[i] : 0;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, v, o);
            if ((threadIdx.x & 31) >= o) v += t;
        }
        if ((threadIdx.x & 31) == 31) warp_sum[threadIdx.x >> 5] = v;
        __syncthreads();
        if (threadIdx.x < 32) {
            int w = threadIdx.x < (blockDim.x >> 5) ? warp_sum[threadIdx.x] : 0;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, w, o);
                if (threadIdx.x >= o) w += t;
            }
            warp_sum[threadIdx.x] = w;
        }
        __syncthreads();
        const int before = carry + ((threadIdx.x >> 5) ? warp_sum[(threadIdx.x >> 5) - 1] : 0);
        if (i < n) { counts[i] = before + v; fill[i] = before + v; }
        __syncthreads();
        if (threadIdx.x == blockDim.x - 1) carry = before + v;
        __syncthreads();
    }
}
__global__ void dq_list_fill_kernel(CsrView csr, const float* scales, int row_start, int row_stop, int KT, int* fill, int2* ent) {
    const int m = row_start + blockIdx.x * blockDim.x + threadIdx.x;
    if (m >= row_stop) return;
    const int rt = (m - row_start) / kDqBlockM, row = (m - row_start) % kDqBlockM;
    // The reference adds the outlier row sum AFTER the row scale (ojasx_lut_cpu.cpp:178-182, 127), so an outlier
    // folded into the weight tile is pre-divided by the scale that the epilogue applies.
    const float sc = scales ? scales[m] : 1.0f;
    for (int j = csr.row_ptrs[m]; j < csr.row_ptrs[m + 1]; ++j) {
        const int col = csr.cols[j], kt = col / kDqBlockK;
        if (kt >= KT) continue;
        const float v = sc != 0.0f ? csr.vals[j] / sc : 0.0f;
        // slot kt of the row tile holds the END of tile kt - 1 = start of tile kt after the scan
        const int pos = atomicAdd(&fill[(size_t)rt * (KT + 1) + kt], 1);
        ent[pos] = make_int2((row << 8) | (col & (kDqBlockK - 1)), __float_as_int(v));
    }
}

DqLists::~DqLists() { cudaFree(off); cudaFree(ent); }

// Builds (or reuses) the lists for rows [row_start, row_stop) of the layer behind L.  Returns false when they cannot be
// used for this launch (no outliers, a stream capture in progress before they exist, an allocation that failed).
static bool ensure_dq_lists(DqLists* d, const LinearProblem& L, unsigned generation, cudaStream_t stream) {
    if (!d || L.csr.nnz <= 0) return false;
    const int KT = L.K / kDqBlockK, rows = L.row_stop - L.row_start, row_tiles = (rows + kDqBlockM - 1) / kDqBlockM;
    if (d->valid && d->generation == generation && d->row_start == L.row_start && d->row_stop == L.row_stop && d->csr_vals == L.csr.vals)
        return true;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) return false;
    d->valid = false;
    const size_t n_off = (size_t)row_tiles * (KT + 1) + 1;
    if (n_off > d->off_cap) {
        cudaFree(d->off);
        d->off = nullptr; d->off_cap = 0;
        if (cudaMalloc((void**)&d->off, sizeof(int) * 2 * n_off) != cudaSuccess) { cudaGetLastError(); return false; }
        d->off_cap = n_off;
    }
    if ((size_t)L.csr.nnz > d->ent_cap) {
        cudaFree(d->ent);
        d->ent = nullptr; d->ent_cap = 0;
        if (cudaMalloc((void**)&d->ent, sizeof(int2) * (size_t)L.csr.nnz) != cudaSuccess) { cudaGetLastError(); return false; }
        d->ent_cap = (size_t)L.csr.nnz;
    }
    int* fill = d->off + d->off_cap;
    if (cudaMemsetAsync(d->off, 0, sizeof(int) * n_off, stream) != cudaSuccess) return false;
    const int blocks = (rows + 255) / 256;
    dq_list_count_kernel<<<blocks, 256, 0, stream>>>(L.csr, L.row_start, L.row_stop, KT, d->off);
    dq_list_scan_kernel<<<1, 1024, 0, stream>>>(d->off, fill, (int)n_off, 0);
    // after the inclusive scan slot (rt, kt + 1) holds the end of tile (rt, kt): shift by one slot when reading, i.e.
    // tile (rt, kt) = [slot(rt, kt), slot(rt, kt + 1)) -- slot (rt, 0) is the end of the previous row tile
    dq_list_fill_kernel<<<blocks, 256, 0, stream>>>(L.csr, L.scales, L.row_start, L.row_stop, KT, fill, d->ent);
    if (cudaGetLastError() != cudaSuccess) return false;
    count_launch(3);
    d->row_start = L.row_start; d->row_stop = L.row_stop; d->generation = generation; d->csr_vals = L.csr.vals;
    d->valid = true;
    return true;
}

// cuTensorMapEncodeTiled through the runtime's driver entry point lookup (no link against the driver library).
using TensorMapEncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                       const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                       CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static TensorMapEncodeFn tensor_map_encoder() {
    static TensorMapEncodeFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            p = nullptr;
        }
        return reinterpret_cast<TensorMapEncodeFn>(p);
    }();
    return fn;
}
// X [batch, K] bf16 row-major as a 2-D tensor (columns innermost), box = 64 columns x n_pad rows, 128-byte swizzle;
// rows past the batch read as zero.
static bool encode_x_map(CUtensorMap* map, const void* x, int K, int batch, int n_pad) {
    TensorMapEncodeFn enc = tensor_map_encoder();
    if (!enc) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)batch};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kDqBlockK, (cuuint32_t)n_pad};
    const cuuint32_t estr[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int launch_dequant_gemm(const LinearProblem& L, cudaStream_t stream, DqLists* lists, unsigned generation) {
    DequantGemmProblem P{};
    int* error_flag = nullptr;
    OJX_CUDA_TRY(cudaGetSymbolAddress((void**)&error_flag, g_dq_error));
    P.codes = L.codes; P.codebook = L.codebook; P.scales = L.scales; P.bias = L.bias; P.csr = L.csr;
    P.x = static_cast<const __nv_bfloat16*>(L.x); P.y = static_cast<__nv_bfloat16*>(L.y);
    P.error_flag = error_flag;
    P.K = L.K; P.G = L.G; P.row_start = L.row_start; P.row_stop = L.row_stop; P.batch = L.batch;
    const int nb = L.batch < 256 ? L.batch : 256;
    P.n_pad = round_up(nb, 16);
    int cols = 32;
    while (cols < P.n_pad) cols <<= 1;
    P.tmem_cols = cols;
    // Outlier lists of the layer (built once) spare every CTA the sort in its prologue and the shared memory for it.
    const bool glists = L.K / kDqBlockK <= kDqMaxTiles && !getenv("OJASX_B200_TENSOR_NO_LISTS") && ensure_dq_lists(lists, L, generation, stream);
    if (glists) { P.tile_off = lists->off; P.tile_ent = lists->ent; }
    // Batches of several 256-column tiles: two row tiles per CTA share every X tile (vq_dequant_gemm256_kernel), when
    // the tile pairs fill the GPU without a split along K.  OJASX_B200_TENSOR_ROWS=128 / 256 forces one kernel or the
    // other (256: with a split if the grid is small).
    {
        const char* rows_env = getenv("OJASX_B200_TENSOR_ROWS");
        const char* tma_off = getenv("OJASX_B200_TENSOR_TMA");
        const int rows = L.row_stop - L.row_start, forced = rows_env ? atoi(rows_env) : 0;
        dim3 grid((rows + 2 * kDqBlockM - 1) / (2 * kDqBlockM), (L.batch + 255) / 256, 1);
        const bool fills = (int)(grid.x * grid.y) * 3 >= num_sms() * 2;
        CUtensorMap xmap{};
        if ((forced == 256 || (forced != 128 && fills)) && !(tma_off && tma_off[0] == '0') && (glists || L.csr.nnz == 0) &&
            rows > kDqBlockM && P.n_pad >= 64 && dequant_gemm256_smem(P.n_pad) <= kDqSmemBudget &&
            encode_x_map(&xmap, L.x, L.K, L.batch, P.n_pad)) {
            int z = 1, per = L.K / kDqBlockK;
            if (forced == 256 && !getenv("OJASX_B200_TENSOR_NO_KSPLIT")) plan_ksplit((int)(grid.x * grid.y), L.K / kDqBlockK, num_sms(), 8, &z, &per);
            if ((z > 1 ? per : L.K / kDqBlockK) <= kDqMaxTiles) {
                P.ksplit = z;
                P.tiles_per_split = z > 1 ? per : L.K / kDqBlockK;
                int cols2 = 32;
                while (cols2 < 2 * P.n_pad) cols2 <<= 1;
                P.tmem_cols = cols2;
                P.stages = kDq2Stages;
                P.use_tma = 1;
                const size_t smem = dequant_gemm256_smem(P.n_pad);
                static thread_local size_t configured2[64] = {};
                int dev = 0;
                OJX_CUDA_TRY(cudaGetDevice(&dev));
                if (dev < 0 || dev >= 64 || smem > configured2[dev]) {
                    OJX_CUDA_TRY(cudaFuncSetAttribute(vq_dequant_gemm256_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                    if (dev >= 0 && dev < 64) configured2[dev] = smem;
                }
                grid.z = z;
                cudaLaunchConfig_t cfg{};
                cfg.gridDim = grid;
                cfg.blockDim = dim3(kDq2Threads);
                cfg.dynamicSmemBytes = smem;
                cfg.stream = stream;
                cudaLaunchAttribute attr[1];
                attr[0].id = cudaLaunchAttributeClusterDimension;
                attr[0].val.clusterDim.x = 1;
                attr[0].val.clusterDim.y = 1;
                attr[0].val.clusterDim.z = grid.z;
                cfg.attrs = attr;
                cfg.numAttrs = 1;
                OJX_CUDA_TRY(cudaLaunchKernelEx(&cfg, vq_dequant_gemm256_kernel, P, xmap));
                count_launch(1);
                return OJX_OK;
            }
        }
    }
    // Stage buffers: at least one per producer group.  (A group waits on a stage's "empty" barrier by phase
    // parity; with fewer stages than groups a group could be two phases ahead of a stage it shares with
    // another group, and a parity wait cannot tell "two ahead" from "done".)  More stages when the batch
    // tile is narrow; room for at least 1024 staged outlier entries is kept when every CTA lists its own.
    P.stages = kDqGroups;
    if (dequant_gemm_smem(P.n_pad, P.stages, glists ? 0 : 1024) > kDqSmemBudget) return OJX_ERR_UNSUPPORTED;
    while (P.stages < kDqStages && dequant_gemm_smem(P.n_pad, P.stages + 1, glists ? 0 : 4096) <= kDqSmemBudget) ++P.stages;
    // shared-memory room for the outliers of 128 rows: whatever is left, up to 8192 entries; the
    // kernel reads entries beyond that from global memory
    P.csr_cap = 0;
    if (L.csr.nnz > 0 && !glists) {
        const size_t left = kDqSmemBudget - dequant_gemm_smem(P.n_pad, P.stages, 0);
        P.csr_cap = (int)(left / 8 < 8192 ? left / 8 : 8192);
    }
    const size_t smem = dequant_gemm_smem(P.n_pad, P.stages, P.csr_cap);
    // the opt-in is a per-device attribute of the kernel: remember what each device was given
    static thread_local size_t configured[64] = {};
    int cur_dev = 0;
    OJX_CUDA_TRY(cudaGetDevice(&cur_dev));
    if (cur_dev < 0 || cur_dev >= 64 || smem > configured[cur_dev]) {
        OJX_CUDA_TRY(cudaFuncSetAttribute(vq_dequant_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (cur_dev >= 0 && cur_dev < 64) configured[cur_dev] = smem;
    }
    const int rows = L.row_stop - L.row_start;
    dim3 grid((rows + kDqBlockM - 1) / kDqBlockM, (L.batch + 255) / 256, 1);
    P.ksplit = 1;
    P.tiles_per_split = L.K / kDqBlockK;
    if (!getenv("OJASX_B200_TENSOR_NO_KSPLIT")) {
        int z = 1, per = P.tiles_per_split;
        plan_ksplit((int)(grid.x * grid.y), L.K / kDqBlockK, num_sms(), 4, &z, &per);
        if (z > 1) {
            P.ksplit = z;
            P.tiles_per_split = per;
            grid.z = z;
        }
    }
    // X tiles by the copy engine when the tensor map can be made (OJASX_B200_TENSOR_TMA=0 keeps the 16-byte copies)
    CUtensorMap xmap{};
    const char* tma_env = getenv("OJASX_B200_TENSOR_TMA");
    P.use_tma = !(tma_env && tma_env[0] == '0') && encode_x_map(&xmap, L.x, L.K, L.batch, P.n_pad) ? 1 : 0;
    // the K splits of a tile are one cluster (they exchange partial sums through distributed shared memory)
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kDqThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = grid.z;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    OJX_CUDA_TRY(cudaLaunchKernelEx(&cfg, vq_dequant_gemm_kernel, P, xmap));
    count_launch(1);
    return OJX_OK;
}

}  // namespace ojx

