// Row walk of the split-manifold LUT path with conflict-free table gathers.
//
// RowWalker (lut_core.cuh) gives every lane one row: the 32 gathers of a warp instruction hit
// random banks of the table and cost about four shared-memory wavefronts.  Here the 32 lanes of a
// warp share one row instead: lane l owns the four groups 4l..4l+3 of the table slice, and the
// slice is stored code-major with lane l's entries in bank l, so a gather instruction is one
// wavefront whatever the codes are.
//
// The reference adds a row's table entries in ascending group order into one fp32 accumulator
// (split_manifold_lut_experiment/native/src/ojasx_lut_cpu.cpp:161-175).  That order is kept by
// passing the running sum of a row from lane to lane: in step t lane l works on row t - l, takes
// the sum that lane l - 1 produced for that row one step earlier (one shuffle), adds its four
// entries in order and hands the sum on.  Thirty-two rows are in flight in a warp, each one lane
// further than the next; lane 0 starts a row from the sum parked in shared memory (zero in the
// first slice) and the last active lane parks it again.
//
// Shared memory, by absolute shared-space address (the walker is used only when the dynamic area
// starts at 1024, which is checked at run time):
//     1024  parked row sums           f32[6912]
//    28672  activations of the slice  f32[2048], element d of group p at d*SG + p
//    36864  code rings of warps 0..6  (4 KB each)
//    65536  table, groups j = 0, 1    entry (code k, j, lane l) at 65536 + k*256 + j*128 + l*4
//   131072  table, groups j = 2, 3    entry at 131072 + k*256 + (j-2)*128 + l*4
//   196608  code rings of warps 7..15
// Both table halves start on a 64 KB boundary, so the address of an entry is the constant word
// (half | l*4) with the code byte dropped into bits 8..15: one byte-permute instruction per gather.
//
// Code bytes: a warp owns a contiguous run of rows and a ring of 32 slots of 128 bytes, slot
// (row & 31) holding the row's bytes of the current slice, so lane l finds its four codes in word
// l of the slot (bank l again).  The bytes are requested with 16-byte cp.async pieces, each piece
// kLead steps before the first lane needs it: the eight lanes 8k..8k+7 use their 32-byte sector of
// row u in steps u+8k .. u+8k+7, so that sector is requested in step u+8k-kLead.  A lane reads its
// word two steps before it uses it; with kLead = 22 a piece lands at least two steps after the last
// read of the slot's previous row and is complete six steps before its first read.
//
// Rows outside the warp's run (while the chain fills and drains) are walked like the others with
// whatever bytes the slot holds: every byte is a valid table index, their sums travel only along
// their own diagonal, and nothing of them is stored.
#pragma once
#include "lut_core.cuh"

namespace ojx {

constexpr uint32_t kChAcc = 1024, kChXs = 28672, kChRingLo = 36864, kChTab = 65536, kChRingHi = 196608;
constexpr int kChRingBytes = 4096, kChLoWarps = 7;
static_assert(kChAcc + kAccRows * 4 == kChXs && kChXs + kXsFloats * 4 == kChRingLo, "front area");
static_assert(kChRingLo + kChLoWarps * kChRingBytes == kChTab, "rings of the first warps end at the table");
static_assert(kChRingHi + (kWarps - kChLoWarps) * kChRingBytes == kChAcc + sizeof(CoreSmem), "whole dynamic area");
static_assert(kChTab + kSliceGroups * 256 * 4 == kChRingHi, "table");

__device__ __forceinline__ uint32_t ch_prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
template <int OFF>
__device__ __forceinline__ float ch_lds_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1+%2];" : "=f"(v) : "r"(addr), "n"(OFF));
    return v;
}
__device__ __forceinline__ uint32_t ch_lds_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

template <int D>
struct ChainWalker {
    static constexpr int SG = slice_groups<D>();
    static constexpr int kSlots = 32;
    static constexpr int kSlotBytes = 128;
    static constexpr int kLead = 22;
    static constexpr int kPrologue = 24;  // kLead rounded up to the request cadence of four steps
    static_assert(kSlots * kSlotBytes == kChRingBytes, "ring");
    static_assert(SG <= 128 && SG % 16 == 0, "a slice is at most 32 lanes x 4 groups");

    unsigned char* const raw;  // start of the dynamic shared memory (shared address 1024)
    const uint8_t* base;       // code row 0 of the work item
    const int n, G;
    const int warp, lane, nslices;

    __device__ ChainWalker(unsigned char* raw_, const uint8_t* base_, int n_, int G_)
        : raw(raw_), base(base_), n(n_), G(G_), warp(threadIdx.x >> 5), lane(threadIdx.x & 31),
          nslices((G_ + SG - 1) / SG) {}

    template <class T>
    __device__ __forceinline__ T* at(uint32_t shared_addr) const { return reinterpret_cast<T*>(raw + (shared_addr - kChAcc)); }
    __device__ __forceinline__ float* acc() const { return at<float>(kChAcc); }
    __device__ __forceinline__ float* table() const { return at<float>(kChTab); }
    __device__ __forceinline__ int* ring_hi_ints() const { return at<int>(kChRingHi); }

    // The walker needs whole 16-byte pieces of every row, four groups per lane and the layout above.
    __device__ static __forceinline__ bool usable(const unsigned char* raw, const uint8_t* codes, const float* codebook, int G) {
        return D <= 16 && (G & 15) == 0 && ((reinterpret_cast<uintptr_t>(codes) & 15) == 0) &&
               ((reinterpret_cast<uintptr_t>(codebook) & 7) == 0) &&
               static_cast<uint32_t>(__cvta_generic_to_shared(raw)) == kChAcc;
    }

    // Table slice of groups [g0, g0 + ng): entry (k, j, l) = sum_d x[(g0+4l+j)*D + d] * cb[k*D + d], d ascending,
    // separate multiply and add (the arithmetic of RowWalker::build_slice, so the same bits).  A thread keeps the
    // activations of its four groups in registers and runs over the centroids, whose coordinates every lane of a
    // warp reads from the same address.  `xr` holds this thread's share of the slice's activations, loaded before
    // the barrier that precedes the build (load_x).
    static constexpr int kXPerThread = kXsFloats / kThreads;
    __device__ __forceinline__ void load_x(int g0, int ng, const XLoad& xl, float (&xr)[kXPerThread]) const {
#pragma unroll
        for (int q = 0; q < kXPerThread; ++q) {
            const int i = threadIdx.x + q * kThreads;
            xr[q] = 0.0f;
            if (i < ng * D) {
                const int d = i / ng, pos = i - d * ng;
                xr[q] = xl((g0 + pos) * D + d);
            }
        }
    }
    // Centroids of a warp: warp w builds the entries of centroids w, w+16, ..., 16 rows of D floats = 32 lanes x D/2
    // floats.  Every lane loads its D/2 floats once per work item; the build broadcasts them with shuffles, so its
    // loop has no global loads (a load per centroid from L2 cost about 700 clocks each under the code stream).
    static constexpr int kCbRegs = D / 2;
    static_assert(D % 4 == 0 && kCbRegs >= 2, "centroid pieces");
    __device__ __forceinline__ void load_centroids(const float* __restrict__ codebook, int Kcb, float (&cr)[kCbRegs]) const {
        const int flat = lane * kCbRegs;             // position in the warp's [16][D] array
        const int k = warp + kWarps * (flat / D);
        const float* src = codebook + (size_t)k * D + (flat % D);
#pragma unroll
        for (int r = 0; r < kCbRegs; r += 2) {
            float2 v = make_float2(0.0f, 0.0f);
            if (k < Kcb) v = __ldg(reinterpret_cast<const float2*>(src + r));
            cr[r] = v.x;
            cr[r + 1] = v.y;
        }
    }
    __device__ __forceinline__ void build_slice(int ng, const float (&xr)[kXPerThread], const float (&cr)[kCbRegs], int Kcb) const {
        float* xs = at<float>(kChXs);
#pragma unroll
        for (int q = 0; q < kXPerThread; ++q) {
            const int i = threadIdx.x + q * kThreads;
            if (i < ng * D) {
                const int d = i / ng, pos = i - d * ng;
                xs[d * SG + pos] = xr[q];
            }
        }
        __syncthreads();
        const int lpos = ng <= 64 ? (lane & 15) : lane;  // a slice of <= 64 groups is kept twice: lanes 16..31 mirror 0..15
        const bool mine = 4 * lpos < ng;
        float xg[4][D];
#pragma unroll
        for (int d = 0; d < D; ++d) {
            float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (mine) v = *reinterpret_cast<const float4*>(xs + d * SG + 4 * lpos);
            xg[0][d] = v.x; xg[1][d] = v.y; xg[2][d] = v.z; xg[3][d] = v.w;
        }
        float* out = table() + lane;
        if (ng <= 64) {
            // both halves of the warp hold the same groups: each half computes every second centroid and writes
            // the entry into both copies (its own lane's bank and the mirror lane's)
            float* mir = table() + (lane ^ 16);
            const int h = lane >> 4;
#pragma unroll 2
            for (int ii = 0; ii < 128 / kWarps; ++ii) {
                const int i = 2 * ii + h, k = warp + kWarps * i;
                float c[D];
#pragma unroll
                for (int d = 0; d < D; ++d) c[d] = __shfl_sync(0xffffffffu, cr[d % kCbRegs], 2 * i + (d >= kCbRegs ? 1 : 0));
                float dot[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    dot[j] = __fmul_rn(xg[j][0], c[0]);
#pragma unroll
                    for (int d = 1; d < D; ++d) dot[j] = __fadd_rn(dot[j], __fmul_rn(xg[j][d], c[d]));
                    if (k >= Kcb) dot[j] = 0.0f;
                }
                if (mine) {
                    out[k * 64] = dot[0];
                    out[k * 64 + 32] = dot[1];
                    out[k * 64 + 16384] = dot[2];
                    out[k * 64 + 16384 + 32] = dot[3];
                    mir[k * 64] = dot[0];
                    mir[k * 64 + 32] = dot[1];
                    mir[k * 64 + 16384] = dot[2];
                    mir[k * 64 + 16384 + 32] = dot[3];
                }
            }
            __syncthreads();
            return;
        }
#pragma unroll 2
        for (int i = 0; i < 256 / kWarps; ++i) {
            const int k = warp + kWarps * i;
            float c[D];
#pragma unroll
            for (int d = 0; d < D; ++d) c[d] = __shfl_sync(0xffffffffu, cr[d % kCbRegs], 2 * i + (d >= kCbRegs ? 1 : 0));
            float dot[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                dot[j] = __fmul_rn(xg[j][0], c[0]);
#pragma unroll
                for (int d = 1; d < D; ++d) dot[j] = __fadd_rn(dot[j], __fmul_rn(xg[j][d], c[d]));
                if (k >= Kcb) dot[j] = 0.0f;
            }
            if (mine) {
                out[k * 64] = dot[0];
                out[k * 64 + 32] = dot[1];
                out[k * 64 + 16384] = dot[2];
                out[k * 64 + 16384 + 32] = dot[3];
            }
        }
        __syncthreads();
    }

    struct Entries { float v0, v1, v2, v3; };
    __device__ __forceinline__ Entries gather(uint32_t w, uint32_t tb) const {
        Entries e;
        e.v0 = ch_lds_f32<0>(ch_prmt(w, tb, 0x7604));
        e.v1 = ch_lds_f32<128>(ch_prmt(w, tb, 0x7614));
        e.v2 = ch_lds_f32<65536>(ch_prmt(w, tb, 0x7624));
        e.v3 = ch_lds_f32<65536 + 128>(ch_prmt(w, tb, 0x7634));
        return e;
    }

    // How this lane takes part in the walk of one slice.  A slice of at most 64 groups needs only 16 lanes per
    // row, so the warp runs two chains (lanes 0..15 on the first part of its rows, lanes 16..31 on the rest); a
    // ring slot then holds one row of each chain in its two halves.
    struct Plan {
        int rb, nu, nu0, nact;     // first row and row count of the warp, rows of chain 0, lanes of a chain
        int pos, mine;             // place of the lane in its chain, chain of the lane
        uint32_t ring;
        // requests: the lane copies 16-byte piece (lane>>3)*2 + (lane&1) of a slot, rows four apart in time
        int k8, delta, rnu;
        bool piece_ok;
        const uint8_t* gpiece;
        uint32_t rpiece;
    };
    __device__ __forceinline__ Plan make_plan(int s, int W) const {
        Plan p;
        const int per = ((n + kWarps - 1) / kWarps + 3) & ~3;
        p.rb = min(n, warp * per);
        p.nu = min(n, p.rb + per) - p.rb;
        const bool half = W <= 64;
        p.nact = W >> 2;
        p.nu0 = half ? min(p.nu, (((p.nu + 1) >> 1) + 3) & ~3) : p.nu;
        p.pos = half ? (lane & 15) : lane;
        p.mine = half ? (lane >> 4) : 0;
        p.ring = warp < kChLoWarps ? kChRingLo + warp * kChRingBytes : kChRingHi + (warp - kChLoWarps) * kChRingBytes;
        const int piece = 2 * (lane >> 3) + (lane & 1);
        p.delta = (lane & 7) >> 1;
        p.k8 = half ? ((lane >> 3) & 1) * 8 : (lane >> 3) * 8;
        const int src_byte = half ? (piece & 3) * 16 : piece * 16;
        p.rnu = p.mine ? p.nu - p.nu0 : p.nu0;
        p.piece_ok = src_byte < W;
        p.gpiece = base + (size_t)(p.rb + (p.mine ? p.nu0 : 0)) * G + s * SG + src_byte;
        p.rpiece = p.ring + piece * 16;
        return p;
    }
    __device__ __forceinline__ void request(const Plan& p, int t) const {
        const int u = t + kLead - p.k8 + p.delta;
        if (p.piece_ok && (unsigned)u < (unsigned)p.rnu) {
            const uint32_t dst = p.rpiece + (u & (kSlots - 1)) * kSlotBytes;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(p.gpiece + (size_t)u * G) : "memory");
        }
        cp_async_commit();
    }
    // First requests of a slice; the warp's ring is idle since its previous walk ended, so this runs before the
    // table build and the memory latency hides behind it.
    __device__ __forceinline__ void prefetch(int s, int W) const {
        const Plan p = make_plan(s, W);
#pragma unroll
        for (int t = -kPrologue; t < 0; t += 4) request(p, t);
    }

    // State of a lane between steps of the walk.
    struct Lane {
        uint32_t pr;        // shared address of the lane's word in the slot of the row it reads next
        uint32_t tb;        // table half 0 | lane*4
        Entries cur;        // entries of the step about to be added
        uint32_t wnext;     // code word of the step after
        float run;          // sum after the lane's last step
        // requests (incremental: row index, slot address, source address)
        int ru;
        unsigned rlim;
        uint32_t rdst;
        const uint8_t* rsrc;
        size_t rstride;
    };
    __device__ __forceinline__ uint32_t next_word(Lane& L) const {
        const uint32_t w = ch_lds_u32(L.pr);
        L.pr = (L.pr & ~(uint32_t)(kChRingBytes - 1)) | ((L.pr + kSlotBytes) & (kChRingBytes - 1));
        return w;
    }
    __device__ __forceinline__ void next_request(Lane& L) const {
        asm volatile(
            "{\n .reg .pred p;\n setp.lt.u32 p, %2, %3;\n @p cp.async.cg.shared.global [%0], [%1], 16;\n cp.async.commit_group;\n}\n" ::"r"(L.rdst),
            "l"(L.rsrc), "r"(L.ru), "r"(L.rlim)
            : "memory");
        L.ru += 4;
        L.rsrc += L.rstride;
        L.rdst = (L.rdst & ~(uint32_t)(kChRingBytes - 1)) | ((L.rdst + 4 * kSlotBytes) & (kChRingBytes - 1));
    }
    // Four steps.  `use` holds the sums the head lane starts the four rows from; the tail lane parks the four sums
    // that the previous four steps completed (rows ub .. ub+3, ub a multiple of 4; rows past the chain's last one
    // belong to nobody -- row counts of warps and chains are multiples of 4 except at the end of the work item).
    __device__ __forceinline__ void four_steps(Lane& L, const float4& use, bool head, uint32_t park_addr, int ub, unsigned park_lim) const {
        float hold[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t w2 = next_word(L);
            hold[i] = L.run;
            float sum = __shfl_up_sync(0xffffffffu, L.run, 1);
            if (head) sum = i == 0 ? use.x : i == 1 ? use.y : i == 2 ? use.z : use.w;
            const Entries nxt = gather(L.wnext, L.tb);
            sum = __fadd_rn(sum, L.cur.v0);
            sum = __fadd_rn(sum, L.cur.v1);
            sum = __fadd_rn(sum, L.cur.v2);
            sum = __fadd_rn(sum, L.cur.v3);
            L.run = sum;
            L.cur = nxt;
            L.wnext = w2;
        }
        asm volatile("{\n .reg .pred p;\n setp.lt.u32 p, %5, %6;\n @p st.shared.v4.f32 [%0], {%1, %2, %3, %4};\n}\n" ::"r"(park_addr),
                     "f"(hold[0]), "f"(hold[1]), "f"(hold[2]), "f"(hold[3]), "r"(ub), "r"(park_lim)
                     : "memory");
    }

    // Adds the entries of slice s (W groups) to the parked sums of this warp's rows (after prefetch(s, W)).
    template <bool FIRST>
    __device__ __forceinline__ void walk(int s, int W) const {
        const Plan p = make_plan(s, W);
        if (p.nu <= 0) {
            cp_async_wait<0>();
            return;
        }
        cp_async_wait<5>();
        __syncwarp();

        Lane L;
        L.tb = kChTab | (lane * 4);
        L.pr = p.ring + (((0 - p.pos) & (kSlots - 1)) * kSlotBytes) + lane * 4;
        L.cur = gather(next_word(L), L.tb);   // step 0
        L.wnext = next_word(L);               // step 1
        L.run = 0.0f;
        L.ru = kLead - p.k8 + p.delta;        // request of step 0
        L.rlim = p.piece_ok ? (unsigned)p.rnu : 0u;
        L.rdst = p.rpiece + (L.ru & (kSlots - 1)) * kSlotBytes;
        L.rsrc = p.gpiece + (ptrdiff_t)L.ru * G;
        L.rstride = (size_t)4 * G;
        const int mynu = p.mine ? p.nu - p.nu0 : p.nu0;
        const int row0 = p.rb + ((p.mine && mynu > 0) ? p.nu0 : 0);   // a multiple of 4: rb and nu0 are
        const float* accw = acc() + row0;
        const bool head = p.pos == 0;
        const bool tail = p.pos == p.nact - 1;
        const unsigned park_lim = tail ? (unsigned)mynu : 0u;
        int ub = -1 - p.pos;                                           // row whose sum `run` holds at step 0
        uint32_t park = kChAcc + (uint32_t)(row0 + ub) * 4;
        // sums to start rows step .. step+3 from (used by the head lane); reads past the warp's rows stay inside shared memory
        float4 sa = make_float4(0.0f, 0.0f, 0.0f, 0.0f), sb = sa;
        if (!FIRST) sa = *reinterpret_cast<const float4*>(accw);
        const int steps = p.nu0 + p.nact - 1;
        int t0 = 0;
        for (; t0 < steps; t0 += 8) {
            next_request(L);
            cp_async_wait<5>();
            __syncwarp();
            if (!FIRST) sb = *reinterpret_cast<const float4*>(accw + t0 + 4);
            four_steps(L, sa, head, park, ub, park_lim);
            next_request(L);
            cp_async_wait<5>();
            __syncwarp();
            if (!FIRST) sa = *reinterpret_cast<const float4*>(accw + t0 + 8);
            four_steps(L, sb, head, park + 16, ub + 4, park_lim);
            ub += 8;
            park += 32;
        }
        if (tail && (unsigned)ub < (unsigned)mynu) acc()[row0 + ub] = L.run;
        cp_async_wait<0>();
    }

    // Epilogue of the warp's own rows (ojasx_lut_cpu.cpp:178-182 then :117-127): y = (sum * scale + bias) + outlier
    // row sum, the outlier sum formed on its own from zero in entry order, multiply then add.  Each warp finishes
    // the rows it walked, so apart from the staging of x there is no CTA-wide barrier: the warp copies its row
    // pointers into its (idle) code ring, then takes 128 rows at a time -- all lanes multiply the entries of those
    // rows into the warp's part of the (idle) table area with coalesced loads of (col, val), then lane l adds the
    // products of rows l, l+32, l+64, l+96 in order.  `xsm` is x staged in shared memory by the CTA (null: x is read
    // from global memory).  Call after a __syncthreads() that follows the staging.
    static constexpr int kEpiRows = 128;
    static constexpr int kEpiProducts = 1536;   // products per pass of a warp: (128 KB - 32 KB of x) / 16 warps
    static constexpr int kEpiUnroll = 16;
    __device__ __forceinline__ float* epilogue_x() const { return table(); }
    // `rp_all`: the work item's row pointers (local row r at rp_all[r], n + 1 of them) already in shared memory, or null.
    template <class Store>
    __device__ __forceinline__ void warp_epilogue(const CsrView& csr, int row0, const float* __restrict__ scales,
                                                  const float* __restrict__ bias, const float* xsm, const XLoad& xl,
                                                  Store store, const int* rp_all = nullptr) const {
        const int per = ((n + kWarps - 1) / kWarps + 3) & ~3;
        const int rb = min(n, warp * per);
        const int nu = min(n, rb + per) - rb;
        if (nu <= 0) return;
        const bool has = csr.nnz > 0;
        const uint32_t ring = warp < kChLoWarps ? kChRingLo + warp * kChRingBytes : kChRingHi + (warp - kChLoWarps) * kChRingBytes;
        const int* rpw = rp_all ? rp_all + rb : at<int>(ring);       // nu + 1 <= 433 row pointers
        float* prod = table() + kCsrXFloats + warp * kEpiProducts;
        const float* accw = acc() + rb;
        if (has) {
            if (!rp_all) {
                int* w = at<int>(ring);
                for (int i = lane; i <= nu; i += 32) w[i] = csr.row_ptrs[row0 + rb + i];
                __syncwarp();
            }
            // ask for all of the warp's entries at once (a 128-byte line per lane and step), so that the loads
            // below find them on their way or in L2 instead of paying a DRAM round trip per batch
            for (int j = (rpw[0] & ~31) + lane * 32; j < rpw[nu]; j += 32 * 32) {
                asm volatile("prefetch.global.L2 [%0];" ::"l"(csr.cols + j));
                asm volatile("prefetch.global.L2 [%0];" ::"l"(csr.vals + j));
            }
        }
        for (int q0 = 0; q0 < nu; q0 += kEpiRows) {
            const int R = min(kEpiRows, nu - q0);
            float osum[kEpiRows / 32], sc[kEpiRows / 32], bs[kEpiRows / 32];
#pragma unroll
            for (int i = 0; i < kEpiRows / 32; ++i) {   // scale and bias of the rows: asked for now, used after the outlier sums
                const int row = q0 + lane + 32 * i;
                osum[i] = 0.0f;
                sc[i] = (scales && row < q0 + R) ? scales[row0 + rb + row] : 1.0f;
                bs[i] = (bias && row < q0 + R) ? bias[row0 + rb + row] : 0.0f;
            }
            if (has) {
                const int jb = rpw[q0], je = rpw[q0 + R];
                for (int jc = jb; jc < je; jc += kEpiProducts) {
                    const int ce = min(jc + kEpiProducts, je);
                    for (int base = jc + lane; base < ce; base += 32 * kEpiUnroll) {
                        int col[kEpiUnroll];
                        float val[kEpiUnroll];
#pragma unroll
                        for (int u = 0; u < kEpiUnroll; ++u) {
                            const int j = base + u * 32;
                            col[u] = j < ce ? csr.cols[j] : 0;
                            val[u] = j < ce ? csr.vals[j] : 0.0f;
                        }
#pragma unroll
                        for (int u = 0; u < kEpiUnroll; ++u) {
                            const int j = base + u * 32;
                            const float xv = xsm ? xsm[col[u]] : xl(col[u]);
                            if (j < ce) prod[j - jc] = __fmul_rn(val[u], xv);
                        }
                    }
                    __syncwarp();
#pragma unroll
                    for (int i = 0; i < kEpiRows / 32; ++i) {
                        const int row = q0 + lane + 32 * i;
                        if (row < q0 + R) {
                            const int sb = max(rpw[row], jc), se = min(rpw[row + 1], ce);
                            float a = osum[i];
                            for (int j = sb; j < se; ++j) a = __fadd_rn(a, prod[j - jc]);
                            osum[i] = a;
                        }
                    }
                    __syncwarp();
                }
            }
#pragma unroll
            for (int i = 0; i < kEpiRows / 32; ++i) {
                const int row = q0 + lane + 32 * i;
                if (row < q0 + R) {
                    const int m = row0 + rb + row;
                    float res = accw[row];
                    if (scales) res = __fmul_rn(res, sc[i]);
                    if (bias) res = __fadd_rn(res, bs[i]);
                    if (has) res = __fadd_rn(res, osum[i]);
                    store(m, res);
                }
            }
        }
    }

    // The same epilogue with the outlier entries streamed in by the copy engine.  Per-thread loads keep too few bytes
    // in flight for the (col, val) arrays (about 18 bytes per clock and SM); here every warp brings its own entries
    // into its part of the table area in chunks of kStreamChunk entries, two chunks in flight per warp (96 KB per SM),
    // and walks its rows in order as the chunks land: products in place, then one lane per row adds a row's products
    // in entry order.  A row whose entries end inside the chunk is finished and stored; the one row that straddles
    // the end of a chunk carries its partial sum into the next chunk (same additions in the same order).  Scale and
    // bias are applied to the parked sums beforehand, so finishing a row is one addition.
    // `jbw`, `jew`: row_ptrs of the warp's first row and of the row after its last one (read before the walk, so no
    // round trip is left in front of the first copy).  Needs x in shared memory and 16-byte aligned (col, val) arrays.
    static constexpr int kStreamChunk = kEpiProducts / 4;   // entries; a buffer is cols[kStreamChunk] | vals[kStreamChunk]
    __device__ __forceinline__ int warp_first_row() const { return min(n, warp * (((n + kWarps - 1) / kWarps + 3) & ~3)); }
    __device__ __forceinline__ int warp_row_count() const {
        const int per = ((n + kWarps - 1) / kWarps + 3) & ~3;
        return min(n, warp_first_row() + per) - warp_first_row();
    }
    __device__ static __forceinline__ bool stream_ok(const CsrView& csr) {
        return ((reinterpret_cast<uintptr_t>(csr.cols) | reinterpret_cast<uintptr_t>(csr.vals)) & 15) == 0;
    }
    template <class Store>
    __device__ __forceinline__ void warp_epilogue_stream(const CsrView& csr, int row0, const float* __restrict__ scales,
                                                         const float* __restrict__ bias, const float* xsm, int jbw, int jew,
                                                         Store store) const {
        const int rb = warp_first_row(), nu = warp_row_count();
        if (nu <= 0) return;
        constexpr int CH = kStreamChunk;
        const uint32_t ring = warp < kChLoWarps ? kChRingLo + warp * kChRingBytes : kChRingHi + (warp - kChLoWarps) * kChRingBytes;
        int* rpw = at<int>(ring);
        float* accw = acc() + rb;
        float* region = table() + kCsrXFloats + warp * kEpiProducts;
        unsigned char* bars = at<unsigned char>(kChXs) + warp * 16;   // the activation area is idle until the next table build
        const int jc0 = jbw & ~3;
        const int nch = max(1, (jew - jc0 + CH - 1) / CH);
        auto issue = [&](int c) {   // lane 0
            const int jc = jc0 + c * CH;
            int cnt = min(CH, (jew - jc + 3) & ~3);
            cnt = max(0, min(cnt, (csr.nnz - jc) & ~3));   // never past the end of the arrays: the last entries come by plain loads
            float* buf = region + (c & 1) * 2 * CH;
            void* bar = bars + (c & 1) * 8;
            bulk_expect(bar, (unsigned)cnt * 8u);
            if (cnt > 0) {
                bulk_copy_add(bar, buf, csr.cols + jc, (unsigned)cnt * 4u);
                bulk_copy_add(bar, buf + CH, csr.vals + jc, (unsigned)cnt * 4u);
            }
        };
        if (lane == 0) {
            bulk_bar_init(bars);
            bulk_bar_init(bars + 8);
        }
        // row pointers of the warp's rows into its idle code ring; scale and bias onto the parked sums
        for (int i0 = lane; i0 <= nu; i0 += 32 * 8) {
            int v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = i0 + 32 * u <= nu ? csr.row_ptrs[row0 + rb + i0 + 32 * u] : 0;
#pragma unroll
            for (int u = 0; u < 8; ++u) if (i0 + 32 * u <= nu) rpw[i0 + 32 * u] = v[u];
        }
        __syncwarp();
        // Normally the entries of 32 consecutive rows fit a buffer (384 entries are 12 per row): then a chunk is exactly
        // the entries of the next 32 rows, every lane finishes one whole row per chunk and nothing straddles.
        const int nblk = (nu + 31) >> 5;
        bool fits = true;
        for (int k = lane; k < nblk; k += 32) fits = fits && (rpw[min(32 * k + 32, nu)] - (rpw[32 * k] & ~3)) <= CH;
        fits = __all_sync(0xffffffffu, fits);
        auto count_of = [&](int k, int& jc) {   // entries the copy engine brings for block k, from entry jc on
            jc = rpw[32 * k] & ~3;
            const int want = (rpw[min(32 * k + 32, nu)] - jc + 3) & ~3;
            return max(0, min(want, (csr.nnz - jc) & ~3));
        };
        auto issue_block = [&](int k) {   // lane 0
            int jc;
            const int cnt = count_of(k, jc);
            float* buf = region + (k & 1) * 2 * CH;
            void* bar = bars + (k & 1) * 8;
            bulk_expect(bar, (unsigned)cnt * 8u);
            if (cnt > 0) {
                bulk_copy_add(bar, buf, csr.cols + jc, (unsigned)cnt * 4u);
                bulk_copy_add(bar, buf + CH, csr.vals + jc, (unsigned)cnt * 4u);
            }
        };
        if (lane == 0) {   // the first two chunks are on their way while scale and bias are applied
            if (fits) {
                issue_block(0);
                if (nblk > 1) issue_block(1);
            } else {       // a block of rows with more entries than a buffer: fixed-size chunks, rows finished as their entries land
                issue(0);
                if (nch > 1) issue(1);
            }
        }
        if (scales || bias) {
            for (int i0 = lane; i0 < nu; i0 += 32 * 8) {
                float sc[8], bs[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int r = i0 + 32 * u;
                    sc[u] = (scales && r < nu) ? scales[row0 + rb + r] : 1.0f;
                    bs[u] = (bias && r < nu) ? bias[row0 + rb + r] : 0.0f;
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int r = i0 + 32 * u;
                    if (r < nu) {
                        float res = accw[r];
                        if (scales) res = __fmul_rn(res, sc[u]);
                        if (bias) res = __fadd_rn(res, bs[u]);
                        accw[r] = res;
                    }
                }
            }
        }
        __syncwarp();
        if (fits) {
            for (int k = 0; k < nblk; ++k) {
                const int r = 32 * k + lane, ee = rpw[min(32 * k + 32, nu)];
                int jc;
                const int got = count_of(k, jc);
                int* cols = reinterpret_cast<int*>(region + (k & 1) * 2 * CH);
                float* vals = region + (k & 1) * 2 * CH + CH;
                if (lane < 4 && jc + got + lane < ee) {   // entries the copy left out because the arrays end inside their 16-byte piece
                    cols[got + lane] = csr.cols[jc + got + lane];
                    vals[got + lane] = csr.vals[jc + got + lane];
                }
                bulk_copy_wait(bars + (k & 1) * 8, (unsigned)((k >> 1) & 1));
                __syncwarp();
                const int m = ee - jc;
#pragma unroll 4
                for (int i = lane; i < m; i += 32) vals[i] = __fmul_rn(vals[i], xsm[cols[i]]);
                __syncwarp();
                if (r < nu) {
                    float a = 0.0f;
                    for (int j = rpw[r]; j < rpw[r + 1]; ++j) a = __fadd_rn(a, vals[j - jc]);
                    store(row0 + rb + r, __fadd_rn(accw[r], a));
                }
                __syncwarp();
                if (lane == 0 && k + 2 < nblk) issue_block(k + 2);
            }
            __syncwarp();
            if (lane == 0) {
                bulk_bar_inval(bars);
                bulk_bar_inval(bars + 8);
            }
            return;
        }
        __syncwarp();
        int cur = 0;             // first row not finished yet
        float carry = 0.0f;      // partial outlier sum of row `cur` when it began in an earlier chunk
        bool has_carry = false;
        for (int c = 0; c < nch; ++c) {
            const int jc = jc0 + c * CH, ce = min(jc + CH, jew);
            int* cols = reinterpret_cast<int*>(region + (c & 1) * 2 * CH);
            float* vals = region + (c & 1) * 2 * CH + CH;
            {   // entries the copy left out because the arrays end inside their 16-byte piece
                const int got = max(0, min(min(CH, (jew - jc + 3) & ~3), (csr.nnz - jc) & ~3));
                const int j = jc + got + lane;
                if (lane < 4 && j < ce) {
                    cols[got + lane] = csr.cols[j];
                    vals[got + lane] = csr.vals[j];
                }
            }
            bulk_copy_wait(bars + (c & 1) * 8, (unsigned)((c >> 1) & 1));
            __syncwarp();
            const int m = ce - jc;
#pragma unroll 4
            for (int i = lane; i < m; i += 32) vals[i] = __fmul_rn(vals[i], xsm[cols[i]]);
            __syncwarp();
            for (;;) {
                const int r = cur + lane;
                const bool complete = r < nu && rpw[r + 1] <= ce;
                const int cnt = __popc(__ballot_sync(0xffffffffu, complete));
                if (complete) {
                    float a = (lane == 0 && has_carry) ? carry : 0.0f;
                    for (int j = max(rpw[r], jc); j < rpw[r + 1]; ++j) a = __fadd_rn(a, vals[j - jc]);
                    store(row0 + rb + r, __fadd_rn(accw[r], a));
                }
                if (cnt == 32) {
                    cur += 32;
                    has_carry = false;
                    continue;
                }
                float a = (cnt == 0 && has_carry) ? carry : 0.0f;
                if (lane == cnt && r < nu)
                    for (int j = max(rpw[r], jc); j < ce; ++j) a = __fadd_rn(a, vals[j - jc]);
                carry = __shfl_sync(0xffffffffu, a, cnt);
                has_carry = true;
                cur += cnt;
                break;
            }
            __syncwarp();
            if (lane == 0 && c + 2 < nch) issue(c + 2);
        }
        __syncwarp();
        if (lane == 0) {
            bulk_bar_inval(bars);
            bulk_bar_inval(bars + 8);
        }
    }

    // The same with table slices that were built beforehand (unlike run(), this form ends with a __syncthreads()): `images` holds, for every slice, the 128 KB image of the
    // table area (the layout above, a slice of at most 64 groups stored twice), so a slice is brought in by ONE bulk copy
    // of the copy engine instead of being computed.  `before_last` runs once the last slice's table is in.  The mbarrier sits in the activation area, which this form does
    // not use.
    static constexpr int kImageFloats = kSliceGroups * 256;
    template <class F>
    __device__ void run_prebuilt(const float* __restrict__ images, F before_last) const {
        void* bar = at<void>(kChXs);
        if (threadIdx.x == 0) bulk_bar_init(bar);
        for (int s = 0; s < nslices; ++s) {
            const int g0 = s * SG, ng = min(SG, G - g0);
            __syncthreads();  // every warp has left the previous slice's table; the barrier is initialised
            prefetch(s, ng);
            if (threadIdx.x == 0) bulk_copy_issue(bar, table(), images + (size_t)s * kImageFloats, (unsigned)(kImageFloats * sizeof(float)));
            bulk_copy_wait(bar, (unsigned)(s & 1));
            if (s == nslices - 1) before_last();
            if (s == 0) walk<true>(s, ng);
            else walk<false>(s, ng);
        }
        __syncthreads();   // walks over (the caller needs this barrier too); the barrier is set up afresh by the next call
        if (threadIdx.x == 0) bulk_bar_inval(bar);
    }

    // Leaves acc()[lr] = sum_{g<G} LUT_x[g, code[lr, g]] for lr < n.  All threads of the CTA must call it; on
    // return a __syncthreads() has NOT yet been executed.  `before_last` runs once, after the table of the last
    // slice is built.
    template <class F>
    __device__ void run(const XLoad& xl, const float* __restrict__ codebook, int Kcb, F before_last) const {
        float cr[kCbRegs];
        load_centroids(codebook, Kcb, cr);
        for (int s = 0; s < nslices; ++s) {
            const int g0 = s * SG, ng = min(SG, G - g0);
            float xr[kXPerThread];
            load_x(g0, ng, xl, xr);
            __syncthreads();  // every warp has left the previous slice's table and activations
            prefetch(s, ng);
            build_slice(ng, xr, cr, Kcb);
            if (s == nslices - 1) before_last();
            if (s == 0) walk<true>(s, ng);
            else walk<false>(s, ng);
        }
    }
};

}  // namespace ojx
