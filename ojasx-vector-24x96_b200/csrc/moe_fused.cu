// Expert pass of the top-k MoE for batches of tokens: one work item is one routed expert with up to
// four of the tokens that routed to it, gate/up projection, SiLU gate and down projection fused.
// Replaces the per-token loops of SplitManifoldMoE::forward_cpu
// (split_manifold_lut_experiment/native/src/ojasx_lut_cpu.cpp:213-365) for every (token, expert)
// pair at once; results per pair do not depend on which other tokens share the work item.
//
// Why whole experts: an expert has only 2I + H code rows (1280 + 2560 at hidden 2560 / inter 640), so
// whatever is done once per work item -- bringing in lookup tables, filling and draining the lane
// chains, outlier epilogues, CTA barriers -- has to be spread over as many table gathers as possible.
//
// Row walk (same idea as ChainWalker in lut_chain.cuh, generalised): the 32 lanes of a warp form
// 32/LC chains of LC lanes; a lane owns four consecutive groups of the table slice and one bank of
// shared memory, so every gather instruction is one wavefront.  The running sum of a row travels
// from lane to lane inside a chain (one shuffle per step), which keeps the reference's summation
// order g = 0..G-1 with one fp32 accumulator per row (ojasx_lut_cpu.cpp:293-322, 348-363).  The
// chains of a warp are shared out between the C tokens of the work item (each token has its own
// table, all read the same code bytes: one row of code bytes serves C tokens) and, when C chains do
// not fill the warp, between R parts of the warp's rows.  LC * C * R = 32; a slice is 4*LC groups.
//
// Tables.  Gate/up: the table of a token depends only on the token, so it is built once per token
// by moe_prebuild (in 16-group blocks laid out so that 16-byte pieces go straight to their banks)
// and copied per slice with cp.async.  Down: the table of a pair depends on the pair's intermediate
// vector, which this work item has just produced in shared memory, so it is built in place.
#include "lut_chain.cuh"
#include "launch.h"
#include "handles.h"
#include "peer.cuh"

#include <cstdlib>

namespace ojx {

// ---- shared memory, by absolute shared-space address (the dynamic area must start at 1024):
//     1024  control words
//     1152  parked row sums f32[C][nAcc], then the intermediate vectors f32[C][I], then the code
//           rings of the warps that do not fit behind the table (only when C = 1)
//    65536  table (as in lut_chain.cuh: entry (code k, j, lane l) at 65536 + (j>>1)*65536 + k*256 + (j&1)*128 + l*4)
//   196608  code rings (32 slots of 128/C bytes per warp)
constexpr uint32_t kMcCtl = 1024, kMcAcc = 1152, kMcBack = 196608, kMcEnd = 233472;
constexpr int kMcBackBytes = (int)(kMcEnd - kMcBack);
constexpr int kMcLead = 22, kMcPrologue = 24;
constexpr size_t kMcSmemBytes = kMcEnd - 1024;
static_assert(kMcSmemBytes == sizeof(CoreSmem), "same dynamic shared memory size as the other table kernels");

__device__ int g_moe_fused_error;   // 1: the dynamic shared memory did not start at shared address 1024

struct McChunk { int expert, first, C, pad; };

// Where things live for a work item of C tokens.
struct McLayout {
    uint32_t acc, inter, ring;   // absolute shared addresses; ring = this warp's code ring
    int nAcc;                    // floats per token in the parked sums
};

__host__ __device__ inline int mc_ring_bytes(int C) { return 4096 / C; }
// Floats per token in the parked sums: the rows, room for the head lanes' reads past a warp's rows, and a
// remainder of 8 modulo 32 so that the C tokens' sums of one row sit in different banks.
__host__ __device__ inline int mc_nacc_for(int rows) {
    const int base = (rows + 3) / 4 * 4 + 64;
    return base + ((8 - base % 32) + 32) % 32;
}

// Front-area bytes needed for C tokens (host and device agree on the map).
__host__ __device__ inline uint32_t mc_front_end(int C, int nAcc, int I, uint32_t* inter_out, uint32_t* ring_front_out, int* n_back_out) {
    const uint32_t inter = kMcAcc + (uint32_t)C * nAcc * 4;
    const uint32_t after = inter + (uint32_t)C * I * 4;
    const int rb = mc_ring_bytes(C);
    int n_back = kMcBackBytes / rb;
    if (n_back > kWarps) n_back = kWarps;
    const uint32_t ring_front = (after + rb - 1) / rb * rb;    // rings wrap by address arithmetic: aligned to their size
    if (inter_out) *inter_out = inter;
    if (ring_front_out) *ring_front_out = ring_front;
    if (n_back_out) *n_back_out = n_back;
    return n_back == kWarps ? after : ring_front + (uint32_t)(kWarps - n_back) * rb;
}

struct McCtx {
    unsigned char* raw;     // dynamic shared memory (shared address 1024)
    const uint8_t* base;    // code row 0 of the matrix block walked
    int n, G;               // rows, code bytes per row
    uint64_t stream_policy; // L2 policy of the code bytes: each row is read once by a work item, so it should not push
                            // the tokens' tables (read by every expert a token routes to) out of L2
    McLayout L;
    template <class T>
    __device__ __forceinline__ T* at(uint32_t shared_addr) const { return reinterpret_cast<T*>(raw + (shared_addr - 1024)); }
    __device__ __forceinline__ float* table() const { return at<float>(kChTab); }
};

// Rows of a warp and of its parts.
struct McRows {
    int rb, nu, nuR;
    __device__ __forceinline__ McRows(int n, int R) {
        const int warp = threadIdx.x >> 5;
        const int per = ((n + kWarps - 1) / kWarps + 3) & ~3;
        rb = min(n, warp * per);
        nu = min(n, rb + per) - rb;
        nuR = R == 1 ? nu : ((((nu + R - 1) / R) + 3) & ~3);
    }
    __device__ __forceinline__ int part_rows(int r) const { return max(0, min(nuR, nu - r * nuR)); }
};

template <int C, int LC>
struct McMode {
    static_assert(C * LC <= 32 && 32 % (C * LC) == 0, "chains fill the warp");
    static constexpr int R = 32 / (C * LC);        // parts of the warp's rows
    static constexpr int W = 4 * LC;                // groups (code bytes) per row in a slice
    static constexpr int SLOT = R * W;              // bytes per ring slot (= 128 / C)
    static constexpr int RING = 32 * SLOT;
    static constexpr int PPP = W / 16;              // 16-byte pieces per part
    static constexpr int NPIECE = SLOT / 16;
};

// Code-byte requests of a lane: 16-byte piece `piece` of a slot, rows four apart in time.
template <int C, int LC>
struct McReq {
    using M = McMode<C, LC>;
    bool ok;
    int k8, delta, rnu;
    const uint8_t* gpiece;
    uint32_t rpiece;
    __device__ __forceinline__ McReq(const McCtx& X, const McRows& rows, int col0) {
        const int lane = threadIdx.x & 31;
        const int piece = 2 * (lane >> 3) + (lane & 1);
        delta = (lane & 7) >> 1;
        ok = piece < M::NPIECE;
        const int part = piece / M::PPP, sub = piece % M::PPP;
        k8 = (sub >> 1) * 8;                        // first lane of a chain that reads the piece's 32-byte sector
        rnu = ok ? rows.part_rows(part) : 0;
        gpiece = X.base + (size_t)(rows.rb + part * rows.nuR) * X.G + col0 + sub * 16;
        rpiece = X.L.ring + piece * 16;
    }
};

template <int C, int LC>
__device__ __forceinline__ void mc_prefetch(const McCtx& X, int col0) {
    using M = McMode<C, LC>;
    const McRows rows(X.n, M::R);
    const McReq<C, LC> q(X, rows, col0);
#pragma unroll
    for (int t = -kMcPrologue; t < 0; t += 4) {
        const int u = t + kMcLead - q.k8 + q.delta;
        if (q.ok && (unsigned)u < (unsigned)q.rnu) {
            const uint32_t dst = q.rpiece + (u & 31) * M::SLOT;
            asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(q.gpiece + (size_t)u * X.G), "l"(X.stream_policy) : "memory");
        }
        cp_async_commit();
    }
}

struct McEntries { float v0, v1, v2, v3; };
__device__ __forceinline__ McEntries mc_gather(uint32_t w, uint32_t tb) {
    McEntries e;
    e.v0 = ch_lds_f32<0>(ch_prmt(w, tb, 0x7604));
    e.v1 = ch_lds_f32<128>(ch_prmt(w, tb, 0x7614));
    e.v2 = ch_lds_f32<65536>(ch_prmt(w, tb, 0x7624));
    e.v3 = ch_lds_f32<65536 + 128>(ch_prmt(w, tb, 0x7634));
    return e;
}

// Adds the table entries of the slice that starts at code byte col0 to the parked sums of the warp's
// rows, for the C tokens of the work item (after mc_prefetch<C, LC>(X, col0) and with the slice's
// table in place).  FIRST: the sums start from zero.
template <int C, int LC, bool FIRST>
__device__ __forceinline__ void mc_walk(const McCtx& X, int col0) {
    using M = McMode<C, LC>;
    const int lane = threadIdx.x & 31;
    const McRows rows(X.n, M::R);
    if (rows.nu <= 0) {
        cp_async_wait<0>();
        return;
    }
    const McReq<C, LC> q(X, rows, col0);
    const int pos = lane % LC, cr = lane / LC, c = cr % C, r = cr / C;
    const int mynu = rows.part_rows(r);
    cp_async_wait<5>();
    __syncwarp();

    // lane state
    uint32_t pr = X.L.ring + (((0 - pos) & 31) * M::SLOT) + r * M::W + pos * 4;   // word of the row read next
    const uint32_t tb = kChTab | (lane * 4);
    auto next_word = [&]() {
        const uint32_t w = ch_lds_u32(pr);
        pr = (pr & ~(uint32_t)(M::RING - 1)) | ((pr + M::SLOT) & (M::RING - 1));
        return w;
    };
    McEntries cur = mc_gather(next_word(), tb);   // step 0
    uint32_t wnext = next_word();                 // step 1
    float run = 0.0f;
    int ru = kMcLead - q.k8 + q.delta;            // request of step 0
    const unsigned rlim = (unsigned)q.rnu;
    uint32_t rdst = q.rpiece + (ru & 31) * M::SLOT;
    const uint8_t* rsrc = q.gpiece + (ptrdiff_t)ru * X.G;
    const size_t rstride = (size_t)4 * X.G;
    const uint64_t pol = X.stream_policy;
    auto next_request = [&]() {
        asm volatile(
            "{\n .reg .pred p;\n setp.lt.u32 p, %2, %3;\n @p cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %4;\n cp.async.commit_group;\n}\n" ::"r"(rdst),
            "l"(rsrc), "r"(ru), "r"(rlim), "l"(pol)
            : "memory");
        ru += 4;
        rsrc += rstride;
        rdst = (rdst & ~(uint32_t)(M::RING - 1)) | ((rdst + 4 * M::SLOT) & (M::RING - 1));
    };
    const int row0 = rows.rb + (mynu > 0 ? r * rows.nuR : 0);
    const float* accw = X.at<float>(X.L.acc) + c * X.L.nAcc + row0;
    const bool head = pos == 0, tail = pos == LC - 1;
    const unsigned park_lim = tail ? (unsigned)mynu : 0u;
    int ub = -1 - pos;                             // row whose sum `run` holds at step 0
    uint32_t park = X.L.acc + (uint32_t)(c * X.L.nAcc + row0 + ub) * 4;
    auto four_steps = [&](const float4& use, uint32_t park_addr, int ubase) {
        float hold[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t w2 = next_word();
            hold[i] = run;
            float sum = __shfl_up_sync(0xffffffffu, run, 1);
            if (head) sum = i == 0 ? use.x : i == 1 ? use.y : i == 2 ? use.z : use.w;
            const McEntries nxt = mc_gather(wnext, tb);
            sum = __fadd_rn(sum, cur.v0);
            sum = __fadd_rn(sum, cur.v1);
            sum = __fadd_rn(sum, cur.v2);
            sum = __fadd_rn(sum, cur.v3);
            run = sum;
            cur = nxt;
            wnext = w2;
        }
        asm volatile("{\n .reg .pred p;\n setp.lt.u32 p, %5, %6;\n @p st.shared.v4.f32 [%0], {%1, %2, %3, %4};\n}\n" ::"r"(park_addr),
                     "f"(hold[0]), "f"(hold[1]), "f"(hold[2]), "f"(hold[3]), "r"(ubase), "r"(park_lim)
                     : "memory");
    };
    float4 sa = make_float4(0.0f, 0.0f, 0.0f, 0.0f), sb = sa;
    if (!FIRST) sa = *reinterpret_cast<const float4*>(accw);
    const int steps = rows.part_rows(0) + LC - 1;
    for (int t0 = 0; t0 < steps; t0 += 8) {
        next_request();
        cp_async_wait<5>();
        __syncwarp();
        if (!FIRST) sb = *reinterpret_cast<const float4*>(accw + t0 + 4);
        four_steps(sa, park, ub);
        next_request();
        cp_async_wait<5>();
        __syncwarp();
        if (!FIRST) sa = *reinterpret_cast<const float4*>(accw + t0 + 8);
        four_steps(sb, park + 16, ub + 4);
        ub += 8;
        park += 32;
    }
    if (tail && (unsigned)ub < (unsigned)mynu) X.at<float>(X.L.acc)[c * X.L.nAcc + row0 + ub] = run;
    cp_async_wait<0>();
}

// Copies the slice of the C tokens' prebuilt tables that starts at 16-group block blk0 into the table
// area.  tok = table of token mc_unit_token() of the work item, block layout of moe_prebuild.
// Unit u = lane & 7 is a run of four lanes = (chain, 16-group block of the chain); a thread copies the
// 16-byte pieces (code k, j) of its unit, 64 threads per unit and 16 pieces each.  Reads: 64 contiguous
// bytes per unit and instruction; writes: eight units = eight different 16-byte columns of a 128-byte row.
template <int C, int LC>
__device__ __forceinline__ int mc_unit_token() { return (int)(((threadIdx.x & 7) / (LC / 4)) % C); }
template <int C, int LC>
__device__ __forceinline__ void mc_copy_table(const float* tok, int blk0) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int u = lane & 7, bl = u % (LC / 4);
    const float* src = tok + (size_t)(blk0 + bl) * 4096;
#pragma unroll
    for (int it = 0; it < 16; ++it) {
        const int kj = it * 64 + warp * 4 + (lane >> 3);
        const int k = kj >> 2, j = kj & 3;
        const uint32_t dst = kChTab + (uint32_t)(j >> 1) * 65536u + (uint32_t)k * 256u + (uint32_t)(j & 1) * 128u + (uint32_t)u * 16u;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src + kj * 4) : "memory");
    }
    cp_async_commit();
}

// Centroids of a warp for mc_build_table: warp w builds the entries of centroids w, w+16, ...; the 16 x D
// floats are spread over the lanes (D/2 each) and broadcast with shuffles inside the build loop.
template <int D>
__device__ __forceinline__ void mc_load_centroids(const float* __restrict__ codebook, int Kcb, float (&cbreg)[D / 2]) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int flat = lane * (D / 2);
    const int k = warp + kWarps * (flat / D);
    const float* src = codebook + (size_t)k * D + (flat % D);
#pragma unroll
    for (int q = 0; q < D / 2; q += 2) {
        float2 v = make_float2(0.0f, 0.0f);
        if (k < Kcb) v = __ldg(reinterpret_cast<const float2*>(src + q));
        cbreg[q] = v.x;
        cbreg[q + 1] = v.y;
    }
}

// Builds the slice of the C tokens' tables that starts at group g0 from activations held in shared
// memory (xs: f32 [C][K], K = row length): entry (k, j, lane) = sum_d x[(g0 + 4*pos + j)*D + d] * cb[k*D + d],
// d ascending, separate multiply and add (ojasx_lut_cpu.cpp:330-342 compiles to that on baseline x86-64).
// The R parts of a warp need the same entries: part r computes every R-th centroid and writes all copies.
template <int D, int C, int LC>
__device__ __forceinline__ void mc_build_table(const McCtx& X, const float* xs, int K, int g0, const float* __restrict__ codebook, int Kcb) {
    using M = McMode<C, LC>;
    constexpr int kCbRegs = D / 2;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float cbreg[kCbRegs];
    mc_load_centroids<D>(codebook, Kcb, cbreg);
    const int pos = lane % LC, cr = lane / LC, c = cr % C, r = cr / C;
    float xg[4][D];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float4* xp = reinterpret_cast<const float4*>(xs + (size_t)c * K + (size_t)(g0 + 4 * pos + j) * D);
#pragma unroll
        for (int q = 0; q < D / 4; ++q) {
            const float4 v = xp[q];
            xg[j][4 * q] = v.x; xg[j][4 * q + 1] = v.y; xg[j][4 * q + 2] = v.z; xg[j][4 * q + 3] = v.w;
        }
    }
    float* tab = X.table();
#pragma unroll 2
    for (int ii = 0; ii < 16 / M::R; ++ii) {
        const int i = M::R * ii + r, k = warp + kWarps * i;
        float cv[D];
#pragma unroll
        for (int d = 0; d < D; ++d) cv[d] = __shfl_sync(0xffffffffu, cbreg[d % kCbRegs], 2 * i + (d >= kCbRegs ? 1 : 0));
        float dot[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            dot[j] = __fmul_rn(xg[j][0], cv[0]);
#pragma unroll
            for (int d = 1; d < D; ++d) dot[j] = __fadd_rn(dot[j], __fmul_rn(xg[j][d], cv[d]));
            if (k >= Kcb) dot[j] = 0.0f;
        }
#pragma unroll
        for (int r2 = 0; r2 < M::R; ++r2) {
            float* out = tab + ((r2 * C + c) * LC + pos) + k * 64;
            out[0] = dot[0];
            out[32] = dot[1];
            out[16384] = dot[2];
            out[16384 + 32] = dot[3];
        }
    }
}

// Finishes the rows a warp walked, for the C tokens of the work item: res = sum * scale + (outlier row . x),
// the outlier sum formed on its own from zero in entry order, multiply then add (ojasx_lut_cpu.cpp:117-127
// applied to the expert's rows).  The entries (col, val) are loaded once and multiplied with the C tokens'
// activations.  rpw: the warp's row pointers (nu + 1 ints, filled by the caller when the matrix has
// outliers), prod: the warp's product scratch (nprod floats, shared out between the tokens), xsm: the
// activations in shared memory, token c at xsm + c * xstride.  Rows go to `store(c, row_in_block, value)`.
template <int C, class Store>
__device__ __forceinline__ void mc_epilogue(const McCtx& X, const CsrView& csr, size_t absrow0,
                                            const float* __restrict__ scales, const float* xsm, int xstride,
                                            const int* rpw, float* prod, int nprod, Store store) {
    constexpr int kRows = 128, kUnroll = 16;
    const int lane = threadIdx.x & 31;
    const McRows rows(X.n, 1);
    if (rows.nu <= 0) return;
    const bool has = csr.nnz > 0;
    const int np = (nprod / C) & ~3;            // products per token and pass
    const float* accw = X.at<float>(X.L.acc) + rows.rb;
    for (int q0 = 0; q0 < rows.nu; q0 += kRows) {
        const int Rn = min(kRows, rows.nu - q0);
        float osum[C][kRows / 32];
#pragma unroll
        for (int c = 0; c < C; ++c)
#pragma unroll
            for (int i = 0; i < kRows / 32; ++i) osum[c][i] = 0.0f;
        if (has) {
            const int jb = rpw[q0], je = rpw[q0 + Rn];
            for (int jc = jb; jc < je; jc += np) {
                const int ce = min(jc + np, je);
                for (int base = jc + lane; base < ce; base += 32 * kUnroll) {
                    int col[kUnroll];
                    float val[kUnroll];
#pragma unroll
                    for (int u = 0; u < kUnroll; ++u) {
                        const int j = base + u * 32;
                        col[u] = j < ce ? csr.cols[j] : 0;
                        val[u] = j < ce ? csr.vals[j] : 0.0f;
                    }
#pragma unroll
                    for (int u = 0; u < kUnroll; ++u) {
                        const int j = base + u * 32;
                        if (j < ce) {
#pragma unroll
                            for (int c = 0; c < C; ++c) prod[c * np + j - jc] = __fmul_rn(val[u], xsm[c * xstride + col[u]]);
                        }
                    }
                }
                __syncwarp();
#pragma unroll
                for (int i = 0; i < kRows / 32; ++i) {
                    const int row = q0 + lane + 32 * i;
                    if (row < q0 + Rn) {
                        const int sb = max(rpw[row], jc), se = min(rpw[row + 1], ce);
#pragma unroll
                        for (int c = 0; c < C; ++c) {
                            float a = osum[c][i];
                            for (int j = sb; j < se; ++j) a = __fadd_rn(a, prod[c * np + j - jc]);
                            osum[c][i] = a;
                        }
                    }
                }
                __syncwarp();
            }
        }
#pragma unroll
        for (int i = 0; i < kRows / 32; ++i) {
            const int row = q0 + lane + 32 * i;
            if (row < q0 + Rn) {
                const float sc = scales ? scales[absrow0 + rows.rb + row] : 1.0f;
#pragma unroll
                for (int c = 0; c < C; ++c) {
                    float res = accw[c * X.L.nAcc + row];
                    if (scales) res = __fmul_rn(res, sc);
                    if (has) res = __fadd_rn(res, osum[c][i]);
                    store(c, rows.rb + row, res);
                }
            }
        }
    }
}

// Asks L2 for the 16-group blocks [blk0, blk0 + nblk) of the C tokens' prebuilt tables (the slice that will be
// copied after the walk that is about to start), 128 bytes per thread and step.  tok_of(c): table of token c.
template <class TokOf>
__device__ __forceinline__ void mc_table_to_l2(int C, int blk0, int nblk, TokOf tok_of) {
    const int lines = C * nblk * 128;   // a block is 16 KB
    for (int id = threadIdx.x; id < lines; id += kThreads) {
        const int tb = id >> 7, line = id & 127;
        const int c = tb / nblk, bl = tb - c * nblk;
        const float* p = tok_of(c) + (size_t)(blk0 + bl) * 4096 + line * 32;
        asm volatile("prefetch.global.L2::evict_last [%0];" ::"l"(p));
    }
}

__device__ __forceinline__ float mc_silu(float v) {
    // v / (1 + exp(-v)), ojasx_lut_cpu.cpp:209-211; exp in double, rounded once
    const float e = (float)exp((double)(-v));
    return __fdiv_rn(v, __fadd_rn(1.0f, e));
}

// Lanes per chain for the next slice: the widest chain that the C tokens leave room for and the
// remaining groups (a multiple of 16) fill.
__device__ __forceinline__ int mc_pick_lc(int C, int remaining_groups) {
    int lc = C == 1 ? 16 : 32 / C;
    if (lc > 16) lc = 16;
    while (4 * lc > remaining_groups) lc >>= 1;
    return lc;
}

#define MC_DISPATCH(C_, LC_, ...)                                   \
    do {                                                            \
        if ((C_) == 4) {                                            \
            if ((LC_) == 8) { constexpr int MC = 4, ML = 8; __VA_ARGS__; } \
            else { constexpr int MC = 4, ML = 4; __VA_ARGS__; }            \
        } else if ((C_) == 2) {                                     \
            if ((LC_) == 16) { constexpr int MC = 2, ML = 16; __VA_ARGS__; } \
            else if ((LC_) == 8) { constexpr int MC = 2, ML = 8; __VA_ARGS__; } \
            else { constexpr int MC = 2, ML = 4; __VA_ARGS__; }            \
        } else {                                                    \
            if ((LC_) == 16) { constexpr int MC = 1, ML = 16; __VA_ARGS__; } \
            else if ((LC_) == 8) { constexpr int MC = 1, ML = 8; __VA_ARGS__; } \
            else { constexpr int MC = 1, ML = 4; __VA_ARGS__; }            \
        }                                                           \
    } while (0)

template <int D>
__global__ void __launch_bounds__(kThreads, 1) moe_fused_kernel(const __grid_constant__ MoeProblem P,
                                                                  const __grid_constant__ PeerLink link) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    if (static_cast<uint32_t>(__cvta_generic_to_shared(smem_raw)) != 1024u) {
        if (threadIdx.x == 0) atomicExch(&g_moe_fused_error, 1);
        return;
    }
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int* plan = P.plan;
    const int n_chunks = plan[0];
    int* counter = const_cast<int*>(plan) + 1;
    const int* sorted = plan + 4;
    const McChunk* chunks = reinterpret_cast<const McChunk*>(plan + 4 + P.n_tokens * P.k_active);
    const int H = P.H, I = P.I, G = P.G, Gi = P.Gi;
    const int nAcc = P.mc_nacc;
    const size_t esz = P.io_dtype == OJX_BF16 ? 2 : 4;
    McCtx X;
    X.raw = smem_raw;
    if (P.mc_debug & 64) asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(X.stream_policy));
    else asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(X.stream_policy));
    volatile int* ctl = X.at<volatile int>(kMcCtl);
    const int NB = G / 16;   // 16-group blocks per token table

    // Control words: ctl[0], ctl[1] = ids of the current and the next work item (alternating); ctl[8 + 8*slot ...] =
    // expert, chunk size and pair ids of the item in `slot`.  The next item is claimed, and its description
    // loaded, while the current one is in progress, so that no work item starts with a chain of global loads.
    auto load_desc = [&](int sl) {   // threads 0..3
        const int it = ctl[sl];
        if (it < n_chunks) {
            const McChunk ch = chunks[it];
            if (tid == 0) { ctl[8 + 8 * sl] = ch.expert; ctl[8 + 8 * sl + 1] = ch.C; }
            ctl[8 + 8 * sl + 2 + tid] = sorted[ch.first + (tid < ch.C ? tid : 0)];
        }
    };
    if (tid == 0) ctl[0] = atomicAdd(counter, 1);
    __syncthreads();
    if (tid < 4) load_desc(0);
    for (int slot = 0;; slot ^= 1) {
        __syncthreads();   // the description in `slot` is visible; every thread has left the previous work item
        const int item = ctl[slot];
        if (item >= n_chunks) break;
        const int expert = ctl[8 + 8 * slot], C = ctl[8 + 8 * slot + 1];
        if (tid == 0) ctl[slot ^ 1] = atomicAdd(counter, 1);
        auto pair_of = [&](int c) { return (int)ctl[8 + 8 * slot + 2 + c]; };
        auto token_of = [&](int c) { return (int)ctl[8 + 8 * slot + 2 + c] / P.k_active; };
        {
            uint32_t inter_a, ring_front;
            int n_back;
            mc_front_end(C, nAcc, I, &inter_a, &ring_front, &n_back);
            X.L.acc = kMcAcc;
            X.L.inter = inter_a;
            X.L.nAcc = nAcc;
            const int rbytes = mc_ring_bytes(C);
            X.L.ring = warp < n_back ? kMcBack + warp * rbytes : ring_front + (warp - n_back) * rbytes;
        }
        float* inter = X.at<float>(X.L.inter);

        // ------------------------------------------------------------ gate and up rows: [e*2I, (e+1)*2I)
        const size_t gu_row0 = (size_t)expert * 2 * I;
        X.base = P.gu_codes + gu_row0 * G;
        X.n = 2 * I;
        X.G = G;
        {
            bool first = true;
            for (int col = 0; col < G;) {
                const int LC = mc_pick_lc(C, G - col);
                MC_DISPATCH(C, LC, (mc_prefetch<MC, ML>(X, col)));
                __syncthreads();   // every warp has left the table area (previous slice, or the previous item's epilogue)
                if (!(P.mc_debug & 1)) MC_DISPATCH(C, LC, (mc_copy_table<MC, ML>(P.lut_in + (size_t)token_of(mc_unit_token<MC, ML>()) * NB * 4096, col / 16)));
                cp_async_wait<0>();
                __syncthreads();
                if (col + 4 * LC < G && !(P.mc_debug & 32)) {   // the next slice's tables towards L2 while this one is walked
                    const int ncol = col + 4 * LC;
                    mc_table_to_l2(C, ncol / 16, mc_pick_lc(C, G - ncol) / 4, [&](int c) { return P.lut_in + (size_t)token_of(c) * NB * 4096; });
                }
                if (P.mc_debug & 2) { cp_async_wait<0>(); }
                else if (first) MC_DISPATCH(C, LC, (mc_walk<MC, ML, true>(X, col)));
                else MC_DISPATCH(C, LC, (mc_walk<MC, ML, false>(X, col)));
                first = false;
                col += 4 * LC;
            }
        }
        __syncthreads();   // walks over: the table area is scratch now
        if (tid < 4) load_desc(slot ^ 1);

        // epilogue of the gate/up rows: activations of the C tokens into the table area, then every warp
        // finishes its rows in place (sum * scale + outliers), then inter = silu(gate) * up
        float* xarea = X.table();
        const int xfloats = C * H;
        const int nprod = ((32768 - xfloats) / kWarps) & ~31;
        float* prod = xarea + xfloats + warp * nprod;
        int* rpw = X.at<int>(X.L.ring);
        const McRows wr(2 * I, 1);
        if (P.gu_csr.nnz > 0) {
            if (P.io_dtype == OJX_F32 && (reinterpret_cast<uintptr_t>(P.x) & 15) == 0) {
                // 16 bytes per thread and step, every load of a thread in flight at once
                const int per_tok = H >> 2, total4 = C * per_tok;
                for (int b0 = tid; b0 < total4; b0 += kThreads * 4) {
                    float4 v[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int i4 = b0 + u * kThreads;
                        if (i4 < total4) {
                            const int c = i4 / per_tok, k4 = i4 - c * per_tok;
                            v[u] = reinterpret_cast<const float4*>(static_cast<const float*>(P.x) + (size_t)token_of(c) * H)[k4];
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int i4 = b0 + u * kThreads;
                        if (i4 < total4) reinterpret_cast<float4*>(xarea)[i4] = v[u];
                    }
                }
            } else {
                for (int idx = tid; idx < xfloats; idx += kThreads) {
                    const int c = idx / H, k = idx - c * H;
                    const XLoad xl{static_cast<const char*>(P.x) + (size_t)token_of(c) * H * esz, H, P.io_dtype};
                    xarea[idx] = xl(k);
                }
            }
            for (int i = lane; i <= wr.nu && wr.nu > 0; i += 32) rpw[i] = P.gu_csr.row_ptrs[gu_row0 + wr.rb + i];
            __syncthreads();
        }
        if (!(P.mc_debug & 8)) {
            float* acc0 = X.at<float>(X.L.acc);
            auto put = [&](int c, int row, float v) { acc0[c * nAcc + row] = v; };
            if (C == 4) mc_epilogue<4>(X, P.gu_csr, gu_row0, P.gu_scales, xarea, H, rpw, prod, nprod, put);
            else if (C == 2) mc_epilogue<2>(X, P.gu_csr, gu_row0, P.gu_scales, xarea, H, rpw, prod, nprod, put);
            else mc_epilogue<1>(X, P.gu_csr, gu_row0, P.gu_scales, xarea, H, rpw, prod, nprod, put);
        }
        __syncthreads();
        for (int idx = tid; idx < C * I; idx += kThreads) {
            const int c = idx / I, i = idx - c * I;
            const float* accc = X.at<float>(X.L.acc) + c * nAcc;
            float gate = accc[i], up = accc[I + i];
            if (P.gate_limit > 0.0f) {
                gate = fminf(gate, P.gate_limit);
                up = fminf(fmaxf(up, -P.gate_limit), P.gate_limit);
            }
            inter[idx] = __fmul_rn(mc_silu(gate), up);
        }

        // ------------------------------------------------------------ down rows: [e*H, (e+1)*H)
        const size_t dn_row0 = (size_t)expert * H;
        X.base = P.dn_codes + dn_row0 * Gi;
        X.n = H;
        X.G = Gi;
        {
            bool first = true;
            for (int col = 0; col < Gi;) {
                const int LC = mc_pick_lc(C, Gi - col);
                MC_DISPATCH(C, LC, (mc_prefetch<MC, ML>(X, col)));
                __syncthreads();   // inter is complete; every warp has left the table area
                if (!(P.mc_debug & 4)) MC_DISPATCH(C, LC, (mc_build_table<D, MC, ML>(X, inter, I, col, P.cb_down, P.Kcb)));
                __syncthreads();
                if (P.mc_debug & 2) { cp_async_wait<0>(); }
                else if (first) MC_DISPATCH(C, LC, (mc_walk<MC, ML, true>(X, col)));
                else MC_DISPATCH(C, LC, (mc_walk<MC, ML, false>(X, col)));
                first = false;
                col += 4 * LC;
            }
        }
        __syncthreads();
        {
            const int nprod2 = (32768 / kWarps) & ~31;
            float* prod2 = X.table() + warp * nprod2;
            const McRows wd(H, 1);
            if (P.dn_csr.nnz > 0) {
                for (int i = lane; i <= wd.nu && wd.nu > 0; i += 32) rpw[i] = P.dn_csr.row_ptrs[dn_row0 + wd.rb + i];
                __syncwarp();
            }
            if (!(P.mc_debug & 8)) {
                float* out[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) out[c] = P.expert_out + (size_t)pair_of(c) * H;
                auto put = [&](int c, int row, float v) { peer_store(link, out[c] + row, v); };
                if (C == 4) mc_epilogue<4>(X, P.dn_csr, dn_row0, P.dn_scales, inter, I, rpw, prod2, nprod2, put);
                else if (C == 2) mc_epilogue<2>(X, P.dn_csr, dn_row0, P.dn_scales, inter, I, rpw, prod2, nprod2, put);
                else mc_epilogue<1>(X, P.dn_csr, dn_row0, P.dn_scales, inter, I, rpw, prod2, nprod2, put);
            }
        }
        // the barrier at the top of the loop (and the one before the next table copy) separates this
        // epilogue from the next work item
    }
    peer_signal_when_last(link, gridDim.x);
}

// Work list of the fused kernel: the (token, expert) pairs this handle evaluates, sorted by expert, cut
// into chunks of 4, 2 and 1 pairs of one expert (the largest chunks first in the list, so that the CTAs
// that start last get the short ones).  plan[0] = chunks, plan[1] = work counter (zeroed), plan[4..] =
// sorted pair ids, then the chunks.  One CTA; counting sort on the local expert id.
__device__ __forceinline__ int block_exclusive_scan(int v, int* warp_tot /* [33] shared */, int* total) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    int inc = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, inc, off);
        if (lane >= off) inc += o;
    }
    __syncthreads();   // warp_tot may still be read from the previous scan
    if (lane == 31) warp_tot[wid] = inc;
    __syncthreads();
    if (wid == 0) {
        int t = lane < nwarp ? warp_tot[lane] : 0;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int o = __shfl_up_sync(0xffffffffu, t, off);
            if (lane >= off) t += o;
        }
        warp_tot[lane] = t;
    }
    __syncthreads();
    *total = warp_tot[nwarp - 1];
    return inc - v + (wid > 0 ? warp_tot[wid - 1] : 0);
}

__device__ __forceinline__ int plan_local_expert(const MoeProblem& P, int pair) {
    const int e = P.topk_idx[pair] - P.expert_offset;
    const float w = P.topk_w[pair];
    // ojasx_lut_cpu.cpp:284-286: ids outside the expert table and |w| < 1e-8 are skipped.
    return (e < 0 || e >= P.E || fabsf(w) < 1e-8f) ? -1 : e;
}

__global__ void __launch_bounds__(1024) moe_chunk_plan_kernel(const __grid_constant__ MoeProblem P, int* __restrict__ plan) {
    extern __shared__ int plan_smem[];
    int* cnt = plan_smem;            // [E] pairs per local expert
    int* start = plan_smem + P.E;    // [E] next free slot of the expert in the sorted list
    __shared__ int warp_tot[33];
    const int pairs = P.n_tokens * P.k_active;
    int* sorted = plan + 4;
    McChunk* chunks = reinterpret_cast<McChunk*>(plan + 4 + pairs);
    for (int e = threadIdx.x; e < P.E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = plan_local_expert(P, p);
        if (e >= 0) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    // every thread owns a contiguous run of experts
    const int per = (P.E + (int)blockDim.x - 1) / (int)blockDim.x;
    const int lo = min(P.E, (int)threadIdx.x * per), hi = min(P.E, lo + per);
    const int cmax = P.mc_cmax;
    int np = 0, n4 = 0, n2 = 0, n1 = 0;
    for (int e = lo; e < hi; ++e) {
        int c = cnt[e];
        np += c;
        if (cmax >= 4) { n4 += c >> 2; c &= 3; }
        if (cmax >= 2) { n2 += c >> 1; c &= 1; }
        n1 += c;
    }
    int tp, t4, t2, t1;
    int bp = block_exclusive_scan(np, warp_tot, &tp);
    int b4 = block_exclusive_scan(n4, warp_tot, &t4);
    int b2 = block_exclusive_scan(n2, warp_tot, &t2);
    int b1 = block_exclusive_scan(n1, warp_tot, &t1);
    for (int e = lo; e < hi; ++e) {
        int c = cnt[e], at = bp;
        start[e] = bp;
        bp += c;
        if (cmax >= 4) {
            for (int j = 0; j < (c >> 2); ++j) { chunks[b4++] = McChunk{e, at, 4, 0}; at += 4; }
            c &= 3;
        }
        if (cmax >= 2) {
            for (int j = 0; j < (c >> 1); ++j) { chunks[t4 + b2++] = McChunk{e, at, 2, 0}; at += 2; }
            c &= 1;
        }
        for (int j = 0; j < c; ++j) { chunks[t4 + t2 + b1++] = McChunk{e, at, 1, 0}; at += 1; }
    }
    if (threadIdx.x == 0) {
        plan[0] = t4 + t2 + t1;
        plan[1] = 0;
        plan[2] = tp;
        plan[3] = 0;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = plan_local_expert(P, p);
        if (e >= 0) sorted[atomicAdd(&start[e], 1)] = p;
    }
}

// Table of one activation vector in 16-group blocks: out[t][blk][k][j][i] = <x_t[group 16*blk + 4*i + j], cb[k]>
// with the arithmetic of RowWalker::build_slice (d ascending, separate multiply and add).  A 16-byte piece
// (k, j) holds the entries of four lanes of a chain, i.e. it goes to one bank column of the table area
// whatever the chain length.  grid = (G / 16, n_vectors), 256 threads (thread = centroid).
template <int D>
__device__ __forceinline__ void moe_prebuild_block(const void* __restrict__ x, int io_dtype, int K, int G,
                                                   const float* __restrict__ codebook, int Kcb, float* __restrict__ out,
                                                   int blk, int t, float* xs /* shared, 16 * D floats */) {
    const int kc = threadIdx.x;
    const size_t esz = io_dtype == OJX_BF16 ? 2 : 4;
    const XLoad xl{static_cast<const char*>(x) + (size_t)t * K * esz, K, io_dtype};
    for (int i = threadIdx.x; i < 16 * D; i += 256) xs[i] = xl(blk * 16 * D + i);
    float c[D];
#pragma unroll
    for (int d = 0; d < D; ++d) c[d] = kc < Kcb ? codebook[kc * D + d] : 0.0f;
    __syncthreads();
    float4* o = reinterpret_cast<float4*>(out + (((size_t)t * (G / 16) + blk) * 256 + kc) * 16);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float dot[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float* xg = xs + (4 * i + j) * D;
            float a = __fmul_rn(xg[0], c[0]);
#pragma unroll
            for (int d = 1; d < D; ++d) a = __fadd_rn(a, __fmul_rn(xg[d], c[d]));
            dot[i] = kc < Kcb ? a : 0.0f;
        }
        o[j] = make_float4(dot[0], dot[1], dot[2], dot[3]);
    }
}

template <int D>
__global__ void __launch_bounds__(256) moe_prebuild_kernel(const void* __restrict__ x, int io_dtype, int K, int G,
                                                           const float* __restrict__ codebook, int Kcb,
                                                           float* __restrict__ out) {
    __shared__ float xs[16 * D];
    moe_prebuild_block<D>(x, io_dtype, K, G, codebook, Kcb, out, blockIdx.x, blockIdx.y, xs);
}

// ------------------------------------------------------------------------------- host side
// Largest chunk (4, 2, 1) whose shared-memory map fits this shape; 0: the fused kernel does not apply.
int moe_fused_cmax(const MoeProblem& P) {
    if (P.D != 4 && P.D != 8 && P.D != 16) return 0;
    if (P.G <= 0 || P.Gi <= 0 || (P.G & 15) || (P.Gi & 15) || P.Kcb > 256) return 0;
    if ((reinterpret_cast<uintptr_t>(P.gu_codes) & 15) || (reinterpret_cast<uintptr_t>(P.dn_codes) & 15)) return 0;
    if ((reinterpret_cast<uintptr_t>(P.cb_down) & 7) || (P.I & 3) || (P.H & 3)) return 0;
    const int rows = P.H > 2 * P.I ? P.H : 2 * P.I;
    const int nAcc = mc_nacc_for(rows);
    const int per = round_up((rows + kWarps - 1) / kWarps, 4);
    int best = 0;
    for (int C = 1; C <= 4; C *= 2) {
        if (mc_front_end(C, nAcc, P.I, nullptr, nullptr, nullptr) > kChTab) break;
        if ((per + 1) * 4 > mc_ring_bytes(C)) break;                 // row pointers of a warp are staged in its ring
        if ((size_t)C * P.H > 16384) break;                          // activations of the chunk next to the product scratch
        best = C;
    }
    return best;
}

bool moe_fused_wanted(const MoeProblem& P) {
    // OJASX_B200_MOE_FUSED_MIN_PAIRS: routed pairs expected on this handle from which the whole-expert kernel
    // is used (read on every call so tests can switch paths).  Measured on B200 at hidden 2560 / inter 640 it
    // ties with the per-pair kernels at 2560 pairs and loses below that, so it is off unless asked for.
    const char* env = getenv("OJASX_B200_MOE_FUSED_MIN_PAIRS");
    const int g_fused_min_pairs = env ? atoi(env) : (1 << 30);
    if (!P.lut_in || !P.plan) return false;
    const long long pairs = (long long)P.n_tokens * P.k_active;
    const long long expect = P.E_total > P.E ? (pairs * P.E + P.E_total - 1) / P.E_total : pairs;
    if (expect < g_fused_min_pairs) return false;
    return moe_fused_cmax(P) > 0;
}

template <int D>
static int launch_moe_fused_t(MoeProblem P, cudaStream_t s, const PeerLink& link) {
    static thread_local bool opted[64] = {};
    int dev = 0;
    OJX_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !opted[dev]) {
        OJX_CUDA_TRY(cudaFuncSetAttribute(moe_fused_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMcSmemBytes));
        const size_t hs = sizeof(int) * 2 * 4096;
        OJX_CUDA_TRY(cudaFuncSetAttribute(moe_chunk_plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)hs));
        if (dev >= 0 && dev < 64) opted[dev] = true;
    }
    int launches = 0;
    if (P.E > 4096) return OJX_ERR_TOO_LARGE;
    moe_chunk_plan_kernel<<<1, 1024, sizeof(int) * 2 * (size_t)P.E, s>>>(P, const_cast<int*>(P.plan));
    OJX_CUDA_TRY(cudaGetLastError());
    ++launches;
    if (!P.lut_ready) {
        moe_prebuild_kernel<D><<<dim3(P.G / 16, P.n_tokens), 256, 0, s>>>(P.x, P.io_dtype, P.H, P.G, P.cb_in, P.Kcb,
                                                                          const_cast<float*>(P.lut_in));
        OJX_CUDA_TRY(cudaGetLastError());
        ++launches;
    }
    const long long pairs = (long long)P.n_tokens * P.k_active;
    const int sms = num_sms();
    const int grid = (int)(pairs < sms ? pairs : sms);
    moe_fused_kernel<D><<<grid, kThreads, kMcSmemBytes, s>>>(P, link);
    OJX_CUDA_TRY(cudaGetLastError());
    ++launches;
    count_launch(launches);
    return OJX_OK;
}

// Plan + (tables) + fused experts; the caller adds the combine pass.  P.lut_in must be in block layout
// when P.lut_ready is set.
int launch_moe_fused(MoeProblem P, cudaStream_t s, const PeerLink* lk) {
    const PeerLink none{};
    const PeerLink& link = lk ? *lk : none;
    P.mc_cmax = moe_fused_cmax(P);
    if (P.mc_cmax <= 0) return OJX_ERR_UNSUPPORTED;
    { const char* e = getenv("OJX_MC_DEBUG"); P.mc_debug = e ? atoi(e) : 0; const char* c = getenv("OJX_MC_CMAX"); if (c && atoi(c) < P.mc_cmax) P.mc_cmax = atoi(c); }
    const int rows = P.H > 2 * P.I ? P.H : 2 * P.I;
    P.mc_nacc = mc_nacc_for(rows);
    switch (P.D) {
        case 4: return launch_moe_fused_t<4>(P, s, link);
        case 8: return launch_moe_fused_t<8>(P, s, link);
        case 16: return launch_moe_fused_t<16>(P, s, link);
        default: return OJX_ERR_UNSUPPORTED;
    }
}

// The tables of the tokens in block layout, for callers that build them together with something else.
int launch_moe_prebuild_blocks(const void* x, int io_dtype, int n_tokens, int H, int D, const float* codebook, int Kcb,
                               float* out, cudaStream_t s) {
    const int G = H / D;
    if (G & 15) return OJX_ERR_UNSUPPORTED;
    switch (D) {
        case 4: moe_prebuild_kernel<4><<<dim3(G / 16, n_tokens), 256, 0, s>>>(x, io_dtype, H, G, codebook, Kcb, out); break;
        case 8: moe_prebuild_kernel<8><<<dim3(G / 16, n_tokens), 256, 0, s>>>(x, io_dtype, H, G, codebook, Kcb, out); break;
        case 16: moe_prebuild_kernel<16><<<dim3(G / 16, n_tokens), 256, 0, s>>>(x, io_dtype, H, G, codebook, Kcb, out); break;
        default: return OJX_ERR_UNSUPPORTED;
    }
    OJX_CUDA_TRY(cudaGetLastError());
    count_launch(1);
    return OJX_OK;
}

int take_moe_fused_error(int* out) {
    int v = 0, zero = 0;
    OJX_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_moe_fused_error, sizeof(int)));
    if (v) OJX_CUDA_TRY(cudaMemcpyToSymbol(g_moe_fused_error, &zero, sizeof(int)));
    *out = v;
    return OJX_OK;
}

}  // namespace ojx
