// Core of the split-manifold LUT path: build an fp32 lookup-table slice in shared memory and
// accumulate, for a set of code rows, sum_g LUT[g, code[row, g]] in ascending g with one fp32
// accumulator per row -- the evaluation order of the reference's CPU kernel
// (split_manifold_lut_experiment/native/src/ojasx_lut_cpu.cpp:93-100 for the table,
// :161-175 for the row sum), so results are bit-identical to it.
//
// Shape of the computation on one SM (one 512-thread CTA, all 227 KB of shared memory; two
// 256-thread CTAs with half-size tables were measured and were not faster):
//   * the table of one token is G*256 fp32 and does not fit, so the group axis is cut into
//     slices of <= 128 groups (128 KB); slices are processed in ascending order and the
//     per-row accumulators are parked in shared memory between slices, which keeps the
//     summation order of a row strictly g = 0..G-1;
//   * inside a slice each warp owns 32-row blocks; lane l walks row l of the block, so the
//     row sum stays sequential; code bytes arrive through a per-warp 4-stage cp.async ring
//     of 32 rows x 32 bytes, loaded as coalesced 16-byte pieces and read back as two
//     conflict-free 128-bit shared loads per lane;
//   * the only CTA-wide barriers are around the table build of each slice; the code stream
//     of a warp runs ahead across slice boundaries.
#pragma once
#include "common.cuh"

namespace ojx {

constexpr int kThreads = 512;
constexpr int kCtasPerSm = 1;
constexpr int kWarps = kThreads / 32;
constexpr int kSliceGroups = 128;            // table slice: 128 groups x 256 entries x 4 B = 128 KB
constexpr int kXsFloats = kSliceGroups * 16; // x slice staging (block_dim <= 16 at 128 groups)
constexpr int kAccRows = 6912;               // rows per work item that can park an accumulator
constexpr int kChunk = 32;                   // code bytes per row per ring stage
constexpr int kStages = 4;
constexpr int kStageBytes = 32 * kChunk;     // 32 rows x 32 bytes

struct alignas(16) CoreSmem {
    float lut[kSliceGroups * 256];
    float acc[kAccRows];
    float xs[kXsFloats];
    uint8_t ring[kWarps * kStages * kStageBytes];
};
static_assert(kCtasPerSm * (sizeof(CoreSmem) + 1024) <= 228 * 1024, "shared memory budget of one SM");

// Rows of a work item: local row lr < n0 lives at base0 + lr*G, the rest at base1 + (lr-n0)*G
// (two ranges so that an expert's gate rows and up rows can share one table pass).
struct RowSet {
    const uint8_t* base0;
    const uint8_t* base1;
    int n0;
    int n;        // total local rows (<= kAccRows)
    int G;        // code bytes per row
    int aligned;  // 1: G % 16 == 0 and both bases 16-byte aligned -> cp.async path
};

// Reads element k of the activation vector as fp32; k >= K reads as zero (the reference's
// LUT GEMM pads the feature axis with zeros, ojasx_24x96/math_engine.py:166-171).
struct XLoad {
    const void* p;
    int K;
    int dtype;
    __device__ __forceinline__ float operator()(int k) const {
        if (k >= K) return 0.0f;
        if (dtype == OJX_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[k]);
        return reinterpret_cast<const float*>(p)[k];
    }
};

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, int src_bytes) {
    unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(gsrc), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

template <int D>
constexpr int slice_groups() { return (kXsFloats / D) < kSliceGroups ? (kXsFloats / D) : kSliceGroups; }

// ---- bulk copy of a contiguous run of global memory into shared memory by the copy engine (TMA), tracked by an
// mbarrier.  Used where a whole table slice is brought in at once: per-thread 16-byte copies keep too few bytes
// in flight per SM for that (about 18 bytes per clock measured), the copy engine does not have that limit.
// Every wait is bounded; a wait that runs out raises g_bulk_copy_timeout and carries on.
static __device__ int g_bulk_copy_timeout;   // one per translation unit; moe.cu is the one that copies tables this way
constexpr int kBulkSpin = 1 << 22;
__device__ __forceinline__ void bulk_bar_init(void* bar) {
    const unsigned a = static_cast<unsigned>(__cvta_generic_to_shared(bar));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(a) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// One thread, after a barrier that follows the last wait: the location may be initialised again afterwards.
__device__ __forceinline__ void bulk_bar_inval(void* bar) {
    const unsigned a = static_cast<unsigned>(__cvta_generic_to_shared(bar));
    asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(a) : "memory");
}
// One thread: global [src, src + bytes) -> shared dst; src, dst and bytes are multiples of 16, bytes < 1 MiB.
__device__ __forceinline__ void bulk_copy_issue(void* bar, void* dst, const void* src, unsigned bytes) {
    const unsigned b = static_cast<unsigned>(__cvta_generic_to_shared(bar));
    const unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(dst));
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // earlier generic accesses to dst come first
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(b), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(d), "l"(src),
                 "r"(bytes), "r"(b)
                 : "memory");
}
// The two halves of bulk_copy_issue, for several copies that complete one phase of a barrier: one bulk_expect with
// the sum of their sizes (zero completes the phase at once), then a bulk_copy_add per copy.
__device__ __forceinline__ void bulk_expect(void* bar, unsigned bytes) {
    const unsigned b = static_cast<unsigned>(__cvta_generic_to_shared(bar));
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // earlier generic accesses to the destinations come first
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(b), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_copy_add(void* bar, void* dst, const void* src, unsigned bytes) {
    const unsigned b = static_cast<unsigned>(__cvta_generic_to_shared(bar));
    const unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(dst));
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(d), "l"(src),
                 "r"(bytes), "r"(b)
                 : "memory");
}
__device__ __forceinline__ bool bulk_copy_wait(void* bar, unsigned parity) {
    const unsigned b = static_cast<unsigned>(__cvta_generic_to_shared(bar));
    for (int i = 0; i < kBulkSpin; ++i) {
        unsigned done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(b), "r"(parity)
            : "memory");
        if (done) return true;
    }
    atomicExch(&g_bulk_copy_timeout, 1);
    return false;
}

// Position of a warp's code stream: slice s, row block rb, 32-byte chunk cc inside the slice.
struct StagePos {
    int s, rb, cc;
    bool valid;
};

template <int D>
struct RowWalker {
    static constexpr int SG = slice_groups<D>();

    CoreSmem& sm;
    const RowSet rs;
    const int warp, lane, nrb, nslices;

    __device__ RowWalker(CoreSmem& sm_, const RowSet& rs_)
        : sm(sm_), rs(rs_), warp(threadIdx.x >> 5), lane(threadIdx.x & 31), nrb((rs_.n + 31) >> 5),
          nslices((rs_.G + SG - 1) / SG) {}

    __device__ __forceinline__ int slice_ng(int s) const { int r = rs.G - s * SG; return r < SG ? r : SG; }
    __device__ __forceinline__ int slice_chunks(int s) const { return (slice_ng(s) + kChunk - 1) / kChunk; }

    __device__ __forceinline__ StagePos first() const { return StagePos{0, warp, 0, warp < nrb && nslices > 0}; }
    __device__ __forceinline__ void advance(StagePos& p) const {
        if (!p.valid) return;
        if (++p.cc == slice_chunks(p.s)) {
            p.cc = 0;
            p.rb += kWarps;
            if (p.rb >= nrb) {
                p.rb = warp;
                if (++p.s == nslices) p.valid = false;
            }
        }
    }
    __device__ __forceinline__ const uint8_t* row_ptr(int lr) const {
        return lr < rs.n0 ? rs.base0 + (size_t)lr * rs.G : rs.base1 + (size_t)(lr - rs.n0) * rs.G;
    }

    // Fill ring slot `slot` of this warp with stage p (no-op when p is past the end).
    __device__ __forceinline__ void issue(const StagePos& p, int slot) const {
        if (p.valid) {
            uint8_t* st = sm.ring + (warp * kStages + slot) * kStageBytes;
            const int col_end = p.s * SG + slice_ng(p.s);
            const int col0 = p.s * SG + p.cc * kChunk;
            if (rs.aligned) {
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    const int piece = lane + 32 * q;
                    const int row = piece >> 1, half = piece & 1;
                    const int lr = p.rb * 32 + row;
                    const int col = col0 + half * 16;
                    const bool ok = lr < rs.n && col < col_end;
                    const uint8_t* src = ok ? row_ptr(lr) + col : rs.base0;
                    cp_async16(st + row * kChunk + ((half ^ ((row >> 2) & 1)) << 4), src, ok ? 16 : 0);
                }
            } else {
                const int lr = p.rb * 32 + lane;
                const uint8_t* src = lr < rs.n ? row_ptr(lr) : nullptr;
#pragma unroll 4
                for (int j = 0; j < kChunk; ++j) {
                    const int col = col0 + j;
                    const uint8_t v = (src && col < col_end) ? src[col] : (uint8_t)0;
                    st[lane * kChunk + ((((j >> 4) ^ ((lane >> 2) & 1)) << 4) | (j & 15))] = v;
                }
            }
        }
        cp_async_commit();
    }

    // Build table slice s: lut[gl*256 + k] = sum_d x[(g0+gl)*D + d] * cb[k*D + d], d ascending,
    // separate multiply and add (no fused multiply-add), as ojasx_lut_cpu.cpp:93-100 compiles
    // to on a baseline x86-64 build.  c[] holds this thread's centroid (tid & 255).  Four groups
    // are in flight per thread so that the four dependent add chains overlap.
    // (The packed fp32x2 forms of sm_100 are not used: ptxas contracts a packed mul.rn + add.rn
    // pair into one FMA -- 76 % of 8-term dot products changed in a direct test -- also when
    // they are spelled as a*b+(-0) and a*1+b, and that changes table values.)
    __device__ __forceinline__ void build_slice(int s, const XLoad& xl, const float (&c)[D], int Kcb,
                                                const float* __restrict__ prebuilt) const {
        constexpr int U = 4;
        const int g0 = s * SG, ng = slice_ng(s);
        if (prebuilt) {
            // The table of this activation vector was built once by lut_prebuild_kernel (same
            // arithmetic, so the same bits); this slice of it is one contiguous run: one bulk copy
            // (the mbarrier sits in the x staging area, which the prebuilt path does not use).
            if (threadIdx.x == 0) bulk_copy_issue(sm.xs, sm.lut, prebuilt + (size_t)g0 * 256, (unsigned)ng * 1024u);
            bulk_copy_wait(sm.xs, (unsigned)(s & 1));
            return;
        }
        for (int i = threadIdx.x; i < ng * D; i += kThreads) sm.xs[i] = xl(g0 * D + i);
        __syncthreads();
        const int kc = threadIdx.x & 255;
        const bool ok = kc < Kcb;
        constexpr int GS = kThreads / 256;  // groups advanced per step by the CTA's two halves
        for (int gb = threadIdx.x >> 8; gb < ng; gb += GS * U) {
            float dot[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int gl = gb + u * GS;
                const float4* xp = reinterpret_cast<const float4*>(sm.xs + (gl < ng ? gl : gb) * D);
#pragma unroll
                for (int q = 0; q < D / 4; ++q) {
                    const float4 xx = xp[q];
                    if (q == 0) dot[u] = __fmul_rn(xx.x, c[0]);
                    else dot[u] = __fadd_rn(dot[u], __fmul_rn(xx.x, c[4 * q]));
                    dot[u] = __fadd_rn(dot[u], __fmul_rn(xx.y, c[4 * q + 1]));
                    dot[u] = __fadd_rn(dot[u], __fmul_rn(xx.z, c[4 * q + 2]));
                    dot[u] = __fadd_rn(dot[u], __fmul_rn(xx.w, c[4 * q + 3]));
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int gl = gb + u * GS;
                if (gl < ng) sm.lut[gl * 256 + kc] = ok ? dot[u] : 0.0f;
            }
        }
        __syncthreads();
    }

    // Consume one landed stage: add the (up to 32) table entries of this lane's row, in order.
    __device__ __forceinline__ float consume(const StagePos& p, int slot, float acc) const {
        const uint8_t* st = sm.ring + (warp * kStages + slot) * kStageBytes + lane * kChunk;
        const int ng = slice_ng(p.s);
        const int swz = (lane >> 2) & 1;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int gl0 = p.cc * kChunk + h * 16;
            if (gl0 >= ng) break;
            const uint4 w = *reinterpret_cast<const uint4*>(st + ((h ^ swz) << 4));
            const float* lp = sm.lut + gl0 * 256;
            const unsigned ws[4] = {w.x, w.y, w.z, w.w};
            if (gl0 + 16 <= ng) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const unsigned code = (ws[j >> 2] >> ((j & 3) * 8)) & 0xffu;
                    acc = __fadd_rn(acc, lp[j * 256 + code]);
                }
            } else {
                const int nb = ng - gl0;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    if (j < nb) {
                        const unsigned code = (ws[j >> 2] >> ((j & 3) * 8)) & 0xffu;
                        acc = __fadd_rn(acc, lp[j * 256 + code]);
                    }
                }
            }
        }
        return acc;
    }

    // Leaves sm.acc[lr] = sum_{g<G} LUT_x[g, code[lr, g]] for lr < rs.n.  All threads of the
    // CTA must call it; on return a __syncthreads() has NOT yet been executed.  `before_last`
    // runs once, right after the table of the last slice is built (used to ask L2 for the data
    // the epilogue will want).
    template <class F>
    __device__ void run(const XLoad& xl, const float* __restrict__ codebook, int Kcb, F before_last,
                        const float* __restrict__ prebuilt = nullptr) const {
        float c[D];
        {
            const int kc = threadIdx.x & 255;
#pragma unroll
            for (int d = 0; d < D; ++d) c[d] = kc < Kcb ? codebook[kc * D + d] : 0.0f;
        }
        if (prebuilt && threadIdx.x == 0) bulk_bar_init(sm.xs);   // first used after the slice loop's barrier
        StagePos prod = first();
        StagePos cons = prod;
        int issued = 0, consumed = 0;
#pragma unroll
        for (int i = 0; i < kStages - 1; ++i) {
            issue(prod, issued % kStages);
            advance(prod);
            ++issued;
        }
        for (int s = 0; s < nslices; ++s) {
            __syncthreads();  // every warp has left the previous slice's table (and sm.xs)
            build_slice(s, xl, c, Kcb, prebuilt);
            if (s == nslices - 1) before_last();
            const int nch = slice_chunks(s);
            for (int rb = warp; rb < nrb; rb += kWarps) {
                const int lr = rb * 32 + lane;
                float acc = s == 0 ? 0.0f : sm.acc[lr];
                for (int cc = 0; cc < nch; ++cc) {
                    cp_async_wait<kStages - 2>();
                    __syncwarp();
                    issue(prod, issued % kStages);
                    advance(prod);
                    ++issued;
                    acc = consume(cons, consumed % kStages, acc);
                    advance(cons);
                    ++consumed;
                }
                sm.acc[lr] = acc;
            }
        }
        cp_async_wait<0>();
        if (prebuilt) {   // the barrier is set up afresh by the next call
            __syncthreads();
            if (threadIdx.x == 0) bulk_bar_inval(sm.xs);
        }
    }
};

// Whole table of one activation vector, built once and shared by every work item that uses that
// vector (the routed experts of a token): out[t, g, k] with the arithmetic of build_slice.
// grid = (ceil(G / 16), n_vectors), 256 threads (thread = centroid).
template <int D>
__device__ __forceinline__ void lut_prebuild_block(const void* __restrict__ x, int io_dtype, int K, int G,
                                                   const float* __restrict__ codebook, int Kcb, float* __restrict__ out,
                                                   int gx, int t, float* xs /* shared, 16 * D floats */) {
    const int g0 = gx * 16, ng = min(16, G - g0), kc = threadIdx.x;
    const size_t esz = io_dtype == OJX_BF16 ? 2 : 4;
    const XLoad xl{static_cast<const char*>(x) + (size_t)t * K * esz, K, io_dtype};
    for (int i = threadIdx.x; i < ng * D; i += 256) xs[i] = xl(g0 * D + i);
    float c[D];
#pragma unroll
    for (int d = 0; d < D; ++d) c[d] = kc < Kcb ? codebook[kc * D + d] : 0.0f;
    __syncthreads();
    float* o = out + ((size_t)t * G + g0) * 256 + kc;
    for (int gl = 0; gl < ng; ++gl) {
        const float* xg = xs + gl * D;
        float dot = __fmul_rn(xg[0], c[0]);
#pragma unroll
        for (int d = 1; d < D; ++d) dot = __fadd_rn(dot, __fmul_rn(xg[d], c[d]));
        o[(size_t)gl * 256] = kc < Kcb ? dot : 0.0f;
    }
}

template <int D>
__global__ void __launch_bounds__(256) lut_prebuild_kernel(const void* __restrict__ x, int io_dtype, int K, int G,
                                                           const float* __restrict__ codebook, int Kcb,
                                                           float* __restrict__ out) {
    __shared__ float xs[16 * D];
    lut_prebuild_block<D>(x, io_dtype, K, G, codebook, Kcb, out, blockIdx.x, blockIdx.y, xs);
}

// CSR outlier row sums for the rows [row0, row0+n) of a work item, reference order
// (ojasx_lut_cpu.cpp:117-126): acc = 0; j ascending; acc += val * x[col], multiply then add.
// The products are independent of one another, so they are computed by all threads with
// coalesced loads of (col, val) and staged in the table area of shared memory (free once the
// row walk is over); only the short in-order additions run one row per thread.  Results land in
// sm.lut[oacc_off + lr].  Every thread of the CTA must call it, after a __syncthreads() that
// follows the row walk; it ends with a __syncthreads().
constexpr int kCsrOaccFloats = 8192;                                   // >= kAccRows
constexpr int kCsrXFloats = 8192;                                      // activations staged when K fits
constexpr int kCsrChunk = kSliceGroups * 256 - kCsrOaccFloats - kCsrXFloats;  // products per pass
constexpr int kCsrUnroll = 16;
static_assert(kCsrOaccFloats >= kAccRows, "outlier sums need one slot per row");
static_assert((kAccRows + 1) * sizeof(int) <= sizeof(CoreSmem::ring), "row pointers are staged in the ring area");

// Ask L2 for the CSR arrays of rows [row0, row0+n) (called before the row walk, so the data is
// near by the time the epilogue wants it).
__device__ __forceinline__ void csr_prefetch_l2(const CsrView& csr, int row0, int n) {
    const int jb = csr.row_ptrs[row0], je = csr.row_ptrs[row0 + n];
    for (int j = jb + threadIdx.x * 32; j < je; j += kThreads * 32) {
        asm volatile("prefetch.global.L2 [%0];" ::"l"(csr.cols + j));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(csr.vals + j));
    }
    for (int r = threadIdx.x * 32; r <= n; r += kThreads * 32) asm volatile("prefetch.global.L2 [%0];" ::"l"(csr.row_ptrs + row0 + r));
}

// `area` is a 128 KB region of shared memory that is idle after the row walk (the table), `rp` room for n + 1 ints.
__device__ __forceinline__ void csr_rows_to_area(float* area, int* rp, const CsrView& csr, int row0, int n, int oacc_off,
                                                 const XLoad& xl) {
    float* oacc = area + oacc_off;
    float* xsm = area + kCsrOaccFloats;
    float* prod = xsm + kCsrXFloats;
    const bool x_in_smem = xl.K <= kCsrXFloats;
    // loads first, stores after: the compiler cannot tell that the shared stores leave the global arrays alone
    for (int b0 = threadIdx.x; b0 <= n; b0 += kThreads * kCsrUnroll) {
        int v[kCsrUnroll];
#pragma unroll
        for (int u = 0; u < kCsrUnroll; ++u) {
            const int lr = b0 + u * kThreads;
            v[u] = lr <= n ? csr.row_ptrs[row0 + lr] : 0;
        }
#pragma unroll
        for (int u = 0; u < kCsrUnroll; ++u) {
            const int lr = b0 + u * kThreads;
            if (lr <= n) rp[lr] = v[u];
            if (lr < n) oacc[lr] = 0.0f;
        }
    }
    if (x_in_smem) {
        for (int b0 = threadIdx.x; b0 < xl.K; b0 += kThreads * kCsrUnroll) {
            float v[kCsrUnroll];
#pragma unroll
            for (int u = 0; u < kCsrUnroll; ++u) {
                const int k = b0 + u * kThreads;
                v[u] = k < xl.K ? xl(k) : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < kCsrUnroll; ++u) {
                const int k = b0 + u * kThreads;
                if (k < xl.K) xsm[k] = v[u];
            }
        }
    }
    __syncthreads();
    const int jb = rp[0], je = rp[n];
    for (int jc = jb; jc < je; jc += kCsrChunk) {
        const int ce = min(jc + kCsrChunk, je);
        for (int base = jc + threadIdx.x; base < ce; base += kThreads * kCsrUnroll) {
            int col[kCsrUnroll];
            float val[kCsrUnroll];
#pragma unroll
            for (int u = 0; u < kCsrUnroll; ++u) {
                const int j = base + u * kThreads;
                col[u] = j < ce ? csr.cols[j] : 0;
                val[u] = j < ce ? csr.vals[j] : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < kCsrUnroll; ++u) {
                const int j = base + u * kThreads;
                const float xv = x_in_smem ? xsm[col[u]] : xl(col[u]);
                if (j < ce) prod[j - jc] = __fmul_rn(val[u], xv);
            }
        }
        __syncthreads();
        for (int lr = threadIdx.x; lr < n; lr += kThreads) {
            const int s = max(rp[lr], jc), e = min(rp[lr + 1], ce);
            if (s < e) {
                float acc = oacc[lr];
                for (int j = s; j < e; ++j) acc = __fadd_rn(acc, prod[j - jc]);
                oacc[lr] = acc;
            }
        }
        __syncthreads();
    }
}

__device__ __forceinline__ void csr_rows_to_smem(CoreSmem& sm, const CsrView& csr, int row0, int n, int oacc_off,
                                                 const XLoad& xl) {
    // the code ring is idle between row walks
    csr_rows_to_area(sm.lut, reinterpret_cast<int*>(sm.ring), csr, row0, n, oacc_off, xl);
}

}  // namespace ojx
