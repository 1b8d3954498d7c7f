/*
 * oracle_port.c -- CPU restatement of the reference's split-manifold LUT path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker that the GPU path is compared with.
 * It is compiled into oracle/liboracle_port.so and loaded only by tests/,
 * __graft_entry__.smoke() and the cpu_baseline / "--impl reference" legs of bench.py.
 * The shipped library never links, loads or calls it.
 *
 * Parity pin: every function that restates reference code is checked bit-for-bit against
 * the reference's own library (oracle/_ref/libojasx_lut.so, compiled from the reference
 * sources with the reference Makefile's default flags) by tests/test_oracle_pin.py and
 * against the committed vectors under tests/golden/ (made by tests/golden/make_golden.py
 * from that same library).  Functions marked "restatement, unpinned in the reference"
 * have no reference implementation to be checked against; they are pinned against
 * torch-CPU formulas instead (same test file).
 *
 * Arithmetic is plain IEEE fp32, one operation per C statement, sequential order, and the
 * build uses -ffp-contract=off, so results do not depend on the host's FMA support.
 *
 * File:line citations are paths inside the reference project.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------------------
 * LUT build.  split_manifold_lut_experiment/native/src/ojasx_lut_cpu.cpp:18-102; the
 * branch that runs on x86-64 with default flags is the portable loop at :93-100:
 * dot = 0; for d: dot += x_g[d] * c[d]   (fp32, d ascending, separate multiply and add).
 * ---------------------------------------------------------------------------------- */
static void build_lut(const float* x, const float* codebook, int G, int D, int Kcb, float* lut)
{
    for (int g = 0; g < G; ++g) {
        const float* xg = x + (size_t)g * D;
        float* lg = lut + (size_t)g * Kcb;
        for (int k = 0; k < Kcb; ++k) {
            const float* c = codebook + (size_t)k * D;
            float dot = 0.0f;
            for (int d = 0; d < D; ++d) {
                float p = xg[d] * c[d];
                dot = dot + p;
            }
            lg[k] = dot;
        }
    }
}

API void oracle_build_lut(const float* x, const float* codebook, int G, int D, int Kcb, float* lut)
{
    build_lut(x, codebook, G, D, Kcb, lut);
}

/* Row gather: ojasx_lut_cpu.cpp:161-175.  One fp32 accumulator, g ascending.  (The
 * reference unrolls by 4 but keeps a single accumulator, so the order is unchanged.) */
static float gather_row(const float* lut, const uint8_t* code_row, int G, int Kcb)
{
    float sum = 0.0f;
    for (int g = 0; g < G; ++g) sum = sum + lut[(size_t)g * Kcb + code_row[g]];
    return sum;
}

/* CSR outlier row: ojasx_lut_cpu.cpp:117-126.  acc = 0; for j ascending: acc += val*x[col]. */
static float csr_row(const int* row_ptrs, const int* cols, const float* vals, int m, const float* x)
{
    float acc = 0.0f;
    for (int j = row_ptrs[m]; j < row_ptrs[m + 1]; ++j) {
        float p = vals[j] * x[cols[j]];
        acc = acc + p;
    }
    return acc;
}

/* ------------------------------------------------------------------------------------
 * Linear forward.  ojasx_lut_cpu.cpp:132-206 (forward_cpu) followed by :104-130
 * (forward_outliers_cpu; skipped when nnz == 0, :109).
 *   y[b,m] = (sum_g lut_b[g, codes[m,g]]) * scales[m] (+ bias[m]);  then  y[b,m] += csr_row.
 * G = in_features / block_dim (integer division, ojasx_lut.h:92).
 * scales == NULL means all ones (ojasx_lut.h:97), bias == NULL means no bias.
 * row_start/row_stop select output rows [row_start,row_stop); y is [batch, row_stop-row_start]
 * (the row-slice contract of ojasx_24x96/native/ojasx_backend_abi.h:97-111).
 * ---------------------------------------------------------------------------------- */
API int oracle_linear_forward(int in_features, int out_features, int block_dim, int codebook_size,
                              const float* codebook, const uint8_t* codes, const float* scales,
                              const float* bias, int nnz, const int* row_ptrs, const int* cols,
                              const float* vals, const float* x, float* y, int batch,
                              int row_start, int row_stop)
{
    if (!codebook || !codes || !x || !y) return -1;
    const int G = in_features / block_dim;
    const int Kcb = codebook_size;
    float* lut = (float*)malloc(sizeof(float) * (size_t)(G > 0 ? G : 1) * Kcb);
    if (!lut) return -3;
    const int rows = row_stop - row_start;
    for (int b = 0; b < batch; ++b) {
        const float* xb = x + (size_t)b * in_features;
        float* yb = y + (size_t)b * rows;
        build_lut(xb, codebook, G, block_dim, Kcb, lut);
        for (int m = row_start; m < row_stop; ++m) {
            float sum = gather_row(lut, codes + (size_t)m * G, G, Kcb);
            float res = sum * (scales ? scales[m] : 1.0f);
            if (bias) res = res + bias[m];
            yb[m - row_start] = res;
        }
    }
    if (nnz > 0 && row_ptrs && cols && vals) {
        for (int b = 0; b < batch; ++b) {
            const float* xb = x + (size_t)b * in_features;
            float* yb = y + (size_t)b * rows;
            for (int m = row_start; m < row_stop; ++m) {
                float acc = csr_row(row_ptrs, cols, vals, m, xb);
                yb[m - row_start] = yb[m - row_start] + acc;
            }
        }
    }
    free(lut);
    return 0;
}

/* fast_silu: ojasx_lut_cpu.cpp:209-211,  x / (1 + exp(-x)) with the C library's expf. */
static float silu(float v) { return v / (1.0f + expf(-v)); }

/* ------------------------------------------------------------------------------------
 * MoE forward, one token.  ojasx_lut_cpu.cpp:213-365.
 *   y = 0; lut_in from x once (:234-273); for each routed expert in caller order, skipping
 *   ids outside [0,E) and |w| < 1e-8 (:284-286):
 *     gate = (sum_g lut_in[g, gu[e, i, g]])     * gu_scale[e, i]          (:293-308)
 *     up   = (sum_g lut_in[g, gu[e, I+i, g]])   * gu_scale[e, I+i]        (:310-322)
 *     inter[i] = silu(gate) * up                                            (:325)
 *     lut_down from inter with down_codebook                                (:330-342)
 *     y[h] += ((sum_gi lut_down[gi, dn[e, h, gi]]) * dn_scale[e, h]) * w    (:348-363)
 *
 * Extension with no counterpart in the reference (restatement, unpinned in the reference):
 * optional CSR outliers on the expert matrices, composed exactly as the linear layer
 * composes them (ojasx_lut_cpu.cpp:104-130): the flattened gate_up matrix [E*2I, H] and the
 * flattened down matrix [E*H, I] each carry one CSR whose row r belongs to expert r/(2I)
 * (resp. r/H); the outlier row sum is added after the scale, before silu / the routing weight.
 * With both nnz == 0 the function is the reference's forward_cpu.
 * ---------------------------------------------------------------------------------- */
API int oracle_moe_forward(int E, int H, int I, int block_dim, int codebook_size,
                           const float* cb_in, const float* cb_down,
                           const uint8_t* gu_codes, const float* gu_scales,
                           const uint8_t* dn_codes, const float* dn_scales,
                           int gu_nnz, const int* gu_row_ptrs, const int* gu_cols, const float* gu_vals,
                           int dn_nnz, const int* dn_row_ptrs, const int* dn_cols, const float* dn_vals,
                           const float* x, const int* idx, const float* w, int k_active, float* y)
{
    if (!x || !idx || !w || !y) return -1;
    if (k_active <= 0) return 0;
    const int G = H / block_dim, Gi = I / block_dim, Kcb = codebook_size;
    for (int h = 0; h < H; ++h) y[h] = 0.0f;
    float* lut_in = (float*)malloc(sizeof(float) * (size_t)G * Kcb);
    float* lut_dn = (float*)malloc(sizeof(float) * (size_t)(Gi > 0 ? Gi : 1) * Kcb);
    float* inter = (float*)malloc(sizeof(float) * (size_t)I);
    if (!lut_in || !lut_dn || !inter) { free(lut_in); free(lut_dn); free(inter); return -3; }
    build_lut(x, cb_in, G, block_dim, Kcb, lut_in);
    for (int kk = 0; kk < k_active; ++kk) {
        const int e = idx[kk];
        const float we = w[kk];
        if (e < 0 || e >= E || fabsf(we) < 1e-8f) continue;
        const size_t gu_off = (size_t)e * 2 * I * G, gs_off = (size_t)e * 2 * I;
        for (int i = 0; i < I; ++i) {
            float gate = gather_row(lut_in, gu_codes + gu_off + (size_t)i * G, G, Kcb);
            gate = gate * (gu_scales ? gu_scales[gs_off + i] : 1.0f);
            float up = gather_row(lut_in, gu_codes + gu_off + (size_t)(I + i) * G, G, Kcb);
            up = up * (gu_scales ? gu_scales[gs_off + I + i] : 1.0f);
            if (gu_nnz > 0) {
                gate = gate + csr_row(gu_row_ptrs, gu_cols, gu_vals, (int)gs_off + i, x);
                up = up + csr_row(gu_row_ptrs, gu_cols, gu_vals, (int)gs_off + I + i, x);
            }
            inter[i] = silu(gate) * up;
        }
        build_lut(inter, cb_down, Gi, block_dim, Kcb, lut_dn);
        const size_t dn_off = (size_t)e * H * Gi, ds_off = (size_t)e * H;
        for (int h = 0; h < H; ++h) {
            float s = gather_row(lut_dn, dn_codes + dn_off + (size_t)h * Gi, Gi, Kcb);
            float eh = s * (dn_scales ? dn_scales[ds_off + h] : 1.0f);
            if (dn_nnz > 0) eh = eh + csr_row(dn_row_ptrs, dn_cols, dn_vals, (int)ds_off + h, inter);
            float contrib = eh * we;
            y[h] = y[h] + contrib;
        }
    }
    free(lut_in); free(lut_dn); free(inter);
    return 0;
}

/* ------------------------------------------------------------------------------------
 * Router (restatement, unpinned in the reference; formula from
 * split_manifold_lut_experiment/tools/run_full_48_layers_and_generate.py:172-175):
 *   logits = x W^T ; p = softmax(logits) ; (w, idx) = topk(p, k) ; w /= sum(w).
 * Fixed evaluation order, chosen so that a 32-lane warp can reproduce it bit for bit:
 *   logit[e]: 32 interleaved fp32 partial sums, partial[j] accumulates W[e,c]*x[c] for
 *             c = j, j+32, ... ascending (separate multiply and add), then the partials are
 *             combined by a butterfly: for off in 16,8,4,2,1: partial[j] += partial[j^off].
 *   softmax : m = max logit; q[e] = (float)exp((double)(logit[e]-m)); s = sum of q in
 *             ascending e (fp32); p[e] = q[e] / s.
 *   top-k   : k rounds of arg-max over p, ties to the lower index; w = p[idx];
 *             wsum = sum of the k weights in selection order; w[i] = w[i] / wsum.
 * ---------------------------------------------------------------------------------- */
static float dot32(const float* w, const float* x, int n)
{
    float part[32];
    for (int j = 0; j < 32; ++j) part[j] = 0.0f;
    for (int c = 0; c < n; ++c) {
        float p = w[c] * x[c];
        part[c & 31] = part[c & 31] + p;
    }
    for (int off = 16; off >= 1; off >>= 1) {
        float nxt[32];
        for (int j = 0; j < 32; ++j) nxt[j] = part[j] + part[j ^ off];
        memcpy(part, nxt, sizeof(part));
    }
    return part[0];
}

API int oracle_router_topk(const float* x, const float* Wr, int B, int H, int E, int k,
                           int* idx_out, float* w_out, float* probs_out /* may be NULL, [B,E] */)
{
    if (!x || !Wr || !idx_out || !w_out || k > E) return -1;
    float* p = (float*)malloc(sizeof(float) * (size_t)E);
    if (!p) return -3;
    for (int b = 0; b < B; ++b) {
        const float* xb = x + (size_t)b * H;
        float m = -INFINITY;
        for (int e = 0; e < E; ++e) {
            p[e] = dot32(Wr + (size_t)e * H, xb, H);
            if (p[e] > m) m = p[e];
        }
        float s = 0.0f;
        for (int e = 0; e < E; ++e) {
            p[e] = (float)exp((double)(p[e] - m));
            s = s + p[e];
        }
        for (int e = 0; e < E; ++e) p[e] = p[e] / s;
        if (probs_out) memcpy(probs_out + (size_t)b * E, p, sizeof(float) * (size_t)E);
        float wsum = 0.0f;
        for (int r = 0; r < k; ++r) {
            int best = -1;
            float bv = -INFINITY;
            for (int e = 0; e < E; ++e) {
                int taken = 0;
                for (int q = 0; q < r; ++q) if (idx_out[(size_t)b * k + q] == e) { taken = 1; break; }
                if (taken) continue;
                if (p[e] > bv) { bv = p[e]; best = e; }
            }
            idx_out[(size_t)b * k + r] = best;
            w_out[(size_t)b * k + r] = bv;
            wsum = wsum + bv;
        }
        for (int r = 0; r < k; ++r) w_out[(size_t)b * k + r] = w_out[(size_t)b * k + r] / wsum;
    }
    free(p);
    return 0;
}

/* ------------------------------------------------------------------------------------
 * Reference KV cache, as shipped (scalar int8 of each block's first coordinate).
 *   append : split_manifold_lut_experiment/native/src/ojasx_lut_kv_cache.cpp:16-65
 *   logits : ojasx_lut_kv_cache.cpp:67-108
 *   softmax: split_manifold_lut_experiment/native/src/ojasx_lut_c_api.cpp:178-191
 *   context: ojasx_lut_kv_cache.cpp:110-132
 * Codes/scales are caller-held arrays: k_codes,v_codes [T,G] uint8, k_scales,v_scales [T].
 * ---------------------------------------------------------------------------------- */
API void oracle_kv_legacy_append(const float* k, const float* v, int head_dim, int block_dim,
                                 uint8_t* k_code_row, uint8_t* v_code_row, float* k_scale, float* v_scale)
{
    const int G = head_dim / block_dim;
    const float* src[2] = {k, v};
    uint8_t* dst[2] = {k_code_row, v_code_row};
    float* sc[2] = {k_scale, v_scale};
    for (int s = 0; s < 2; ++s) {
        float mx = 1e-8f;
        for (int d = 0; d < head_dim; ++d) { float a = fabsf(src[s][d]); if (a > mx) mx = a; }
        float scale = mx / 127.0f;
        *sc[s] = scale;
        for (int g = 0; g < G; ++g) {
            float val = src[s][g * block_dim];
            int q = (int)roundf(val / scale);
            if (q > 127) q = 127;
            if (q < -128) q = -128;
            dst[s][g] = (uint8_t)(q + 128);
        }
    }
}

API void oracle_kv_legacy_attention(const float* q, int head_dim, int block_dim, int T,
                                    const uint8_t* k_codes, const uint8_t* v_codes,
                                    const float* k_scales, const float* v_scales,
                                    float scale_factor, float* out)
{
    if (T == 0) return;                                  /* ojasx_lut_c_api.cpp:173 */
    const int G = head_dim / block_dim, D = block_dim;
    if (scale_factor <= 0.0f) scale_factor = 1.0f / sqrtf((float)head_dim);
    float* lut = (float*)malloc(sizeof(float) * (size_t)G * 256);
    float* logit = (float*)malloc(sizeof(float) * (size_t)T);
    for (int g = 0; g < G; ++g)
        for (int c = 0; c < 256; ++c) lut[g * 256 + c] = q[g * D] * (float)(c - 128);
    for (int t = 0; t < T; ++t) {
        float s = 0.0f;
        for (int g = 0; g < G; ++g) s = s + lut[g * 256 + k_codes[(size_t)t * G + g]];
        float r = s * k_scales[t];
        logit[t] = r * scale_factor;
    }
    float mx = logit[0];
    for (int t = 1; t < T; ++t) if (logit[t] > mx) mx = logit[t];
    float sum = 0.0f;
    for (int t = 0; t < T; ++t) { logit[t] = expf(logit[t] - mx); sum = sum + logit[t]; }
    float inv = 1.0f / sum;
    for (int t = 0; t < T; ++t) logit[t] = logit[t] * inv;
    memset(out, 0, sizeof(float) * (size_t)head_dim);
    for (int t = 0; t < T; ++t) {
        float wgt = logit[t] * v_scales[t];
        if (wgt == 0.0f) continue;
        for (int g = 0; g < G; ++g) {
            float val = (float)((int)v_codes[(size_t)t * G + g] - 128) * wgt;
            out[g * D] = out[g * D] + val;
        }
    }
    free(lut); free(logit);
}

/* ------------------------------------------------------------------------------------
 * Codebook-VQ KV cache (restatement, unpinned in the reference: the reference allocates
 * k_codebook / v_codebook, ojasx_lut_kv_cache.h:33-35, but never reads them).
 *
 * Append: nearest centroid per block_dim-wide sub-vector, rule of
 * ojasx_24x96/codec.py:217-224 (_nearest): argmin_c ( |v|^2 - 2 v.C_c + |C_c|^2 ), first
 * minimum.  Fixed fp32 order: each of the three terms is a sequential sum over d
 * (separate multiply and add); dist = (vv - 2*vc) + cc.
 * ---------------------------------------------------------------------------------- */
API void oracle_kvq_encode(const float* vec, int head_dim, int block_dim, const float* codebook,
                           int Kcb, uint8_t* codes_out)
{
    const int G = head_dim / block_dim, D = block_dim;
    for (int g = 0; g < G; ++g) {
        const float* v = vec + g * D;
        float vv = 0.0f;
        for (int d = 0; d < D; ++d) { float p = v[d] * v[d]; vv = vv + p; }
        int best = 0;
        float bd = INFINITY;
        for (int c = 0; c < Kcb; ++c) {
            const float* cv = codebook + (size_t)c * D;
            float vc = 0.0f, cc = 0.0f;
            for (int d = 0; d < D; ++d) { float p = v[d] * cv[d]; vc = vc + p; }
            for (int d = 0; d < D; ++d) { float p = cv[d] * cv[d]; cc = cc + p; }
            float t = 2.0f * vc;
            float dist = vv - t;
            dist = dist + cc;
            if (dist < bd) { bd = dist; best = c; }
        }
        codes_out[g] = (uint8_t)best;
    }
}

/* Decode attention of one KV head against n_q query heads that share it (GQA), in fp64:
 * structure of ojasx_lut_kv_cache.cpp:86-107 (per-group LUT of q against the codebook, then
 * logit[t] = scale * sum_g lut[g, k_codes[t,g]]) and the exact online softmax of
 * ojasx_24x96/long_context.py:92-176 (running max m, normaliser l, accumulator O in fp64,
 * kv blocks of `kv_block` tokens, no causal mask at decode since every cached key precedes
 * the query).  V is codebook[v_code].  q is given in fp32 (already rounded from bf16 by the
 * caller when the bf16 path is being checked).  out is [n_q, head_dim] fp64. */
API void oracle_kvq_decode(const float* q, int n_q, int head_dim, int block_dim, int T,
                           const uint8_t* k_codes, const uint8_t* v_codes,
                           const float* k_cb, const float* v_cb, double scale, int kv_block,
                           double* out)
{
    const int G = head_dim / block_dim, D = block_dim;
    if (scale <= 0.0) scale = 1.0 / sqrt((double)head_dim);
    if (kv_block <= 0) kv_block = 256;
    double* lut = (double*)malloc(sizeof(double) * (size_t)G * 256);
    double* s = (double*)malloc(sizeof(double) * (size_t)kv_block);
    for (int h = 0; h < n_q; ++h) {
        const float* qh = q + (size_t)h * head_dim;
        double* oh = out + (size_t)h * head_dim;
        for (int g = 0; g < G; ++g)
            for (int c = 0; c < 256; ++c) {
                double dsum = 0.0;
                for (int d = 0; d < D; ++d) dsum += (double)qh[g * D + d] * (double)k_cb[(size_t)c * D + d];
                lut[g * 256 + c] = dsum;
            }
        double m = -INFINITY, l = 0.0;
        for (int d = 0; d < head_dim; ++d) oh[d] = 0.0;
        for (int t0 = 0; t0 < T; t0 += kv_block) {
            int n = T - t0 < kv_block ? T - t0 : kv_block;
            double mb = -INFINITY;
            for (int i = 0; i < n; ++i) {
                double acc = 0.0;
                for (int g = 0; g < G; ++g) acc += lut[g * 256 + k_codes[(size_t)(t0 + i) * G + g]];
                s[i] = acc * scale;
                if (s[i] > mb) mb = s[i];
            }
            double mn = m > mb ? m : mb;
            double alpha = isinf(m) ? 0.0 : exp(m - mn);
            l *= alpha;
            for (int d = 0; d < head_dim; ++d) oh[d] *= alpha;
            for (int i = 0; i < n; ++i) {
                double p = exp(s[i] - mn);
                l += p;
                const uint8_t* vc = v_codes + (size_t)(t0 + i) * G;
                for (int g = 0; g < G; ++g) {
                    const float* cv = v_cb + (size_t)vc[g] * D;
                    for (int d = 0; d < D; ++d) oh[g * D + d] += p * (double)cv[d];
                }
            }
            m = mn;
        }
        double ls = l > 0.0 ? l : 1.0;
        for (int d = 0; d < head_dim; ++d) oh[d] /= ls;
    }
    free(lut); free(s);
}

/* fp64 evaluation of the linear layer (no reference counterpart; used only to report how far
 * both the reference's fp32 order and the GPU are from the exact sum). */
API int oracle_linear_forward_f64(int in_features, int out_features, int block_dim, int codebook_size,
                                  const float* codebook, const uint8_t* codes, const float* scales,
                                  const float* bias, int nnz, const int* row_ptrs, const int* cols,
                                  const float* vals, const float* x, double* y, int batch)
{
    const int G = in_features / block_dim, D = block_dim, Kcb = codebook_size;
    double* lut = (double*)malloc(sizeof(double) * (size_t)(G > 0 ? G : 1) * Kcb);
    if (!lut) return -3;
    for (int b = 0; b < batch; ++b) {
        const float* xb = x + (size_t)b * in_features;
        for (int g = 0; g < G; ++g)
            for (int k = 0; k < Kcb; ++k) {
                double dsum = 0.0;
                for (int d = 0; d < D; ++d) dsum += (double)xb[g * D + d] * (double)codebook[(size_t)k * D + d];
                lut[(size_t)g * Kcb + k] = dsum;
            }
        for (int m = 0; m < out_features; ++m) {
            double sum = 0.0;
            for (int g = 0; g < G; ++g) sum += lut[(size_t)g * Kcb + codes[(size_t)m * G + g]];
            sum *= scales ? (double)scales[m] : 1.0;
            if (bias) sum += (double)bias[m];
            if (nnz > 0)
                for (int j = row_ptrs[m]; j < row_ptrs[m + 1]; ++j) sum += (double)vals[j] * (double)xb[cols[j]];
            y[(size_t)b * out_features + m] = sum;
        }
    }
    free(lut);
    return 0;
}
