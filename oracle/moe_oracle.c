/*
 * moe_oracle.c: CPU restatement of the reference's arithmetic for the quantized MoE expert path.
 *
 * TEST INFRASTRUCTURE ONLY. Nothing in the product library links, loads or calls this file. The
 * parity tests, the smoke check and the CPU-baseline leg of the benchmark are its only users; they
 * use it as the checker, never as the thing measured or shipped.
 *
 * Parity pin: every function below is compared, on seeded inputs, with the reference's own code
 * compiled from its sources (the `_ref` recipe in this folder's Makefile) by tests/test_oracle_pin.py,
 * and with committed golden vectors produced by that code (tests/golden/). The W4 and activation-piece
 * functions have no reference counterpart and say so ("parity unpinned") where they are defined.
 *
 * Paths cited are relative to the reference project root.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_BLOCK 128u

static float f32_of_bits(uint32_t b) { float f; memcpy(&f, &b, 4); return f; }
static uint32_t bits_of_f32(float f) { uint32_t b; memcpy(&b, &f, 4); return b; }

/* ------------------------------------------------------------------ number formats */

/* bf16 -> f32: the 16 bits are the top half of the f32 (src/omega_blackwell_matmul.h:60). */
float orc_bf16_to_f32(uint16_t b) { return f32_of_bits((uint32_t)b << 16); }

/* f32 -> bf16, round to nearest even, NaN kept quiet (src/omega_blackwell_matmul.h:63-75). */
uint16_t orc_f32_to_bf16(float f) {
    uint32_t x = bits_of_f32(f);
    if ((x & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((x >> 16) | 0x0040u);
    return (uint16_t)((x + 0x7fffu + ((x >> 16) & 1u)) >> 16);
}

/* e4m3 decode: sign 7, exponent 6..3 (bias 7), mantissa 2..0; exponent 0 is m * 2^-9; 0x7f and 0xff
 * are NaN (src/omega_gpu_fp8_pack.c:15-22). */
float orc_e4m3_decode(uint8_t b) {
    const int e = (b >> 3) & 15, m = b & 7;
    const float s = (b & 0x80) ? -1.0f : 1.0f;
    if (e == 15 && m == 7) return NAN;
    if (e == 0) return s * (float)m * ldexpf(1.0f, -9);
    return s * (1.0f + (float)m / 8.0f) * ldexpf(1.0f, e - 7);
}

/* f32 -> e4m3, round to nearest even, saturating at 448 and never producing the NaN code
 * (src/omega_gpu_fp8_api.c:702-721). Written from the definition: pick the nearest of the 127
 * non-negative finite codes, ties to the even code. */
uint8_t orc_e4m3_encode(float v) {
    const uint8_t s = (bits_of_f32(v) >> 24) & 0x80u;
    const float a = fabsf(v);
    if (!(a < 448.0f)) return (uint8_t)(s | 0x7eu); /* NaN and anything at or past the top saturate */
    int e; (void)frexpf(a, &e); e -= 1;           /* a in [2^e, 2^(e+1)) for a > 0 */
    if (a == 0.0f || e < -6) e = -6;               /* subnormal grid: units of 2^-9 */
    const float unit = ldexpf(1.0f, e - 3);
    const float q = a / unit;                       /* exact: power-of-two division */
    float r = nearbyintf(q);                        /* default rounding mode: to nearest even */
    uint32_t code;
    if (e == -6 && r < 8.0f) code = (uint32_t)r;    /* subnormal codes 0..7 */
    else {
        if (r >= 16.0f) { r = 8.0f; e += 1; }
        code = ((uint32_t)(e + 7) << 3) | ((uint32_t)r - 8u);
    }
    if (code > 0x7eu) code = 0x7eu;
    return (uint8_t)(s | code);
}

/* Weight quantiser: per 128 x 128 block scale = amax / 448 rounded UP to bf16 (1.0 for a zero block),
 * code = encode(w / scale). Returns -1 for an inf/NaN weight or bad dims (src/omega_gpu_fp8_api.c:723-754). */
int orc_quantize_bf16(uint32_t n, uint32_t k, const uint16_t *w, uint8_t *w8, uint16_t *scale) {
    if (!w || !w8 || !scale || !n || !k || n % ORC_BLOCK || k % ORC_BLOCK) return -1;
    const uint32_t kb = k / ORC_BLOCK;
    for (uint32_t bn = 0; bn < n / ORC_BLOCK; bn++) for (uint32_t bk = 0; bk < kb; bk++) {
        float amax = 0.0f;
        for (uint32_t r = 0; r < ORC_BLOCK; r++) for (uint32_t c = 0; c < ORC_BLOCK; c++) {
            const float f = fabsf(orc_bf16_to_f32(w[((size_t)bn * ORC_BLOCK + r) * k + bk * ORC_BLOCK + c]));
            if (!(f <= 3.0e38f)) return -1;
            if (f > amax) amax = f;
        }
        uint16_t sb = 0x3f80u;
        if (amax > 0.0f) {
            const uint32_t b = bits_of_f32(amax / 448.0f);
            sb = (uint16_t)((b >> 16) + ((b & 0xffffu) ? 1u : 0u));
        }
        scale[(size_t)bn * kb + bk] = sb;
        const float sc = orc_bf16_to_f32(sb);
        for (uint32_t r = 0; r < ORC_BLOCK; r++) for (uint32_t c = 0; c < ORC_BLOCK; c++) {
            const size_t at = ((size_t)bn * ORC_BLOCK + r) * k + bk * ORC_BLOCK + c;
            w8[at] = orc_e4m3_encode(orc_bf16_to_f32(w[at]) / sc);
        }
    }
    return 0;
}

/* ------------------------------------------------------------------ FP8 GEMV / grouped GEMM */

/* Double-precision GEMV: y[r] = sum_c decode(w[r][c]) * x[c] * scale[r/128][c/128], also sum |terms|
 * (src/omega_gpu_fp8_pack.c:59-76). rows [r0, r1) only, so callers can thread it. */
void orc_gemv_rows(const uint8_t *w, const uint16_t *scale, uint32_t k, uint32_t r0, uint32_t r1,
                   const float *x, double *y, double *ymag) {
    const uint32_t kb = k / ORC_BLOCK;
    float lut[256];
    for (int i = 0; i < 256; i++) lut[i] = orc_e4m3_decode((uint8_t)i);
    for (uint32_t r = r0; r < r1; r++) {
        double acc = 0.0, mag = 0.0;
        const uint8_t *row = w + (size_t)r * k;
        const uint16_t *srow = scale + (size_t)(r / ORC_BLOCK) * kb;
        for (uint32_t b = 0; b < kb; b++) {
            const double s = (double)orc_bf16_to_f32(srow[b]);
            for (uint32_t c = b * ORC_BLOCK; c < (b + 1) * ORC_BLOCK; c++) {
                const double p = (double)lut[row[c]] * (double)x[c] * s;
                acc += p; mag += fabs(p);
            }
        }
        y[r] = acc;
        if (ymag) ymag[r] = mag;
    }
}
void orc_gemv(const uint8_t *w, const uint16_t *scale, uint32_t n, uint32_t k, const float *x, double *y, double *ymag) {
    orc_gemv_rows(w, scale, k, 0, n, x, y, ymag);
}

/* The reference kernel's exact f32 summation order for one output row (tests/gpu_fp8gemm_test.c:48-69):
 * 32 lanes, lane L owns lb contiguous columns per K step of 32 * lb columns; dot = fma chain over those
 * bytes; acc = fma(dot, scale, acc) per step; then a shuffle-down tree 16, 8, 4, 2, 1 read at lane 0.
 * The reference folds 2^-120, 2^64 and 2^56 into w, x and scale; those are exact powers of two whose
 * product is 1, so the unfolded chain below gives the same bits. lb is 16 when k % 512 == 0, 8 when k % 256 == 0.
 * The reference kernel refuses any other k (it falls back to a general GEMM); the library extends the same order
 * with lb = 4 there, which this function mirrors (no reference counterpart for that case). */
float orc_gemv_emu_row(const uint8_t *w, const uint16_t *s, const float *x, uint32_t k) {
    const uint32_t lb = (k % 512u == 0) ? 16u : (k % 256u == 0) ? 8u : 4u, steps = k / (32u * lb);
    float a[32];
    for (uint32_t lane = 0; lane < 32; lane++) {
        float acc = 0.0f;
        for (uint32_t st = 0; st < steps; st++) {
            float dot = 0.0f; const uint32_t c0 = st * 32u * lb + lane * lb;
            for (uint32_t b = 0; b < lb; b++) dot = fmaf(orc_e4m3_decode(w[c0 + b]), x[c0 + b], dot);
            acc = fmaf(dot, orc_bf16_to_f32(s[c0 / ORC_BLOCK]), acc);
        }
        a[lane] = acc;
    }
    for (uint32_t o = 16; o >= 1; o /= 2) for (uint32_t l = 0; l + o < 32; l++) a[l] += a[l + o];
    return a[0];
}
void orc_gemv_emu(const uint8_t *w, const uint16_t *scale, uint32_t n, uint32_t k, const float *x, float *y) {
    for (uint32_t r = 0; r < n; r++)
        y[r] = orc_gemv_emu_row(w + (size_t)r * k, scale + (size_t)(r / ORC_BLOCK) * (k / ORC_BLOCK), x, k);
}

/* ------------------------------------------------------------------ router top-k */

/* Top-k over `experts` logits: k rounds of a strict greater-than scan in ascending index, so the lowest
 * index wins ties; ids come out in descending-logit order. Weights: softmax over all experts, then divided
 * by the sum of the selected ones when norm_topk (tests/gpu_router_test.c:62-79). Double precision. */
void orc_topk(const float *logits, uint32_t experts, uint32_t topk, int norm_topk, uint32_t *ids, double *wts) {
    double mx = -1e300, sum = 0.0, sk = 0.0;
    for (uint32_t e = 0; e < experts; e++) if ((double)logits[e] > mx) mx = (double)logits[e];
    for (uint32_t e = 0; e < experts; e++) sum += exp((double)logits[e] - mx);
    uint8_t *taken = calloc(experts, 1);
    for (uint32_t r = 0; r < topk; r++) {
        int best = -1;
        for (uint32_t e = 0; e < experts; e++) if (!taken[e] && (best < 0 || logits[e] > logits[best])) best = (int)e;
        ids[r] = (uint32_t)best; taken[best] = 1;
        wts[r] = exp((double)logits[best] - mx) / sum; sk += wts[r];
    }
    if (norm_topk) for (uint32_t r = 0; r < topk; r++) wts[r] /= sk;
    free(taken);
}

/* Router front half for one residual row (tests/gpu_router_test.c:62-79; kernel contract src/omega_blackwell_codegen_router.h:15-33):
 * xn = x * (1 / sqrt(mean(x^2) + eps)) * norm_w, logits[e] = sum_k bf16(gate[e][k]) * xn[k], then the top-k rule of orc_topk on
 * the double logits. margin = last selected logit minus the best unselected one (an id difference below a small margin is a
 * near-tie, not an error). Everything in double. xn, logits: outputs. */
void orc_router(const float *x, const float *norm_w, const uint16_t *gate_bf16, uint32_t hidden, uint32_t experts, uint32_t topk, float eps,
                int norm_topk, double *xn, double *logits, uint32_t *ids, double *wts, double *margin) {
    double ss = 0.0;
    for (uint32_t i = 0; i < hidden; i++) ss += (double)x[i] * x[i];
    const double r = 1.0 / sqrt(ss / (double)hidden + (double)eps);
    for (uint32_t i = 0; i < hidden; i++) xn[i] = (double)x[i] * r * (double)norm_w[i];
    double mx = -1e300, sum = 0.0, sk = 0.0;
    for (uint32_t e = 0; e < experts; e++) {
        double l = 0.0;
        for (uint32_t k = 0; k < hidden; k++) l += (double)orc_bf16_to_f32(gate_bf16[(size_t)e * hidden + k]) * xn[k];
        logits[e] = l; if (l > mx) mx = l;
    }
    for (uint32_t e = 0; e < experts; e++) sum += exp(logits[e] - mx);
    uint8_t *taken = calloc(experts, 1);
    for (uint32_t rr = 0; rr <= topk && rr < experts; rr++) {
        int best = -1;
        for (uint32_t e = 0; e < experts; e++) if (!taken[e] && (best < 0 || logits[e] > logits[best])) best = (int)e;
        if (rr < topk) { ids[rr] = (uint32_t)best; taken[best] = 1; wts[rr] = exp(logits[best] - mx) / sum; sk += wts[rr]; }
        else if (margin) *margin = logits[ids[topk - 1]] - logits[best];
    }
    if (norm_topk) for (uint32_t rr = 0; rr < topk; rr++) wts[rr] /= sk;
    free(taken);
}

/* ------------------------------------------------------------------ SwiGLU and combine */

/* act[c] = g / (1 + exp(-g)) * up, gate = columns [0, I), up = [I, 2I) of one gate|up row
 * (tests/gpu_decode_graph_test.c:61-66; src/omega_blackwell_codegen_dec.h:17-19). */
void orc_swiglu(const float *gu, uint32_t inter, float *act) {
    for (uint32_t j = 0; j < inter; j++) { const float v = gu[j]; act[j] = v / (1.0f + expf(-v)) * gu[inter + j]; }
}

/* Router-weighted sum in slot order, multiply then add, never fused: m = w0*d0; m = m + w_g*d_g
 * (src/omega_blackwell_codegen_dec.c:226-255; host form tests/gpu_decode_graph_test.c:144-146).
 * d: slots rows of `hidden` f32. Built with -ffp-contract=off so the compiler cannot fuse it either. */
void orc_combine(const float *w, const float *d, uint32_t slots, uint32_t hidden, float *out) {
    for (uint32_t i = 0; i < hidden; i++) {
        float m = 0.0f;
        for (uint32_t g = 0; g < slots; g++) { const float p = w[g] * d[(size_t)g * hidden + i]; m = g ? m + p : p; }
        out[i] = m;
    }
}

/* The prefill form of the same combine (src/omega_blackwell_codegen_pfhost.h:23-31; host loop mc_ref,
 * tests/gpu_pfhost_test.c:38-49): the accumulator starts at +0.0 and row s of token r is down[inv[r*K+s]].
 * Equal to orc_combine except for the sign of an exact zero. */
void orc_combine_mc(const float *down, const uint32_t *inv, const float *wt, uint32_t rows, uint32_t hidden, uint32_t K, float *out) {
    for (uint32_t r = 0; r < rows; r++)
        for (uint32_t c = 0; c < hidden; c++) {
            float acc = 0.0f;
            for (uint32_t g = 0; g < K; g++) { const float p = wt[(size_t)r * K + g] * down[(size_t)inv[(size_t)r * K + g] * hidden + c]; acc = acc + p; }
            out[(size_t)r * hidden + c] = acc;
        }
}

/* RMSNorm as the reference host glue computes it: sum of squares in double, one f32 factor, then
 * x * s * w (tests/gpu_decode_graph_test.c:56-60). w may be NULL (all ones). */
void orc_rmsnorm(const float *x, const float *w, uint32_t hidden, float eps, float *out) {
    double sq = 0.0;
    for (uint32_t i = 0; i < hidden; i++) sq += (double)x[i] * x[i];
    const float s = (float)(1.0 / sqrt(sq / hidden + (double)eps));
    for (uint32_t i = 0; i < hidden; i++) out[i] = x[i] * s * (w ? w[i] : 1.0f);
}

/* ------------------------------------------------------------------ routing plan (ABI1 logical words) */

/* Stable counting scatter, order expert, then token, then original slot; one shared-expert row per token
 * as the last segment (om/moe/moe_plan.om:139-159). cfg = {version 1, tokens <= 128, slots <= 8,
 * experts 1..256, shared id == experts, work capacity <= 1152, segment capacity <= 257, map capacity
 * <= 1160}. ids dense token*slots, 0xFFFFFFFF = absent. Returns 0, or 1 bad cfg, 2 bad id, 3 capacity;
 * a refusal writes nothing. work: 9 words per row; seg: 4 per segment; maps: X at 0, Y at 1160;
 * meta = {work, segs, routed, tokens, 1, 0, 0, 0}. */
uint64_t orc_moe_plan(const uint64_t *cfg, const uint64_t *ids, uint64_t *work, uint64_t *seg, uint64_t *maps, uint64_t *meta) {
    const uint64_t T = cfg[1], S = cfg[2], E = cfg[3];
    if (cfg[0] != 1 || T > 128 || S > 8 || E == 0 || E > 256 || cfg[4] != E) return 1;
    if (cfg[5] > 1152 || cfg[6] > 257 || cfg[7] > 1160) return 1;
    uint64_t cnt[257] = {0}, start[257], cur[257], routed = 0;
    for (uint64_t i = 0; i < T * S; i++) {
        const uint64_t v = ids[i];
        if (v == 0xffffffffull) continue;
        if (v >= E) return 2;
        cnt[v]++; routed++;
    }
    cnt[E] = T;
    uint64_t ns = 0, nw = 0;
    for (uint64_t e = 0; e <= E; e++) { start[e] = cur[e] = nw; if (cnt[e]) { ns++; nw += cnt[e]; } }
    if (nw > cfg[5] || ns > cfg[6] || nw + 8 > cfg[7]) return 3;
    uint64_t z = 0;
    for (uint64_t e = 0; e <= E; e++) if (cnt[e]) { seg[z * 4] = e; seg[z * 4 + 1] = start[e]; seg[z * 4 + 2] = cnt[e]; seg[z * 4 + 3] = e == E; z++; }
#define ORC_WORK(p, e, t, s) do { uint64_t *r_ = work + (p) * 9; r_[0] = (e); r_[1] = (t); r_[2] = (t); r_[3] = (s); r_[4] = (s); \
        r_[5] = start[e]; r_[6] = cnt[e]; r_[7] = (t) * (S + 1) + (s); r_[8] = (s); } while (0)
    for (uint64_t i = 0; i < T * S; i++) {
        const uint64_t v = ids[i];
        if (v == 0xffffffffull) continue;
        const uint64_t p = cur[v]++; ORC_WORK(p, v, i / S, i % S);
    }
    for (uint64_t t = 0; t < T; t++) ORC_WORK(routed + t, E, t, S);
#undef ORC_WORK
    for (uint64_t p = 0; p < nw; p++) { maps[p] = work[p * 9 + 1]; maps[1160 + p] = work[p * 9 + 7]; }
    for (uint64_t p = 0; p < 8; p++) { maps[nw + p] = 0; maps[1160 + nw + p] = 0; }
    meta[0] = nw; meta[1] = ns; meta[2] = routed; meta[3] = T; meta[4] = 1; meta[5] = meta[6] = meta[7] = 0;
    return 0;
}

/* LE u32 picks -> logical words, n active entries (om/moe/moe_ids32.om:4-16). */
uint64_t orc_moe_ids32(const uint8_t *src, uint64_t n, uint64_t *ids) {
    if (n > 1024) return 1;
    for (uint64_t i = 0; i < n; i++) ids[i] = (uint64_t)src[i * 4] | (uint64_t)src[i * 4 + 1] << 8 | (uint64_t)src[i * 4 + 2] << 16 | (uint64_t)src[i * 4 + 3] << 24;
    return 0;
}

/* Logical maps -> LE u32 map bytes, work + 8 entries of each map, validated first (om/moe/moe_maps32.om:9-28). */
uint64_t orc_moe_maps32(const uint64_t *meta, const uint64_t *maps, uint8_t *out) {
    if (meta[0] > 1152) return 1;
    const uint64_t n = meta[0] + 8;
    for (uint64_t zz = 0; zz < 2; zz++) for (uint64_t i = 0; i < n; i++) if (maps[zz * 1160 + i] > 0xffffffffull) return 2;
    for (uint64_t zz = 0; zz < 2; zz++) for (uint64_t i = 0; i < n; i++) {
        const uint64_t p = zz * 1160 + i, v = maps[p];
        for (int b = 0; b < 4; b++) out[p * 4 + b] = (uint8_t)(v >> (8 * b));
    }
    return 0;
}

/* Logical segments + 257-pair {weight, scale} directory -> 32-byte records {w_va, s_va, row0 u32, cnt u32,
 * 0 u64} (om/moe/moe_segs32.om:22-72). 1 bad meta, 2 bad segment, 3 bad directory entry. */
uint64_t orc_moe_segs32(const uint64_t *seg, const uint64_t *meta, const uint64_t *dir, uint8_t *out) {
    if (meta[1] > 257 || meta[0] > 1152) return 1;
    uint64_t pos = 0;
    for (uint64_t z = 0; z < meta[1]; z++) {
        const uint64_t e = seg[z * 4];
        if (e > 256 || seg[z * 4 + 1] != pos || seg[z * 4 + 2] == 0 || seg[z * 4 + 2] > meta[0]) return 2;
        pos += seg[z * 4 + 2];
        if (pos > meta[0]) return 2;
        for (int q = 0; q < 2; q++) { const uint64_t v = dir[e * 2 + q]; if (v == 0 || v % 8) return 3; }
    }
    if (pos != meta[0]) return 2;
    for (uint64_t z = 0; z < meta[1]; z++) {
        const uint64_t e = seg[z * 4];
        const uint64_t rec[4] = { dir[e * 2], dir[e * 2 + 1], seg[z * 4 + 1] | seg[z * 4 + 2] << 32, 0 };
        for (int q = 0; q < 4; q++) for (int b = 0; b < 8; b++) out[z * 32 + q * 8 + b] = (uint8_t)(rec[q] >> (8 * b));
    }
    return 0;
}

/* Token windows with tokens * 9 <= 128 over at most 128 tokens (om/moe/moe_windows.om:29-67).
 * cfg = {1, tokens, 2048, 512, 9, router stride, window capacity <= 128, 0}. */
uint64_t orc_moe_windows(const uint64_t *c, uint64_t *o, uint64_t *m) {
    if (c[0] != 1 || c[1] > 128 || c[2] != 2048 || c[3] != 512 || c[4] != 9) return 1;
    if (c[5] == 0 || c[5] > 0xffffffffull || c[5] % 16 || c[6] > 128 || c[7] != 0) return 1;
    const uint64_t take = 128 / 9, nw = (c[1] + take - 1) / take;
    if (nw > c[6]) return 2;
    uint64_t first = 0;
    for (uint64_t z = 0; z < nw; z++) {
        uint64_t count = c[1] - first; if (count > take) count = take;
        uint64_t *v = o + z * 8;
        v[0] = first; v[1] = count; v[2] = count * c[4];
        v[3] = first * c[2] * 4; v[4] = first * c[4] * c[3] * 8; v[5] = first * c[4] * c[3] * 4;
        v[6] = first * c[4] * c[2] * 4; v[7] = first * c[5];
        first += count;
    }
    m[0] = nw; m[1] = c[1]; m[2] = c[1] * 9; m[3] = 1;
    return 0;
}

/* GROUP launch words: validate 16 request words, emit 16 LE u32 (om/moe/moe_group.om:55-101). */
static uint64_t grp_extent(const uint64_t *r, uint64_t i) {
    if (i < 3) return (r[8] - 1) * r[7] + (i == 0 ? 8u * 4u : 9u * 16u);
    if (i < 5) return r[8] * 9 * 32;
    return (r[8] * 9 + 8) * 4;
}
uint64_t orc_moe_group(const uint64_t *r, uint8_t *o) {
    if (r[8] > 128) return 1;
    const uint64_t rows = r[8] * 9;
    if (r[8] == 0 || rows > 128 || r[11] != 9 || r[15] != 256) return 1;
    if (r[9] < rows || r[10] < rows + 8) return 2;
    if (r[7] == 0 || r[7] > 0xffffffffull || r[7] < 9 * 16) return 2;
    if (r[7] % 16) return 3;
    for (int i = 0; i < 7; i++) if (r[i] == 0 || r[i] % 8) return 3;
    if (r[12] != r[13] || r[14] != 1) return 4;
    for (uint64_t i = 0; i < 7; i++) if (r[i] > UINT64_MAX - grp_extent(r, i)) return 5;
    for (uint64_t j = 0; j < 4; j++) for (uint64_t i = 0; i < j + 3; i++) {
        const uint64_t a = r[i], al = grp_extent(r, i), b = r[j + 3], bl = grp_extent(r, j + 3);
        if (a < b + bl && b < a + al) return 5;
    }
    uint32_t w[16];
    for (int i = 0; i < 7; i++) { w[i * 2] = (uint32_t)r[i]; w[i * 2 + 1] = (uint32_t)(r[i] >> 32); }
    w[14] = (uint32_t)r[7]; w[15] = (uint32_t)r[8];
    for (int i = 0; i < 16; i++) for (int b = 0; b < 4; b++) o[i * 4 + b] = (uint8_t)(w[i] >> (8 * b));
    return 0;
}

/* The same ordering rule at any capacity, in the device's u32 form (the incumbent host GROUP,
 * src/omega_gpu_q36_graph.c:1107-1144, without its `& 255` mask and 256-expert cap): counts per expert,
 * exclusive starts, xmap[p] = token, ymap[p] = token * ystride + slot, 8 zero pads after the last row,
 * segments {expert, row0, cnt} for non-empty experts in ascending id. Absent ids (0xFFFFFFFF) are skipped.
 * Returns the segment count, or -1 on an id >= experts. */
int64_t orc_plan_global(uint32_t tokens, uint32_t slots, uint32_t experts, uint32_t ystride, const uint32_t *ids,
                        uint32_t *counts, uint32_t *starts, uint32_t *xmap, uint32_t *ymap, uint32_t *seg3, uint32_t *rows_out) {
    memset(counts, 0, (size_t)experts * 4);
    for (size_t i = 0; i < (size_t)tokens * slots; i++) { if (ids[i] == 0xffffffffu) continue; if (ids[i] >= experts) return -1; counts[ids[i]]++; }
    uint32_t row = 0; int64_t segs = 0;
    uint32_t *cur = malloc((size_t)experts * 4);
    for (uint32_t e = 0; e < experts; e++) {
        starts[e] = cur[e] = row;
        if (counts[e]) { seg3[segs * 3] = e; seg3[segs * 3 + 1] = row; seg3[segs * 3 + 2] = counts[e]; segs++; row += counts[e]; }
    }
    for (uint32_t t = 0; t < tokens; t++) for (uint32_t s = 0; s < slots; s++) {
        const uint32_t e = ids[(size_t)t * slots + s];
        if (e == 0xffffffffu) continue;
        const uint32_t p = cur[e]++; xmap[p] = t; ymap[p] = t * ystride + s;
    }
    for (uint32_t p = row; p < row + 8; p++) { xmap[p] = 0; ymap[p] = 0; }
    *rows_out = row;
    free(cur);
    return segs;
}

/* ------------------------------------------------------------------ activation quantisers */

/* Per 128-wide group: amax = max(|x|, 2^-100); scale = smallest power of two with amax / scale <= 448;
 * q = e4m3_rne_satfinite(x / scale) (src/omega_blackwell_codegen_qg.h:7-15; tests/gpu_qgemm_test.c:24-35). */
static float pq_scale(float amax) {
    if (!(amax > ldexpf(1.0f, -100))) amax = ldexpf(1.0f, -100);
    const uint32_t mb = bits_of_f32(amax), E = mb >> 23, M = mb & 0x7fffffu, c = (M + 0x1fffffu) >> 23;
    return f32_of_bits((E + c - 8u) << 23);
}
void orc_act_quant(const float *x, uint32_t k, uint8_t *q, float *s) {
    for (uint32_t b = 0; b < k / ORC_BLOCK; b++) {
        float m = 0.0f;
        for (uint32_t j = 0; j < ORC_BLOCK; j++) m = fmaxf(m, fabsf(x[ORC_BLOCK * b + j]));
        const float sc = pq_scale(m);
        s[b] = sc;
        for (uint32_t j = 0; j < ORC_BLOCK; j++) q[ORC_BLOCK * b + j] = orc_e4m3_encode(x[ORC_BLOCK * b + j] / sc);
    }
}
/* Multi-piece form (no reference counterpart: parity unpinned; it is this library's own activation
 * format). Piece 0 is orc_act_quant; piece p encodes the residual left by pieces 0..p-1 at scale / 16^p:
 * r_0 = x / scale; q_p = encode(r_p * 16^p ... ) with r_{p+1} = r_p - decode(q_p) / 16^p. Every step is an
 * exact f32 operation (power-of-two scalings and a difference of nearby values). q: pieces rows of k. */
void orc_act_pieces(const float *x, uint32_t k, uint32_t pieces, uint8_t *q, float *s) {
    for (uint32_t b = 0; b < k / ORC_BLOCK; b++) {
        float m = 0.0f;
        for (uint32_t j = 0; j < ORC_BLOCK; j++) m = fmaxf(m, fabsf(x[ORC_BLOCK * b + j]));
        const float sc = pq_scale(m);
        s[b] = sc;
        for (uint32_t j = 0; j < ORC_BLOCK; j++) {
            float r = x[ORC_BLOCK * b + j] / sc;
            for (uint32_t p = 0; p < pieces; p++) {
                const uint8_t c = orc_e4m3_encode(r);
                q[(size_t)p * k + ORC_BLOCK * b + j] = c;
                r = (r - orc_e4m3_decode(c)) * 16.0f;
            }
        }
    }
}
/* value the pieces stand for (double): scale * sum_p decode(q_p) / 16^p */
void orc_act_pieces_decode(const uint8_t *q, const float *s, uint32_t k, uint32_t pieces, double *x) {
    for (uint32_t c = 0; c < k; c++) {
        double v = 0.0, f = 1.0;
        for (uint32_t p = 0; p < pieces; p++) { v += (double)orc_e4m3_decode(q[(size_t)p * k + c]) * f; f /= 16.0; }
        x[c] = v * (double)s[c / ORC_BLOCK];
    }
}

/* ------------------------------------------------------------------ W4 (no reference implementation) */

/* fp16 helpers for the W4 scale (IEEE binary16, round to nearest even). */
uint16_t orc_f32_to_f16(float f) {
    const uint32_t x = bits_of_f32(f), sign = (x >> 16) & 0x8000u;
    const uint32_t ax = x & 0x7fffffffu;
    if (ax >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | (ax > 0x7f800000u ? 0x200u : 0u));
    if (ax >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);              /* rounds past 65504 -> inf */
    if (ax < 0x33000001u) return (uint16_t)sign;                           /* below half the smallest subnormal */
    int e = (int)(ax >> 23) - 127; uint32_t m = (ax & 0x7fffffu) | 0x800000u;
    int shift = e < -14 ? 13 + (-14 - e) : 13;
    uint32_t q = m >> shift, rem = m & ((1u << shift) - 1u), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) q++;
    if (e < -14) return (uint16_t)(sign | q);
    return (uint16_t)(sign | (((uint32_t)(e + 15) << 10) + (q - 0x400u)));
}
float orc_f16_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 31u, m = h & 0x3ffu;
    if (e == 0) return f32_of_bits(sign) + (sign ? -1.0f : 1.0f) * (float)m * ldexpf(1.0f, -24);
    if (e == 31) return f32_of_bits(sign | 0x7f800000u | (m << 13));
    return f32_of_bits(sign | ((e + 112u) << 23) | (m << 13));
}
/* Signed int4 group quantiser as the benchmark configuration defines it (the reference refuses integer
 * W4, docs/models/QUANT.md:62: PARITY UNPINNED, self-oracle). Per row, per 32-element K group:
 * scale = fp16(amax / 7) (1.0 for a zero group); q = clamp(rint(w / scale), -8, 7); two per byte along K,
 * low nibble = even column (the reference's only nibble convention, docs/models/QUANT.md:57). */
void orc_w4_quantize(uint32_t n, uint32_t k, const float *w, uint8_t *packed, uint16_t *scale_f16) {
    for (uint32_t r = 0; r < n; r++) for (uint32_t g = 0; g < k / 32; g++) {
        float amax = 0.0f;
        for (uint32_t j = 0; j < 32; j++) amax = fmaxf(amax, fabsf(w[(size_t)r * k + g * 32 + j]));
        uint16_t sh = amax > 0.0f ? orc_f32_to_f16(amax / 7.0f) : 0x3c00u;
        if ((sh & 0x7fffu) == 0) sh = 0x3c00u;
        scale_f16[(size_t)r * (k / 32) + g] = sh;
        const float sc = orc_f16_to_f32(sh);
        for (uint32_t j = 0; j < 32; j += 2) {
            int q[2];
            for (int h = 0; h < 2; h++) {
                float v = nearbyintf(w[(size_t)r * k + g * 32 + j + h] / sc);
                q[h] = v < -8.0f ? -8 : v > 7.0f ? 7 : (int)v;
            }
            packed[((size_t)r * k + g * 32 + j) / 2] = (uint8_t)((q[0] & 15) | ((q[1] & 15) << 4));
        }
    }
}
/* y[m][r] = sum_c x[m][c] * q[r][c] * scale[r][c/32], double accumulate; rows [r0, r1). */
void orc_w4_gemm_rows(const uint8_t *packed, const uint16_t *scale_f16, uint32_t k, uint32_t r0, uint32_t r1,
                      uint32_t n, const float *x, uint32_t m_rows, double *y) {
    for (uint32_t r = r0; r < r1; r++) for (uint32_t m = 0; m < m_rows; m++) {
        double acc = 0.0;
        for (uint32_t g = 0; g < k / 32; g++) {
            const double sc = (double)orc_f16_to_f32(scale_f16[(size_t)r * (k / 32) + g]);
            double part = 0.0;
            for (uint32_t j = 0; j < 32; j++) {
                const uint32_t c = g * 32 + j; const uint8_t b = packed[((size_t)r * k + c) / 2];
                int q = (c & 1u) ? (b >> 4) : (b & 15); if (q > 7) q -= 16;
                part += (double)x[(size_t)m * k + c] * (double)q;
            }
            acc += part * sc;
        }
        y[(size_t)m * n + r] = acc;
    }
}

/* ------------------------------------------------------------------ MXFP4 (E2M1 nibble + E8M0 scale per 32 elements) */

/* One MXFP4 element as exact IEEE binary32 bits: what the reference's scalar decoder returns (native/models/mxfp4.om; contract
 * docs/models/MXFP4.md:4-9; its verification oracle tests/models/mxfp4-check.py:30-35: ldexp(FP4_VALUES[nibble], scale - 127), values the
 * format cannot hold finitely become signed infinity, signed zero kept, small results become subnormals). nib 0..15 (bit 3 = sign, bits 2..1
 * exponent, bit 0 mantissa), scale 0..254 biased by 127; 255 is the reserved NaN block and is refused by the callers. Integer arithmetic only. */
uint32_t orc_mxfp4_bits(uint32_t nib, uint32_t scale) {
    const uint32_t sign = (nib & 8u) << 28, m = nib & 7u;
    if (m == 0) return sign;
    /* value = mag * 2^(scale - 127) with mag in {0.5, 1, 1.5, 2, 3, 4, 6} = (2 + man) * 2^(exp - 2) for exp >= 1, and 0.5 = 2^-1 for m = 1 */
    int e; uint32_t frac;   /* value = (1 + frac / 2) * 2^e */
    if (m == 1) { e = -1; frac = 0; } else { e = (int)(m >> 1) - 1; frac = m & 1u; }
    e += (int)scale - 127;
    if (e > 127) return sign | 0x7f800000u;
    if (e >= -126) return sign | ((uint32_t)(e + 127) << 23) | (frac << 22);
    /* subnormal: (1 + frac / 2) * 2^e = (2 + frac) * 2^(e - 1); one unit is 2^-149 */
    const int sh = e - 1 + 149;
    if (sh < 0) return sign;   /* cannot occur: the smallest element is 0.5 * 2^-127 = 2^-128 = 2^21 units */
    return sign | ((2u + frac) << sh);
}
/* y[m][r] = sum over groups of 2^(scale - 127) * sum_c x[m][c] * e2m1(nibble[r][c]) in double; low nibble = even column (gpt-oss order). rows [r0, r1) */
void orc_mxfp4_gemm_rows(const uint8_t *packed, const uint8_t *scale_e8m0, uint32_t k, uint32_t r0, uint32_t r1,
                         uint32_t n, const float *x, uint32_t m_rows, double *y) {
    for (uint32_t r = r0; r < r1; r++) for (uint32_t m = 0; m < m_rows; m++) {
        double acc = 0.0;
        for (uint32_t c = 0; c < k; c++) {
            const uint8_t b = packed[((size_t)r * k + c) / 2];
            const uint32_t bits = orc_mxfp4_bits((c & 1u) ? (b >> 4) : (b & 15u), scale_e8m0[(size_t)r * (k / 32) + c / 32]);
            float w; memcpy(&w, &bits, 4);
            acc += (double)x[(size_t)m * k + c] * (double)w;
        }
        y[(size_t)m * n + r] = acc;
    }
}

/* ------------------------------------------------------------------ NVFP4 (E2M1 nibble + unsigned E4M3 scale per 16 elements) */

/* One NVFP4 element times its block scale as exact IEEE binary32 bits: what the reference's scalar decoder returns (native/models/nvfp4.om,
 * nvfp4bits; contract docs/models/MXFMT.md: "nvfp4bits nib scale gives the exact binary32 bits of element x scale"; its verification oracle
 * tests/models/mxfmt-check.py:287-300 compares with the ml_dtypes product float4_e2m1fn x float8_e4m3fn and with exact rationals).
 * nib 0..15 (bit 3 = sign), scale 0..126: an E4M3 code with the sign bit clear; 127 (NaN) and 128..255 (sign set) are refused by that unit
 * (trap 5): here they return 0xffffffff, which no valid pair produces. Signed zero kept. Integer arithmetic and one exact ldexp. */
uint32_t orc_nvfp4_bits(uint32_t nib, uint32_t scale) {
    if (nib > 15u || scale > 126u) return 0xffffffffu;
    const uint32_t sign = (nib & 8u) << 28, m = nib & 7u;
    const uint32_t twice = m < 4u ? m : (2u + (m & 1u)) << ((m >> 1) - 1u);        /* 2 x {0, .5, 1, 1.5, 2, 3, 4, 6} */
    const uint32_t se = scale >> 3, sig = se ? ((scale & 7u) | 8u) : (scale & 7u);   /* scale = sig * 2^(se ? se - 10 : -9) */
    if (twice == 0 || sig == 0) return sign;
    const float v = ldexpf((float)(twice * sig), (se ? (int)se - 10 : -9) - 1);     /* at most 12 * 15 = 180: exact, and never subnormal */
    uint32_t bits; memcpy(&bits, &v, 4);
    return sign | bits;
}
/* y[m][r] = sum over columns of x[m][c] * (element[r][c] * scale[r][c / 16]) in double, columns in order; low nibble = even column
 * (native/models/nvfp4.om: "element 2i is the low nibble of byte i"). rows [r0, r1) */
void orc_nvfp4_gemm_rows(const uint8_t *packed, const uint8_t *scale_ue4m3, uint32_t k, uint32_t r0, uint32_t r1,
                         uint32_t n, const float *x, uint32_t m_rows, double *y) {
    for (uint32_t r = r0; r < r1; r++) for (uint32_t m = 0; m < m_rows; m++) {
        double acc = 0.0;
        for (uint32_t c = 0; c < k; c++) {
            const uint8_t b = packed[((size_t)r * k + c) / 2];
            const uint32_t bits = orc_nvfp4_bits((c & 1u) ? (b >> 4) : (b & 15u), scale_ue4m3[(size_t)r * (k / 16) + c / 16]);
            float w; memcpy(&w, &bits, 4);
            acc += (double)x[(size_t)m * k + c] * (double)w;
        }
        y[(size_t)m * n + r] = acc;
    }
}

/* NVFP4 encoder of the reference (native/models/nvfp4.om: nvfp4enc, nvfp4scale, nvfp4nib; contract docs/models/MXFMT.md; checked there against a
 * binary64 quotient oracle, exact rationals around every threshold and ml_dtypes, tests/models/mxfmt-check.py:302-352).
 * orc_nvfp4_enc: the nearest-even E2M1 nibble of x / scale, found by comparing |x| with scale x {1, 3, 5, 7, 10, 14, 20} / 4 (each exact in
 * binary32); above 6 and infinity saturate to 6; scale 0 gives a signed zero; 0xff where the unit traps (NaN input, scale above 126).
 * orc_nvfp4_scale: the block scale, e4m3 (round to nearest even, saturating at 448) of the binary32 quotient amax / 6; 0xff for a NaN amax.
 * orc_nvfp4_block: 16 binary32 values -> scale code and 8 packed bytes (element 2i in the low nibble of byte i); 0xff if any value is NaN. */
uint32_t orc_nvfp4_enc(uint32_t bits, uint32_t scale) {
    static const uint32_t mid[7] = {1, 3, 5, 7, 10, 14, 20};
    if (scale > 126u) return 0xffu;
    const uint32_t sign = (bits >> 28) & 8u, a = bits & 0x7fffffffu;
    if (a > 0x7f800000u) return 0xffu;
    const uint32_t se = scale >> 3, sig = se ? ((scale & 7u) | 8u) : (scale & 7u);
    if (sig == 0) return sign;
    const int ex = (se ? (int)se - 10 : -9) - 2;
    float av; memcpy(&av, &a, 4);
    uint32_t c = 0;
    for (uint32_t k = 0; k < 7; k++) {
        const float t = ldexpf((float)(sig * mid[k]), ex);   /* at most 15 * 20 = 300: exact */
        if (av < t) break;
        if (av > t) { c = k + 1; continue; }
        if (k & 1u) c = k + 1;                               /* a tie goes to the even code */
        break;
    }
    return sign | c;
}
uint32_t orc_nvfp4_scale(uint32_t amax_bits) {
    if (amax_bits > 0x7f800000u) return 0xffu;
    float a; memcpy(&a, &amax_bits, 4);
    const volatile float q = a / 6.0f;                       /* one binary32 division, as the unit does */
    return (uint32_t)orc_e4m3_encode(q) & 0x7fu;
}
uint32_t orc_nvfp4_block(const uint32_t *x, uint8_t *q) {
    uint32_t amax = 0;
    for (int i = 0; i < 16; i++) { const uint32_t a = x[i] & 0x7fffffffu; if (a > 0x7f800000u) return 0xffu; if (a > amax) amax = a; }
    const uint32_t sc = orc_nvfp4_scale(amax);
    for (int j = 0; j < 8; j++) q[j] = (uint8_t)(orc_nvfp4_enc(x[2 * j], sc) | (orc_nvfp4_enc(x[2 * j + 1], sc) << 4));
    return sc;
}
void orc_nvfp4_enc_many(const uint32_t *bits, size_t n, uint32_t scale, uint8_t *out) { for (size_t i = 0; i < n; i++) out[i] = (uint8_t)orc_nvfp4_enc(bits[i], scale); }
void orc_nvfp4_scale_many(const uint32_t *amax, size_t n, uint8_t *out) { for (size_t i = 0; i < n; i++) out[i] = (uint8_t)orc_nvfp4_scale(amax[i]); }
/* rows x k binary32 values (k a multiple of 16) -> packed [rows][k / 2] and scales [rows][k / 16]; returns the number of blocks refused (NaN) */
size_t orc_nvfp4_quantize(const uint32_t *x, size_t rows, size_t k, uint8_t *packed, uint8_t *scales) {
    size_t bad = 0;
    for (size_t r = 0; r < rows; r++) for (size_t b = 0; b < k / 16; b++) {
        const uint32_t sc = orc_nvfp4_block(x + r * k + b * 16, packed + r * (k / 2) + b * 8);
        scales[r * (k / 16) + b] = (uint8_t)sc;
        if (sc == 0xffu) bad++;
    }
    return bad;
}

/* ------------------------------------------------------------------ block-scaled product C = A B^T of two quantised operands */

/* The reference's definition of a block-scaled GEMM (native/models/mxdot.om `mxmm`, contract docs/models/MXFMT.md: "Each block term is exact ...
 * Block terms are added left to right in binary64"; its verification oracle tests/models/mxfmt-check.py:392-411, `mx_reference`).
 * fmt 0: NVFP4 (E2M1 nibbles, low nibble first, unsigned E4M3 scale per 16); fmt 1: MXFP4 (E2M1, E8M0 scale per 32); fmt 2: MXFP8 (E4M3 bytes,
 * E8M0 per 32). A is m x k, B is n x k, both K-contiguous; scales [rows][k / block]. C[i][j] = sum over blocks, in order, of
 * (sum_e a_e b_e) * sa * sb, every term exact in binary64 (the inner sums are small integers over 4, or under 2^53 units for E4M3), only the
 * running sum rounds. mag (optional) = sum of |terms|. Returns 0, or 5 where the unit traps: fmt > 2, k = 0 or not a multiple of the block,
 * a NaN element (E4M3 0x7f / 0xff) or scale (E8M0 255, UE4M3 above 126). */
static double mx_elem(uint32_t fmt, const uint8_t *a, size_t i) {
    if (fmt == 2) return (double)orc_e4m3_decode(a[i]);
    const uint32_t nib = (a[i >> 1] >> (4u * (i & 1u))) & 15u, m = nib & 7u;
    const double v = m < 4u ? 0.5 * m : (double)((2u + (m & 1u)) << ((m >> 1) - 1u)) * 0.5;   /* 0 .5 1 1.5 2 3 4 6 */
    return (nib & 8u) ? -v : v;
}
static int mx_scale(uint32_t fmt, uint32_t code, double *out) {
    if (fmt == 0) { if (code > 126u) return 5; *out = (double)orc_e4m3_decode((uint8_t)code); return 0; }
    if (code == 255u) return 5;
    *out = ldexp(1.0, (int)code - 127);
    return 0;
}
int orc_mxmm(uint32_t fmt, uint32_t m, uint32_t n, uint32_t k, const uint8_t *A, const uint8_t *SA, const uint8_t *B, const uint8_t *SB, double *C, double *mag) {
    if (fmt > 2u) return 5;
    const uint32_t bs = fmt == 0 ? 16u : 32u;
    if (k == 0 || k % bs) return 5;
    const uint32_t kb = k / bs;
    if (fmt == 2) for (size_t i = 0; i < (size_t)k * m; i++) if ((A[i] & 127u) == 127u) return 5;
    if (fmt == 2) for (size_t i = 0; i < (size_t)k * n; i++) if ((B[i] & 127u) == 127u) return 5;
    for (uint32_t i = 0; i < m; i++) for (uint32_t j = 0; j < n; j++) {
        double acc = 0.0, ab = 0.0;
        for (uint32_t t = 0; t < kb; t++) {
            double sa, sb, inner = 0.0;
            if (mx_scale(fmt, SA[(size_t)i * kb + t], &sa) || mx_scale(fmt, SB[(size_t)j * kb + t], &sb)) return 5;
            for (uint32_t e = 0; e < bs; e++) inner += mx_elem(fmt, A, ((size_t)i * kb + t) * bs + e) * mx_elem(fmt, B, ((size_t)j * kb + t) * bs + e);
            const double term = inner * sa * sb;
            acc += term; ab += fabs(term);
        }
        C[(size_t)i * n + j] = acc;
        if (mag) mag[(size_t)i * n + j] = ab;
    }
    return 0;
}

/* ------------------------------------------------------------------ one MoE layer, the reference host glue */

/* For sorted row p (expert e, token t, slot s): gu = GEMV(W_gu[e], x[t]) (double dot, stored f32, as a
 * caller of omega_gpu_fp8_gemv_* receives it), act = swiglu(gu), dn = GEMV(W_dn[e], act), written at
 * dn[(t * slots + s)]. Rows [p0, p1) so callers can thread it. hidden = k of gate|up = n of down;
 * inter = n/2 of gate|up = k of down (tests/gpu_decode_graph_test.c:129-147). */
void orc_expert_rows(const uint8_t *wgu, const uint16_t *sgu, const uint8_t *wdn, const uint16_t *sdn,
                     uint32_t hidden, uint32_t inter, const float *x, const uint32_t *row_expert,
                     const uint32_t *row_token, const uint32_t *row_dest, uint32_t p0, uint32_t p1, float *dn_out) {
    const size_t gu_w = (size_t)2 * inter * hidden, gu_s = (size_t)(2 * inter / ORC_BLOCK) * (hidden / ORC_BLOCK);
    const size_t dn_w = (size_t)hidden * inter, dn_s = (size_t)(hidden / ORC_BLOCK) * (inter / ORC_BLOCK);
    double *t = malloc(sizeof(double) * (size_t)(2 * inter > hidden ? 2 * inter : hidden));
    float *gu = malloc(sizeof(float) * 2 * inter), *act = malloc(sizeof(float) * inter);
    for (uint32_t p = p0; p < p1; p++) {
        const uint32_t e = row_expert[p];
        orc_gemv(wgu + e * gu_w, sgu + e * gu_s, 2 * inter, hidden, x + (size_t)row_token[p] * hidden, t, NULL);
        for (uint32_t i = 0; i < 2 * inter; i++) gu[i] = (float)t[i];
        orc_swiglu(gu, inter, act);
        orc_gemv(wdn + e * dn_w, sdn + e * dn_s, hidden, inter, act, t, NULL);
        float *o = dn_out + (size_t)row_dest[p] * hidden;
        for (uint32_t i = 0; i < hidden; i++) o[i] = (float)t[i];
    }
    free(t); free(gu); free(act);
}

/* value (f32, exact) that `pieces` activation pieces stand for; pieces == 0 leaves x as it is */
static void orc_requantise(float *x, uint32_t k, uint32_t pieces) {
    if (!pieces) return;
    uint8_t *q = malloc((size_t)pieces * k); float *s = malloc(sizeof(float) * (k / ORC_BLOCK)); double *d = malloc(sizeof(double) * k);
    orc_act_pieces(x, k, pieces, q, s);
    orc_act_pieces_decode(q, s, k, pieces, d);
    for (uint32_t c = 0; c < k; c++) x[c] = (float)d[c];
    free(q); free(s); free(d);
}
/* orc_expert_rows with the activations passed through the piece quantiser first (x_pieces for the layer input,
 * act_pieces for the gated activations): the arithmetic model of the tensor-core engine, whose FP8 MMA needs FP8
 * activations. The reference's own QMMA path is tested the same way, against a reference that applies its
 * activation quantiser first (tests/gpu_qgemm_test.c:24-35, :231). */
void orc_expert_rows_q(const uint8_t *wgu, const uint16_t *sgu, const uint8_t *wdn, const uint16_t *sdn,
                       uint32_t hidden, uint32_t inter, const float *x, const uint32_t *row_expert,
                       const uint32_t *row_token, const uint32_t *row_dest, uint32_t p0, uint32_t p1, float *dn_out,
                       uint32_t x_pieces, uint32_t act_pieces) {
    const size_t gu_w = (size_t)2 * inter * hidden, gu_s = (size_t)(2 * inter / ORC_BLOCK) * (hidden / ORC_BLOCK);
    const size_t dn_w = (size_t)hidden * inter, dn_s = (size_t)(hidden / ORC_BLOCK) * (inter / ORC_BLOCK);
    double *t = malloc(sizeof(double) * (size_t)(2 * inter > hidden ? 2 * inter : hidden));
    float *gu = malloc(sizeof(float) * 2 * inter), *act = malloc(sizeof(float) * inter), *xq = malloc(sizeof(float) * hidden);
    for (uint32_t p = p0; p < p1; p++) {
        const uint32_t e = row_expert[p];
        memcpy(xq, x + (size_t)row_token[p] * hidden, sizeof(float) * hidden);
        orc_requantise(xq, hidden, x_pieces);
        orc_gemv(wgu + e * gu_w, sgu + e * gu_s, 2 * inter, hidden, xq, t, NULL);
        for (uint32_t i = 0; i < 2 * inter; i++) gu[i] = (float)t[i];
        orc_swiglu(gu, inter, act);
        orc_requantise(act, inter, act_pieces);
        orc_gemv(wdn + e * dn_w, sdn + e * dn_s, hidden, inter, act, t, NULL);
        float *o = dn_out + (size_t)row_dest[p] * hidden;
        for (uint32_t i = 0; i < hidden; i++) o[i] = (float)t[i];
    }
    free(t); free(gu); free(act); free(xq);
}
