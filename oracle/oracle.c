/* CPU oracle for the routed-expert FFN path (numerical mode E-W4A8-v1).
 *
 * TEST INFRASTRUCTURE ONLY. This file restates, in plain C, what the reference
 * computes on this path; it is the checker for the CUDA library, never part of
 * it. Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may
 * build, load or call it.
 *
 * Parity pins (see tests/test_oracle_pins.py): the reference's own golden
 * vectors (oracle/goldens/e4m3_decode_table.json, mxfp4_golden.json, the real
 * block fixture bench/fixtures/expert_nibble_fixture.json), fixtures generated
 * by running the reference's Python lattice oracle and codec
 * (crates/mimo26-repack/tests/lattice_oracle.py, oracle/lattice/quant_v1.py),
 * and the reference's own host-compiled quantiser / planner / reducer
 * (oracle/_ref, built from the sources under the reference tree).
 *
 * Each function cites the reference lines it follows (paths inside the
 * reference repository).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_HIDDEN 4096
#define ORC_INTER 2048
#define ORC_EXPERTS 256
#define ORC_TOPK 8

static inline uint32_t f32_bits(float v) { uint32_t b; memcpy(&b, &v, 4); return b; }
static inline float bits_f32(uint32_t b) { float v; memcpy(&v, &b, 4); return v; }

/* ---- E4M3FN ------------------------------------------------------------------
 * crates/mimo26-load/src/e4m3.rs:19-31, oracle/lattice/quant_v1.py:39-47:
 * [s eeee mmm], bias 7, subnormals m * 2^-9, S.1111.111 = NaN. */
float orc_e4m3_decode(uint8_t c) {
    if ((c & 0x7f) == 0x7f) return NAN;
    const int e = (c >> 3) & 15, m = c & 7;
    const float v = e ? ldexpf(1.0f + (float)m / 8.0f, e - 7) : ldexpf((float)m, -9);
    return (c & 0x80) ? -v : v;
}

/* Smallest k with a <= 448 * 2^k for finite a > 0, exact through frexp
 * (oracle/lattice/quant_v1.py:33-36; the same integer the wire codec's
 * ceil(log2(amax/448)) yields, crates/mimo26-coordinator/src/wire.rs:66-68). */
static int scale_exponent(double a) {
    int e;
    const double m = frexp(a, &e); /* a = m 2^e, m in [0.5,1) */
    return m <= 0.875 ? e - 9 : e - 8;
}

/* Nearest E4M3 magnitude code of y >= 0, ties to even (even != 0) or to the
 * larger magnitude (even == 0), saturating at 448. Subnormal quantum 2^-9.
 * quant_v1.py:50-71 (RNE); e4m3.rs:50-81 (half-up). */
static unsigned e4m3_encode_mag(double y, int even) {
    if (y == 0.0) return 0;
    if (y < 0.015625) { /* below 2^-6 */
        const double q = y * 512.0;
        double r = floor(q);
        const double frac = q - r;
        if (frac > 0.5 || (frac == 0.5 && (!even || fmod(r, 2.0) == 1.0))) r += 1.0;
        return (unsigned)r; /* 8 is the smallest normal's code */
    }
    int g;
    frexp(y, &g);
    int E = g - 1;
    const double q = ldexp(y, 3 - E); /* in [8,16) */
    double r = floor(q);
    const double frac = q - r;
    if (frac > 0.5 || (frac == 0.5 && (!even || fmod(r, 2.0) == 1.0))) r += 1.0;
    if (r == 16.0) { r = 8.0; ++E; }
    if (E > 8 || (E == 8 && r > 14.0)) return 0x7e;
    return (unsigned)((E + 7) * 8 + ((int)r - 8));
}

/* ---- wire quantiser ------------------------------------------------------------
 * crates/mimo26-coordinator/src/wire.rs:53-78: per K32 block amax in f64 (NaN
 * ignored by max), s = 0 for a zero block else clamp(ceil(log2(amax/448)) +
 * 127, 0, 254); payload = encode_e4m3(v * 2^(127-s)) with NaN -> 0, clamp 448,
 * sign only for v < 0 (crates/mimo26-load/src/e4m3.rs:50-81). */
void orc_quant_wire(const float* x, uint64_t n_elems, uint8_t* payload, uint8_t* scales) {
    for (uint64_t b = 0; b < n_elems / 32; ++b) {
        const float* blk = x + b * 32;
        double amax = 0.0;
        for (int k = 0; k < 32; ++k) {
            const double a = fabs((double)blk[k]);
            if (a > amax) amax = a; /* NaN compares false: skipped, as f64::max does */
        }
        int s = 0;
        if (amax != 0.0) {
            if (isinf(amax)) s = 254;
            else {
                s = scale_exponent(amax) + 127;
                s = s < 0 ? 0 : s > 254 ? 254 : s;
            }
        }
        scales[b] = (uint8_t)s;
        for (int k = 0; k < 32; ++k) {
            double v = (double)blk[k];
            if (isnan(v)) v = 0.0;
            v = ldexp(v, 127 - s);
            double mag = fabs(v);
            if (mag > 448.0) mag = 448.0;
            const unsigned sign = v < 0.0 ? 0x80u : 0u;
            payload[b * 32 + k] = (uint8_t)(mag == 0.0 ? 0u : (sign | e4m3_encode_mag(mag, 0)));
        }
    }
}

/* ---- quantiser e4m3fn-k32-v1 ------------------------------------------------------
 * oracle/lattice/quant_v1.py:74-87 and crates/mimo26-expert/kernels/b1/quant_v1.cuh:84-100:
 * a = max(max|h|, 1e-4f); k = smallest integer with a <= 448 2^k; scale byte k + 127;
 * payload = RNE(h 2^-k), -0 kept. Fault 1: nonfinite input; fault 2: payload * 2^k
 * outside FP32. A faulting block writes nothing. Returns the number of faulting blocks. */
uint64_t orc_quant_v1(const float* x, uint64_t n_elems, uint8_t* payload, uint8_t* scales, uint32_t* block_faults) {
    uint64_t bad = 0;
    for (uint64_t b = 0; b < n_elems / 32; ++b) {
        const float* blk = x + b * 32;
        float amax = 1e-4f;
        int fault = 0;
        for (int k = 0; k < 32; ++k) {
            if (!isfinite(blk[k])) { fault = 1; break; }
            const float a = fabsf(blk[k]);
            if (a > amax) amax = a;
        }
        uint8_t codes[32];
        int kexp = 0;
        if (!fault) {
            kexp = scale_exponent((double)amax);
            for (int k = 0; k < 32; ++k) {
                const double y = ldexp((double)blk[k], -kexp);
                const unsigned sign = signbit(blk[k]) ? 0x80u : 0u;
                const unsigned code = e4m3_encode_mag(fabs(y), 1);
                codes[k] = (uint8_t)(sign | code);
                const unsigned field = (code >> 3) & 15u;
                if (field && (int)field - 7 + kexp > 127) fault = 2;
            }
        }
        if (block_faults) block_faults[b] = (uint32_t)fault;
        if (fault) { ++bad; continue; }
        memcpy(payload + b * 32, codes, 32);
        scales[b] = (uint8_t)(kexp + 127);
    }
    return bad;
}

/* oracle/lattice/quant_v1.py:90-102: scale bytes outside 105..247 and NaN codes
 * are faults (return 1); otherwise value = decode(code) * 2^(s-127) as FP32. */
int orc_dequant_v1(const uint8_t* payload, const uint8_t* scales, uint64_t n_elems, float* out) {
    for (uint64_t i = 0; i < n_elems; ++i) {
        const uint8_t s = scales[i / 32];
        if (s < 105 || s > 247 || (payload[i] & 0x7f) == 0x7f) return 1;
        const double v = ldexp((double)orc_e4m3_decode(payload[i]), (int)s - 127);
        if (fabs(v) > 3.4028234663852886e38) return 1;
        out[i] = (float)v;
    }
    return 0;
}

/* ---- MXFP4 -------------------------------------------------------------------------
 * spike/mxfp4.py:59-84, crates/mimo26-expert/src/mxfp4.rs:51-134: codebook by
 * nibble, LOW nibble = even k, scale 2^(min(b,254)-127), product saturated to
 * +-FLT_MAX before the cast, -0 preserved. */
static const double kE2M1[16] = {0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0};
void orc_mxfp4_unpack(const uint8_t* packed, const uint8_t* scales, uint64_t rows, uint64_t in_cols, float* out) {
    for (uint64_t r = 0; r < rows; ++r)
        for (uint64_t k = 0; k < in_cols; ++k) {
            const uint8_t byte = packed[r * (in_cols / 2) + k / 2];
            const int nib = (k & 1) ? (byte >> 4) : (byte & 15);
            const int sb = scales[r * (in_cols / 32) + k / 32];
            double v = kE2M1[nib] * ldexp(1.0, (sb > 254 ? 254 : sb) - 127);
            if (v > 3.4028234663852886e38) v = 3.4028234663852886e38;
            if (v < -3.4028234663852886e38) v = -3.4028234663852886e38;
            out[r * in_cols + k] = (float)v;
        }
}

/* ---- stable route plan ----------------------------------------------------------------
 * crates/mimo26-expert/kernels/b1/group_plan.cu:32-79: reject id outside [0,256),
 * non-resident expert, weight outside [0, FLT_MAX] (NaN included), an expert twice
 * in a row; then a stable counting sort of routes by expert. Returns 0, or 7
 * (metadata) / 8 (nonfinite) as the reference's Status values. */
int orc_plan(const int32_t* ids, const float* w, uint32_t rows, const uint8_t* resident, int32_t* inverse,
             int32_t* original_routes, float* grouped_weights, uint32_t* counts) {
    uint32_t next[ORC_EXPERTS];
    const uint32_t routes = rows * ORC_TOPK;
    memset(counts, 0, ORC_EXPERTS * sizeof(uint32_t));
    for (uint32_t i = 0; i < routes; ++i) {
        const int32_t e = ids[i];
        if (e < 0 || e >= ORC_EXPERTS || !resident[e]) return 7;
        if (!(w[i] >= 0.0f && w[i] <= 3.402823466e+38f)) return 8;
        for (uint32_t j = (i / ORC_TOPK) * ORC_TOPK; j < i; ++j)
            if (ids[j] == e) return 7;
        ++counts[e];
    }
    uint32_t total = 0;
    for (int e = 0; e < ORC_EXPERTS; ++e) { next[e] = total; total += counts[e]; }
    for (uint32_t i = 0; i < routes; ++i) {
        const uint32_t g = next[ids[i]]++;
        inverse[i] = (int32_t)g;
        original_routes[g] = (int32_t)i;
        grouped_weights[g] = w[i];
    }
    return 0;
}

/* ---- activation E-ACT-CR32 --------------------------------------------------------------
 * crates/mimo26-repack/tests/lattice_oracle.py:32-53: e = RN32(exp_f64(-|g|));
 * g >= 0: (g / (1 + e)) * u; g < 0: ((g * e) / (1 + e)) * u; ordered FP32 ops. */
float orc_activation(float g, float u) {
    const float t = g >= 0.0f ? -g : g;
    const float e = (float)exp((double)t);
    volatile float d = 1.0f + e;
    volatile float s;
    if (g >= 0.0f) s = g / d;
    else { volatile float ge = g * e; s = ge / d; }
    volatile float r = s * u;
    return r;
}

/* ---- exact block dot products ---------------------------------------------------------------
 * The lattice oracle takes dots in FP64 and rounds the result to FP32
 * (lattice_oracle.py:66-67,86-87). Every operand is a small integer times a
 * power of two, so a K32 block's sum of products is an exact integer: E4M3
 * value = X * 2^-9 with X = (8+m) << (e-1) (or m for e = 0), E2M1 value =
 * W * 2^-1 with W in {0,1,2,3,4,6,8,12}. Block sums are scaled and added in
 * long double, then rounded to FP64 and to FP32. */
static void e4m3_ints(const uint8_t* codes, uint64_t n, int32_t* out) {
    for (uint64_t i = 0; i < n; ++i) {
        const int e = (codes[i] >> 3) & 15, m = codes[i] & 7;
        const int32_t mag = e ? (int32_t)(8 + m) << (e - 1) : m;
        out[i] = (codes[i] & 0x80) ? -mag : mag;
    }
}
static void e2m1_ints(const uint8_t* packed, uint64_t rows, uint64_t row_bytes, uint64_t byte0, uint64_t nbytes, int8_t* out) {
    static const int8_t t[8] = {0, 1, 2, 3, 4, 6, 8, 12};
    for (uint64_t r = 0; r < rows; ++r)
        for (uint64_t b = 0; b < nbytes; ++b) {
            const uint8_t v = packed[r * row_bytes + byte0 + b];
            const int lo = v & 15, hi = v >> 4;
            out[r * nbytes * 2 + 2 * b] = (int8_t)((lo & 8) ? -t[lo & 7] : t[lo & 7]);
            out[r * nbytes * 2 + 2 * b + 1] = (int8_t)((hi & 8) ? -t[hi & 7] : t[hi & 7]);
        }
}
static float dot_blocks(const int32_t* x, const uint8_t* xs, const int8_t* w, const uint8_t* ws, uint32_t k) {
    long double acc = 0.0L;
    for (uint32_t b = 0; b < k / 32; ++b) {
        int32_t p = 0; /* |x| <= 15 << 14, |w| <= 12: 32 products stay below 2^27 */
        for (int i = 0; i < 32; ++i) p += x[b * 32 + i] * (int32_t)w[b * 32 + i];
        const int wsb = ws[b] > 254 ? 254 : ws[b];
        acc += ldexpl((long double)p, -10 + (int)xs[b] - 127 + wsb - 127);
    }
    return (float)(double)acc;
}

/* One expert on m routed rows, one tensor-parallel slice [i0, i0+il) of the
 * intermediate dimension (lattice_oracle.py:56-90 `expert`, restricted to one
 * rank's rows and columns): gate/up FP64 dots -> FP32, activation, quantiser v1,
 * down FP64 dot over the local K -> FP32 partial. Weights in checkpoint layout:
 * gate_w/up_w u8 [2048][2048] + scales [2048][128]; down_w u8 [4096][1024] +
 * scales [4096][64]. Optional outputs may be NULL. Returns 0, 1 (input fault:
 * NaN code or scale byte outside 105..247) or 2 (intermediate quantiser fault). */
int orc_expert_ffn(const uint8_t* xq, const uint8_t* xs, uint32_t m, const uint8_t* gate_w, const uint8_t* gate_s,
                   const uint8_t* up_w, const uint8_t* up_s, const uint8_t* down_w, const uint8_t* down_s, uint32_t i0,
                   uint32_t il, float* gate_out, float* up_out, float* h_out, uint8_t* mid_q, uint8_t* mid_s, float* y_out) {
    const uint32_t H = ORC_HIDDEN;
    for (uint64_t i = 0; i < (uint64_t)m * H; ++i)
        if ((xq[i] & 0x7f) == 0x7f) return 1;
    for (uint64_t i = 0; i < (uint64_t)m * (H / 32); ++i)
        if (xs[i] < 105 || xs[i] > 247) return 1;
    int32_t* xi = (int32_t*)malloc((size_t)m * H * 4);
    int8_t* gw = (int8_t*)malloc((size_t)il * H);
    int8_t* uw = (int8_t*)malloc((size_t)il * H);
    int8_t* dw = (int8_t*)malloc((size_t)H * il);
    float* gate = (float*)malloc((size_t)m * il * 4);
    float* up = (float*)malloc((size_t)m * il * 4);
    float* h = (float*)malloc((size_t)m * il * 4);
    uint8_t* mq = (uint8_t*)malloc((size_t)m * il);
    uint8_t* msc = (uint8_t*)malloc((size_t)m * (il / 32));
    int32_t* mi = (int32_t*)malloc((size_t)m * il * 4);
    e4m3_ints(xq, (uint64_t)m * H, xi);
    e2m1_ints(gate_w + (size_t)i0 * (H / 2), il, H / 2, 0, H / 2, gw);
    e2m1_ints(up_w + (size_t)i0 * (H / 2), il, H / 2, 0, H / 2, uw);
    e2m1_ints(down_w, H, ORC_INTER / 2, i0 / 2, il / 2, dw);
    int rc = 0;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < (int64_t)il; ++n)
        for (uint32_t t = 0; t < m; ++t) {
            gate[(size_t)t * il + n] = dot_blocks(xi + (size_t)t * H, xs + (size_t)t * (H / 32), gw + (size_t)n * H,
                                                  gate_s + (size_t)(i0 + n) * (H / 32), H);
            up[(size_t)t * il + n] = dot_blocks(xi + (size_t)t * H, xs + (size_t)t * (H / 32), uw + (size_t)n * H,
                                                up_s + (size_t)(i0 + n) * (H / 32), H);
        }
    for (uint64_t i = 0; i < (uint64_t)m * il; ++i) h[i] = orc_activation(gate[i], up[i]);
    if (orc_quant_v1(h, (uint64_t)m * il, mq, msc, NULL)) rc = 2;
    if (!rc) {
        e4m3_ints(mq, (uint64_t)m * il, mi);
#pragma omp parallel for schedule(static)
        for (int64_t n = 0; n < (int64_t)H; ++n)
            for (uint32_t t = 0; t < m; ++t)
                y_out[(size_t)t * H + n] = dot_blocks(mi + (size_t)t * il, msc + (size_t)t * (il / 32), dw + (size_t)n * il,
                                                      down_s + (size_t)n * (ORC_INTER / 32) + i0 / 32, il);
        if (gate_out) memcpy(gate_out, gate, (size_t)m * il * 4);
        if (up_out) memcpy(up_out, up, (size_t)m * il * 4);
        if (h_out) memcpy(h_out, h, (size_t)m * il * 4);
        if (mid_q) memcpy(mid_q, mq, (size_t)m * il);
        if (mid_s) memcpy(mid_s, msc, (size_t)m * (il / 32));
    }
    free(xi); free(gw); free(uw); free(dw); free(gate); free(up); free(h); free(mq); free(msc); free(mi);
    return rc;
}

/* ---- BF16, ordered combine, rank sum ---------------------------------------------------------- */
/* crates/mimo26-wire/src/bf16.rs:28-42 / route_reduce.cu:52-59 */
uint16_t orc_bf16_rne(float v) {
    const uint32_t b = f32_bits(v);
    return (uint16_t)((b + 0x7fffu + ((b >> 16) & 1u)) >> 16);
}
/* crates/mimo26-expert/kernels/b1/route_reduce.cu:61-74: v = add(v, mul(w_j, z_j)), j = 0..7,
 * separate roundings; BF16 RNE; nonfinite w/z/v or BF16 overflow -> 8 (Status::nonfinite). */
int orc_route_reduce_h(const float* y, const float* w, uint32_t rows, uint32_t hidden, float* partial, uint16_t* bf16) {
    const float mx = 3.402823466e+38f;
    for (uint64_t i = 0; i < (uint64_t)rows * hidden; ++i) {
        const uint64_t row = i / hidden, col = i % hidden;
        volatile float v = 0.0f;
        for (int j = 0; j < ORC_TOPK; ++j) {
            const float wt = w[row * ORC_TOPK + j];
            const float z = y[(row * ORC_TOPK + j) * hidden + col];
            if (!(wt >= 0.0f && wt <= mx) || !(z >= -mx && z <= mx)) return 8;
            volatile float prod = wt * z;
            v = v + prod;
            if (!(v >= -mx && v <= mx)) return 8;
        }
        const uint16_t code = orc_bf16_rne(v);
        if ((code & 0x7f80u) == 0x7f80u) return 8;
        if (partial) partial[i] = v;
        bf16[i] = code;
    }
    return 0;
}
int orc_route_reduce(const float* y, const float* w, uint32_t rows, float* partial, uint16_t* bf16) {
    return orc_route_reduce_h(y, w, rows, ORC_HIDDEN, partial, bf16);
}
/* crates/mimo26-coordinator/kernels/glue.cu:202-213, crates/mimo26-wire/src/l4.rs:169-244:
 * s = 0; s += f32(bf16_r) in rank order. planes is [n_ranks][n]. */
void orc_rank_sum(const uint16_t* planes, uint32_t n_ranks, uint64_t n, float* out) {
    for (uint64_t i = 0; i < n; ++i) {
        volatile float s = 0.0f;
        for (uint32_t r = 0; r < n_ranks; ++r) s = s + bits_f32((uint32_t)planes[(uint64_t)r * n + i] << 16);
        out[i] = s;
    }
}

/* ---- router (the caller's step before the path) ---------------------------------------------
 * crates/mimo26-coordinator/src/router.rs:42-80 (router_from_logits), Python twin
 * oracle/mimo26/nn/layers.py::router: FP64 sigmoid of the FP32 logits; the top_k experts by
 * score + bias, descending, a tie going to the lower expert id (stable sort over ascending ids);
 * weights = unbiased scores over their sum, the sum taken in selection order, in FP64, then FP32. */
void orc_router_from_logits(const float* logits, const float* bias, uint32_t rows, uint32_t n_experts, uint32_t top_k,
                            int32_t* idx_out, float* w_out) {
    double* score = (double*)malloc(sizeof(double) * n_experts);
    double* sel = (double*)malloc(sizeof(double) * n_experts);
    for (uint32_t r = 0; r < rows; ++r) {
        for (uint32_t e = 0; e < n_experts; ++e) {
            const double s = (double)logits[(size_t)r * n_experts + e];
            score[e] = 1.0 / (1.0 + exp(-s));
            sel[e] = score[e] + (bias ? (double)bias[e] : 0.0);
        }
        double wsum = 0.0;
        for (uint32_t k = 0; k < top_k; ++k) {          /* k-th pass of a stable descending selection */
            uint32_t best = 0;
            int have = 0;
            for (uint32_t e = 0; e < n_experts; ++e) {
                if (isnan(sel[e])) continue;             /* taken */
                if (!have || sel[e] > sel[best]) { best = e; have = 1; }
            }
            idx_out[(size_t)r * top_k + k] = (int32_t)best;
            wsum += score[best];
            sel[best] = NAN;
        }
        for (uint32_t k = 0; k < top_k; ++k)
            w_out[(size_t)r * top_k + k] = (float)(score[idx_out[(size_t)r * top_k + k]] / wsum);
    }
    free(score);
    free(sel);
}

/* ---- one layer on one rank ------------------------------------------------------------------
 * The reference's rank FFN (crates/mimo26-spark/kernels/b1_serve.cu:312-572) on
 * the lattice above: plan, per-expert FFN on the expert's rows in stable
 * grouped order, unweighted FP32 rows back in original route order, ordered
 * weighted combine, BF16. Weights: checkpoint tensors stacked over experts
 * (only experts that receive a route are touched). Optional dumps in grouped
 * order: h_g [routes][il], midq_g [routes][il], mids_g [routes][il/32].
 * Returns 0, 3 (plan rejected), 4 (numerical fault). */
int orc_ffn_layer(const uint8_t* gate_w, const uint8_t* gate_s, const uint8_t* up_w, const uint8_t* up_s,
                  const uint8_t* down_w, const uint8_t* down_s, uint32_t tp_rank, uint32_t tp_size, const uint8_t* xq,
                  const uint8_t* xs, const int32_t* ids, const float* w, uint32_t rows, float* y_routes, float* partial,
                  uint16_t* bf16, float* h_g, uint8_t* midq_g, uint8_t* mids_g) {
    const uint32_t routes = rows * ORC_TOPK, il = ORC_INTER / tp_size, i0 = tp_rank * il, H = ORC_HIDDEN;
    uint8_t resident[ORC_EXPERTS];
    memset(resident, 1, sizeof resident);
    int32_t* inverse = (int32_t*)malloc((size_t)routes * 4);
    int32_t* original = (int32_t*)malloc((size_t)routes * 4);
    float* gwts = (float*)malloc((size_t)routes * 4);
    uint32_t counts[ORC_EXPERTS];
    int rc = orc_plan(ids, w, rows, resident, inverse, original, gwts, counts) ? 3 : 0;
    uint32_t base = 0;
    for (int e = 0; e < ORC_EXPERTS && !rc; ++e) {
        const uint32_t m = counts[e];
        if (!m) continue;
        uint8_t* xe = (uint8_t*)malloc((size_t)m * H);
        uint8_t* se = (uint8_t*)malloc((size_t)m * (H / 32));
        float* ye = (float*)malloc((size_t)m * H * 4);
        for (uint32_t t = 0; t < m; ++t) {
            const uint32_t token = (uint32_t)original[base + t] / ORC_TOPK;
            memcpy(xe + (size_t)t * H, xq + (size_t)token * H, H);
            memcpy(se + (size_t)t * (H / 32), xs + (size_t)token * (H / 32), H / 32);
        }
        const size_t gw_e = (size_t)e * ORC_INTER * (H / 2), gs_e = (size_t)e * ORC_INTER * (H / 32);
        const size_t dw_e = (size_t)e * H * (ORC_INTER / 2), ds_e = (size_t)e * H * (ORC_INTER / 32);
        const int f = orc_expert_ffn(xe, se, m, gate_w + gw_e, gate_s + gs_e, up_w + gw_e, up_s + gs_e, down_w + dw_e,
                                     down_s + ds_e, i0, il, NULL, NULL, h_g ? h_g + (size_t)base * il : NULL,
                                     midq_g ? midq_g + (size_t)base * il : NULL,
                                     mids_g ? mids_g + (size_t)base * (il / 32) : NULL, ye);
        if (f) rc = 4;
        else
            for (uint32_t t = 0; t < m; ++t) memcpy(y_routes + (size_t)original[base + t] * H, ye + (size_t)t * H, (size_t)H * 4);
        free(xe); free(se); free(ye);
        base += m;
    }
    if (!rc && orc_route_reduce(y_routes, w, rows, partial, bf16)) rc = 4;
    free(inverse); free(original); free(gwts);
    return rc;
}

/* ---- the reference's CPU expert path (timed baseline) -------------------------------------------
 * crates/mimo26-spark/src/main.rs:75-95 (no-cuda serve path): decode_hidden
 * (serve.rs:33-61) -> per-expert gate/up/down with on-the-fly MXFP4 decode and a
 * sequential FP32 accumulator (crates/mimo26-expert/src/grouped.rs:315-334),
 * silu(x) = x / (1 + exp(-x)) (grouped.rs:359-361), no intermediate
 * quantisation -> cpu_reduce_bf16 (crates/mimo26-spark/src/decode.rs:777-792).
 * This is the E-FP32 lattice the reference runs on CPU, threaded here over
 * output rows with OpenMP. Experts [e_lo, e_hi) only, so a bounded sample of a
 * workload can be timed. out_f32 [rows][4096] accumulates w * y over the
 * sampled experts. Returns the number of routed rows processed. */
uint32_t orc_cpu_path(const uint8_t* gate_w, const uint8_t* gate_s, const uint8_t* up_w, const uint8_t* up_s,
                      const uint8_t* down_w, const uint8_t* down_s, const uint8_t* xq, const uint8_t* xs,
                      const int32_t* ids, const float* w, uint32_t rows, uint32_t e_lo, uint32_t e_hi, float* out_f32,
                      uint16_t* out_bf16) {
    const uint32_t H = ORC_HIDDEN, I = ORC_INTER, routes = rows * ORC_TOPK;
    static const float cb[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f, -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};
    double pow2[256];
    for (int b = 0; b < 256; ++b) pow2[b] = ldexp(1.0, (b > 254 ? 254 : b) - 127);
    float* x = (float*)malloc((size_t)rows * H * 4);
    for (uint32_t t = 0; t < rows; ++t)
        for (uint32_t k = 0; k < H; ++k) {
            double v = (double)orc_e4m3_decode(xq[(size_t)t * H + k]) * pow2[xs[(size_t)t * (H / 32) + k / 32]];
            if (v > 3.4028234663852886e38) v = 3.4028234663852886e38;
            if (v < -3.4028234663852886e38) v = -3.4028234663852886e38;
            x[(size_t)t * H + k] = (float)v;
        }
    /* rows of the sampled experts, in expert order; slot[r] = row of route r or -1 */
    int32_t* slot = (int32_t*)malloc((size_t)routes * 4);
    uint32_t total = 0;
    for (uint32_t r = 0; r < routes; ++r) slot[r] = -1;
    for (uint32_t e = e_lo; e < e_hi; ++e)
        for (uint32_t r = 0; r < routes; ++r)
            if (ids[r] == (int32_t)e) slot[r] = (int32_t)total++;
    float* y = (float*)malloc((size_t)(total ? total : 1) * H * 4);
    float* hbuf = (float*)malloc((size_t)rows * I * 4);
    uint32_t* rt = (uint32_t*)malloc((size_t)rows * 4);
    for (uint32_t e = e_lo; e < e_hi; ++e) {
        uint32_t m = 0;
        for (uint32_t r = 0; r < routes; ++r)
            if (ids[r] == (int32_t)e) rt[m++] = r;
        if (!m) continue;
        const uint8_t* gp = gate_w + (size_t)e * I * (H / 2); const uint8_t* gs = gate_s + (size_t)e * I * (H / 32);
        const uint8_t* upp = up_w + (size_t)e * I * (H / 2); const uint8_t* us = up_s + (size_t)e * I * (H / 32);
        const uint8_t* dp = down_w + (size_t)e * H * (I / 2); const uint8_t* ds = down_s + (size_t)e * H * (I / 32);
#pragma omp parallel for schedule(static)
        for (int64_t n = 0; n < (int64_t)I; ++n)
            for (uint32_t t = 0; t < m; ++t) {
                const float* xr = x + (size_t)(rt[t] / ORC_TOPK) * H;
                float g = 0.0f, u = 0.0f;
                for (uint32_t k = 0; k < H; ++k) {
                    const uint8_t gb = gp[(size_t)n * (H / 2) + k / 2], ub = upp[(size_t)n * (H / 2) + k / 2];
                    const float gwv = (float)((double)cb[(k & 1) ? gb >> 4 : gb & 15] * pow2[gs[(size_t)n * (H / 32) + k / 32]]);
                    const float uwv = (float)((double)cb[(k & 1) ? ub >> 4 : ub & 15] * pow2[us[(size_t)n * (H / 32) + k / 32]]);
                    g += gwv * xr[k];
                    u += uwv * xr[k];
                }
                hbuf[(size_t)t * I + n] = (g / (1.0f + expf(-g))) * u;
            }
#pragma omp parallel for schedule(static)
        for (int64_t n = 0; n < (int64_t)H; ++n)
            for (uint32_t t = 0; t < m; ++t) {
                float acc = 0.0f;
                for (uint32_t k = 0; k < I; ++k) {
                    const uint8_t b = dp[(size_t)n * (I / 2) + k / 2];
                    const float wv = (float)((double)cb[(k & 1) ? b >> 4 : b & 15] * pow2[ds[(size_t)n * (I / 32) + k / 32]]);
                    acc += wv * hbuf[(size_t)t * I + k];
                }
                y[(size_t)slot[rt[t]] * H + n] = acc;
            }
    }
    /* cpu_reduce_bf16: token-major, slot order, out += y * w */
    memset(out_f32, 0, (size_t)rows * H * 4);
    for (uint32_t r = 0; r < routes; ++r) {
        if (slot[r] < 0) continue;
        float* o = out_f32 + (size_t)(r / ORC_TOPK) * H;
        const float* yr = y + (size_t)slot[r] * H;
        for (uint32_t n = 0; n < H; ++n) o[n] += yr[n] * w[r];
    }
    if (out_bf16)
        for (uint64_t i = 0; i < (uint64_t)rows * H; ++i) out_bf16[i] = orc_bf16_rne(out_f32[i]);
    free(x); free(hbuf); free(rt); free(slot); free(y);
    return total;
}
