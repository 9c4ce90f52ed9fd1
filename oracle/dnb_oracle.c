/* CPU oracle for the quantised-MoE expert path -- TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of denno-beta's own CPU implementation of the path
 * (crates/denno-engine/src/...), function by function, in the same fp32
 * operation order.  It is what the CUDA library is checked against; it is not
 * part of the library and nothing the library ships may call it.  Only the
 * tests, the smoke check and the benchmark's CPU-baseline leg load it.
 *
 * Parity pins: every dequantiser below is checked bit-for-bit against the
 * llama.cpp-generated vectors of the reference's tests/data/dequant_ref.bin,
 * and the MoE order against the hard-coded answers of model/moe.rs's tests
 * (see tests/test_oracle_*.py).
 *
 * Build: gcc -O2 -ffp-contract=off (no fast-math: the sequential fp32 order is
 * the contract).  The *_mt functions are the timed multi-threaded variants and
 * are compiled in the same unit with OpenMP.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "dnb_iq_tables.h"
#include "dnb_synth.h"
#include "dnb_oracle.h"

#define QK_K 256

/* ---- scalar helpers ------------------------------------------------------ */

/* IEEE binary16 -> binary32, exact (subnormals included).
 * Reference: kquant.rs:224-227 (half::f16::to_f32). */
static float f16_to_f32(const uint8_t* p) {
    const uint32_t h = (uint32_t)p[0] | ((uint32_t)p[1] << 8);
    const uint32_t sign = (h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do { man <<= 1; ++e; } while ((man & 0x400u) == 0);
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

static uint32_t rd_u32(const uint8_t* b) {
    return (uint32_t)b[0] | ((uint32_t)b[1] << 8) | ((uint32_t)b[2] << 16) | ((uint32_t)b[3] << 24);
}

/* kquant.rs:172-217 */
int orc_blck_size(int type) {
    switch (type) {
        case 0: return 1;
        case 2: case 7: case 8: case 20: return 32;
        case 42: return 64;
        case 12: case 13: case 14: case 18: case 21: case 22: case 23: return 256;
        default: return 0;
    }
}

int orc_type_size(int type) {
    switch (type) {
        case 0: return 4;
        case 2: return 18;   /* Q4_0 */
        case 7: return 24;   /* Q5_1 */
        case 8: return 34;   /* Q8_0 */
        case 12: return 144; /* Q4_K */
        case 13: return 176; /* Q5_K */
        case 14: return 210; /* Q6_K */
        case 18: return 98;  /* IQ3_XXS */
        case 20: return 18;  /* IQ4_NL */
        case 21: return 110; /* IQ3_S */
        case 22: return 82;  /* IQ2_S */
        case 23: return 136; /* IQ4_XS */
        case 42: return 18;  /* Q2_0 */
        default: return 0;
    }
}

/* moe_expert.rs:84-100 (row_bytes): bytes of one row of n_in elements, or -1. */
long orc_row_bytes(int type, long n_in) {
    const int bs = orc_blck_size(type), ts = orc_type_size(type);
    if (bs == 0 || ts == 0 || n_in <= 0 || n_in % bs != 0) return -1;
    return (n_in / bs) * ts;
}

/* kquant.rs:878-887 */
static void get_scale_min_k4(int j, const uint8_t* q, uint8_t* sc, uint8_t* m) {
    if (j < 4) {
        *sc = q[j] & 63;
        *m = q[j + 4] & 63;
    } else {
        *sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

/* One block -> blck_size floats.  Reference: kquant.rs:341-874 (dequant_block),
 * same element order and the same association of every product.  The sign of
 * the IQ formats is applied as a negation of (db * grid): for every finite
 * value that equals the reference's multiplication by +-1.0, and it is also what
 * the golden vectors hold for NaN scales (the sign bit of the NaN flips). */
static void dequant_block(int type, const uint8_t* x, float* y) {
    switch (type) {
        case 42: { /* Q2_0, kquant.rs:347-354 */
            const float d = f16_to_f32(x);
            for (int j = 0; j < 64; ++j) {
                const int q = (x[2 + j / 4] >> ((j % 4) * 2)) & 3;
                y[j] = (float)(q - 1) * d;
            }
        } break;
        case 2: { /* Q4_0, kquant.rs:357-365 */
            const float d = f16_to_f32(x);
            for (int j = 0; j < 16; ++j) {
                y[j] = (float)((x[2 + j] & 0x0F) - 8) * d;
                y[j + 16] = (float)((x[2 + j] >> 4) - 8) * d;
            }
        } break;
        case 7: { /* Q5_1, kquant.rs:394-406 */
            const float d = f16_to_f32(x), m = f16_to_f32(x + 2);
            const uint32_t qh = rd_u32(x + 4);
            for (int j = 0; j < 16; ++j) {
                const int xh0 = (int)(((qh >> j) << 4) & 0x10);
                const int xh1 = (int)((qh >> (j + 12)) & 0x10);
                const int x0 = (x[8 + j] & 0x0F) | xh0;
                const int x1 = (x[8 + j] >> 4) | xh1;
                y[j] = (float)x0 * d + m;
                y[j + 16] = (float)x1 * d + m;
            }
        } break;
        case 8: { /* Q8_0, kquant.rs:409-414 */
            const float d = f16_to_f32(x);
            for (int j = 0; j < 32; ++j) y[j] = (float)(int8_t)x[2 + j] * d;
        } break;
        case 12: { /* Q4_K, kquant.rs:505-526 */
            const float d = f16_to_f32(x), dmin = f16_to_f32(x + 2);
            int yi = 0, is = 0;
            for (int j = 0; j < QK_K; j += 64) {
                const uint8_t* q = x + 16 + j / 2;
                uint8_t sc, m;
                get_scale_min_k4(is, x + 4, &sc, &m);
                const float d1 = d * (float)sc, m1 = dmin * (float)m;
                get_scale_min_k4(is + 1, x + 4, &sc, &m);
                const float d2 = d * (float)sc, m2 = dmin * (float)m;
                for (int l = 0; l < 32; ++l) y[yi++] = d1 * (float)(q[l] & 0xF) - m1;
                for (int l = 0; l < 32; ++l) y[yi++] = d2 * (float)(q[l] >> 4) - m2;
                is += 2;
            }
        } break;
        case 13: { /* Q5_K, kquant.rs:529-558 */
            const float d = f16_to_f32(x), dmin = f16_to_f32(x + 2);
            const uint8_t* qh = x + 16;
            int yi = 0, is = 0;
            uint8_t u1 = 1, u2 = 2;
            for (int j = 0; j < QK_K; j += 64) {
                const uint8_t* ql = x + 48 + j / 2;
                uint8_t sc, m;
                get_scale_min_k4(is, x + 4, &sc, &m);
                const float d1 = d * (float)sc, m1 = dmin * (float)m;
                get_scale_min_k4(is + 1, x + 4, &sc, &m);
                const float d2 = d * (float)sc, m2 = dmin * (float)m;
                for (int l = 0; l < 32; ++l) {
                    const float v = (float)((ql[l] & 0xF) + ((qh[l] & u1) ? 16 : 0));
                    y[yi++] = d1 * v - m1;
                }
                for (int l = 0; l < 32; ++l) {
                    const float v = (float)((ql[l] >> 4) + ((qh[l] & u2) ? 16 : 0));
                    y[yi++] = d2 * v - m2;
                }
                is += 2;
                u1 <<= 2;
                u2 <<= 2;
            }
        } break;
        case 14: { /* Q6_K, kquant.rs:561-583 */
            const float d = f16_to_f32(x + 208);
            int yi = 0;
            for (int n = 0; n < QK_K; n += 128) {
                const uint8_t* ql = x + n / 2;
                const uint8_t* qh = x + 128 + n / 4;
                const int8_t* sc = (const int8_t*)(x + 192 + n / 16);
                for (int l = 0; l < 32; ++l) {
                    const int is = l / 16;
                    const int q1 = ((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
                    const int q2 = ((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
                    const int q3 = ((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                    const int q4 = ((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                    y[yi + l] = d * (float)sc[is] * (float)q1;
                    y[yi + l + 32] = d * (float)sc[is + 2] * (float)q2;
                    y[yi + l + 64] = d * (float)sc[is + 4] * (float)q3;
                    y[yi + l + 96] = d * (float)sc[is + 6] * (float)q4;
                }
                yi += 128;
            }
        } break;
        case 22: { /* IQ2_S, kquant.rs:632-656 */
            const float d = f16_to_f32(x);
            const uint8_t *qs = x + 2, *qh = x + 66, *signs = x + 34, *scales = x + 74;
            int yi = 0;
            for (int ib = 0; ib < 8; ++ib) {
                const float db0 = d * (0.5f + (float)(scales[ib] & 0xF)) * 0.25f;
                const float db1 = d * (0.5f + (float)(scales[ib] >> 4)) * 0.25f;
                for (int l = 0; l < 4; ++l) {
                    const uint32_t idx = (uint32_t)qs[ib * 4 + l] | (((uint32_t)qh[ib] << (8 - 2 * l)) & 0x300u);
                    const uint64_t grid = dnb_iq2s_grid[idx];
                    const uint8_t sg = signs[ib * 4 + l];
                    const float db = (l / 2 == 0) ? db0 : db1;
                    for (int j = 0; j < 8; ++j) {
                        const float v = db * (float)(uint8_t)(grid >> (8 * j));
                        y[yi + j] = (sg & (1u << j)) ? -v : v;
                    }
                    yi += 8;
                }
            }
        } break;
        case 18: { /* IQ3_XXS, kquant.rs:659-680 */
            const float d = f16_to_f32(x);
            const uint8_t *qs = x + 2, *ss = x + 2 + QK_K / 4;
            int yi = 0;
            for (int ib = 0; ib < 8; ++ib) {
                const uint32_t aux = rd_u32(ss + 4 * ib);
                const float db = d * (0.5f + (float)(aux >> 28)) * 0.5f;
                for (int l = 0; l < 4; ++l) {
                    const uint8_t sg = dnb_ksigns_iq2xs[(aux >> (7 * l)) & 127];
                    const uint32_t g1 = dnb_iq3xxs_grid[qs[ib * 8 + 2 * l]];
                    const uint32_t g2 = dnb_iq3xxs_grid[qs[ib * 8 + 2 * l + 1]];
                    for (int j = 0; j < 4; ++j) {
                        const float v0 = db * (float)(uint8_t)(g1 >> (8 * j));
                        const float v1 = db * (float)(uint8_t)(g2 >> (8 * j));
                        y[yi + j] = (sg & (1u << j)) ? -v0 : v0;
                        y[yi + j + 4] = (sg & (1u << (j + 4))) ? -v1 : v1;
                    }
                    yi += 8;
                }
            }
        } break;
        case 21: { /* IQ3_S, kquant.rs:683-735 */
            const float d = f16_to_f32(x);
            const uint8_t *qs = x + 2, *qh = x + 66, *signs = x + 74, *scales = x + 106;
            int yi = 0;
            for (int ib = 0; ib < 8; ++ib) {
                const uint8_t scb = scales[ib / 2];
                const float db = d * (1.0f + 2.0f * (float)((ib & 1) ? (scb >> 4) : (scb & 0xF)));
                for (int l = 0; l < 4; ++l) {
                    const uint32_t g1 = dnb_iq3s_grid[(uint32_t)qs[ib * 8 + 2 * l] | (((uint32_t)qh[ib] << (8 - 2 * l)) & 256u)];
                    const uint32_t g2 = dnb_iq3s_grid[(uint32_t)qs[ib * 8 + 2 * l + 1] | (((uint32_t)qh[ib] << (7 - 2 * l)) & 256u)];
                    const uint8_t sg = signs[ib * 4 + l];
                    for (int j = 0; j < 4; ++j) {
                        const float v0 = db * (float)(uint8_t)(g1 >> (8 * j));
                        const float v1 = db * (float)(uint8_t)(g2 >> (8 * j));
                        y[yi + j] = (sg & (1u << j)) ? -v0 : v0;
                        y[yi + j + 4] = (sg & (1u << (j + 4))) ? -v1 : v1;
                    }
                    yi += 8;
                }
            }
        } break;
        case 20: { /* IQ4_NL, kquant.rs:842-853 */
            const float d = f16_to_f32(x);
            for (int j = 0; j < 16; ++j) {
                y[j] = d * (float)dnb_kvalues_iq4nl[x[2 + j] & 0xF];
                y[j + 16] = d * (float)dnb_kvalues_iq4nl[x[2 + j] >> 4];
            }
        } break;
        case 23: { /* IQ4_XS, kquant.rs:856-872 */
            const float d = f16_to_f32(x);
            const uint32_t scales_h = (uint32_t)x[2] | ((uint32_t)x[3] << 8);
            const uint8_t *scales_l = x + 4, *qs = x + 8;
            int yi = 0;
            for (int ib = 0; ib < 8; ++ib) {
                const int ls = (int)((scales_l[ib / 2] >> (4 * (ib % 2))) & 0xF) | (int)(((scales_h >> (2 * ib)) & 3) << 4);
                const float dl = d * (float)(ls - 32);
                for (int j = 0; j < 16; ++j) {
                    y[yi + j] = dl * (float)dnb_kvalues_iq4nl[qs[ib * 16 + j] & 0xF];
                    y[yi + j + 16] = dl * (float)dnb_kvalues_iq4nl[qs[ib * 16 + j] >> 4];
                }
                yi += 32;
            }
        } break;
        default: break;
    }
}

/* kquant.rs:290-318 (dequant_row_into).  Returns 0, or -1 for an unknown type /
 * a length that is not a whole number of blocks. */
int orc_dequant_row(int type, const uint8_t* blocks, long n, float* out) {
    const int bs = orc_blck_size(type), ts = orc_type_size(type);
    if (bs == 0 || n % bs != 0) return -1;
    if (type == 0) {
        memcpy(out, blocks, (size_t)n * 4);
        return 0;
    }
    for (long i = 0; i < n / bs; ++i) dequant_block(type, blocks + i * ts, out + i * bs);
    return 0;
}

/* moe_expert.rs:107-114 (dot_seq) and moe.rs:64-72 (dot_row): ascending i,
 * one rounding for the product and one for the sum. */
static float dot_seq(const float* w, const float* x, long n) {
    float acc = 0.0f;
    for (long i = 0; i < n; ++i) acc += w[i] * x[i];
    return acc;
}

/* moe_expert.rs:698-713 + 4722-4733 (expert_gemv_scalar). */
int orc_gemv_scalar(int type, const uint8_t* blocks, long n_in, long n_out, const float* x, float* out) {
    const long rb = orc_row_bytes(type, n_in);
    if (rb < 0 || n_out <= 0) return -1;
    float* row = (float*)malloc((size_t)n_in * sizeof(float));
    for (long r = 0; r < n_out; ++r) {
        orc_dequant_row(type, blocks + r * rb, n_in, row);
        out[r] = dot_seq(row, x, n_in);
    }
    free(row);
    return 0;
}

/* The same GEMV with the dot product carried in double: the "truth" used to
 * judge which of two fp32 evaluation orders is closer (moe_expert.rs tests use
 * an f64 reference the same way, moe_expert.rs:8516-8760). */
int orc_gemv_f64(int type, const uint8_t* blocks, long n_in, long n_out, const float* x, double* out) {
    const long rb = orc_row_bytes(type, n_in);
    if (rb < 0 || n_out <= 0) return -1;
    float* row = (float*)malloc((size_t)n_in * sizeof(float));
    for (long r = 0; r < n_out; ++r) {
        orc_dequant_row(type, blocks + r * rb, n_in, row);
        double acc = 0.0;
        for (long i = 0; i < n_in; ++i) acc += (double)row[i] * (double)x[i];
        out[r] = acc;
    }
    free(row);
    return 0;
}

/* tensor.rs:1125-1135 (rmsnorm_into): rows of `cols`. */
void orc_rmsnorm(const float* x, const float* w, long rows, long cols, float eps, float* out) {
    for (long r = 0; r < rows; ++r) {
        const float* xi = x + r * cols;
        float ss = 0.0f;
        for (long i = 0; i < cols; ++i) ss += xi[i] * xi[i];
        ss = ss / (float)cols;
        const float inv = 1.0f / sqrtf(ss + eps);
        for (long i = 0; i < cols; ++i) out[r * cols + i] = xi[i] * inv * w[i];
    }
}

/* tensor.rs:1171-1183 (softmax, max-subtracted, in place). */
void orc_softmax(float* x, long n) {
    float mx = -INFINITY;
    for (long i = 0; i < n; ++i) mx = (x[i] > mx) ? x[i] : mx; /* f32::max ignores NaN on the right */
    float sum = 0.0f;
    for (long i = 0; i < n; ++i) {
        x[i] = expf(x[i] - mx);
        sum += x[i];
    }
    if (sum > 0.0f)
        for (long i = 0; i < n; ++i) x[i] /= sum;
}

/* tensor.rs:1164-1168 (silu) and hyper.rs:112-114 (sigmoid). */
float orc_silu(float v) { return v / (1.0f + expf(-v)); }
float orc_sigmoid(float v) { return 1.0f / (1.0f + expf(-v)); }

/* ---- hyper-connection mix / combine: model/hyper.rs ---------------------------------------------------------------
 * The file states its order of operations as the numeric contract (hyper.rs:13-36); every product and sum below is
 * a separate f32 operation in that order (this file is compiled with contraction off).
 * Pinned by the reference's hard-coded anchor (tests/hyper.rs:321-365: mixed, inject and combine to the bit). */

/* hyper.rs:131-138 (dot_row): sequential f32, multiply then add. */
static float hc_dot_row(const float* w, const float* x, long n) {
    float acc = 0.0f;
    for (long i = 0; i < n; ++i) acc += w[i] * x[i];
    return acc;
}

/* hyper.rs:160-222 (mix_internal with w_down_inject) for one token.
 *   x [hc][e], w_norm [hc][e], w_down_inject [low_rank + hc][hc*e], w_up [hc*e][low_rank]
 *   -> mixed [e], inject [hc]; xn_out (optional) [hc][e]. */
void orc_hc_mix(const float* x, const float* w_norm, const float* w_down_inject, const float* w_up, long hc, long e,
                long low_rank, float eps, float* mixed, float* inject, float* xn_out) {
    const long hc_dim = hc * e;
    float* xn = (float*)malloc(sizeof(float) * (size_t)hc_dim);
    float* lo = (float*)malloc(sizeof(float) * (size_t)low_rank);
    const float inv_hc = 1.0f / (float)hc;
    /* steps 1-3: per-stream rmsnorm, gamma folded into the same x*inv*w product (hyper.rs:144-157) */
    for (long s = 0; s < hc; ++s) orc_rmsnorm(x + s * e, w_norm + s * e, 1, e, eps, xn + s * e);
    /* steps 4-5 (hc_lo_apply, hyper.rs:255-262): 1/hc after the matmul, then silu(v) = v * sigmoid(v) */
    for (long r = 0; r < low_rank; ++r) {
        float v = hc_dot_row(w_down_inject + r * hc_dim, xn, hc_dim);
        v = v * inv_hc;
        lo[r] = v * orc_sigmoid(v);
    }
    /* inject rows: scaled, no silu (hc_inject_apply, hyper.rs:354-359) */
    for (long r = 0; r < hc; ++r) inject[r] = hc_dot_row(w_down_inject + (low_rank + r) * hc_dim, xn, hc_dim) * inv_hc;
    /* steps 6-8 (mixed_range, hyper.rs:279-304): the first stream's term starts the sum, 1/hc last */
    for (long d = 0; d < e; ++d) {
        float acc = 0.0f;
        for (long s = 0; s < hc; ++s) {
            const float g = hc_dot_row(w_up + (s * e + d) * low_rank, lo, low_rank);
            const float term = xn[s * e + d] * orc_sigmoid(g);
            acc = (s == 0) ? term : acc + term;
        }
        mixed[d] = acc * inv_hc;
    }
    if (xn_out) memcpy(xn_out, xn, sizeof(float) * (size_t)hc_dim);
    free(lo);
    free(xn);
}

/* hyper.rs:384-416 (hc_combine): out[s][d] = residual[s][d] + block[d] * (2 * sigmoid(inject[s])). */
void orc_hc_combine(const float* residual, const float* block, const float* inject, long hc, long e, float* out) {
    for (long s = 0; s < hc; ++s) {
        const float w = 2.0f * orc_sigmoid(inject[s]);
        for (long d = 0; d < e; ++d) out[s * e + d] = residual[s * e + d] + block[d] * w;
    }
}

/* moe.rs:256-279 (select_topk_scan): k passes, strict '>' so ties keep the lower
 * index, NaN only chosen when nothing else is left; output ascending.  The
 * faster forms in moe.rs:188-250 are specified to return the same set. */
void orc_select_topk(const float* probs, long n, long k, int32_t* out) {
    uint8_t* used = (uint8_t*)calloc((size_t)n, 1);
    for (long s = 0; s < k; ++s) {
        long best = -1;
        for (long i = 0; i < n; ++i) {
            if (used[i]) continue;
            if (best < 0 || probs[i] > probs[best]) best = i;
        }
        used[best] = 1;
        out[s] = (int32_t)best;
    }
    free(used);
    for (long a = 1; a < k; ++a) { /* insertion sort ascending */
        const int32_t v = out[a];
        long b = a - 1;
        while (b >= 0 && out[b] > v) { out[b + 1] = out[b]; --b; }
        out[b + 1] = v;
    }
}

/* qwen4exp.rs:11802-11821 / 17680-17697 (router_renorm). */
void orc_router_renorm(const float* probs, const int32_t* sel, long k, float* w) {
    float sum = 0.0f;
    for (long t = 0; t < k; ++t) sum += probs[sel[t]];
    if (isfinite(sum) && sum > 0.0f) {
        for (long t = 0; t < k; ++t) w[t] = probs[sel[t]] / sum;
    } else {
        const float u = 1.0f / (float)(k > 0 ? k : 1);
        for (long t = 0; t < k; ++t) w[t] = u;
    }
}

/* Router for nt tokens: logits (fp32 rows, sequential dot) + bias -> softmax ->
 * top-k -> renorm.  moe.rs:331-361; qwen4exp.rs:11729-11821 (decode),
 * 17990-18108 (prefill rows).  probs_out (nt*ne) may be NULL. */
void orc_router(const float* x, long nt, long e, const float* w_r, const float* bias, long ne, long k,
                int norm_topk, int32_t* sels, float* wts, float* probs_out) {
    float* probs = (float*)malloc((size_t)ne * sizeof(float));
    for (long t = 0; t < nt; ++t) {
        for (long i = 0; i < ne; ++i) {
            float v = dot_seq(w_r + i * e, x + t * e, e);
            if (bias) v += bias[i];
            probs[i] = v;
        }
        orc_softmax(probs, ne);
        orc_select_topk(probs, ne, k, sels + t * k);
        if (norm_topk) {
            orc_router_renorm(probs, sels + t * k, k, wts + t * k);
        } else {
            for (long s = 0; s < k; ++s) wts[t * k + s] = probs[sels[t * k + s]];
        }
        if (probs_out) memcpy(probs_out + t * ne, probs, (size_t)ne * sizeof(float));
    }
    free(probs);
}

/* ---- fp32 MoE (moe.rs:284-405, moe_ffn) ---------------------------------- */

static void expert_ffn_f32(const float* x, const float* gw, const float* uw, const float* dw, long e, long ff,
                           float* act, float* h) {
    for (long r = 0; r < ff; ++r) act[r] = dot_seq(gw + r * e, x, e);
    for (long r = 0; r < ff; ++r) act[r] = orc_silu(act[r]);
    for (long r = 0; r < ff; ++r) act[r] *= dot_seq(uw + r * e, x, e);
    for (long j = 0; j < e; ++j) h[j] = dot_seq(dw + j * ff, act, ff);
}

void orc_moe_ffn_f32(const float* x, long e, long ff, long ne, long k, int norm_topk, const float* gate_inp,
                     const float* bias, const float* gate_exps, const float* up_exps, const float* down_exps,
                     const float* sh_gate, const float* sh_up, const float* sh_down, long sff, float* out) {
    int32_t* sel = (int32_t*)malloc((size_t)k * sizeof(int32_t));
    float* wts = (float*)malloc((size_t)k * sizeof(float));
    orc_router(x, 1, e, gate_inp, bias, ne, k, norm_topk, sel, wts, NULL);
    float* act = (float*)malloc((size_t)(ff > sff ? ff : sff) * sizeof(float));
    float* h = (float*)malloc((size_t)e * sizeof(float));
    for (long j = 0; j < e; ++j) out[j] = 0.0f;
    for (long t = 0; t < k; ++t) {
        const long ei = sel[t];
        expert_ffn_f32(x, gate_exps + ei * ff * e, up_exps + ei * ff * e, down_exps + ei * e * ff, e, ff, act, h);
        for (long j = 0; j < e; ++j) out[j] += wts[t] * h[j];
    }
    if (sh_gate && sh_up && sh_down) {
        expert_ffn_f32(x, sh_gate, sh_up, sh_down, e, sff, act, h);
        for (long j = 0; j < e; ++j) out[j] += h[j];
    }
    free(sel); free(wts); free(act); free(h);
}

/* ---- quantised experts ---------------------------------------------------- */

/* One expert FFN on GGUF blocks: gate, silu, up, product, down, each GEMV being
 * expert_gemv_scalar.  qwen4exp.rs:12170-12181 (statement order gate -> silu ->
 * up -> mul -> down). */
static void expert_ffn_q(const float* x, int ty_g, const uint8_t* wg, int ty_u, const uint8_t* wu, int ty_d,
                         const uint8_t* wd, long e, long ff, float* act, float* up, float* h) {
    orc_gemv_scalar(ty_g, wg, e, ff, x, act);
    for (long r = 0; r < ff; ++r) act[r] = orc_silu(act[r]);
    orc_gemv_scalar(ty_u, wu, e, ff, x, up);
    for (long r = 0; r < ff; ++r) act[r] *= up[r];
    orc_gemv_scalar(ty_d, wd, ff, e, act, h);
}


/* One MoE block for nt tokens, token by token, exactly the decode order:
 * (RMSNorm) -> router -> experts ascending -> out += w*h -> shared expert.
 * qwen4exp.rs:11659-12411 (moe_ffn_quant_impl); moe.rs:313-405.
 * sels_out / wts_out (nt*k) may be NULL. */
int orc_moe_block(const orc_moe_layer* L, const float* hin, long nt, float* out, int32_t* sels_out,
                  float* wts_out) {
    const long e = L->e, ff = L->ff, k = L->k;
    const long rb_g = orc_row_bytes(L->ty_gate, e), rb_u = orc_row_bytes(L->ty_up, e), rb_d = orc_row_bytes(L->ty_down, ff);
    if (rb_g < 0 || rb_u < 0 || rb_d < 0) return -1;
    float* x = (float*)malloc((size_t)e * sizeof(float));
    float* act = (float*)malloc((size_t)(ff > L->sff ? ff : L->sff) * sizeof(float));
    float* up = (float*)malloc((size_t)(ff > L->sff ? ff : L->sff) * sizeof(float));
    float* h = (float*)malloc((size_t)e * sizeof(float));
    int32_t* sel = (int32_t*)malloc((size_t)k * sizeof(int32_t));
    float* wts = (float*)malloc((size_t)k * sizeof(float));
    for (long t = 0; t < nt; ++t) {
        if (L->norm_w) orc_rmsnorm(hin + t * e, L->norm_w, 1, e, L->eps, x);
        else memcpy(x, hin + t * e, (size_t)e * sizeof(float));
        orc_router(x, 1, e, L->router_w, L->router_bias, L->ne, k, L->norm_topk, sel, wts, NULL);
        float* o = out + t * e;
        for (long j = 0; j < e; ++j) o[j] = 0.0f;
        for (long s = 0; s < k; ++s) {
            const long ei = sel[s];
            expert_ffn_q(x, L->ty_gate, L->gate + ei * ff * rb_g, L->ty_up, L->up + ei * ff * rb_u, L->ty_down,
                         L->down + ei * e * rb_d, e, ff, act, up, h);
            for (long j = 0; j < e; ++j) o[j] += wts[s] * h[j];
        }
        if (L->sgate && L->sup && L->sdown) {
            expert_ffn_q(x, L->ty_sgate, L->sgate, L->ty_sup, L->sup, L->ty_sdown, L->sdown, e, L->sff, act, up, h);
            float coef = 1.0f;
            if (L->shared_gate_row) coef = orc_sigmoid(dot_seq(L->shared_gate_row, x, e));
            if (L->shared_gate_row) { for (long j = 0; j < e; ++j) o[j] += h[j] * coef; }
            else { for (long j = 0; j < e; ++j) o[j] += h[j]; }
        }
        if (sels_out) memcpy(sels_out + t * k, sel, (size_t)k * sizeof(int32_t));
        if (wts_out) memcpy(wts_out + t * k, wts, (size_t)k * sizeof(float));
    }
    free(x); free(act); free(up); free(h); free(sel); free(wts);
    return 0;
}

/* The experts + weighted sum only, with the selection given (used to re-evaluate
 * the oracle under the GPU's selection when two router probabilities tie to
 * within rounding).  x is the (already normalised) expert input. */
int orc_moe_experts_given(const orc_moe_layer* L, const float* x, long nt, const int32_t* sels, const float* wts,
                          float* out) {
    const long e = L->e, ff = L->ff, k = L->k;
    const long rb_g = orc_row_bytes(L->ty_gate, e), rb_u = orc_row_bytes(L->ty_up, e), rb_d = orc_row_bytes(L->ty_down, ff);
    if (rb_g < 0 || rb_u < 0 || rb_d < 0) return -1;
    float* act = (float*)malloc((size_t)(ff > L->sff ? ff : L->sff) * sizeof(float));
    float* up = (float*)malloc((size_t)(ff > L->sff ? ff : L->sff) * sizeof(float));
    float* h = (float*)malloc((size_t)e * sizeof(float));
    for (long t = 0; t < nt; ++t) {
        const float* xt = x + t * e;
        float* o = out + t * e;
        for (long j = 0; j < e; ++j) o[j] = 0.0f;
        for (long s = 0; s < k; ++s) {
            const long ei = sels[t * k + s];
            expert_ffn_q(xt, L->ty_gate, L->gate + ei * ff * rb_g, L->ty_up, L->up + ei * ff * rb_u, L->ty_down,
                         L->down + ei * e * rb_d, e, ff, act, up, h);
            for (long j = 0; j < e; ++j) o[j] += wts[t * k + s] * h[j];
        }
        if (L->sgate && L->sup && L->sdown) {
            expert_ffn_q(xt, L->ty_sgate, L->sgate, L->ty_sup, L->sup, L->ty_sdown, L->sdown, e, L->sff, act, up, h);
            if (L->shared_gate_row) {
                const float coef = orc_sigmoid(dot_seq(L->shared_gate_row, xt, e));
                for (long j = 0; j < e; ++j) o[j] += h[j] * coef;
            } else {
                for (long j = 0; j < e; ++j) o[j] += h[j];
            }
        }
    }
    free(act); free(up); free(h);
    return 0;
}

/* ---- grouped (prefill) form ------------------------------------------------ */

/* orc_segment (moe_expert.rs:8272-8281) is declared in dnb_oracle.h */

/* moe_expert.rs:8309-8390 (build_grouped_batch) from a routing table: by_expert
 * lists are (token ascending) per expert; segments sorted m descending, ties
 * expert ascending; rows[] receives (token, slot) per gathered row.
 * Returns the number of segments; m_total through *m_total_out. */
long orc_build_segments(const int32_t* sels, long nt, long k, long ne, orc_segment* segs, int32_t* row_token,
                        int32_t* row_slot, long* m_total_out) {
    long* cnt = (long*)calloc((size_t)ne, sizeof(long));
    for (long i = 0; i < nt * k; ++i) cnt[sels[i]]++;
    long nseg = 0;
    for (long ei = 0; ei < ne; ++ei)
        if (cnt[ei] > 0) { segs[nseg].expert = (uint32_t)ei; segs[nseg].m = (uint32_t)cnt[ei]; nseg++; }
    for (long a = 1; a < nseg; ++a) { /* stable insertion sort: m desc, expert asc */
        const orc_segment v = segs[a];
        long b = a - 1;
        while (b >= 0 && segs[b].m < v.m) { segs[b + 1] = segs[b]; --b; }
        segs[b + 1] = v;
    }
    long row = 0;
    for (long s = 0; s < nseg; ++s) {
        segs[s].x_off = (uint32_t)row;   /* in rows; callers scale by n_in / n_out */
        segs[s].out_off = (uint32_t)row;
        for (long t = 0; t < nt; ++t)
            for (long j = 0; j < k; ++j)
                if ((uint32_t)sels[t * k + j] == segs[s].expert) { row_token[row] = (int32_t)t; row_slot[row] = (int32_t)j; row++; }
    }
    *m_total_out = row;
    free(cnt);
    return nseg;
}

/* moe_expert.rs:8455-8513 (grouped_expert_gemm_cpu): xs / outs are row-packed in
 * segment order; segment offsets here are in rows. */
int orc_grouped_gemm(int type, const uint8_t* w_all, long n_in, long n_out, const orc_segment* segs, long nseg,
                     const float* xs, float* outs) {
    const long rb = orc_row_bytes(type, n_in);
    if (rb < 0) return -1;
    float* w = (float*)malloc((size_t)n_in * sizeof(float));
    for (long s = 0; s < nseg; ++s) {
        const uint8_t* blocks = w_all + (long)segs[s].expert * n_out * rb;
        const long m = segs[s].m, x0 = (long)segs[s].x_off * n_in, o0 = (long)segs[s].out_off * n_out;
        for (long r = 0; r < n_out; ++r) {
            orc_dequant_row(type, blocks + r * rb, n_in, w);
            for (long t = 0; t < m; ++t) outs[o0 + t * n_out + r] = dot_seq(w, xs + x0 + t * n_in, n_in);
        }
    }
    free(w);
    return 0;
}

/* One MoE block for a chunk of nt tokens in the grouped form: router rows ->
 * by_expert -> segments -> gather -> gate/up GEMM -> SwiGLU -> down GEMM ->
 * scatter (expert ascending, rows of the expert in token order) -> shared expert.
 * qwen4exp.rs:17921-18350 (moe_ffn_quant_batch_full); moe_grouped_gpu.rs:395-442
 * (reference_h_with_weights), 454-566 (ScatterPlan).  Must equal orc_moe_block
 * token for token (qwen4exp.rs:28259 tests batch == sequential). */
int orc_moe_block_grouped(const orc_moe_layer* L, const float* hin, long nt, float* out, int32_t* sels_out,
                          float* wts_out) {
    const long e = L->e, ff = L->ff, k = L->k, ne = L->ne;
    float* x = (float*)malloc((size_t)(nt * e) * sizeof(float));
    if (L->norm_w) orc_rmsnorm(hin, L->norm_w, nt, e, L->eps, x);
    else memcpy(x, hin, (size_t)(nt * e) * sizeof(float));
    int32_t* sels = (int32_t*)malloc((size_t)(nt * k) * sizeof(int32_t));
    float* wts = (float*)malloc((size_t)(nt * k) * sizeof(float));
    orc_router(x, nt, e, L->router_w, L->router_bias, ne, k, L->norm_topk, sels, wts, NULL);
    orc_segment* segs = (orc_segment*)malloc((size_t)ne * sizeof(orc_segment));
    int32_t* rtok = (int32_t*)malloc((size_t)(nt * k) * sizeof(int32_t));
    int32_t* rslot = (int32_t*)malloc((size_t)(nt * k) * sizeof(int32_t));
    long m_total = 0;
    const long nseg = orc_build_segments(sels, nt, k, ne, segs, rtok, rslot, &m_total);
    float* gx = (float*)malloc((size_t)(m_total * e) * sizeof(float));
    for (long r = 0; r < m_total; ++r) memcpy(gx + r * e, x + (long)rtok[r] * e, (size_t)e * sizeof(float));
    float* g = (float*)malloc((size_t)(m_total * ff) * sizeof(float));
    float* u = (float*)malloc((size_t)(m_total * ff) * sizeof(float));
    float* hh = (float*)malloc((size_t)(m_total * e) * sizeof(float));
    int rc = orc_grouped_gemm(L->ty_gate, L->gate, e, ff, segs, nseg, gx, g);
    rc |= orc_grouped_gemm(L->ty_up, L->up, e, ff, segs, nseg, gx, u);
    for (long i = 0; i < m_total * ff; ++i) g[i] = g[i] / (1.0f + expf(-g[i])) * u[i];
    rc |= orc_grouped_gemm(L->ty_down, L->down, ff, e, segs, nseg, g, hh);
    for (long i = 0; i < nt * e; ++i) out[i] = 0.0f;
    /* scatter: expert ascending, then the expert's rows in order */
    for (long ei = 0; ei < ne; ++ei)
        for (long s = 0; s < nseg; ++s) {
            if ((long)segs[s].expert != ei) continue;
            for (long r = segs[s].x_off; r < (long)segs[s].x_off + (long)segs[s].m; ++r) {
                const float w = wts[(long)rtok[r] * k + rslot[r]];
                float* dst = out + (long)rtok[r] * e;
                for (long d = 0; d < e; ++d) dst[d] += hh[r * e + d] * w;
            }
        }
    if (L->sgate && L->sup && L->sdown) {
        const long sff = L->sff;
        orc_segment one = {0, (uint32_t)nt, 0, 0};
        float* sg = (float*)malloc((size_t)(nt * sff) * sizeof(float));
        float* su = (float*)malloc((size_t)(nt * sff) * sizeof(float));
        float* sh = (float*)malloc((size_t)(nt * e) * sizeof(float));
        rc |= orc_grouped_gemm(L->ty_sgate, L->sgate, e, sff, &one, 1, x, sg);
        rc |= orc_grouped_gemm(L->ty_sup, L->sup, e, sff, &one, 1, x, su);
        for (long i = 0; i < nt * sff; ++i) sg[i] = sg[i] / (1.0f + expf(-sg[i])) * su[i];
        rc |= orc_grouped_gemm(L->ty_sdown, L->sdown, sff, e, &one, 1, sg, sh);
        for (long t = 0; t < nt; ++t) {
            if (L->shared_gate_row) {
                const float coef = orc_sigmoid(dot_seq(L->shared_gate_row, x + t * e, e));
                for (long j = 0; j < e; ++j) out[t * e + j] += sh[t * e + j] * coef;
            } else {
                for (long j = 0; j < e; ++j) out[t * e + j] += sh[t * e + j];
            }
        }
        free(sg); free(su); free(sh);
    }
    if (sels_out) memcpy(sels_out, sels, (size_t)(nt * k) * sizeof(int32_t));
    if (wts_out) memcpy(wts_out, wts, (size_t)(nt * k) * sizeof(float));
    free(x); free(sels); free(wts); free(segs); free(rtok); free(rslot); free(gx); free(g); free(u); free(hh);
    return rc;
}

/* ---- timed CPU baseline (multi-threaded) ----------------------------------- */

/* Lane-split dot: 8 independent partial sums, the shape of the reference's
 * AVX2 kernels (moe_expert.rs:188-280 gemv_q4k_avx2 keeps 8 fp32 lanes and
 * reduces once per row).  Not bit-equal to dot_seq (rel ~1e-6), like theirs. */
static float dot_lanes(const float* w, const float* x, long n) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (long i = 0; i + 8 <= n; i += 8)
        for (int l = 0; l < 8; ++l) acc[l] += w[i + l] * x[i + l];
    return ((acc[0] + acc[4]) + (acc[2] + acc[6])) + ((acc[1] + acc[5]) + (acc[3] + acc[7]));
}

/* Row-parallel GEMV (rayon rows in moe_expert.rs:815-907). */
int orc_gemv_mt(int type, const uint8_t* blocks, long n_in, long n_out, const float* x, float* out) {
    const long rb = orc_row_bytes(type, n_in);
    if (rb < 0) return -1;
#pragma omp parallel
    {
        float* row = (float*)malloc((size_t)n_in * sizeof(float));
#pragma omp for schedule(static)
        for (long r = 0; r < n_out; ++r) {
            orc_dequant_row(type, blocks + r * rb, n_in, row);
            out[r] = dot_lanes(row, x, n_in);
        }
        free(row);
    }
    return 0;
}

/* Experts + weighted sum for nt tokens with the selection given, experts
 * evaluated in parallel per token and summed in ascending order afterwards
 * (qwen4exp.rs:11959-12042 expert_contribs_par + 12126-12216). */
int orc_moe_block_mt(const orc_moe_layer* L, const float* hin, long nt, float* out) {
    const long e = L->e, ff = L->ff, k = L->k;
    const long rb_g = orc_row_bytes(L->ty_gate, e), rb_u = orc_row_bytes(L->ty_up, e), rb_d = orc_row_bytes(L->ty_down, ff);
    if (rb_g < 0 || rb_u < 0 || rb_d < 0) return -1;
    const int has_sh = (L->sgate && L->sup && L->sdown) ? 1 : 0;
    float* x = (float*)malloc((size_t)e * sizeof(float));
    float* probs = (float*)malloc((size_t)L->ne * sizeof(float));
    int32_t* sel = (int32_t*)malloc((size_t)k * sizeof(int32_t));
    float* wts = (float*)malloc((size_t)k * sizeof(float));
    float* hs = (float*)malloc((size_t)((k + 1) * e) * sizeof(float));
    for (long t = 0; t < nt; ++t) {
        if (L->norm_w) orc_rmsnorm(hin + t * e, L->norm_w, 1, e, L->eps, x);
        else memcpy(x, hin + t * e, (size_t)e * sizeof(float));
#pragma omp parallel for schedule(static)
        for (long i = 0; i < L->ne; ++i) {
            float v = dot_lanes(L->router_w + i * e, x, e);
            if (L->router_bias) v += L->router_bias[i];
            probs[i] = v;
        }
        orc_softmax(probs, L->ne);
        orc_select_topk(probs, L->ne, k, sel);
        orc_router_renorm(probs, sel, k, wts);
        float* acts = (float*)malloc((size_t)((k + 1) * ff) * sizeof(float));
        /* gate/up rows of all selected experts in one parallel sweep */
#pragma omp parallel
        {
            float* row = (float*)malloc((size_t)(e > ff ? e : ff) * sizeof(float));
#pragma omp for schedule(static)
            for (long idx = 0; idx < (k + has_sh) * ff; ++idx) {
                const long s = idx / ff, r = idx % ff;
                const uint8_t* wg = (s < k) ? L->gate + ((long)sel[s] * ff + r) * rb_g : L->sgate + r * rb_g;
                const uint8_t* wu = (s < k) ? L->up + ((long)sel[s] * ff + r) * rb_u : L->sup + r * rb_u;
                orc_dequant_row(s < k ? L->ty_gate : L->ty_sgate, wg, e, row);
                const float gv = dot_lanes(row, x, e);
                orc_dequant_row(s < k ? L->ty_up : L->ty_sup, wu, e, row);
                const float uv = dot_lanes(row, x, e);
                acts[idx] = orc_silu(gv) * uv;
            }
#pragma omp for schedule(static)
            for (long idx = 0; idx < (k + has_sh) * e; ++idx) {
                const long s = idx / e, j = idx % e;
                const uint8_t* wd = (s < k) ? L->down + ((long)sel[s] * e + j) * rb_d : L->sdown + j * rb_d;
                orc_dequant_row(s < k ? L->ty_down : L->ty_sdown, wd, ff, row);
                hs[idx] = dot_lanes(row, acts + s * ff, ff);
            }
            free(row);
        }
        free(acts);
        float* o = out + t * e;
        const float sh_coef = (has_sh && L->shared_gate_row) ? orc_sigmoid(dot_lanes(L->shared_gate_row, x, e)) : 1.0f;
        for (long j = 0; j < e; ++j) {
            float a = 0.0f;
            for (long s = 0; s < k; ++s) a += wts[s] * hs[s * e + j];
            if (has_sh) a += hs[k * e + j] * sh_coef;
            o[j] = a;
        }
    }
    free(x); free(probs); free(sel); free(wts); free(hs);
    return 0;
}

/* ---- synthetic inputs (shared generator, see dnb_synth.h) ------------------- */

void orc_synth_blocks(int type, uint64_t seed, uint64_t tensor_id, uint8_t* dst, uint64_t n_blocks) {
    dnb_synth_fill_blocks_host(type, seed, tensor_id, dst, n_blocks);
}
void orc_synth_normal(uint64_t seed, uint64_t tensor_id, float sigma, float* dst, uint64_t n) {
    dnb_synth_fill_normal_host(seed, tensor_id, sigma, dst, n);
}
void orc_synth_zipf_bias(uint64_t seed, uint64_t tensor_id, double s, float* bias, uint32_t n) {
    dnb_synth_zipf_bias_host(seed, tensor_id, s, bias, n);
}
