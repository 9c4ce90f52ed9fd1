/* Timed CPU baseline -- TEST / BENCHMARK INFRASTRUCTURE ONLY, never the parity oracle.
 *
 * An AVX2+FMA restatement of the kernels denno-beta's CPU path runs in production (the
 * reference's Rust cannot be built here: no cargo), so that the benchmark's CPU leg is
 * not a strawman:
 *   fast_gemv_q4k      model/moe_expert.rs:188-280   gemv_q4k_avx2 (8-lane FMA on nibbles
 *                      scaled by d*sc, per-block horizontal sum, min term through the
 *                      32-element sums of x)
 *   fast_gemv_iq3xxs   model/moe_expert.rs:1583-1603 iq_vec8<3> + :1624-1667 gemv_iq<3>
 *                      (8 weights = two grid words + sign byte, two accumulators by parity)
 *   fast_gemm_q4k      model/moe_expert.rs:5709-5860 gemm_q4k_avx2 (k-chunked so that the
 *                      tokens' x chunk stays in L1: :5672-5689 gemm_k_blocks; a block is
 *                      decoded once and applied to every token)
 *   fast_gemm_iq3xxs   the same loop structure with the IQ3_XXS decode (gemm_iq_v2, :2002)
 *   scheduling         rows in parallel chunks of 64 over all selected experts
 *                      (qwen4exp.rs:19325 DECODE_FLAT_ROWS, :15770 MOE_FLAT_ROWS;
 *                      :16311-16787 moe_experts_flat) -- OpenMP here, rayon there
 * Results are checked against the sequential oracle within the reference's own bound for
 * these kernels (1e-4 + 1e-5*|ref|, moe_expert.rs:8755-8758) by tests/test_oracle_fast.py.
 * Other block formats take a generic path (row dequantised by the oracle, 8-lane FMA dot).
 *
 * Build: gcc -O3 -mavx2 -mfma -mf16c -fopenmp (contraction allowed).
 */
#include <immintrin.h>
#include <math.h>
#include <omp.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "dnb_iq_tables.h"
#include "dnb_oracle.h"

#define T_Q4_K 12
#define T_IQ3_XXS 18
#define FLAT_ROWS 64

static int g_threads = 0; /* 0 = OpenMP's default */

void orc_set_threads(int n) {
    g_threads = n > 0 ? n : 0;
    if (n > 0) omp_set_num_threads(n);
}
int orc_get_threads(void) { return g_threads > 0 ? g_threads : omp_get_max_threads(); }

static inline float hsum8(__m256 v) {
    __m128 s = _mm_add_ps(_mm256_castps256_ps128(v), _mm256_extractf128_ps(v, 1));
    s = _mm_add_ps(s, _mm_movehl_ps(s, s));
    s = _mm_add_ss(s, _mm_shuffle_ps(s, s, 0x55));
    return _mm_cvtss_f32(s);
}
static inline float f16f(const uint8_t* p) {
    uint16_t h;
    memcpy(&h, p, 2);
    return _cvtsh_ss(h);
}
static inline void scale_min_k4(int j, const uint8_t* q, uint8_t* sc, uint8_t* m) {
    if (j < 4) {
        *sc = q[j] & 63;
        *m = q[j + 4] & 63;
    } else {
        *sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}
/* sums of x over groups of 32, ascending */
static void group_sums_32(const float* x, long n, float* g) {
    for (long c = 0; c < n / 32; ++c) {
        float s = 0.f;
        for (int i = 0; i < 32; ++i) s += x[c * 32 + i];
        g[c] = s;
    }
}
static inline __m256 u8x8_to_ps(__m128i v) { return _mm256_cvtepi32_ps(_mm256_cvtepu8_epi32(v)); }

/* 64 elements of one nibble plane (32 bytes already masked) against x, scaled by dv */
static inline __m256 fma32(__m256 acc, __m256i nib, const float* xp, __m256 dv) {
    const __m128i l = _mm256_castsi256_si128(nib), h = _mm256_extracti128_si256(nib, 1);
    acc = _mm256_fmadd_ps(_mm256_mul_ps(u8x8_to_ps(l), dv), _mm256_loadu_ps(xp), acc);
    acc = _mm256_fmadd_ps(_mm256_mul_ps(u8x8_to_ps(_mm_srli_si128(l, 8)), dv), _mm256_loadu_ps(xp + 8), acc);
    acc = _mm256_fmadd_ps(_mm256_mul_ps(u8x8_to_ps(h), dv), _mm256_loadu_ps(xp + 16), acc);
    acc = _mm256_fmadd_ps(_mm256_mul_ps(u8x8_to_ps(_mm_srli_si128(h, 8)), dv), _mm256_loadu_ps(xp + 24), acc);
    return acc;
}

static void fast_gemv_q4k(const uint8_t* blocks, long n_in, long r0, long r1, const float* x, const float* gsum,
                          float* out) {
    const long nb = n_in / 256, rb = nb * 144;
    const __m256i m4 = _mm256_set1_epi8(0x0f);
    for (long r = r0; r < r1; ++r) {
        const uint8_t* row = blocks + r * rb;
        float total = 0.f;
        for (long b = 0; b < nb; ++b) {
            const uint8_t* blk = row + b * 144;
            const float d = f16f(blk), dmin = f16f(blk + 2);
            __m256 acc0 = _mm256_setzero_ps(), acc1 = _mm256_setzero_ps();
            float minsum = 0.f;
            for (int j = 0; j < 4; ++j) {
                uint8_t s0, m0, s1, m1;
                scale_min_k4(2 * j, blk + 4, &s0, &m0);
                scale_min_k4(2 * j + 1, blk + 4, &s1, &m1);
                const __m256i qv = _mm256_loadu_si256((const __m256i*)(blk + 16 + j * 32));
                const __m256i lo = _mm256_and_si256(qv, m4), hi = _mm256_and_si256(_mm256_srli_epi16(qv, 4), m4);
                const float* xb = x + b * 256 + j * 64;
                acc0 = fma32(acc0, lo, xb, _mm256_set1_ps(d * (float)s0));
                acc1 = fma32(acc1, hi, xb + 32, _mm256_set1_ps(d * (float)s1));
                minsum += dmin * (float)m0 * gsum[b * 8 + 2 * j];
                minsum += dmin * (float)m1 * gsum[b * 8 + 2 * j + 1];
            }
            total += hsum8(_mm256_add_ps(acc0, acc1)) - minsum;
        }
        out[r] = total;
    }
}

/* 8 weights of an IQ3_XXS block: group h (0..31) = sub-block h/4, quarter h%4 */
static inline __m256 iq3xxs_vec8(const uint8_t* p, int h, float d) {
    const int ib = h >> 2, l = h & 3;
    uint32_t aux;
    memcpy(&aux, p + 66 + 4 * ib, 4);
    const float db = d * (0.5f + (float)(aux >> 28)) * 0.5f;
    const int sg = dnb_ksigns_iq2xs[(aux >> (7 * l)) & 127];
    const uint64_t g = (uint64_t)dnb_iq3xxs_grid[p[2 + 8 * ib + 2 * l]] | ((uint64_t)dnb_iq3xxs_grid[p[2 + 8 * ib + 2 * l + 1]] << 32);
    const __m256 v = _mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(_mm_cvtsi64_si128((long long)g)));
    const __m256i hit = _mm256_and_si256(_mm256_set1_epi32(sg), _mm256_setr_epi32(1, 2, 4, 8, 16, 32, 64, 128));
    const __m256i pos = _mm256_cmpeq_epi32(hit, _mm256_setzero_si256());
    const __m256i neg = _mm256_andnot_si256(pos, _mm256_set1_epi32((int)0x80000000u));
    return _mm256_mul_ps(_mm256_xor_ps(v, _mm256_castsi256_ps(neg)), _mm256_set1_ps(db));
}

static void fast_gemv_iq3xxs(const uint8_t* blocks, long n_in, long r0, long r1, const float* x, float* out) {
    const long nb = n_in / 256, rb = nb * 98;
    for (long r = r0; r < r1; ++r) {
        const uint8_t* row = blocks + r * rb;
        __m256 a0 = _mm256_setzero_ps(), a1 = _mm256_setzero_ps();
        for (long b = 0; b < nb; ++b) {
            const uint8_t* p = row + b * 98;
            const float d = f16f(p);
            const float* xb = x + b * 256;
            for (int h = 0; h < 32; h += 2) {
                a0 = _mm256_fmadd_ps(iq3xxs_vec8(p, h, d), _mm256_loadu_ps(xb + h * 8), a0);
                a1 = _mm256_fmadd_ps(iq3xxs_vec8(p, h + 1, d), _mm256_loadu_ps(xb + h * 8 + 8), a1);
            }
        }
        out[r] = hsum8(_mm256_add_ps(a0, a1));
    }
}

static void fast_gemv_generic(int type, const uint8_t* blocks, long n_in, long r0, long r1, const float* x, float* out,
                              float* rowbuf) {
    const long rb = orc_row_bytes(type, n_in);
    for (long r = r0; r < r1; ++r) {
        orc_dequant_row(type, blocks + r * rb, n_in, rowbuf);
        __m256 a0 = _mm256_setzero_ps(), a1 = _mm256_setzero_ps();
        long i = 0;
        for (; i + 16 <= n_in; i += 16) {
            a0 = _mm256_fmadd_ps(_mm256_loadu_ps(rowbuf + i), _mm256_loadu_ps(x + i), a0);
            a1 = _mm256_fmadd_ps(_mm256_loadu_ps(rowbuf + i + 8), _mm256_loadu_ps(x + i + 8), a1);
        }
        float s = hsum8(_mm256_add_ps(a0, a1));
        for (; i < n_in; ++i) s += rowbuf[i] * x[i];
        out[r] = s;
    }
}

/* rows [r0, r1) of one matrix against one vector */
static void gemv_rows(int type, const uint8_t* w, long n_in, long r0, long r1, const float* x, const float* gsum, float* out,
                      float* rowbuf) {
    if (type == T_Q4_K) fast_gemv_q4k(w, n_in, r0, r1, x, gsum, out);
    else if (type == T_IQ3_XXS) fast_gemv_iq3xxs(w, n_in, r0, r1, x, out);
    else fast_gemv_generic(type, w, n_in, r0, r1, x, out, rowbuf);
}

/* Row-parallel single-matrix GEMV (moe_expert.rs:815-907 for_each_row_chunk). */
int orc_fast_gemv(int type, const uint8_t* blocks, long n_in, long n_out, const float* x, float* out) {
    if (orc_row_bytes(type, n_in) < 0) return -1;
    float* gsum = (float*)malloc((size_t)(n_in / 32 + 1) * sizeof(float));
    group_sums_32(x, n_in, gsum);
    const long chunks = (n_out + FLAT_ROWS - 1) / FLAT_ROWS;
#pragma omp parallel
    {
        float* rowbuf = (float*)malloc((size_t)n_in * sizeof(float));
#pragma omp for schedule(dynamic, 1)
        for (long c = 0; c < chunks; ++c) {
            const long r0 = c * FLAT_ROWS, r1 = r0 + FLAT_ROWS < n_out ? r0 + FLAT_ROWS : n_out;
            gemv_rows(type, blocks, n_in, r0, r1, x, gsum, out, rowbuf);
        }
        free(rowbuf);
    }
    free(gsum);
    return 0;
}

static float dot_avx(const float* a, const float* b, long n) {
    __m256 a0 = _mm256_setzero_ps(), a1 = _mm256_setzero_ps();
    long i = 0;
    for (; i + 16 <= n; i += 16) {
        a0 = _mm256_fmadd_ps(_mm256_loadu_ps(a + i), _mm256_loadu_ps(b + i), a0);
        a1 = _mm256_fmadd_ps(_mm256_loadu_ps(a + i + 8), _mm256_loadu_ps(b + i + 8), a1);
    }
    float s = hsum8(_mm256_add_ps(a0, a1));
    for (; i < n; ++i) s += a[i] * b[i];
    return s;
}

/* Router of nt tokens: rows in parallel, softmax / top-k / renorm by the oracle's functions. */
static void fast_router(const orc_moe_layer* L, const float* x, long nt, int32_t* sels, float* wts) {
    const long e = L->e, ne = L->ne, k = L->k;
    float* logits = (float*)malloc((size_t)(nt * ne) * sizeof(float));
#pragma omp parallel for schedule(static)
    for (long i = 0; i < ne; ++i)
        for (long t = 0; t < nt; ++t) {
            float v = dot_avx(L->router_w + i * e, x + t * e, e);
            if (L->router_bias) v += L->router_bias[i];
            logits[t * ne + i] = v;
        }
#pragma omp parallel for schedule(static)
    for (long t = 0; t < nt; ++t) {
        float* p = logits + t * ne;
        orc_softmax(p, ne);
        orc_select_topk(p, ne, k, sels + t * k);
        if (L->norm_topk) orc_router_renorm(p, sels + t * k, k, wts + t * k);
        else
            for (long s = 0; s < k; ++s) wts[t * k + s] = p[sels[t * k + s]];
    }
    free(logits);
}

/* One MoE block, decode form: per token, the gate/up rows of all selected experts (+ shared) as
 * one flat parallel sweep in chunks of 64 rows, then the down rows likewise, then the weighted
 * sum in ascending expert order (qwen4exp.rs:11659-12411, 19325). */
int orc_fast_moe_block(const orc_moe_layer* L, const float* hin, long nt, float* out) {
    const long e = L->e, ff = L->ff, k = L->k;
    const long rb_g = orc_row_bytes(L->ty_gate, e), rb_u = orc_row_bytes(L->ty_up, e), rb_d = orc_row_bytes(L->ty_down, ff);
    if (rb_g < 0 || rb_u < 0 || rb_d < 0) return -1;
    const int has_sh = (L->sgate && L->sup && L->sdown) ? 1 : 0;
    if (has_sh && L->sff != ff) return -1;
    const long ns = k + has_sh;
    float* x = (float*)malloc((size_t)e * sizeof(float));
    int32_t* sel = (int32_t*)malloc((size_t)k * sizeof(int32_t));
    float* wts = (float*)malloc((size_t)k * sizeof(float));
    float* g = (float*)malloc((size_t)(ns * ff) * sizeof(float));
    float* u = (float*)malloc((size_t)(ns * ff) * sizeof(float));
    float* hs = (float*)malloc((size_t)(ns * e) * sizeof(float));
    float* gsx = (float*)malloc((size_t)(e / 32 + 1) * sizeof(float));
    float* gsa = (float*)malloc((size_t)(ns * (ff / 32 + 1)) * sizeof(float));
    const long cg = ff / FLAT_ROWS > 0 ? (ff + FLAT_ROWS - 1) / FLAT_ROWS : 1, cd = (e + FLAT_ROWS - 1) / FLAT_ROWS;
    for (long t = 0; t < nt; ++t) {
        if (L->norm_w) orc_rmsnorm(hin + t * e, L->norm_w, 1, e, L->eps, x);
        else memcpy(x, hin + t * e, (size_t)e * sizeof(float));
        fast_router(L, x, 1, sel, wts);
        group_sums_32(x, e, gsx);
#pragma omp parallel
        {
            float* rowbuf = (float*)malloc((size_t)(e > ff ? e : ff) * sizeof(float));
#pragma omp for schedule(dynamic, 1)
            for (long idx = 0; idx < 2 * ns * cg; ++idx) {
                const long mat = idx / (ns * cg), s = (idx / cg) % ns, c = idx % cg;
                const long r0 = c * FLAT_ROWS, r1 = r0 + FLAT_ROWS < ff ? r0 + FLAT_ROWS : ff;
                const uint8_t* w;
                int ty;
                if (mat == 0) { w = s < k ? L->gate + (long)sel[s] * ff * rb_g : L->sgate; ty = s < k ? L->ty_gate : L->ty_sgate; }
                else { w = s < k ? L->up + (long)sel[s] * ff * rb_u : L->sup; ty = s < k ? L->ty_up : L->ty_sup; }
                gemv_rows(ty, w, e, r0, r1, x, gsx, (mat == 0 ? g : u) + s * ff, rowbuf);
            }
#pragma omp for schedule(static)
            for (long i = 0; i < ns * ff; ++i) g[i] = g[i] / (1.0f + expf(-g[i])) * u[i];
#pragma omp for schedule(static)
            for (long s = 0; s < ns; ++s) group_sums_32(g + s * ff, ff, gsa + s * (ff / 32 + 1));
#pragma omp for schedule(dynamic, 1)
            for (long idx = 0; idx < ns * cd; ++idx) {
                const long s = idx / cd, c = idx % cd;
                const long r0 = c * FLAT_ROWS, r1 = r0 + FLAT_ROWS < e ? r0 + FLAT_ROWS : e;
                const uint8_t* w = s < k ? L->down + (long)sel[s] * e * rb_d : L->sdown;
                gemv_rows(s < k ? L->ty_down : L->ty_sdown, w, ff, r0, r1, g + s * ff, gsa + s * (ff / 32 + 1), hs + s * e, rowbuf);
            }
            free(rowbuf);
        }
        float* o = out + t * e;
        const float coef = (has_sh && L->shared_gate_row) ? orc_sigmoid(dot_avx(L->shared_gate_row, x, e)) : 1.0f;
        for (long j = 0; j < e; ++j) {
            float a = 0.f;
            for (long s = 0; s < k; ++s) a += wts[s] * hs[s * e + j];
            if (has_sh) a += hs[k * e + j] * coef;
            o[j] = a;
        }
    }
    free(x); free(sel); free(wts); free(g); free(u); free(hs); free(gsx); free(gsa);
    return 0;
}

/* ---- batch kernels (prefill) ------------------------------------------------------ */

#define GEMM_X_L1_BUDGET (16 * 1024)
#define GEMM_TOK_TILE 16

static long gemm_k_blocks(long blk_elems, long m, long cap) {
    long v = GEMM_X_L1_BUDGET / (blk_elems * 4 * (m > 0 ? m : 1));
    return v < 1 ? 1 : (v > cap ? cap : v);
}

/* rows [r0, r1) x m tokens (m <= GEMM_TOK_TILE): out[t*stride + (r - r0)], k-chunked, a block decoded
 * once and applied to every token; per (row, token) the per-block sums are added in ascending
 * block order, as in the one-token kernel */
static void fast_gemm_q4k(const uint8_t* blocks, long n_in, long r0, long r1, const float* xs, long m, const float* gsums,
                          float* out, long stride, float* total /* [rows*m] */) {
    const long nb = n_in / 256, rb = nb * 144, rows = r1 - r0, ng32 = n_in / 32;
    const __m256i m4 = _mm256_set1_epi8(0x0f);
    __m256 a0[GEMM_TOK_TILE], a1[GEMM_TOK_TILE];
    float minsum[GEMM_TOK_TILE];
    memset(total, 0, (size_t)(rows * m) * sizeof(float));
    const long kb = gemm_k_blocks(256, m, 4);
    for (long b0 = 0; b0 < nb; b0 += kb) {
        const long b1 = b0 + kb < nb ? b0 + kb : nb;
        for (long r = r0; r < r1; ++r) {
            const uint8_t* row = blocks + r * rb;
            float* tot = total + (r - r0) * m;
            for (long b = b0; b < b1; ++b) {
                const uint8_t* blk = row + b * 144;
                const float d = f16f(blk), dmin = f16f(blk + 2);
                for (long t = 0; t < m; ++t) { a0[t] = _mm256_setzero_ps(); a1[t] = _mm256_setzero_ps(); minsum[t] = 0.f; }
                for (int j = 0; j < 4; ++j) {
                    uint8_t s0, m0, s1, m1;
                    scale_min_k4(2 * j, blk + 4, &s0, &m0);
                    scale_min_k4(2 * j + 1, blk + 4, &s1, &m1);
                    const __m256 dv0 = _mm256_set1_ps(d * (float)s0), dv1 = _mm256_set1_ps(d * (float)s1);
                    const __m256i qv = _mm256_loadu_si256((const __m256i*)(blk + 16 + j * 32));
                    const __m256i lo = _mm256_and_si256(qv, m4), hi = _mm256_and_si256(_mm256_srli_epi16(qv, 4), m4);
                    const __m128i lol = _mm256_castsi256_si128(lo), loh = _mm256_extracti128_si256(lo, 1);
                    const __m128i hil = _mm256_castsi256_si128(hi), hih = _mm256_extracti128_si256(hi, 1);
                    const __m256 w0 = _mm256_mul_ps(u8x8_to_ps(lol), dv0), w1 = _mm256_mul_ps(u8x8_to_ps(_mm_srli_si128(lol, 8)), dv0);
                    const __m256 w2 = _mm256_mul_ps(u8x8_to_ps(loh), dv0), w3 = _mm256_mul_ps(u8x8_to_ps(_mm_srli_si128(loh, 8)), dv0);
                    const __m256 w4 = _mm256_mul_ps(u8x8_to_ps(hil), dv1), w5 = _mm256_mul_ps(u8x8_to_ps(_mm_srli_si128(hil, 8)), dv1);
                    const __m256 w6 = _mm256_mul_ps(u8x8_to_ps(hih), dv1), w7 = _mm256_mul_ps(u8x8_to_ps(_mm_srli_si128(hih, 8)), dv1);
                    const long gi = b * 8 + j * 2;
                    const float c0m = dmin * (float)m0, c1m = dmin * (float)m1;
                    for (long t = 0; t < m; ++t) {
                        const float* xb = xs + t * n_in + b * 256 + j * 64;
                        __m256 c0 = a0[t], c1 = a1[t];
                        c0 = _mm256_fmadd_ps(w0, _mm256_loadu_ps(xb), c0);
                        c0 = _mm256_fmadd_ps(w1, _mm256_loadu_ps(xb + 8), c0);
                        c0 = _mm256_fmadd_ps(w2, _mm256_loadu_ps(xb + 16), c0);
                        c0 = _mm256_fmadd_ps(w3, _mm256_loadu_ps(xb + 24), c0);
                        c1 = _mm256_fmadd_ps(w4, _mm256_loadu_ps(xb + 32), c1);
                        c1 = _mm256_fmadd_ps(w5, _mm256_loadu_ps(xb + 40), c1);
                        c1 = _mm256_fmadd_ps(w6, _mm256_loadu_ps(xb + 48), c1);
                        c1 = _mm256_fmadd_ps(w7, _mm256_loadu_ps(xb + 56), c1);
                        a0[t] = c0;
                        a1[t] = c1;
                        minsum[t] += c0m * gsums[t * ng32 + gi];
                        minsum[t] += c1m * gsums[t * ng32 + gi + 1];
                    }
                }
                for (long t = 0; t < m; ++t) tot[t] += hsum8(_mm256_add_ps(a0[t], a1[t])) - minsum[t];
            }
        }
    }
    for (long t = 0; t < m; ++t)
        for (long ri = 0; ri < rows; ++ri) out[t * stride + ri] = total[ri * m + t];
}

static void fast_gemm_iq3xxs(const uint8_t* blocks, long n_in, long r0, long r1, const float* xs, long m, float* out,
                             long stride) {
    const long nb = n_in / 256, rb = nb * 98;
    __m256 a0[GEMM_TOK_TILE], a1[GEMM_TOK_TILE];
    for (long r = r0; r < r1; ++r) {
        const uint8_t* row = blocks + r * rb;
        for (long t = 0; t < m; ++t) { a0[t] = _mm256_setzero_ps(); a1[t] = _mm256_setzero_ps(); }
        for (long b = 0; b < nb; ++b) {
            const uint8_t* p = row + b * 98;
            const float d = f16f(p);
            for (int h = 0; h < 32; h += 2) {
                const __m256 v0 = iq3xxs_vec8(p, h, d), v1 = iq3xxs_vec8(p, h + 1, d);
                for (long t = 0; t < m; ++t) {
                    const float* xb = xs + t * n_in + b * 256 + h * 8;
                    a0[t] = _mm256_fmadd_ps(v0, _mm256_loadu_ps(xb), a0[t]);
                    a1[t] = _mm256_fmadd_ps(v1, _mm256_loadu_ps(xb + 8), a1[t]);
                }
            }
        }
        for (long t = 0; t < m; ++t) out[t * stride + (r - r0)] = hsum8(_mm256_add_ps(a0[t], a1[t]));
    }
}

/* rows [r0, r1) of one matrix against m packed token rows; out[t*n_out + r] */
static void gemm_rows(int type, const uint8_t* w, long n_in, long n_out, long r0, long r1, const float* xs, long m,
                      const float* gsums, float* out, float* scratch /* FLAT_ROWS*TILE + n_in */) {
    for (long t0 = 0; t0 < m; t0 += GEMM_TOK_TILE) {
        const long mt = m - t0 < GEMM_TOK_TILE ? m - t0 : GEMM_TOK_TILE;
        if (type == T_Q4_K) {
            fast_gemm_q4k(w, n_in, r0, r1, xs + t0 * n_in, mt, gsums + t0 * (n_in / 32), out + t0 * n_out + r0, n_out, scratch);
        } else if (type == T_IQ3_XXS) {
            fast_gemm_iq3xxs(w, n_in, r0, r1, xs + t0 * n_in, mt, out + t0 * n_out + r0, n_out);
        } else {
            for (long t = t0; t < t0 + mt; ++t)
                fast_gemv_generic(type, w, n_in, r0, r1, xs + t * n_in, out + t * n_out, scratch + FLAT_ROWS * GEMM_TOK_TILE);
        }
    }
}

/* One MoE block for a chunk of nt tokens, grouped by expert: router, expert-major packed rows,
 * tasks = (segment, 64-row chunk) run in parallel with the batch kernels, scatter in ascending
 * expert order, shared expert as one more segment (qwen4exp.rs:17921-18350, 16311-16787). */
int orc_fast_moe_block_grouped(const orc_moe_layer* L, const float* hin, long nt, float* out) {
    const long e = L->e, ff = L->ff, k = L->k, ne = L->ne;
    const long rb_g = orc_row_bytes(L->ty_gate, e), rb_u = orc_row_bytes(L->ty_up, e), rb_d = orc_row_bytes(L->ty_down, ff);
    if (rb_g < 0 || rb_u < 0 || rb_d < 0) return -1;
    const int has_sh = (L->sgate && L->sup && L->sdown) ? 1 : 0;
    if (has_sh && L->sff != ff) return -1;
    float* x = (float*)malloc((size_t)(nt * e) * sizeof(float));
    if (L->norm_w) {
#pragma omp parallel for schedule(static)
        for (long t = 0; t < nt; ++t) orc_rmsnorm(hin + t * e, L->norm_w, 1, e, L->eps, x + t * e);
    } else {
        memcpy(x, hin, (size_t)(nt * e) * sizeof(float));
    }
    int32_t* sels = (int32_t*)malloc((size_t)(nt * k) * sizeof(int32_t));
    float* wts = (float*)malloc((size_t)(nt * k) * sizeof(float));
    fast_router(L, x, nt, sels, wts);
    orc_segment* segs = (orc_segment*)malloc((size_t)(ne + 1) * sizeof(orc_segment));
    int32_t* rtok = (int32_t*)malloc((size_t)(nt * (k + 1)) * sizeof(int32_t));
    int32_t* rslot = (int32_t*)malloc((size_t)(nt * (k + 1)) * sizeof(int32_t));
    long m_total = 0;
    long nseg = orc_build_segments(sels, nt, k, ne, segs, rtok, rslot, &m_total);
    if (has_sh) { /* the shared expert: one more segment over all tokens */
        segs[nseg].expert = (uint32_t)ne; segs[nseg].m = (uint32_t)nt; segs[nseg].x_off = segs[nseg].out_off = (uint32_t)m_total;
        for (long t = 0; t < nt; ++t) { rtok[m_total + t] = (int32_t)t; rslot[m_total + t] = (int32_t)k; }
        m_total += nt;
        nseg++;
    }
    float* gx = (float*)malloc((size_t)(m_total * e) * sizeof(float));
    float* gs = (float*)malloc((size_t)(m_total * (e / 32)) * sizeof(float));
#pragma omp parallel for schedule(static)
    for (long r = 0; r < m_total; ++r) {
        memcpy(gx + r * e, x + (long)rtok[r] * e, (size_t)e * sizeof(float));
        group_sums_32(gx + r * e, e, gs + r * (e / 32));
    }
    float* g = (float*)malloc((size_t)(m_total * ff) * sizeof(float));
    float* u = (float*)malloc((size_t)(m_total * ff) * sizeof(float));
    float* hh = (float*)malloc((size_t)(m_total * e) * sizeof(float));
    float* ga = (float*)malloc((size_t)(m_total * (ff / 32)) * sizeof(float));
    const long cg = (ff + FLAT_ROWS - 1) / FLAT_ROWS, cd = (e + FLAT_ROWS - 1) / FLAT_ROWS;
#pragma omp parallel
    {
        float* scratch = (float*)malloc((size_t)(FLAT_ROWS * GEMM_TOK_TILE + (e > ff ? e : ff)) * sizeof(float));
#pragma omp for schedule(dynamic, 1)
        for (long idx = 0; idx < 2 * nseg * cg; ++idx) {
            const long mat = idx % 2, s = (idx / 2) / cg, c = (idx / 2) % cg;
            const long r0 = c * FLAT_ROWS, r1 = r0 + FLAT_ROWS < ff ? r0 + FLAT_ROWS : ff;
            const int shared = (long)segs[s].expert == ne;
            const uint8_t* w = mat == 0 ? (shared ? L->sgate : L->gate + (long)segs[s].expert * ff * rb_g)
                                        : (shared ? L->sup : L->up + (long)segs[s].expert * ff * rb_u);
            const int ty = mat == 0 ? (shared ? L->ty_sgate : L->ty_gate) : (shared ? L->ty_sup : L->ty_up);
            const long row = segs[s].x_off;
            gemm_rows(ty, w, e, ff, r0, r1, gx + row * e, segs[s].m, gs + row * (e / 32), (mat == 0 ? g : u) + row * ff, scratch);
        }
#pragma omp for schedule(static)
        for (long r = 0; r < m_total; ++r) {
            for (long i = 0; i < ff; ++i) g[r * ff + i] = g[r * ff + i] / (1.0f + expf(-g[r * ff + i])) * u[r * ff + i];
            group_sums_32(g + r * ff, ff, ga + r * (ff / 32));
        }
#pragma omp for schedule(dynamic, 1)
        for (long idx = 0; idx < nseg * cd; ++idx) {
            const long s = idx / cd, c = idx % cd;
            const long r0 = c * FLAT_ROWS, r1 = r0 + FLAT_ROWS < e ? r0 + FLAT_ROWS : e;
            const int shared = (long)segs[s].expert == ne;
            const uint8_t* w = shared ? L->sdown : L->down + (long)segs[s].expert * e * rb_d;
            const long row = segs[s].x_off;
            gemm_rows(shared ? L->ty_sdown : L->ty_down, w, ff, e, r0, r1, g + row * ff, segs[s].m, ga + row * (ff / 32),
                      hh + row * e, scratch);
        }
        free(scratch);
    }
    /* scatter per token: slots in ascending order = ascending expert, then the shared expert */
    long* pos = (long*)malloc((size_t)(nt * (k + 1)) * sizeof(long));
    for (long r = 0; r < m_total; ++r) pos[(long)rtok[r] * (k + 1) + rslot[r]] = r;
#pragma omp parallel for schedule(static)
    for (long t = 0; t < nt; ++t) {
        float* o = out + t * e;
        const float coef = (has_sh && L->shared_gate_row) ? orc_sigmoid(dot_avx(L->shared_gate_row, x + t * e, e)) : 1.0f;
        for (long j = 0; j < e; ++j) {
            float a = 0.f;
            for (long s = 0; s < k; ++s) a += wts[t * k + s] * hh[pos[t * (k + 1) + s] * e + j];
            if (has_sh) a += hh[pos[t * (k + 1) + k] * e + j] * coef;
            o[j] = a;
        }
    }
    free(pos); free(x); free(sels); free(wts); free(segs); free(rtok); free(rslot); free(gx); free(gs);
    free(g); free(u); free(hh); free(ga);
    return 0;
}
