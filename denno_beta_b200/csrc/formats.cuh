// GGUF block formats on the device: how a row's bytes map to 32-element "units"
// and how one unit is decoded to fp32 in registers.
//
// A unit is the 32 elements one lane handles at a time.  Its elements are not
// always 32 consecutive elements of the row: for each format the unit is chosen
// so that the bytes a lane needs are contiguous (Q4_K: one 16-byte slice of qs
// holds 16 low-nibble and 16 high-nibble elements that lie 32 apart).  The
// activation vector is staged in shared memory in the matching "slot" order
// (slot_of), as float4 rows indexed [k][unit], so consecutive lanes read
// consecutive 16-byte words without bank conflicts.
//
// Block layouts follow crates/denno-engine/src/kquant.rs:341-887 of the
// reference (dequant_block); the arithmetic of every element is the same
// expression, evaluated in fp32.
#pragma once
#include "dnb_common.cuh"

namespace dnb {

__device__ __forceinline__ float h2f(uint16_t bits) { return __half2float(__ushort_as_half(bits)); }
__device__ __forceinline__ uint32_t ld16(const uint8_t* p) { return *reinterpret_cast<const uint16_t*>(p); }

// Shared lookup tables of the IQ formats (copied into shared memory per CTA).  The kernels
// pass one pointer; what lies behind it depends on the format.
// The IQ3_XXS codebook is held kLutRep times, entry i of copy r at word i * kLutRep + r: a
// lane reads copy (lane & (kLutRep - 1)), so the 32 random lookups of a warp spread over the banks
// instead of piling up on the few banks a single 1 KB table offers them.
constexpr int kLutRep = 16;
struct IqLut {
    uint32_t grid3xxs[256 * kLutRep];
    __device__ __forceinline__ uint32_t at(uint32_t idx, int rep) const { return grid3xxs[idx * kLutRep + rep]; }
    __device__ __forceinline__ void fill(const uint32_t* table, int tid, int nthr) {
        for (int i = tid; i < 256 * kLutRep; i += nthr) grid3xxs[i] = table[i / kLutRep];
    }
};
struct IqLut3s { uint32_t grid[512]; };
struct IqLut2s { uint64_t grid[1024]; };
struct IqLut4 { int8_t kv[16]; };
template <int T>
__host__ __device__ constexpr int lut_bytes_of() {
    return T == T_IQ3_XXS ? (int)sizeof(IqLut) : T == T_IQ3_S ? (int)sizeof(IqLut3s) : T == T_IQ2_S ? (int)sizeof(IqLut2s)
         : (T == T_IQ4_NL || T == T_IQ4_XS) ? (int)sizeof(IqLut4) : 0;
}

// (unit, slot) of element i of a row, per format.
template <int T>
__device__ __forceinline__ void slot_of(int i, int& u, int& s) {
    if constexpr (T == T_Q4_K || T == T_Q5_K) {
        const int b = i >> 8, r = i & 255, j = r >> 6, p = r & 63, nib = p >> 5, l = p & 31;
        u = b * 8 + j * 2 + (l >> 4);
        s = nib * 16 + (l & 15);
    } else if constexpr (T == T_Q6_K) {
        const int b = i >> 8, r = i & 255, half = r >> 7, p = r & 127, qi = p >> 5, l = p & 31;
        u = b * 8 + half * 4 + (l >> 3);
        s = qi * 8 + (l & 7);
    } else {  // IQ3_XXS, Q8_0, Q5_1: 32 consecutive elements
        u = i >> 5;
        s = i & 31;
    }
}

// Position of element i in the slot-ordered staging of a vector of `nunits` units, for a
// format known only at run time.
__device__ __forceinline__ int slot_index(int type, int i, int nunits) {
    int u, s;
    if (type == T_Q4_K || type == T_Q5_K) slot_of<T_Q4_K>(i, u, s);
    else if (type == T_Q6_K) slot_of<T_Q6_K>(i, u, s);
    else slot_of<T_IQ3_XXS>(i, u, s);
    return (((s >> 2) * nunits + u) << 2) + (s & 3);
}

// kquant.rs:878-887 (get_scale_min_k4) on the 12 scale bytes at `q`.
__device__ __forceinline__ void scale_min_k4(int j, const uint8_t* q, int& sc, int& m) {
    if (j < 4) {
        sc = q[j] & 63;
        m = q[j + 4] & 63;
    } else {
        sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
        m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
    }
}

// Decode unit `u` of a row (bytes in shared memory) into w[32] in slot order.
template <int T>
__device__ __forceinline__ void decode_unit(const uint8_t* row, int u, const IqLut* lut, float (&w)[32]) {
    if constexpr (T == T_Q4_K) {  // kquant.rs:505-526
        const int b = u >> 3, j = (u >> 1) & 3, h = u & 1;
        const uint8_t* blk = row + b * 144;
        const float d = h2f(ld16(blk)), dmin = h2f(ld16(blk + 2));
        int sc1, m1, sc2, m2;
        scale_min_k4(2 * j, blk + 4, sc1, m1);
        scale_min_k4(2 * j + 1, blk + 4, sc2, m2);
        const float d1 = d * (float)sc1, mm1 = dmin * (float)m1, d2 = d * (float)sc2, mm2 = dmin * (float)m2;
        const uint4 qv = *reinterpret_cast<const uint4*>(blk + 16 + 32 * j + 16 * h);
        const uint32_t qw[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint32_t byte = (qw[i >> 2] >> (8 * (i & 3))) & 0xFF;
            w[i] = d1 * (float)(byte & 0xF) - mm1;
            w[16 + i] = d2 * (float)(byte >> 4) - mm2;
        }
    } else if constexpr (T == T_Q5_K) {  // kquant.rs:529-558
        const int b = u >> 3, j = (u >> 1) & 3, h = u & 1;
        const uint8_t* blk = row + b * 176;
        const float d = h2f(ld16(blk)), dmin = h2f(ld16(blk + 2));
        int sc1, m1, sc2, m2;
        scale_min_k4(2 * j, blk + 4, sc1, m1);
        scale_min_k4(2 * j + 1, blk + 4, sc2, m2);
        const float d1 = d * (float)sc1, mm1 = dmin * (float)m1, d2 = d * (float)sc2, mm2 = dmin * (float)m2;
        const uint4 qv = *reinterpret_cast<const uint4*>(blk + 48 + 32 * j + 16 * h);
        const uint4 hv = *reinterpret_cast<const uint4*>(blk + 16 + 16 * h);
        const uint32_t qw[4] = {qv.x, qv.y, qv.z, qv.w};
        const uint32_t hw[4] = {hv.x, hv.y, hv.z, hv.w};
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint32_t byte = (qw[i >> 2] >> (8 * (i & 3))) & 0xFF;
            const uint32_t hb = (hw[i >> 2] >> (8 * (i & 3))) & 0xFF;
            w[i] = d1 * (float)((byte & 0xF) + (((hb >> (2 * j)) & 1) << 4)) - mm1;
            w[16 + i] = d2 * (float)((byte >> 4) + (((hb >> (2 * j + 1)) & 1) << 4)) - mm2;
        }
    } else if constexpr (T == T_IQ3_XXS) {  // kquant.rs:659-680
        const int b = u >> 3, ib = u & 7;
        const uint8_t* blk = row + b * 98;
        const float d = h2f(ld16(blk));
        const uint32_t aux = ld16(blk + 66 + 4 * ib) | (ld16(blk + 68 + 4 * ib) << 16);
        const float db = d * (0.5f + (float)(aux >> 28)) * 0.5f;
#pragma unroll
        for (int l = 0; l < 4; ++l) {
            const uint32_t idx = ld16(blk + 2 + 8 * ib + 2 * l);
            const uint32_t code = (aux >> (7 * l)) & 127;
            const uint32_t sg = code | ((__popc(code) & 1) << 7);  // KSIGNS_IQ2XS[code]: bit 7 = parity
            const int rep = (int)(threadIdx.x & (kLutRep - 1));
            const uint32_t g1 = lut->at(idx & 0xFF, rep), g2 = lut->at(idx >> 8, rep);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float v0 = db * (float)((g1 >> (8 * j)) & 0xFF);
                const float v1 = db * (float)((g2 >> (8 * j)) & 0xFF);
                w[8 * l + j] = (sg >> j) & 1 ? -v0 : v0;
                w[8 * l + 4 + j] = (sg >> (j + 4)) & 1 ? -v1 : v1;
            }
        }
    } else if constexpr (T == T_Q6_K) {  // kquant.rs:561-583
        const int b = u >> 3, half = (u >> 2) & 1, lg = u & 3, l0 = lg * 8;
        const uint8_t* blk = row + b * 210;
        const uint8_t* ql = blk + 64 * half;
        const uint8_t* qh = blk + 128 + 32 * half;
        const int8_t* sc = reinterpret_cast<const int8_t*>(blk + 192 + 8 * half);
        const float d = h2f(ld16(blk + 208));
        const int is = lg >> 1;
        const float s1 = d * (float)sc[is], s2 = d * (float)sc[is + 2], s3 = d * (float)sc[is + 4],
                    s4 = d * (float)sc[is + 6];
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const uint32_t a = ld16(ql + l0 + 2 * p), c = ld16(ql + 32 + l0 + 2 * p), hh = ld16(qh + l0 + 2 * p);
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const uint32_t qa = (a >> (8 * q)) & 0xFF, qc = (c >> (8 * q)) & 0xFF, qb = (hh >> (8 * q)) & 0xFF;
                const int li = 2 * p + q;
                w[li] = s1 * (float)((int)((qa & 0xF) | (((qb >> 0) & 3) << 4)) - 32);
                w[8 + li] = s2 * (float)((int)((qc & 0xF) | (((qb >> 2) & 3) << 4)) - 32);
                w[16 + li] = s3 * (float)((int)((qa >> 4) | (((qb >> 4) & 3) << 4)) - 32);
                w[24 + li] = s4 * (float)((int)((qc >> 4) | (((qb >> 6) & 3) << 4)) - 32);
            }
        }
    } else if constexpr (T == T_Q8_0) {  // kquant.rs:409-414
        const uint8_t* blk = row + u * 34;
        const float d = h2f(ld16(blk));
#pragma unroll
        for (int p = 0; p < 16; ++p) {
            const uint32_t v = ld16(blk + 2 + 2 * p);
            w[2 * p] = (float)(int)(int8_t)(v & 0xFF) * d;
            w[2 * p + 1] = (float)(int)(int8_t)(v >> 8) * d;
        }
    } else if constexpr (T == T_Q4_0) {  // kquant.rs:357-365
        const uint8_t* blk = row + u * 18;
        const float d = h2f(ld16(blk));
#pragma unroll
        for (int p = 0; p < 8; ++p) {
            const uint32_t v = ld16(blk + 2 + 2 * p);
            w[2 * p] = (float)((int)(v & 0xF) - 8) * d;
            w[2 * p + 1] = (float)((int)((v >> 8) & 0xF) - 8) * d;
            w[16 + 2 * p] = (float)((int)((v >> 4) & 0xF) - 8) * d;
            w[16 + 2 * p + 1] = (float)((int)(v >> 12) - 8) * d;
        }
    } else if constexpr (T == T_Q2_0) {  // kquant.rs:347-354: 64 elements per block, two units
        const uint8_t* blk = row + (u >> 1) * 18;
        const float d = h2f(ld16(blk));
        const uint8_t* q = blk + 2 + 8 * (u & 1);
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const uint32_t v = ld16(q + 2 * p);
#pragma unroll
            for (int j = 0; j < 8; ++j) w[8 * p + j] = (float)((int)((v >> (2 * j)) & 3) - 1) * d;
        }
    } else if constexpr (T == T_IQ4_NL) {  // kquant.rs:842-853
        const IqLut4* l4 = reinterpret_cast<const IqLut4*>(lut);
        const uint8_t* blk = row + u * 18;
        const float d = h2f(ld16(blk));
#pragma unroll
        for (int p = 0; p < 8; ++p) {
            const uint32_t v = ld16(blk + 2 + 2 * p);
            w[2 * p] = d * (float)l4->kv[v & 0xF];
            w[2 * p + 1] = d * (float)l4->kv[(v >> 8) & 0xF];
            w[16 + 2 * p] = d * (float)l4->kv[(v >> 4) & 0xF];
            w[16 + 2 * p + 1] = d * (float)l4->kv[v >> 12];
        }
    } else if constexpr (T == T_IQ4_XS) {  // kquant.rs:856-872
        const IqLut4* l4 = reinterpret_cast<const IqLut4*>(lut);
        const int b = u >> 3, ib = u & 7;
        const uint8_t* blk = row + b * 136;
        const float d = h2f(ld16(blk));
        const uint32_t scales_h = ld16(blk + 2);
        const uint32_t sl = blk[4 + (ib >> 1)];
        const int ls = (int)((sl >> (4 * (ib & 1))) & 0xF) | (int)(((scales_h >> (2 * ib)) & 3) << 4);
        const float dl = d * (float)(ls - 32);
        const uint8_t* q = blk + 8 + 16 * ib;
#pragma unroll
        for (int p = 0; p < 8; ++p) {
            const uint32_t v = ld16(q + 2 * p);
            w[2 * p] = dl * (float)l4->kv[v & 0xF];
            w[2 * p + 1] = dl * (float)l4->kv[(v >> 8) & 0xF];
            w[16 + 2 * p] = dl * (float)l4->kv[(v >> 4) & 0xF];
            w[16 + 2 * p + 1] = dl * (float)l4->kv[v >> 12];
        }
    } else if constexpr (T == T_IQ3_S) {  // kquant.rs:683-735
        const IqLut3s* l3 = reinterpret_cast<const IqLut3s*>(lut);
        const int b = u >> 3, ib = u & 7;
        const uint8_t* blk = row + b * 110;
        const float d = h2f(ld16(blk));
        const uint8_t *qs = blk + 2, *qh = blk + 66, *signs = blk + 74, *scales = blk + 106;
        const uint32_t scb = scales[ib >> 1];
        const float db = d * (1.0f + 2.0f * (float)((ib & 1) ? (scb >> 4) : (scb & 0xF)));
        const uint32_t qhb = qh[ib];
#pragma unroll
        for (int l = 0; l < 4; ++l) {
            const uint32_t idx = ld16(qs + 8 * ib + 2 * l);
            const uint32_t g1 = l3->grid[(idx & 0xFF) | ((qhb << (8 - 2 * l)) & 256u)];
            const uint32_t g2 = l3->grid[(idx >> 8) | ((qhb << (7 - 2 * l)) & 256u)];
            const uint32_t sg = signs[4 * ib + l];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float v0 = db * (float)((g1 >> (8 * j)) & 0xFF);
                const float v1 = db * (float)((g2 >> (8 * j)) & 0xFF);
                w[8 * l + j] = (sg >> j) & 1 ? -v0 : v0;
                w[8 * l + 4 + j] = (sg >> (j + 4)) & 1 ? -v1 : v1;
            }
        }
    } else if constexpr (T == T_IQ2_S) {  // kquant.rs:632-656
        const IqLut2s* l2 = reinterpret_cast<const IqLut2s*>(lut);
        const int b = u >> 3, ib = u & 7;
        const uint8_t* blk = row + b * 82;
        const float d = h2f(ld16(blk));
        const uint8_t *qs = blk + 2, *signs = blk + 34, *qh = blk + 66, *scales = blk + 74;
        const uint32_t sc = scales[ib];
        const float db0 = d * (0.5f + (float)(sc & 0xF)) * 0.25f, db1 = d * (0.5f + (float)(sc >> 4)) * 0.25f;
        const uint32_t qhb = qh[ib];
#pragma unroll
        for (int l = 0; l < 4; ++l) {
            const uint32_t idx = (uint32_t)qs[4 * ib + l] | ((qhb << (8 - 2 * l)) & 0x300u);
            const uint64_t g = l2->grid[idx];
            const uint32_t sg = signs[4 * ib + l];
            const float db = l < 2 ? db0 : db1;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float v = db * (float)((uint32_t)(g >> (8 * j)) & 0xFF);
                w[8 * l + j] = (sg >> j) & 1 ? -v : v;
            }
        }
    } else if constexpr (T == T_Q5_1) {  // kquant.rs:394-406
        const uint8_t* blk = row + u * 24;
        const float d = h2f(ld16(blk)), m = h2f(ld16(blk + 2));
        const uint32_t qh = *reinterpret_cast<const uint32_t*>(blk + 4);
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const uint32_t qv = *reinterpret_cast<const uint32_t*>(blk + 8 + 4 * p);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int j = 4 * p + q;
                const uint32_t byte = (qv >> (8 * q)) & 0xFF;
                const int x0 = (int)(byte & 0xF) | (int)(((qh >> j) << 4) & 0x10);
                const int x1 = (int)(byte >> 4) | (int)((qh >> (j + 12)) & 0x10);
                w[j] = (float)x0 * d + m;
                w[j + 16] = (float)x1 * d + m;
            }
        }
    }
}

// ---- decode fast path: x in registers, factored dot products ------------------
// For one-token GEMVs a lane keeps the 32 activations of a unit in registers and
// streams rows past them.  unit_dot returns sum_i w_i * x_i over the unit without
// materialising w_i, using conversions that cost one or two instructions per
// element and are exact:
//   Q4_K   : a nibble q is placed in byte 2 of the float 0x43000000, which is
//            128 + q exactly; sum (128+q) x is corrected by 128 * sum x, a per-lane
//            constant, and the sub-block scale and min are applied to the sums
//            (d1*S - (128*d1 + m1)*Sx).  About five of fp32's 24 bits go to the
//            bias, leaving the result far inside the 1e-3 bar.
//   IQ3_XXS: two grid bytes become the fp16 pair (1024+g0, 1024+g1) by a byte
//            permute, one half2 subtract removes the bias exactly, the two sign bits
//            are moved to bits 15/31 by one integer multiply and applied by xor,
//            and db multiplies the sub-block sum once.
// Other formats decode to registers and use the same fma order as decode_unit.
template <int T>
struct XUnit {
    float x[32];
    float s0, s1;  // sums of slots 0-15 / 16-31 (Q4_K, Q5_K)
};

template <int T>
__device__ __forceinline__ void load_x_unit(const float4* __restrict__ xs4, int nunits, int u, XUnit<T>& X) {
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const float4 v = xs4[k * nunits + u];
        X.x[4 * k] = v.x;
        X.x[4 * k + 1] = v.y;
        X.x[4 * k + 2] = v.z;
        X.x[4 * k + 3] = v.w;
    }
    X.s0 = 0.f;
    X.s1 = 0.f;
    if constexpr (T == T_Q4_K) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            X.s0 += X.x[i];
            X.s1 += X.x[16 + i];
        }
    }
}

// float(128 + byte j of w), w holding one value < 128 per byte
template <int J>
__device__ __forceinline__ float magic128(uint32_t w) {
    return __uint_as_float(__byte_perm(w, 0x43000000u, 0x7054u | (J << 8)));
}

template <int T>
__device__ __forceinline__ float unit_dot(const uint8_t* row, int u, const IqLut* lut, const XUnit<T>& X) {
    if constexpr (T == T_Q4_K) {
        const int b = u >> 3, j = (u >> 1) & 3, h = u & 1;
        const uint8_t* blk = row + b * 144;
        const float d = h2f(ld16(blk)), dmin = h2f(ld16(blk + 2));
        int sc1, m1, sc2, m2;
        scale_min_k4(2 * j, blk + 4, sc1, m1);
        scale_min_k4(2 * j + 1, blk + 4, sc2, m2);
        const uint4 qv = *reinterpret_cast<const uint4*>(blk + 16 + 32 * j + 16 * h);
        const uint32_t qw[4] = {qv.x, qv.y, qv.z, qv.w};
        float slo = 0.f, shi = 0.f;
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
            const uint32_t lo = qw[wi] & 0x0F0F0F0Fu, hi = (qw[wi] >> 4) & 0x0F0F0F0Fu;
            slo = fmaf(magic128<0>(lo), X.x[4 * wi], slo);
            slo = fmaf(magic128<1>(lo), X.x[4 * wi + 1], slo);
            slo = fmaf(magic128<2>(lo), X.x[4 * wi + 2], slo);
            slo = fmaf(magic128<3>(lo), X.x[4 * wi + 3], slo);
            shi = fmaf(magic128<0>(hi), X.x[16 + 4 * wi], shi);
            shi = fmaf(magic128<1>(hi), X.x[16 + 4 * wi + 1], shi);
            shi = fmaf(magic128<2>(hi), X.x[16 + 4 * wi + 2], shi);
            shi = fmaf(magic128<3>(hi), X.x[16 + 4 * wi + 3], shi);
        }
        const float d1 = d * (float)sc1, d2 = d * (float)sc2;
        const float c1 = fmaf(128.0f, d1, dmin * (float)m1), c2 = fmaf(128.0f, d2, dmin * (float)m2);
        float r = d1 * slo;
        r = fmaf(-c1, X.s0, r);
        r = fmaf(d2, shi, r);
        r = fmaf(-c2, X.s1, r);
        return r;
    } else if constexpr (T == T_IQ3_XXS) {
        const int b = u >> 3, ib = u & 7;
        const uint8_t* blk = row + b * 98;
        const float d = h2f(ld16(blk));
        const uint32_t aux = ld16(blk + 66 + 4 * ib) | (ld16(blk + 68 + 4 * ib) << 16);
        const float db = d * (0.5f + (float)(aux >> 28)) * 0.5f;
        const __half2 k1024 = __half2half2(__ushort_as_half((unsigned short)0x6400));
        float acc = 0.f;
#pragma unroll
        for (int l = 0; l < 4; ++l) {
            const uint32_t idx = ld16(blk + 2 + 8 * ib + 2 * l);
            const uint32_t code = (aux >> (7 * l)) & 127u;
            const uint32_t sg = code | ((__popc(code) & 1u) << 7);
            const int rep = (int)(threadIdx.x & (kLutRep - 1));
            const uint32_t g1 = lut->at(idx & 0xFFu, rep), g2 = lut->at(idx >> 8, rep);
            uint32_t p[4];
            p[0] = __byte_perm(g1, 0x64646464u, 0x5140u);
            p[1] = __byte_perm(g1, 0x64646464u, 0x7362u);
            p[2] = __byte_perm(g2, 0x64646464u, 0x5140u);
            p[3] = __byte_perm(g2, 0x64646464u, 0x7362u);
            const uint32_t mul[4] = {0x40008000u, 0x10002000u, 0x04000800u, 0x01000200u};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                __half2 hv = __hsub2(*reinterpret_cast<const __half2*>(&p[q]), k1024);
                uint32_t hb = *reinterpret_cast<const uint32_t*>(&hv);
                hb ^= (sg * mul[q]) & 0x80008000u;
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hb));
                acc = fmaf(f.x, X.x[8 * l + 2 * q], acc);
                acc = fmaf(f.y, X.x[8 * l + 2 * q + 1], acc);
            }
        }
        return db * acc;
    } else {
        float w[32];
        decode_unit<T>(row, u, lut, w);
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) acc = fmaf(w[i], X.x[i], acc);
        return acc;
    }
}

}  // namespace dnb
