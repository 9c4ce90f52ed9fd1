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

// Shared lookup tables of the IQ formats (copied into shared memory per CTA).
struct IqLut {
    uint32_t grid3xxs[256];
};

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
            const uint32_t g1 = lut->grid3xxs[idx & 0xFF], g2 = lut->grid3xxs[idx >> 8];
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

}  // namespace dnb
