// IQ3_XXS decode into mma.sync fragments: what the one-token kernels of gemv_mma.cu and
// decode_fused.cu share.  Each translation unit that includes this header owns a copy of
// the bf16 codebook and uploads it once per device.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "dnb_common.cuh"
#include "formats.cuh"
#include "bulk.cuh"
#include "dnb_iq_tables.h"

// Sub-blocks of the K loops that are unrolled together (more independent work per warp, more registers).
#ifndef DNB_IQ3_UNROLL
#define DNB_IQ3_UNROLL 2
#endif

namespace dnb {

constexpr int kGmRows = 8;     // rows of one matrix per group (x2 matrices = the 16 mma rows)
constexpr int kGmKs = 4;       // warps that split K within a group
constexpr int kGmGroups = 5;   // groups a CTA can hold
constexpr int kGmThreads = kGmGroups * kGmKs * 32;
constexpr int kGmSplit = 3;    // bf16 terms per activation value
constexpr int kIq3Unroll = 2;  // sub-blocks of the gate/up K loop unrolled together

// What a CTA copies into shared memory in one bulk copy: the IQ3_XXS codebook as bf16 pairs,
// entry e of copy r at [e * kLutRep + r]; .x = elements 0,1, .y = elements 2,3.  (A second table
// with ready-made sign masks was tried: its 16-byte lookups cost more shared-memory cycles than
// the multiply-and-mask below costs issue slots, and the kernels got slower.)
struct Iq3Tables {
    uint2 grid[256 * kLutRep];
};
static __device__ __align__(16) Iq3Tables g_iq3_tables;
static bool g_tables_m[64] = {false};

static int upload_tables_m(int device) {
    if (device < 0 || device >= 64) return DNB_ERR_ARG;
    if (g_tables_m[device]) return DNB_OK;
    static Iq3Tables tb;
    for (int e = 0; e < 256; ++e) {
        const uint32_t w = dnb_iq3xxs_grid[e];
        uint32_t h[4];
        for (int j = 0; j < 4; ++j) {
            const float f = (float)((w >> (8 * j)) & 0xFFu);  // <= 62: its fp32 pattern has nothing below bit 16
            uint32_t bits;
            memcpy(&bits, &f, 4);
            h[j] = bits >> 16;
        }
        for (int r = 0; r < kLutRep; ++r) tb.grid[e * kLutRep + r] = make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16));
    }
    DNB_CUDA(cudaMemcpyToSymbol(g_iq3_tables, &tb, sizeof(tb)));
    g_tables_m[device] = true;
    return DNB_OK;
}
// A lane's view of the table in shared memory: its own copy
struct Iq3Lane {
    const uint2* grid;
    __device__ __forceinline__ Iq3Lane(const Iq3Tables* tb, int lane) : grid(tb->grid + (lane & (kLutRep - 1))) {}
};

__device__ __forceinline__ uint32_t bf16_bits(float v) { return __bfloat16_as_ushort(__float2bfloat16_rn(v)); }
__device__ __forceinline__ float silu_m(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float bf16_val(uint32_t h) { return __uint_as_float(h << 16); }

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Eight weights of one IQ3_XXS sub-block as four signed bf16 pairs (without the scale):
// `idx` = the two codebook indices of this lane's quarter, `code` = its 7 sign bits.
__device__ __forceinline__ void iq3_pairs(const Iq3Lane& L, uint32_t idx, uint32_t code, uint32_t (&p)[4]) {
    const uint32_t sg = code | ((__popc(code) & 1u) << 7);  // bit 7 makes the number of minus signs even
    const uint2 g1 = L.grid[(idx & 0xFFu) * kLutRep], g2 = L.grid[(idx >> 8) * kLutRep];
    p[0] = g1.x ^ ((sg * 0x40008000u) & 0x80008000u);
    p[1] = g1.y ^ ((sg * 0x10002000u) & 0x80008000u);
    p[2] = g2.x ^ ((sg * 0x04000800u) & 0x80008000u);
    p[3] = g2.y ^ ((sg * 0x01000200u) & 0x80008000u);
}

// C = A * B with a zero accumulator
__device__ __forceinline__ void mma_bf16_z(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

// One sub-block (32 elements) of two IQ3_XXS rows against the B columns: the lane (g, t) decodes
// elements 8t .. 8t+7 of row `ba` (mma rows 0-7) and of row `bb` (mma rows 8-15); `y` holds the
// lane's B column for those eight elements.  c[0], c[1] = row g of `ba`, columns 2t, 2t+1;
// c[2], c[3] = row g of `bb`.  aux_a, aux_b return the sub-block words (scale in the top 4 bits).
__device__ __forceinline__ void iq3_subblock_mma(const uint8_t* ba, const uint8_t* bb, int ib, int t, const Iq3Lane& lutp,
                                                 const uint4& y, float (&c)[4], uint32_t& aux_a, uint32_t& aux_b) {
    aux_a = ld16(ba + 66 + 4 * ib) | (ld16(ba + 68 + 4 * ib) << 16);
    aux_b = ld16(bb + 66 + 4 * ib) | (ld16(bb + 68 + 4 * ib) << 16);
    const uint32_t ida = ld16(ba + 2 + 8 * ib + 2 * t), idb = ld16(bb + 2 + 8 * ib + 2 * t);
    uint32_t p[4], u4[4];
    iq3_pairs(lutp, ida, (aux_a >> (7 * t)) & 127u, p);
    iq3_pairs(lutp, idb, (aux_b >> (7 * t)) & 127u, u4);
    mma_bf16_z(c, p[0], u4[0], p[1], u4[1], y.x, y.y);
    mma_bf16(c, p[2], u4[2], p[3], u4[3], y.z, y.w);
}
// d * (0.5 + s) * 0.5 = (d / 4) * (2 s + 1), exact in fp32 either way (kquant.rs:667); dq = d / 4
__device__ __forceinline__ float iq3_scale(float dq, uint32_t aux) { return fmaf((float)(aux >> 28), dq + dq, dq); }

// Three-way bf16 split of an fp32 value: three 8-bit mantissas carry its 24 bits, and bf16 has fp32's
// exponent range, so v = h0 + h1 + h2 holds for every finite v (the subtractions are exact).
__device__ __forceinline__ void split3(float v, uint32_t (&h)[kGmSplit]) {
#pragma unroll
    for (int n = 0; n < kGmSplit; ++n) {
        h[n] = bf16_bits(v);
        v -= bf16_val(h[n]);
    }
}
// A gate/up group's share of one warp: blocks [b0, b1) of 8 gate rows (rowg: this lane's row g)
// and 8 up rows.  After the call lanes t = 0 and t = 1 of every row hold the row's two totals.
__device__ __forceinline__ void gate_up_warp(const uint8_t* rowg, const uint8_t* rowu, const Iq3Lane& lutp,
                                             const uint16_t* xb, bool has_col, int b0, int b1, int t, float& accg,
                                             float& accu) {
    for (int b = b0; b < b1; ++b) {
        const uint8_t* bg = rowg + b * 98;
        const uint8_t* bu = rowu + b * 98;
        const float dg = h2f(ld16(bg)) * 0.25f, du = h2f(ld16(bu)) * 0.25f;
#pragma unroll kIq3Unroll
        for (int ib = 0; ib < 8; ++ib) {
            uint4 y = make_uint4(0u, 0u, 0u, 0u);
            if (has_col) y = *reinterpret_cast<const uint4*>(xb + (b * 8 + ib) * 32);
            float c[4];
            uint32_t auxg, auxu;
            iq3_subblock_mma(bg, bu, ib, t, lutp, y, c, auxg, auxu);
            accg = fmaf(iq3_scale(dg, auxg), c[0] + c[1], accg);
            accu = fmaf(iq3_scale(du, auxu), c[2] + c[3], accu);
        }
    }
    // lane t = 0 holds the hi and lo columns, t = 1 the lo2 column, t = 2, 3 nothing
    accg += __shfl_xor_sync(0xffffffffu, accg, 1);
    accu += __shfl_xor_sync(0xffffffffu, accu, 1);
}

// Barrier of the kGmKs warps of gate/up group q (named barriers 1 .. kGmGroups).  The ids are
// immediates so that the kernel reserves only the barriers it uses, not all sixteen.
__device__ __forceinline__ void group_barrier(int q) {
    switch (q) {
        case 0: asm volatile("bar.sync 1, %0;" ::"n"(kGmKs * 32) : "memory"); break;
        case 1: asm volatile("bar.sync 2, %0;" ::"n"(kGmKs * 32) : "memory"); break;
        case 2: asm volatile("bar.sync 3, %0;" ::"n"(kGmKs * 32) : "memory"); break;
        case 3: asm volatile("bar.sync 4, %0;" ::"n"(kGmKs * 32) : "memory"); break;
        default: asm volatile("bar.sync 5, %0;" ::"n"(kGmKs * 32) : "memory"); break;
    }
}

}  // namespace dnb
