/* Seeded synthetic inputs for the quantised-MoE expert path.
 *
 * One counter-based generator, usable from C, C++ and CUDA (host and device),
 * so that a CPU checker and the GPU library can materialise the same tensor
 * from (seed, tensor id) alone.  Nothing here is part of the arithmetic under
 * test: it only fabricates GGUF-format blocks and fp32 activations with the
 * value distributions the benchmark configurations prescribe.
 *
 *   stream key   k   = splitmix64(seed ^ (tensor_id * 0x9E3779B97F4A7C15))
 *   draw i of k      = splitmix64(k + i * 0xD1B54A32D192ED03)
 *   payload bytes    : byte j of a tensor = byte (j & 7) of draw (j >> 3)
 *   normals          : Box-Muller in double on draws (2i, 2i+1) of key k ^ NORMAL
 *
 * Block tensors are payload bytes with the floating-point header fields
 * overwritten per block (see dnb_synth_fix_block).
 */
#ifndef DNB_SYNTH_H
#define DNB_SYNTH_H

#include <stdint.h>
#include <math.h>

#if defined(__CUDACC__)
#define DNB_HD __host__ __device__ static inline
#else
#define DNB_HD static inline
#endif

/* ggml type ids handled by the generator (same values as the GGUF enum). */
#define DNB_TYPE_F32 0
#define DNB_TYPE_Q5_1 7
#define DNB_TYPE_Q8_0 8
#define DNB_TYPE_Q4_K 12
#define DNB_TYPE_Q5_K 13
#define DNB_TYPE_Q6_K 14
#define DNB_TYPE_IQ3_XXS 18
#define DNB_TYPE_Q4_0 2
#define DNB_TYPE_IQ4_NL 20
#define DNB_TYPE_IQ3_S 21
#define DNB_TYPE_IQ2_S 22
#define DNB_TYPE_IQ4_XS 23
#define DNB_TYPE_Q2_0 42

#define DNB_SYNTH_NORMAL_SALT 0x6E6F726D616C2121ull

DNB_HD uint64_t dnb_splitmix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

DNB_HD uint64_t dnb_synth_key(uint64_t seed, uint64_t tensor_id) {
    return dnb_splitmix64(seed ^ (tensor_id * 0x9E3779B97F4A7C15ull));
}

DNB_HD uint64_t dnb_synth_draw(uint64_t key, uint64_t i) {
    return dnb_splitmix64(key + i * 0xD1B54A32D192ED03ull);
}

/* Standard normal number i of the stream `key` (double precision Box-Muller). */
DNB_HD double dnb_synth_normal(uint64_t key, uint64_t i) {
    const uint64_t k = key ^ DNB_SYNTH_NORMAL_SALT;
    const double u1 = ((double)(dnb_synth_draw(k, 2 * i) >> 11) + 0.5) * (1.0 / 9007199254740992.0);
    const double u2 = ((double)(dnb_synth_draw(k, 2 * i + 1) >> 11) + 0.5) * (1.0 / 9007199254740992.0);
    return sqrt(-2.0 * log(u1)) * cos(6.283185307179586476925 * u2);
}

/* fp32 -> IEEE binary16 bits, round to nearest even (finite inputs). */
DNB_HD uint16_t dnb_f32_to_f16_bits(float f) {
    union { float f; uint32_t u; } v;
    v.f = f;
    const uint32_t sign = (v.u >> 16) & 0x8000u;
    const uint32_t a = v.u & 0x7FFFFFFFu;
    if (a >= 0x47800000u) return (uint16_t)(sign | 0x7C00u);      /* overflow -> inf */
    if (a < 0x33000000u) return (uint16_t)sign;                    /* < 2^-25 -> 0 */
    if (a < 0x38800000u) {                                         /* subnormal half */
        const uint32_t shift = 126u - (a >> 23);                   /* 14..24 */
        const uint32_t mant = (a & 0x7FFFFFu) | 0x800000u;
        uint32_t h = mant >> shift;
        const uint32_t rem = mant & ((1u << shift) - 1u);
        const uint32_t half = 1u << (shift - 1u);
        if (rem > half || (rem == half && (h & 1u))) h++;
        return (uint16_t)(sign | h);
    }
    uint32_t h = ((a - 0x38000000u) >> 13);
    const uint32_t rem = a & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) h++;
    return (uint16_t)(sign | h);
}

DNB_HD int dnb_synth_type_size(int type) {
    switch (type) {
        case DNB_TYPE_F32: return 4;
        case DNB_TYPE_Q5_1: return 24;
        case DNB_TYPE_Q8_0: return 34;
        case DNB_TYPE_Q4_K: return 144;
        case DNB_TYPE_Q5_K: return 176;
        case DNB_TYPE_Q6_K: return 210;
        case DNB_TYPE_IQ3_XXS: return 98;
        case DNB_TYPE_Q4_0: case DNB_TYPE_IQ4_NL: case DNB_TYPE_Q2_0: return 18;
        case DNB_TYPE_IQ3_S: return 110;
        case DNB_TYPE_IQ2_S: return 82;
        case DNB_TYPE_IQ4_XS: return 136;
        default: return 0;
    }
}

DNB_HD int dnb_synth_block_size(int type) {
    switch (type) {
        case DNB_TYPE_F32: return 1;
        case DNB_TYPE_Q5_1: case DNB_TYPE_Q8_0: case DNB_TYPE_Q4_0: case DNB_TYPE_IQ4_NL: return 32;
        case DNB_TYPE_Q2_0: return 64;
        case DNB_TYPE_Q4_K: case DNB_TYPE_Q5_K: case DNB_TYPE_Q6_K: case DNB_TYPE_IQ3_XXS:
        case DNB_TYPE_IQ3_S: case DNB_TYPE_IQ2_S: case DNB_TYPE_IQ4_XS: return 256;
        default: return 0;
    }
}

DNB_HD uint8_t dnb_synth_byte(uint64_t key, uint64_t j) {
    return (uint8_t)(dnb_synth_draw(key, j >> 3) >> (8 * (j & 7)));
}

/* Overwrite the header fields of block `b` (already holding payload bytes):
 *   Q4_K / Q5_K : d, dmin = f16(|N(0,1)| * 0.01); the 12 scale bytes stay uniform,
 *                 which makes all sixteen 6-bit scales/mins uniform on 0..63
 *   IQ3_XXS     : d = f16(|N(0,1)| * 0.02); grid indices, 7-bit sign codes and the
 *                 4-bit sub-block scales stay uniform
 *   Q6_K        : d = f16(|N(0,1)| * 0.01) at byte 208; 16 int8 scales = (byte & 63) - 32
 *   Q8_0        : d = f16(|N(0,1)| * 0.01)
 *   Q5_1        : d, m = f16(|N(0,1)| * 0.01)                                        */
DNB_HD void dnb_synth_fix_block(int type, uint64_t key, uint64_t b, uint8_t* blk) {
    const double scale = (type == DNB_TYPE_IQ3_XXS) ? 0.02 : 0.01;
    const uint16_t d = dnb_f32_to_f16_bits((float)(fabs(dnb_synth_normal(key, 2 * b)) * scale));
    const uint16_t d2 = dnb_f32_to_f16_bits((float)(fabs(dnb_synth_normal(key, 2 * b + 1)) * scale));
    switch (type) {
        case DNB_TYPE_Q4_K: case DNB_TYPE_Q5_K: case DNB_TYPE_Q5_1:
            blk[0] = (uint8_t)d; blk[1] = (uint8_t)(d >> 8);
            blk[2] = (uint8_t)d2; blk[3] = (uint8_t)(d2 >> 8);
            break;
        case DNB_TYPE_IQ3_XXS: case DNB_TYPE_Q8_0:
        case DNB_TYPE_Q4_0: case DNB_TYPE_IQ4_NL: case DNB_TYPE_IQ3_S: case DNB_TYPE_IQ2_S: case DNB_TYPE_IQ4_XS:
        case DNB_TYPE_Q2_0:  /* d first in all of these, everything else uniform bytes */
            blk[0] = (uint8_t)d; blk[1] = (uint8_t)(d >> 8);
            break;
        case DNB_TYPE_Q6_K:
            for (int i = 0; i < 16; ++i) blk[192 + i] = (uint8_t)(int8_t)((int)(blk[192 + i] & 63) - 32);
            blk[208] = (uint8_t)d; blk[209] = (uint8_t)(d >> 8);
            break;
        default: break;
    }
}

#ifndef __CUDA_ARCH__
/* Host-side fills (the device versions live in the CUDA library). */
static inline void dnb_synth_fill_blocks_host(int type, uint64_t seed, uint64_t tensor_id,
                                              uint8_t* dst, uint64_t n_blocks) {
    const uint64_t key = dnb_synth_key(seed, tensor_id);
    const uint64_t ts = (uint64_t)dnb_synth_type_size(type);
    const uint64_t bytes = n_blocks * ts;
    for (uint64_t w = 0; w * 8 < bytes; ++w) {
        const uint64_t r = dnb_synth_draw(key, w);
        for (uint64_t j = 0; j < 8 && w * 8 + j < bytes; ++j) dst[w * 8 + j] = (uint8_t)(r >> (8 * j));
    }
    for (uint64_t b = 0; b < n_blocks; ++b) dnb_synth_fix_block(type, key, b, dst + b * ts);
}

/* fp32 tensor of N(0, sigma^2). */
static inline void dnb_synth_fill_normal_host(uint64_t seed, uint64_t tensor_id, float sigma,
                                              float* dst, uint64_t n) {
    const uint64_t key = dnb_synth_key(seed, tensor_id);
    for (uint64_t i = 0; i < n; ++i) dst[i] = (float)(dnb_synth_normal(key, i) * (double)sigma);
}

/* Zipf(s) router bias: a seeded permutation pi of 0..n-1, bias[pi(r)] = -s * ln(r + 1). */
static inline void dnb_synth_zipf_bias_host(uint64_t seed, uint64_t tensor_id, double s,
                                            float* bias, uint32_t n) {
    const uint64_t key = dnb_synth_key(seed, tensor_id);
    for (uint32_t i = 0; i < n; ++i) bias[i] = (float)i;          /* holds pi while shuffling */
    for (uint32_t i = n; i > 1; --i) {                             /* Fisher-Yates */
        const uint32_t j = (uint32_t)(dnb_synth_draw(key, i) % i);
        const float t = bias[i - 1]; bias[i - 1] = bias[j]; bias[j] = t;
    }
    /* bias[r] currently holds pi(r); invert into ranks */
    float tmp[4096];
    if (n > 4096) return;
    for (uint32_t r = 0; r < n; ++r) tmp[(uint32_t)bias[r]] = (float)(-s * log((double)r + 1.0));
    for (uint32_t i = 0; i < n; ++i) bias[i] = tmp[i];
}
#endif

#endif /* DNB_SYNTH_H */
