// Segmented dequant matmul (fp32 lanes): the kernel behind single-matrix GEMV,
// the decode expert GEMVs and the small-m grouped GEMM of prefill.
//
// Reference kernels of the same role: kernels_moe_v3.cu:216-266 (dno_gemv_q4k_v3),
// kernels_seg_k.cu:201-241, kernels_exp_iq_v2.cu:259-319 (segmented m=1),
// kernels_exp_k_pf.cu:188-258 / kernels_exp_iq_pf.cu (m-row prefill).  This is
// a different design: a CTA first stages a contiguous tile of weight rows into
// shared memory with 128-bit coalesced loads (so every format streams HBM the
// same way, whatever its block alignment), stages the activation rows of up to
// TT tokens in a lane-friendly slot order, then each group of LPR lanes owns a
// row: a lane decodes 32-element units into registers once and applies them to
// all staged tokens.  Sums are fixed-order (lane partials in ascending unit
// order, xor-shuffle tree), so results are bit-identical run to run.
#include "dnb_common.cuh"
#include "formats.cuh"
#include "dnb_iq_tables.h"

namespace dnb {

__constant__ uint32_t c_iq3xxs_grid[256];
__constant__ uint32_t c_iq3s_grid[512];
__constant__ unsigned long long c_iq2s_grid[1024];
__constant__ int8_t c_kvalues_iq4nl[16];
static bool g_tables_uploaded[64] = {false};

static int upload_tables(int device) {
    if (device < 0 || device >= 64) return DNB_ERR_ARG;
    if (g_tables_uploaded[device]) return DNB_OK;
    DNB_CUDA(cudaMemcpyToSymbol(c_iq3xxs_grid, dnb_iq3xxs_grid, sizeof(c_iq3xxs_grid)));
    DNB_CUDA(cudaMemcpyToSymbol(c_iq3s_grid, dnb_iq3s_grid, sizeof(c_iq3s_grid)));
    DNB_CUDA(cudaMemcpyToSymbol(c_iq2s_grid, dnb_iq2s_grid, sizeof(c_iq2s_grid)));
    DNB_CUDA(cudaMemcpyToSymbol(c_kvalues_iq4nl, dnb_kvalues_iq4nl, sizeof(c_kvalues_iq4nl)));
    g_tables_uploaded[device] = true;
    return DNB_OK;
}

// The CTA's copy of the format's codebook, behind the one pointer decode_unit takes.
template <int T>
__device__ __forceinline__ void fill_lut(IqLut* lut, int tid, int nthr) {
    if constexpr (T == T_IQ3_XXS) {
        lut->fill(c_iq3xxs_grid, tid, nthr);
    } else if constexpr (T == T_IQ3_S) {
        IqLut3s* l = reinterpret_cast<IqLut3s*>(lut);
        for (int i = tid; i < 512; i += nthr) l->grid[i] = c_iq3s_grid[i];
    } else if constexpr (T == T_IQ2_S) {
        IqLut2s* l = reinterpret_cast<IqLut2s*>(lut);
        for (int i = tid; i < 1024; i += nthr) l->grid[i] = c_iq2s_grid[i];
    } else if constexpr (T == T_IQ4_NL || T == T_IQ4_XS) {
        IqLut4* l = reinterpret_cast<IqLut4*>(lut);
        if (tid < 16) l->kv[tid] = c_kvalues_iq4nl[tid];
    }
}

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }

// Copy `bytes` (even) from global to shared; 128-bit path when both are aligned.
__device__ __forceinline__ void stage_bytes(uint8_t* dst, const uint8_t* src, int bytes, int tid, int nthr) {
    if ((((uintptr_t)src | (uintptr_t)dst) & 15) == 0) {
        const int n16 = bytes >> 4;
        const uint4* s4 = reinterpret_cast<const uint4*>(src);
        uint4* d4 = reinterpret_cast<uint4*>(dst);
        for (int i = tid; i < n16; i += nthr) d4[i] = __ldcs(s4 + i);
        for (int i = (n16 << 4) + 2 * tid; i < bytes; i += 2 * nthr)
            *reinterpret_cast<uint16_t*>(dst + i) = *reinterpret_cast<const uint16_t*>(src + i);
    } else if ((((uintptr_t)src | (uintptr_t)dst) & 3) == 0) {
        const int n4 = bytes >> 2;
        for (int i = tid; i < n4; i += nthr)
            reinterpret_cast<uint32_t*>(dst)[i] = __ldcs(reinterpret_cast<const uint32_t*>(src) + i);
        for (int i = (n4 << 2) + 2 * tid; i < bytes; i += 2 * nthr)
            *reinterpret_cast<uint16_t*>(dst + i) = *reinterpret_cast<const uint16_t*>(src + i);
    } else {
        for (int i = 2 * tid; i < bytes; i += 2 * nthr)
            *reinterpret_cast<uint16_t*>(dst + i) = *reinterpret_cast<const uint16_t*>(src + i);
    }
}

constexpr int kThreads = 256;

// grid = (row tiles, segments).  Dynamic shared memory:
//   [IqLut][weights A tile][weights B tile (fused)][x: TT * n_in floats, slot order]
template <int T, bool FUSED, int LPR, int TT>
__global__ void __launch_bounds__(kThreads)
seg_matmul_kernel(const SegDesc* __restrict__ seg, const int32_t* __restrict__ nseg_dev, int nseg_host, int n_in,
                  int n_out, int rb, int tile_rows, const float* __restrict__ x, int ldx,
                  const int32_t* __restrict__ row_token, float* __restrict__ out, SegDesc single, int tok_chunk) {
    const int s = blockIdx.y;
    const int nseg = nseg_dev ? *nseg_dev : nseg_host;
    if (s >= nseg) return;
    const SegDesc sd = seg ? seg[s] : single;
    if (sd.m == 0) return;
    // blockIdx.z: which tok_chunk tokens of the segment this CTA takes.  A segment with many tokens (the shared
    // expert of a batch, a hot expert of a chunk) is spread over several CTAs instead of being walked by one;
    // a token's arithmetic does not depend on the split.
    const uint32_t t_begin = blockIdx.z * (uint32_t)tok_chunk;
    if (t_begin >= sd.m) return;
    const uint32_t t_end = min(sd.m, t_begin + (uint32_t)tok_chunk);
    const int r0 = blockIdx.x * tile_rows;
    const int rows = min(tile_rows, n_out - r0);
    if (rows <= 0) return;

    extern __shared__ __align__(16) uint8_t smem[];
    IqLut* lut = reinterpret_cast<IqLut*>(smem);
    constexpr int lut_bytes = lut_bytes_of<T>();
    const int tile_bytes = (tile_rows * rb + 15) & ~15;
    uint8_t* wa = smem + lut_bytes;
    uint8_t* wb = wa + tile_bytes;
    float4* xs4 = reinterpret_cast<float4*>(wa + (FUSED ? 2 : 1) * tile_bytes);
    float* xs = reinterpret_cast<float*>(xs4);

    const int tid = threadIdx.x;
    fill_lut<T>(lut, tid, kThreads);
    stage_bytes(wa, sd.wa + (size_t)r0 * rb, rows * rb, tid, kThreads);
    if constexpr (FUSED) stage_bytes(wb, sd.wb + (size_t)r0 * rb, rows * rb, tid, kThreads);

    const int nunits = n_in >> 5;
    const int lane = tid & 31, warp = tid >> 5;
    constexpr int GPW = 32 / LPR;               // row groups per warp
    const int sub = lane % LPR;
    const int grp = warp * GPW + lane / LPR;    // group index in the CTA
    constexpr int NGRP = (kThreads / 32) * GPW;

    for (uint32_t t0 = t_begin; t0 < t_end; t0 += TT) {
        const int nt = min((uint32_t)TT, t_end - t0);
        __syncthreads();  // previous chunk fully consumed (and, first time, nothing)
        for (int tok = 0; tok < nt; ++tok) {
            const uint32_t prow = sd.row0 + t0 + tok;
            const float* xr = x + (size_t)(row_token ? row_token[prow] : (int32_t)prow) * ldx;
            for (int i = tid; i < n_in; i += kThreads) {
                int u, sl;
                slot_of<T>(i, u, sl);
                xs[(((tok * 8 + (sl >> 2)) * nunits + u) << 2) + (sl & 3)] = xr[i];
            }
        }
        __syncthreads();  // weights (first chunk) and x staged

        for (int r = grp; r < rows; r += NGRP) {
            float acc_a[TT], acc_b[TT];
#pragma unroll
            for (int t = 0; t < TT; ++t) { acc_a[t] = 0.f; acc_b[t] = 0.f; }
            const uint8_t* ra = wa + r * rb;
            const uint8_t* rbp = wb + r * rb;
            for (int u = sub; u < nunits; u += LPR) {
                float w[32];
                decode_unit<T>(ra, u, lut, w);
#pragma unroll
                for (int t = 0; t < TT; ++t) {
                    if (t < nt) {
                        float a = acc_a[t];
#pragma unroll
                        for (int k = 0; k < 8; ++k) {
                            const float4 xv = xs4[(t * 8 + k) * nunits + u];
                            a = fmaf(w[4 * k], xv.x, a);
                            a = fmaf(w[4 * k + 1], xv.y, a);
                            a = fmaf(w[4 * k + 2], xv.z, a);
                            a = fmaf(w[4 * k + 3], xv.w, a);
                        }
                        acc_a[t] = a;
                    }
                }
                if constexpr (FUSED) {
                    decode_unit<T>(rbp, u, lut, w);
#pragma unroll
                    for (int t = 0; t < TT; ++t) {
                        if (t < nt) {
                            float a = acc_b[t];
#pragma unroll
                            for (int k = 0; k < 8; ++k) {
                                const float4 xv = xs4[(t * 8 + k) * nunits + u];
                                a = fmaf(w[4 * k], xv.x, a);
                                a = fmaf(w[4 * k + 1], xv.y, a);
                                a = fmaf(w[4 * k + 2], xv.z, a);
                                a = fmaf(w[4 * k + 3], xv.w, a);
                            }
                            acc_b[t] = a;
                        }
                    }
                }
            }
#pragma unroll
            for (int t = 0; t < TT; ++t) {
#pragma unroll
                for (int o = LPR / 2; o > 0; o >>= 1) {
                    acc_a[t] += __shfl_xor_sync(0xffffffffu, acc_a[t], o);
                    if constexpr (FUSED) acc_b[t] += __shfl_xor_sync(0xffffffffu, acc_b[t], o);
                }
            }
            if (sub == 0) {
#pragma unroll
                for (int t = 0; t < TT; ++t) {
                    if (t < nt) {
                        const size_t o = (size_t)(sd.row0 + t0 + t) * n_out + r0 + r;
                        out[o] = FUSED ? silu_f(acc_a[t]) * acc_b[t] : acc_a[t];
                    }
                }
            }
        }
    }
}

template <int T, bool FUSED, int LPR, int TT>
static int launch_cfg(dnb_ctx* c, cudaStream_t st, const SegDesc* seg, const int32_t* nseg_dev, int nseg_max, int n_in,
                      int n_out, const float* x, int ldx, const int32_t* row_token, float* out, SegDesc single, int m_max) {
    const int rb = (int)row_bytes(T, n_in);
    // Aim at ~16 KB of weight bytes per CTA, in whole "group rounds", and keep
    // tile starts 16-byte aligned (tile_rows * rb % 16 == 0) where possible.
    constexpr int NGRP = (kThreads / 32) * (32 / LPR);
    int rounds = (16384 / (FUSED ? 2 : 1)) / (NGRP * rb);
    if (rounds < 1) rounds = 1;
    int tile_rows = NGRP * rounds;
    if (tile_rows > n_out) tile_rows = ((n_out + NGRP - 1) / NGRP) * NGRP;
    const int tile_bytes = (tile_rows * rb + 15) & ~15;
    const size_t smem = (size_t)lut_bytes_of<T>() + (size_t)(FUSED ? 2 : 1) * tile_bytes +
                        (size_t)TT * n_in * sizeof(float);
    auto kern = seg_matmul_kernel<T, FUSED, LPR, TT>;
    static SmemGrant grant;
    if (smem > 200 * 1024) {
        set_error("seg_matmul: shared memory %zu B too large (n_in=%d)", smem, n_in);
        return DNB_DECLINED;
    }
    DNB_CUDA(grant_smem(grant, c->device, kern, smem));
    // Tokens of a segment per CTA.  Chunks of many tokens (a hot expert of a prefill chunk would otherwise be walked
    // by one CTA per row tile) are spread over up to eight CTAs; decode batches are not split: measured at 32 tokens,
    // the empty CTAs of the extra grid dimension cost more (21.2 ms per 48-layer step) than the split saves (18.6 ms).
    int tok_chunk = m_max > 0 ? m_max : 1;
    if (m_max >= 64) tok_chunk = ((m_max + 7) / 8 + TT - 1) / TT * TT;
    const int gz = m_max > tok_chunk ? (m_max + tok_chunk - 1) / tok_chunk : 1;
    dim3 grid((n_out + tile_rows - 1) / tile_rows, nseg_max, gz);
    const bool sh = (st == c->side);
    const char* pname = FUSED ? (TT == 1 ? (sh ? "seg_gate_up_m1_shared" : "seg_gate_up_m1")
                                         : (sh ? "seg_gate_up_m4_shared" : "seg_gate_up_m4"))
                              : (TT == 1 ? (sh ? "seg_matmul_m1_shared" : "seg_matmul_m1")
                                         : (sh ? "seg_matmul_m4_shared" : "seg_matmul_m4"));
    ProfScope prof_(c, st, pname);
    kern<<<grid, kThreads, smem, st>>>(seg, nseg_dev, nseg_max, n_in, n_out, rb, tile_rows, x, ldx, row_token, out,
                                        single, tok_chunk);
    c->launches++;
    DNB_CUDA(cudaGetLastError());
    return DNB_OK;
}

template <int T, bool FUSED>
static int launch_t(dnb_ctx* c, cudaStream_t st, const SegDesc* seg, const int32_t* nseg_dev, int nseg_max, int n_in,
                    int n_out, const float* x, int ldx, const int32_t* row_token, float* out, int m_max,
                    SegDesc single) {
    const int nunits = n_in / 32;
    const bool wide = nunits >= 32;
    if (m_max <= 1) {
        return wide ? launch_cfg<T, FUSED, 32, 1>(c, st, seg, nseg_dev, nseg_max, n_in, n_out, x, ldx, row_token, out, single, m_max)
                    : launch_cfg<T, FUSED, 16, 1>(c, st, seg, nseg_dev, nseg_max, n_in, n_out, x, ldx, row_token, out, single, m_max);
    }
    return wide ? launch_cfg<T, FUSED, 32, 4>(c, st, seg, nseg_dev, nseg_max, n_in, n_out, x, ldx, row_token, out, single, m_max)
                : launch_cfg<T, FUSED, 16, 4>(c, st, seg, nseg_dev, nseg_max, n_in, n_out, x, ldx, row_token, out, single, m_max);
}

int launch_seg_matmul(dnb_ctx* c, cudaStream_t st, int type, bool fused, const SegDesc* seg, const int32_t* nseg_dev,
                      int nseg_max, int n_in, int n_out, const float* x, int ldx, const int32_t* row_token,
                      float* out, int m_max, const SegDesc* single_p) {
    const SegDesc single = single_p ? *single_p : SegDesc{nullptr, nullptr, 0u, 0u};
    if (!seg && !single_p) return DNB_ERR_ARG;
    if (row_bytes(type, n_in) == 0 || n_in % 32 != 0 || n_out <= 0 || nseg_max <= 0) {
        set_error("seg_matmul: unsupported type %d / shape %dx%d", type, n_out, n_in);
        return DNB_DECLINED;
    }
    int rc = upload_tables(c->device);
    if (rc != DNB_OK) return rc;
#define DNB_DISPATCH(TT)                                                                                             \
    case TT:                                                                                                         \
        return fused ? launch_t<TT, true>(c, st, seg, nseg_dev, nseg_max, n_in, n_out, x, ldx, row_token, out, m_max, single) \
                     : launch_t<TT, false>(c, st, seg, nseg_dev, nseg_max, n_in, n_out, x, ldx, row_token, out, m_max, single);
    switch (type) {
        DNB_DISPATCH(T_Q4_K)
        DNB_DISPATCH(T_Q5_K)
        DNB_DISPATCH(T_Q6_K)
        DNB_DISPATCH(T_IQ3_XXS)
        DNB_DISPATCH(T_Q8_0)
        DNB_DISPATCH(T_Q5_1)
        DNB_DISPATCH(T_Q4_0)
        DNB_DISPATCH(T_IQ4_NL)
        DNB_DISPATCH(T_IQ4_XS)
        DNB_DISPATCH(T_IQ3_S)
        DNB_DISPATCH(T_IQ2_S)
        DNB_DISPATCH(T_Q2_0)
        default:
            set_error("seg_matmul: no kernel for ggml type %d", type);
            return DNB_DECLINED;
    }
#undef DNB_DISPATCH
}

// ---- sequential-order GEMV ---------------------------------------------------
// One thread per row: dequantise block by block and accumulate acc += w[i]*x[i]
// in ascending i with separate multiply and add roundings, the order of the
// reference's scalar path (moe_expert.rs:698-713 gemv_scalar_body, dot_seq) and
// of its bit-exact kernels (kernels_moe.cu).  Slow by design; it exists so the
// fast kernels can be checked against CPU-identical bits at any size.
template <int T>
__global__ void gemv_seq_kernel(const uint8_t* __restrict__ w, const float* __restrict__ x, float* __restrict__ out,
                                int n_in, int n_out, int rb) {
    __shared__ __align__(16) uint8_t lut_raw[lut_bytes_of<T>() ? lut_bytes_of<T>() : 16];
    IqLut& lut = *reinterpret_cast<IqLut*>(lut_raw);
    if constexpr (lut_bytes_of<T>() != 0) {
        fill_lut<T>(&lut, threadIdx.x, blockDim.x);
        __syncthreads();
    }
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n_out) return;
    const uint8_t* row = w + (size_t)r * rb;
    float acc = 0.f;
    const int nunits = n_in >> 5;
    // Units are visited so that elements come in ascending row order: for the
    // formats whose unit is not 32 consecutive elements the whole block is
    // decoded into a local buffer first.
    constexpr int BE = block_elems(T);
    if constexpr (BE == 32 || BE == 64) {  // a unit is 32 consecutive elements of the row
        for (int u = 0; u < nunits; ++u) {
            float wv[32];
            decode_unit<T>(row, u, &lut, wv);
            for (int i = 0; i < 32; ++i) acc = __fadd_rn(acc, __fmul_rn(wv[i], x[u * 32 + i]));
        }
    } else {
        for (int b = 0; b < n_in / 256; ++b) {
            float y[256];
            for (int uu = 0; uu < 8; ++uu) {
                float wv[32];
                decode_unit<T>(row, b * 8 + uu, &lut, wv);
                for (int sl = 0; sl < 32; ++sl) {
                    // invert slot_of for this unit
                    int i;
                    if constexpr (T == T_Q4_K || T == T_Q5_K) {
                        const int j = (uu >> 1) & 3, h = uu & 1, nib = sl >> 4, li = sl & 15;
                        i = j * 64 + nib * 32 + h * 16 + li;
                    } else if constexpr (T == T_Q6_K) {
                        const int half = (uu >> 2) & 1, lg = uu & 3, qi = sl >> 3, li = sl & 7;
                        i = half * 128 + qi * 32 + lg * 8 + li;
                    } else {
                        i = uu * 32 + sl;
                    }
                    y[i] = wv[sl];
                }
            }
            for (int i = 0; i < 256; ++i) acc = __fadd_rn(acc, __fmul_rn(y[i], x[b * 256 + i]));
        }
    }
    out[r] = acc;
}

int launch_gemv_seq(dnb_ctx* c, cudaStream_t st, int type, const uint8_t* w, const float* x, float* out, int n_in,
                    int n_out) {
    const int rb = (int)row_bytes(type, n_in);
    if (rb == 0) {
        set_error("gemv_seq: unsupported type %d / n_in %d", type, n_in);
        return DNB_DECLINED;
    }
    int rc = upload_tables(c->device);
    if (rc != DNB_OK) return rc;
    const int thr = 64;
    const int grid = (n_out + thr - 1) / thr;
    switch (type) {
        case T_Q4_K: gemv_seq_kernel<T_Q4_K><<<grid, thr, 0, st>>>(w, x, out, n_in, n_out, rb); break;
        case T_Q5_K: gemv_seq_kernel<T_Q5_K><<<grid, thr, 0, st>>>(w, x, out, n_in, n_out, rb); break;
        case T_Q6_K: gemv_seq_kernel<T_Q6_K><<<grid, thr, 0, st>>>(w, x, out, n_in, n_out, rb); break;
        case T_IQ3_XXS: gemv_seq_kernel<T_IQ3_XXS><<<grid, thr, 0, st>>>(w, x, out, n_in, n_out, rb); break;
        case T_Q8_0: gemv_seq_kernel<T_Q8_0><<<grid, thr, 0, st>>>(w, x, out, n_in, n_out, rb); break;
        case T_Q5_1: gemv_seq_kernel<T_Q5_1><<<grid, thr, 0, st>>>(w, x, out, n_in, n_out, rb); break;
        case T_Q4_0: gemv_seq_kernel<T_Q4_0><<<grid, thr, 0, st>>>(w, x, out, n_in, n_out, rb); break;
        case T_IQ4_NL: gemv_seq_kernel<T_IQ4_NL><<<grid, thr, 0, st>>>(w, x, out, n_in, n_out, rb); break;
        case T_IQ4_XS: gemv_seq_kernel<T_IQ4_XS><<<grid, thr, 0, st>>>(w, x, out, n_in, n_out, rb); break;
        case T_IQ3_S: gemv_seq_kernel<T_IQ3_S><<<grid, thr, 0, st>>>(w, x, out, n_in, n_out, rb); break;
        case T_IQ2_S: gemv_seq_kernel<T_IQ2_S><<<grid, thr, 0, st>>>(w, x, out, n_in, n_out, rb); break;
        case T_Q2_0: gemv_seq_kernel<T_Q2_0><<<grid, thr, 0, st>>>(w, x, out, n_in, n_out, rb); break;
        default: set_error("gemv_seq: no kernel for ggml type %d", type); return DNB_DECLINED;
    }
    c->launches++;
    DNB_CUDA(cudaGetLastError());
    return DNB_OK;
}

}  // namespace dnb
