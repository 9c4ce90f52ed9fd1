// Grouped per-expert GEMM of chunked prefill on the 5th-generation tensor cores.
//
// Reference kernels of this role: kernels_exp_iq_tc.cu:307-527 (wmma bf16, 64x64x32
// tiles, both operands rounded to bf16, "no contract"), kernels_gemm_grouped.cu:
// 134-273 (fp32 FMA), kernels_exp_k_pf.cu:188-258 (m-row fp32).  The reference has
// no tensor-core kernel for Q4_K experts at all.
//
// Design (sm_100a).  One CTA computes, for one expert segment, a tile of 128 weight
// rows x up to 128 token rows over the whole K:
//   D[128 rows][N tokens] (fp32, in TMEM) = W[128][K] * X[N][K]^T
// issued as tcgen05.mma (cta_group::1, kind::f16, M=128, K=16 per instruction) by
// one thread.  W is the A operand and the tokens are the N dimension, so N is only
// as wide as the segment needs (16/32/64/128) and a 3-token expert does not pay
// for a 128-token tile.
//
// Precision.  The path's bar is max|err| <= 1e-3 of the output RMS, which a single
// bf16 rounding of both operands misses by several times.  Each operand is
// therefore split into two bf16 numbers (hi = the value rounded to bf16, lo = the
// exact remainder truncated to bf16), and three MMAs hi*hi + hi*lo + lo*hi
// accumulate into the same TMEM tile; the dropped lo*lo term is about 2^-18
// relative per product.
//
// Operands.
//   A (weights): eight warps dequantise Q4_K bytes straight from global memory,
//      two threads per row and 64 elements per stage, split to hi/lo bf16 and store
//      the two tiles in the K-major 128-byte-swizzled layout the MMA reads.
//   B (activations): a pre-pass gathers the routed token rows into the expert-major
//      packed order and splits them into hi/lo bf16 buffers once per layer; the
//      tiles then arrive by TMA (cp.async.bulk.tensor.2d, 128B swizzle), N rows x 64
//      elements, signalled on the stage's mbarrier.
// Pipeline: `full[s]` (8 producer-warp arrivals + TMA bytes) -> MMA thread ->
// tcgen05.commit -> `empty[s]`; after the last stage a commit on `accum`.
// Epilogue: producer warps 0-3 read their 32 TMEM lanes (= weight rows) with
// tcgen05.ld; gate/up tiles are combined as silu(g)*u and written as hi/lo bf16 in
// packed-row order (the B operand of the down GEMM); down tiles are written as
// fp32 rows for the weighted combine.
//
// Every wait is bounded; a wait that gives up sets *status and the CTA falls
// through to the common teardown (TMEM is always freed).
#include <cuda.h>
#include <cuda_bf16.h>

#include "dnb_common.cuh"
#include "formats.cuh"

namespace dnb {

namespace um {

constexpr int BK = 64;            // K elements per stage (one 128-byte swizzle row of bf16)
constexpr int TILE_M = 128;       // weight rows per CTA
constexpr int A_TILE = TILE_M * BK * 2;   // 16 KB
constexpr int PWARPS = 8;         // producer warps: two threads per weight row (low / high nibble half of a stage)
constexpr int NTHREADS = (PWARPS + 2) * 32;  // warps 0-7 producers (0-3 also epilogue), warp 8 TMA, warp 9 MMA + TMEM

__device__ __forceinline__ uint32_t s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mb_init(uint64_t* b, uint32_t n) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(b)), "r"(n) : "memory");
}
__device__ __forceinline__ void mb_arrive(uint64_t* b) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s32(b)) : "memory");
}
__device__ __forceinline__ void mb_expect_tx(uint64_t* b, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mb_try(uint64_t* b, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(s32(b)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mb_wait(uint64_t* b, uint32_t parity, int* status, int code) {
    for (int i = 0; i < (1 << 21); ++i)
        if (mb_try(b, parity)) return true;
    if (status) atomicExch(status, code);
    return false;
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            s32(dst)),
        "l"(map), "r"(x), "r"(y), "r"(s32(bar))
        : "memory");
}

// K-major, 128-byte swizzle shared memory matrix descriptor (sm_100 format):
// start address >> 4 in bits [0,14), leading byte offset (unused for swizzled
// K-major, set to 1) in [16,30), stride byte offset = 1024 B between 8-row groups in
// [32,46), version 1 in [46,48), layout type 2 (SWIZZLE_128B) in [61,64).
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor, kind::f16: D fp32 (bits 4-5 = 1), A and B bf16 (bits 7-9,
// 10-12 = 1), both K-major (bits 15, 16 = 0), N >> 3 in bits 17-22, M >> 4 in 24-28.
__device__ __forceinline__ uint32_t make_idesc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TILE_M >> 4) << 24);
}

__device__ __forceinline__ void mma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
        : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

struct Maps {            // tensor maps of the B operand: box heights 16, 32, 64, 128 for hi and lo
    CUtensorMap hi[4];
    CUtensorMap lo[4];
};

// Split two fp32 values into bf16 pairs: hi = round-to-nearest bf16, lo = the exact
// remainder a - hi truncated to bf16.  (Rounding hi to nearest halves |lo| compared
// with truncation and so quarters the dropped lo*lo term.)
__device__ __forceinline__ void split2(float a, float b, uint32_t& hi_pair, uint32_t& lo_pair) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);  // .x = a (low half), .y = b
    hi_pair = *reinterpret_cast<const uint32_t*>(&h);
    const float al = a - __uint_as_float(hi_pair << 16), bl = b - __uint_as_float(hi_pair & 0xFFFF0000u);
    lo_pair = __byte_perm(__float_as_uint(al), __float_as_uint(bl), 0x7632);
}

// One stage of one Q4_K row: 64 elements (chunk j of block b) -> hi/lo bf16 rows in
// the swizzled tiles.  hdr = first 16 bytes of the block, q0/q1 = the chunk's 32 qs
// bytes.  Element k of the stage: k < 32 low nibble of byte k, k >= 32 high nibble of
// byte k - 32 (kquant.rs:505-526).
__device__ __forceinline__ void dequant_q4k_stage(const uint4& hdr, const uint4& q0, const uint4& q1, int j, int half,
                                                  uint8_t* tile_hi, uint8_t* tile_lo, int r) {
    const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xFFFF)));
    const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
    // scale bytes 0..11 live in hdr.y, hdr.z, hdr.w
    auto sb = [&](int i) -> uint32_t {
        const uint32_t w = i < 4 ? hdr.y : (i < 8 ? hdr.z : hdr.w);
        return (w >> (8 * (i & 3))) & 0xFFu;
    };
    // this thread's sub-block: 2j (low nibbles, k 0..31) or 2j + 1 (high nibbles, k 32..63)
    const int a = 2 * j + half;
    uint32_t sc, mn;
    if (a < 4) { sc = sb(a) & 63; mn = sb(a + 4) & 63; }
    else { sc = (sb(a + 4) & 0xF) | ((sb(a - 4) >> 6) << 4); mn = (sb(a + 4) >> 4) | ((sb(a) >> 6) << 4); }
    const float d1 = d * (float)sc;
    const float c1 = fmaf(128.0f, d1, dmin * (float)mn);
    const uint32_t rowoff = (uint32_t)(r >> 3) * 1024u + (uint32_t)(r & 7) * 128u;
    const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
    const int sh = half * 4;
#pragma unroll
    for (int g = 0; g < 4; ++g) {  // 8 elements k = 32*half + 8g .. +7 from bytes 8g..8g+7
        uint32_t hv[4], lv[4];
#pragma unroll
        for (int w2 = 0; w2 < 2; ++w2) {
            const uint32_t nib = (qw[2 * g + w2] >> sh) & 0x0F0F0F0Fu;
            // w = d1 * q - m1 evaluated as d1 * (128 + q) - (128 d1 + m1): one fma on an exact float
            const float a0 = fmaf(d1, magic128<0>(nib), -c1), a1 = fmaf(d1, magic128<1>(nib), -c1);
            const float a2 = fmaf(d1, magic128<2>(nib), -c1), a3 = fmaf(d1, magic128<3>(nib), -c1);
            split2(a0, a1, hv[2 * w2], lv[2 * w2]);
            split2(a2, a3, hv[2 * w2 + 1], lv[2 * w2 + 1]);
        }
        const uint32_t col = ((uint32_t)((4 * half + g) ^ (r & 7))) << 4;
        *reinterpret_cast<uint4*>(tile_hi + rowoff + col) = make_uint4(hv[0], hv[1], hv[2], hv[3]);
        *reinterpret_cast<uint4*>(tile_lo + rowoff + col) = make_uint4(lv[0], lv[1], lv[2], lv[3]);
    }
}

// NMAT = 2: gate and up tiles together, SwiGLU epilogue to out_hi / out_lo (bf16 packed rows).
// NMAT = 1: one matrix, fp32 epilogue to out_f32.
// grid = (n_out / 128, segments, token tiles of 128)
template <int NMAT>
__global__ void __launch_bounds__(NTHREADS, 1)
grouped_q4k_umma_kernel(const SegDesc* __restrict__ seg, const int32_t* __restrict__ nseg_dev, int n_in, int n_out,
                        int rb, const __grid_constant__ Maps maps, uint16_t* __restrict__ out_hi,
                        uint16_t* __restrict__ out_lo, float* __restrict__ out_f32, int* status) {
    constexpr int STAGES = (NMAT == 2) ? 2 : 3;
    constexpr int A_BYTES = NMAT * 2 * A_TILE;          // hi + lo per matrix
    constexpr int B_BYTES_MAX = 2 * 128 * BK * 2;       // hi + lo, N = 128
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES_MAX;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* accum = empty + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);

    const int s = blockIdx.y;
    if (s >= *nseg_dev) return;
    const SegDesc sd = seg[s];
    const int t0 = blockIdx.z * 128;
    if ((uint32_t)t0 >= sd.m) return;
    const int m_tile = min(128, (int)sd.m - t0);
    const int nsel = m_tile <= 16 ? 0 : (m_tile <= 32 ? 1 : (m_tile <= 64 ? 2 : 3));
    const int N = 16 << nsel;
    const int r0 = blockIdx.x * TILE_M;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nchunks = n_in / BK;
    constexpr int TM_COLS = (NMAT == 2) ? 256 : 128;

    if (tid == 0) {
        for (int i = 0; i < STAGES; ++i) {
            mb_init(&full[i], PWARPS + 1);  // producer warps + the TMA thread's expect_tx arrival
            mb_init(&empty[i], 1);   // one tcgen05.commit
        }
        mb_init(accum, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == PWARPS + 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(tmem_slot)), "r"(TM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;

    if (warp < PWARPS) {
        // ---------------- producers: two threads per weight row ----------------
        const int r = tid & 127, half = tid >> 7;
        const uint8_t* rowa = sd.wa + (size_t)(r0 + r) * rb;
        const uint8_t* rowb = (NMAT == 2) ? sd.wb + (size_t)(r0 + r) * rb : nullptr;
        // Raw bytes of a stage: header + this stage's 32 qs bytes, per matrix.  Four
        // register buffers keep the loads of three stages ahead in flight (the rows
        // are 1152 or 288 bytes apart, so these are latency-bound 32-byte reads).
        struct Raw { uint4 ha, a0, a1, hb, b0, b1; };
        Raw buf[4];
        auto fetch = [&](Raw& q, int c) {
            const int b = c >> 2, j = c & 3;
            const uint8_t* pa = rowa + b * 144;
            q.ha = __ldg(reinterpret_cast<const uint4*>(pa));
            q.a0 = __ldcs(reinterpret_cast<const uint4*>(pa + 16 + 32 * j));
            q.a1 = __ldcs(reinterpret_cast<const uint4*>(pa + 32 + 32 * j));
            if constexpr (NMAT == 2) {
                const uint8_t* pb = rowb + b * 144;
                q.hb = __ldg(reinterpret_cast<const uint4*>(pb));
                q.b0 = __ldcs(reinterpret_cast<const uint4*>(pb + 16 + 32 * j));
                q.b1 = __ldcs(reinterpret_cast<const uint4*>(pb + 32 + 32 * j));
            }
        };
        fetch(buf[0], 0);
        fetch(buf[1], 1);
        fetch(buf[2], 2);
        for (int c4 = 0; c4 < nchunks && ok; c4 += 4) {  // nchunks is a multiple of 4 (n_in % 256 == 0)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int c = c4 + i;
                if (c + 3 < nchunks) fetch(buf[(i + 3) & 3], c + 3);
                const int st = c % STAGES;
                const uint32_t ph = (uint32_t)(c / STAGES) & 1u;
                if (ok && c >= STAGES) ok = mb_wait(&empty[st], ph ^ 1u, status, 2);
                if (ok) {
                    uint8_t* sa = smem + st * STAGE_BYTES;
                    dequant_q4k_stage(buf[i].ha, buf[i].a0, buf[i].a1, c & 3, half, sa, sa + A_TILE, r);
                    if constexpr (NMAT == 2)
                        dequant_q4k_stage(buf[i].hb, buf[i].b0, buf[i].b1, c & 3, half, sa + 2 * A_TILE, sa + 3 * A_TILE, r);
                    fence_async_smem();   // generic-proxy stores -> visible to the tensor core's async proxy
                    __syncwarp();
                    if (lane == 0) mb_arrive(&full[st]);
                }
            }
        }
        // ---------------- epilogue: TMEM lane = weight row ----------------
        if (ok && warp < 4) ok = mb_wait(accum, 0, status, 3);
        tc_fence_after();
        if (ok && warp < 4) {
            const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
            const size_t prow0 = (size_t)sd.row0 + t0;
            for (int c0 = 0; c0 < N; c0 += 16) {
                uint32_t g[16], u[16];
                tmem_ld16(tmem_base + lane_base + (uint32_t)c0, g);
                if constexpr (NMAT == 2) tmem_ld16(tmem_base + lane_base + (uint32_t)(128 + c0), u);
                tmem_ld_wait();
#pragma unroll
                for (int j2 = 0; j2 < 16; ++j2) {
                    const int t = c0 + j2;
                    if (t < m_tile) {
                        if constexpr (NMAT == 2) {
                            const float gv = __uint_as_float(g[j2]), uv = __uint_as_float(u[j2]);
                            const float a = gv / (1.0f + expf(-gv)) * uv;
                            const uint16_t ah = __bfloat16_as_ushort(__float2bfloat16_rn(a));
                            const float al = a - __uint_as_float((uint32_t)ah << 16);
                            const size_t o = (prow0 + t) * (size_t)n_out + r0 + r;
                            out_hi[o] = ah;
                            out_lo[o] = (uint16_t)(__float_as_uint(al) >> 16);
                        } else {
                            out_f32[(prow0 + t) * (size_t)n_out + r0 + r] = __uint_as_float(g[j2]);
                        }
                    }
                }
            }
        }
        tc_fence_before();
    } else if (warp == PWARPS) {
        // ---------------- TMA: activation tiles ----------------
        if (lane == 0) {
            const CUtensorMap* mh = &maps.hi[nsel];
            const CUtensorMap* ml = &maps.lo[nsel];
            const int yrow = (int)sd.row0 + t0;
            const uint32_t bbytes = (uint32_t)(2 * N * BK * 2);
            for (int c = 0; c < nchunks; ++c) {
                const int st = c % STAGES;
                const uint32_t ph = (uint32_t)(c / STAGES) & 1u;
                if (c >= STAGES && !mb_wait(&empty[st], ph ^ 1u, status, 4)) break;
                uint8_t* sbp = smem + st * STAGE_BYTES + A_BYTES;
                mb_expect_tx(&full[st], bbytes);
                tma_load_2d(sbp, mh, c * BK, yrow, &full[st]);
                tma_load_2d(sbp + N * BK * 2, ml, c * BK, yrow, &full[st]);
            }
        }
    } else {
        // ---------------- MMA issue ----------------
        if (lane == 0) {
            const uint32_t idesc = make_idesc(N);
            for (int c = 0; c < nchunks; ++c) {
                const int st = c % STAGES;
                const uint32_t ph = (uint32_t)(c / STAGES) & 1u;
                if (!mb_wait(&full[st], ph, status, 5)) break;
                tc_fence_after();
                const uint32_t sa = s32(smem + st * STAGE_BYTES);
                const uint32_t sbh = sa + A_BYTES, sbl = sbh + N * BK * 2;
#pragma unroll
                for (int ks = 0; ks < BK / 16; ++ks) {
                    const uint32_t koff = ks * 32;  // 16 bf16 = 32 bytes inside the swizzle row
                    const uint64_t bh = make_desc(sbh + koff), bl = make_desc(sbl + koff);
#pragma unroll
                    for (int mt = 0; mt < NMAT; ++mt) {
                        const uint64_t ah = make_desc(sa + mt * 2 * A_TILE + koff);
                        const uint64_t al = make_desc(sa + mt * 2 * A_TILE + A_TILE + koff);
                        const uint32_t d = tmem_base + (uint32_t)(mt * 128);
                        mma_bf16(d, ah, bh, idesc, (c > 0 || ks > 0) ? 1u : 0u);
                        mma_bf16(d, ah, bl, idesc, 1u);
                        mma_bf16(d, al, bh, idesc, 1u);
                    }
                }
                mma_commit(&empty[st]);   // frees the stage once these MMAs have read it
            }
            mma_commit(accum);            // all MMAs done -> accumulators readable
        }
        __syncwarp();
    }
    __syncthreads();
    if (warp == PWARPS + 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TM_COLS) : "memory");
    }
}

// Gather the routed token rows into packed order and split to hi/lo bf16.
// row_token == null: identity (row p reads x row p).
__global__ void __launch_bounds__(256)
gather_split_kernel(const float* __restrict__ x, int ldx, const int32_t* __restrict__ row_token, int rows, int e,
                    uint16_t* __restrict__ hi, uint16_t* __restrict__ lo) {
    const int p = blockIdx.x;
    if (p >= rows) return;
    const float* xr = x + (size_t)(row_token ? row_token[p] : p) * ldx;
    for (int i = threadIdx.x * 2; i < e; i += 512) {
        const float2 v = *reinterpret_cast<const float2*>(xr + i);
        uint32_t hp, lp;
        split2(v.x, v.y, hp, lp);
        *reinterpret_cast<uint32_t*>(hi + (size_t)p * e + i) = hp;
        *reinterpret_cast<uint32_t*>(lo + (size_t)p * e + i) = lp;
    }
}

}  // namespace um

// ---- host side ---------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// [rows][cols] bf16 row-major, box = 64 columns x box_rows rows, 128-byte swizzle.
static int make_map(CUtensorMap* m, void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        set_error("cuTensorMapEncodeTiled is not available from this driver");
        return DNB_ERR_CUDA;
    }
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {64, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed (%d) for %llu x %llu box %u", (int)r, (unsigned long long)rows,
                  (unsigned long long)cols, box_rows);
        return DNB_ERR_CUDA;
    }
    return DNB_OK;
}

int umma_make_maps(void* hi, void* lo, uint64_t rows, uint64_t cols, UmmaMaps* out) {
    static_assert(sizeof(UmmaMaps) == sizeof(um::Maps), "UmmaMaps must mirror um::Maps");
    um::Maps* m = reinterpret_cast<um::Maps*>(out);
    for (int i = 0; i < 4; ++i) {
        int rc = make_map(&m->hi[i], hi, rows, cols, 16u << i);
        if (rc) return rc;
        if ((rc = make_map(&m->lo[i], lo, rows, cols, 16u << i))) return rc;
    }
    return DNB_OK;
}

int launch_gather_split(dnb_ctx* c, cudaStream_t st, const float* x, int ldx, const int32_t* row_token, int rows, int e,
                        uint16_t* hi, uint16_t* lo) {
    ProfScope prof_(c, st, "gather_split_bf16");
    um::gather_split_kernel<<<rows, 256, 0, st>>>(x, ldx, row_token, rows, e, hi, lo);
    c->launches++;
    DNB_CUDA(cudaGetLastError());
    return DNB_OK;
}

// Grouped Q4_K GEMM on tcgen05.  fused: seg[].wa/wb are gate/up, output silu(g)*u as
// hi/lo bf16 packed rows; otherwise seg[].wa, fp32 output rows.
int launch_grouped_umma(dnb_ctx* c, cudaStream_t st, bool fused, const SegDesc* seg, const int32_t* nseg_dev,
                        int nseg_max, int n_in, int n_out, const UmmaMaps* maps, int nt_max, uint16_t* out_hi,
                        uint16_t* out_lo, float* out_f32) {
    if (n_in % 256 || n_out % um::TILE_M) return DNB_DECLINED;
    const int rb = n_in / 256 * 144;
    const um::Maps& M = *reinterpret_cast<const um::Maps*>(maps);
    const dim3 grid(n_out / um::TILE_M, nseg_max, (nt_max + 127) / 128);
    if (fused) {
        const size_t smem = 2 * (2 * 2 * um::A_TILE + 2 * 128 * um::BK * 2) + 256 + 1024;
        static bool set = false;
        if (!set) {
            DNB_CUDA(cudaFuncSetAttribute(um::grouped_q4k_umma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            set = true;
        }
        ProfScope prof_(c, st, "umma_gate_up");
        um::grouped_q4k_umma_kernel<2><<<grid, um::NTHREADS, smem, st>>>(seg, nseg_dev, n_in, n_out, rb, M, out_hi, out_lo,
                                                                        nullptr, c->status);
    } else {
        const size_t smem = 3 * (2 * um::A_TILE + 2 * 128 * um::BK * 2) + 256 + 1024;
        static bool set = false;
        if (!set) {
            DNB_CUDA(cudaFuncSetAttribute(um::grouped_q4k_umma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            set = true;
        }
        ProfScope prof_(c, st, "umma_down");
        um::grouped_q4k_umma_kernel<1><<<grid, um::NTHREADS, smem, st>>>(seg, nseg_dev, n_in, n_out, rb, M, nullptr, nullptr,
                                                                        out_f32, c->status);
    }
    c->launches++;
    DNB_CUDA(cudaGetLastError());
    return DNB_OK;
}

}  // namespace dnb
