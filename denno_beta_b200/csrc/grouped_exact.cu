// Grouped per-expert GEMM for IQ3_XXS experts on the 5th-generation tensor cores, with the weights
// kept EXACT in bf16 and the block scales applied after the tensor-core sum.
//
// Reference kernels of this role: kernels_exp_iq_tc.cu:307-527 (dno_exp_tc_gu_iq3xxs: wmma bf16 64x64x32,
// weights dequantised to fp32 then rounded to bf16, activations rounded to bf16) and :529-607 (down).
//
// Idea.  An IQ3_XXS weight is  db * g * s  with g one of eight small integers (codebook magnitudes
// <= 62), s = +-1 and db = d * (0.5 + scale) * 0.5 shared by the 32 elements of a sub-block
// (kquant.rs:659-680).  g * s is exact in bf16, so the A operand needs no hi/lo split and no floating
// point arithmetic in its producer: two codebook lookups and four sign masks make eight elements.
// The tensor core sums one sub-block (K = 32) at a time into its own TMEM columns,
//     D_g[row][token] = sum_{k in g} (g*s)[row][k] * x[token][k]        (x as bf16 hi + lo: 2 products),
// and the epilogue warps, which own one weight row per thread, read D_g back and do the fp32
//     acc[row][token] += db[row][g] * D_g[row][token].
// Per sub-block that is 32 FMAs per thread for a 32-token tile - far less than dequantising the
// 128 x 32 weights to fp32 and splitting them, which is what bounds the Q4_K kernel of
// grouped_umma.cu on the small tiles a Zipf router and the decode batches produce.  The products
// are exact (8-bit x 8-bit significands into fp32) and each activation carries 16 significant bits,
// so the result is closer to the sequential fp32 result than the three-product scheme.
//
// Work item: (expert segment, 32-token tile, 128-row tile) over the whole K; the kernel is persistent
// (one CTA per SM walks items i, i + gridDim.x, ...; every item costs the same).
// Roles (832 threads; 16 producer warps because the decode is a chain of dependent shared-memory lookups
// and the epilogue warps mostly wait - measured: with 8 producer warps each scheduler issued 0.4 per cycle):
//   warps 0-15   producers: raw rows arrive by cp.async (16-byte lines that cover the 98-byte blocks, one
//                256-element block ahead, double buffered; the next item's tile is asked into L2 first);
//                decode into the K-major 128-byte swizzled A tiles of a stage (64 K = two sub-blocks);
//                write the sub-block scales
//   warps 16-23  epilogue: TMEM lane quadrant = warp % 4; warps 16-19 own token columns 0-15 of the tile,
//                20-23 columns 16-31, of every matrix: silu(g) * u needs no exchange between warps
//   warp 24      TMA: the stage's activation tiles (hi and lo, 32 rows x 64 K, 128-byte swizzle)
//   warp 25      MMA issue (one elected thread); owns the TMEM allocation
// Barriers: full[s] / empty[s] per stage; tfull[b] / tfree[b] per TMEM buffer (one per stage in flight, both
// of its sub-blocks: one hand-over per stage costs half the waits of one per sub-block, and with everything
// but the barriers left out the kernel still took 40-65 % of its time); sfull[i] per slot of the scale ring (producers -> epilogue).  The down kernel
// has eight TMEM buffers = a whole K = 512 item, so the MMAs of the next item run during an item's stores.
// Every wait is bounded; one that gives up sets *status and the role leaves its loop (the producers
// keep meeting at their named barrier so that none of them is left behind); TMEM is always freed.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "dnb_common.cuh"
#include "dnb_iq_tables.h"
#include "tc_ptx.cuh"

namespace dnb {
namespace ex {
using namespace tcp;

constexpr int BK = 64;                    // K per stage: one 128-byte swizzle row of bf16 = two sub-blocks
constexpr int TILE_M = 128;               // weight rows per item
constexpr int NT = 32;                    // tokens per item
constexpr int A_TILE = TILE_M * BK * 2;   // 16 KB
constexpr int B_TILE = NT * BK * 2;       // 4 KB (hi or lo)
constexpr int STAGE_BYTES = 2 * A_TILE + 2 * B_TILE;
constexpr int STAGES = 3;
constexpr int RAWS = 2;                   // raw slots: one block in flight while one is decoded
constexpr int NB = 8;                     // TMEM buffers at most (one per stage in flight: 2 sub-blocks x NMAT x NT columns);
                                          // the gate/up kernel has 4 (512 columns), the down kernel 8: a whole K = 512 item
constexpr int SCL = 12;                   // slots of the scale ring, one per stage: [2 sub-blocks][NMAT][128]
static_assert(RAWS == 2 && STAGES + NB <= SCL, "a producer must not lap the epilogue on the scale ring");
constexpr int RAW_PITCH = 112;            // seven 16-byte lines cover a 98-byte block at any even offset
constexpr int LUT_REP = 8;
constexpr int PWARPS = 16, EWARPS = 8;
constexpr int W_TMA = PWARPS + EWARPS, W_MMA = W_TMA + 1;
constexpr int NTHREADS = (W_MMA + 1) * 32;
constexpr int kMaxSeg = 1055;
constexpr int kLocalItems = 32;

__constant__ uint32_t c_grid[256];

__device__ __forceinline__ void bar_producers() { asm volatile("bar.sync 1, %0;" ::"n"(PWARPS * 32) : "memory"); }

// Instruction descriptor, kind::f16: D fp32, A and B bf16, both K-major, N >> 3 in bits 17-22, M >> 4 in 24-28.
// (One N = 64 product against the hi and lo rows as one B operand reads the weight tile once but doubles the columns the
// epilogue has to read and add; the kernel is bound by issued instructions, not by shared memory, and it measured the same.)
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NT >> 3) << 17) | ((uint32_t)(TILE_M >> 4) << 24);

__device__ __forceinline__ void mma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t acc) {
    tcp::mma_bf16(d_tmem, adesc, bdesc, kIdesc, acc);
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* r) {
    uint32_t v[16];
    tcp::tmem_ld16(taddr, v);
#pragma unroll
    for (int i = 0; i < 16; ++i) r[i] = __uint_as_float(v[i]);
}
__device__ __forceinline__ uint32_t lds_u16(const uint8_t* p) { return *reinterpret_cast<const uint16_t*>(p); }

struct Maps {  // tensor maps of the B operand: box heights 16, 32, 64, 128 for hi and lo (this kernel uses 32)
    CUtensorMap hi[4];
    CUtensorMap lo[4];
};

struct Item {
    const uint8_t* wa;
    const uint8_t* wb;
    int prow;    // first packed row of the token tile
    int m_tile;  // tokens in the tile (1..NT)
    int r0;      // first weight row
};
__device__ __forceinline__ Item decode_item(int item, int row_tiles, int rows_per_item, int nseg, const int* tile_prefix,
                                            const SegDesc* __restrict__ seg) {
    const int tile = item / row_tiles, rt = item - tile * row_tiles;
    int lo = 0, hi = nseg - 1;
    while (lo < hi) {  // last segment whose first tile is <= tile
        const int mid = (lo + hi + 1) >> 1;
        if (tile_prefix[mid] <= tile) lo = mid; else hi = mid - 1;
    }
    const SegDesc sd = seg[lo];
    const int t0 = (tile - tile_prefix[lo]) * NT;
    Item it;
    it.wa = sd.wa;
    it.wb = sd.wb;
    it.prow = (int)sd.row0 + t0;
    it.m_tile = min(NT, (int)sd.m - t0);
    it.r0 = rt * rows_per_item;
    return it;
}
struct ItemTab {
    const Item* tab;
    const SegDesc* seg;
    const int* tile_prefix;
    int nseg, row_tiles, rows_per_item;
    __device__ __forceinline__ Item get(int k) const {
        if (k < kLocalItems) return tab[k];
        return decode_item((int)blockIdx.x + k * (int)gridDim.x, row_tiles, rows_per_item, nseg, tile_prefix, seg);
    }
};

__device__ __forceinline__ float swiglu_fast(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }

// NMAT = 2: gate and up together, silu(g) * u written as bf16 hi/lo packed rows (the B operand of
// the down GEMM).  NMAT = 1: one matrix, fp32 rows (or peer rows through row_dst).  PAIR (with NMAT = 2):
// the two A tiles of an item are rows r0.. and r0 + 128.. of ONE matrix against the same activation tile, fp32
// rows out: half the stages, hand-overs and activation loads of the NMAT = 1 form.
template <int NMAT, bool PAIR = false>
__global__ void __launch_bounds__(NTHREADS, 1)
grouped_iq3_exact_kernel(const SegDesc* __restrict__ seg, const int32_t* __restrict__ nseg_dev, int n_in, int n_out, int rb,
                         const __grid_constant__ Maps maps, uint16_t* __restrict__ out_hi, uint16_t* __restrict__ out_lo,
                         float* __restrict__ out_f32, int* status, float* const* __restrict__ row_dst) {
    constexpr int TM_COLS = 512;                   // NBUF buffers of 2 * NMAT * NT columns
    constexpr int NBUF = NMAT == 2 ? 4 : 8;
    constexpr int RAW_SLOT = NMAT * TILE_M * RAW_PITCH;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* raw = smem + STAGES * STAGE_BYTES;                        // [2][NMAT][128][RAW_PITCH]
    float* scl = reinterpret_cast<float*>(raw + RAWS * RAW_SLOT);         // [SCL][NMAT][128]
    uint2* lut = reinterpret_cast<uint2*>(scl + SCL * 2 * NMAT * TILE_M);  // [256][LUT_REP]
    uint64_t* full = reinterpret_cast<uint64_t*>(lut + 256 * LUT_REP);
    uint64_t* empty = full + STAGES;
    uint64_t* tfull = empty + STAGES;
    uint64_t* tfree = tfull + NB;
    uint64_t* sfull = tfree + NB;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sfull + SCL);
    int* tile_prefix = reinterpret_cast<int*>(tmem_slot + 4);          // [nseg + 1]
    Item* itab = reinterpret_cast<Item*>(tile_prefix + kMaxSeg + 1);   // [kLocalItems]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nchunks = n_in / BK;
    const int nblocks = n_in / 256;
    constexpr int ROWS_ITEM = PAIR ? 2 * TILE_M : TILE_M;
    const int row_tiles = n_out / ROWS_ITEM;
    const int nseg = min(*nseg_dev, kMaxSeg);

    if (tid == 0) {
        for (int i = 0; i < STAGES; ++i) {
            mb_init(&full[i], PWARPS + 1);  // the producer warps + the TMA thread's expect_tx arrival
            mb_init(&empty[i], 1);          // one tcgen05.commit
        }
        for (int i = 0; i < NB; ++i) {
            mb_init(&tfull[i], 1);
            mb_init(&tfree[i], EWARPS);     // every epilogue warp reads its part of the buffer
        }
        for (int i = 0; i < SCL; ++i) mb_init(&sfull[i], PWARPS);  // every producer warp writes 8 rows of the stage's scales
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = tid; i < 256 * LUT_REP; i += NTHREADS) {  // codebook magnitudes as bf16 pairs (<= 62: exact)
        const uint32_t w = c_grid[i / LUT_REP];
        const uint32_t h0 = __float_as_uint((float)(w & 0xFFu)) >> 16, h1 = __float_as_uint((float)((w >> 8) & 0xFFu)) >> 16;
        const uint32_t h2 = __float_as_uint((float)((w >> 16) & 0xFFu)) >> 16, h3 = __float_as_uint((float)(w >> 24)) >> 16;
        lut[i] = make_uint2(h0 | (h1 << 16), h2 | (h3 << 16));
    }
    for (int i = tid; i < nseg; i += NTHREADS) tile_prefix[i + 1] = ((int)seg[i].m + NT - 1) / NT;
    __syncthreads();
    if (warp == 0) {
        int carry = 0;
        for (int base = 0; base < nseg; base += 32) {
            const int i = base + lane;
            int v = i < nseg ? tile_prefix[i + 1] : 0;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int o = __shfl_up_sync(0xffffffffu, v, d);
                if (lane >= d) v += o;
            }
            if (i < nseg) tile_prefix[i + 1] = carry + v;
            carry += __shfl_sync(0xffffffffu, v, 31);
        }
        if (lane == 0) tile_prefix[0] = 0;
    }
    if (warp == W_MMA) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(tmem_slot)), "r"(TM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int n_items = nseg > 0 ? tile_prefix[nseg] * row_tiles : 0;
    const int GR = gridDim.x;
    const int my_items = (int)blockIdx.x < n_items ? (n_items - (int)blockIdx.x + GR - 1) / GR : 0;
    if (tid < min(my_items, kLocalItems)) itab[tid] = decode_item((int)blockIdx.x + tid * GR, row_tiles, ROWS_ITEM, nseg, tile_prefix, seg);
    __syncthreads();
    const ItemTab items{itab, seg, tile_prefix, nseg, row_tiles, ROWS_ITEM};
    bool ok = true;

    if (warp < PWARPS) {
        // ---------------- producers ----------------
        // Decode: a warp owns 8 rows; its lanes are 8 rows x the 4 eight-element units of a sub-block, so the
        // lanes of a raw-byte load fall in distinct banks (row pitch 28 words) and the unit's 16-byte store
        // is one column of the swizzled row.
        const int l = lane >> 3, l7 = 7 * l;
        const int row0 = warp * 8 + (lane & 7);
        const uint2* lutl = lut + (lane & (LUT_REP - 1));
        const uint32_t colb = ((uint32_t)(l ^ (lane & 7))) << 4;   // column of the unit for sub-block half 0; half 1 flips bit 6
        const uint32_t sa_off = (uint32_t)(row0 >> 3) * 1024u + (uint32_t)(row0 & 7) * 128u;
        const int total_blocks = my_items * nblocks;
        // Part q (0..3) of the fetch of block kb.  Eight consecutive lanes copy the seven 16-byte lines that cover one
        // row's 98-byte block (cp.async; 112-byte bulk copies measured slower, a second block in flight or a lane per
        // row no different), one part per stage of the block before.
        // The tile of the NEXT item (128 rows x row bytes, contiguous in the expert-major layout) is asked into L2 in
        // sixteen large pieces while the current item is decoded, so that HBM sees long requests.
        const int f_line = tid & 7, f_rb = tid >> 3;   // f_rb = 0..63
        auto fetch = [&](int kb, int q) {
            const int rbi = q * 64 + f_rb;             // (matrix, row) of this lane's line
            if (kb < total_blocks && rbi < NMAT * TILE_M && f_line < 7) {
                const int k = kb / nblocks, b = kb - k * nblocks;
                const Item it = items.get(k);
                const int mat = rbi >> 7, frow = rbi & 127;
                const uint8_t* src = (mat && !PAIR) ? it.wb : it.wa;
                const size_t off = ((size_t)(it.r0 + (PAIR ? mat * TILE_M : 0) + frow) * rb + (size_t)98 * b) & ~(size_t)15;
                uint8_t* dst = raw + (kb & 1) * RAW_SLOT + (mat * TILE_M + frow) * RAW_PITCH;
                cp_async16(dst + 16 * f_line, src + off + 16 * f_line);
            }
            if (q == 3) cp_async_commit();
        };
        auto l2_prefetch_item = [&](int k) {
            if (tid < 16 * NMAT && k < my_items) {
                const Item it = items.get(k);
                const uint32_t piece = (uint32_t)(8 * rb);  // a sixteenth of the tile; a multiple of 16 bytes
                const uint8_t* base = PAIR ? it.wa + (size_t)it.r0 * rb + (size_t)tid * piece   // 256 contiguous rows
                                           : ((tid >> 4) ? it.wb : it.wa) + (size_t)it.r0 * rb + (size_t)(tid & 15) * piece;
                asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(base), "r"(piece) : "memory");
            }
        };
        l2_prefetch_item(0);
        for (int q = 0; q < 4; ++q) fetch(0, q);
        int st = 0, slot0 = 0, g = 0;   // stage, first scale slot and running chunk index of the next stage
        uint32_t ph = 0;
        int kblk = 0;                   // block inside the item
        for (int kb = 0; kb < total_blocks; ++kb) {
            cp_async_wait_all();
            bar_producers();  // everybody's lines of block kb have landed; everybody is done with block kb - 1
            if (kblk == 0) l2_prefetch_item(kb / nblocks + 1);
            const uint8_t* rw[NMAT];
            float d[NMAT];
            {
                const int sh = (int)(((size_t)row0 * rb + (size_t)98 * kblk) & 15);
#pragma unroll
                for (int mt = 0; mt < NMAT; ++mt) {
                    rw[mt] = raw + (kb & 1) * RAW_SLOT + (mt * TILE_M + row0) * RAW_PITCH + sh;
                    d[mt] = __half2float(__ushort_as_half((unsigned short)lds_u16(rw[mt])));
                }
            }
            if (++kblk == nblocks) kblk = 0;
#pragma unroll 1
            for (int j = 0; j < 4; ++j) {
                if (ok && g >= STAGES) ok = mb_wait(&empty[st], ph ^ 1u, status, 2);
                if (ok) {
                    uint8_t* sa = smem + st * STAGE_BYTES + sa_off;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int gp = 2 * j + h;  // sub-block inside the 256-element block
#pragma unroll
                        for (int mt = 0; mt < NMAT; ++mt) {
                            const uint8_t* r = rw[mt];
                            const uint32_t aux = lds_u16(r + 66 + 4 * gp) | (lds_u16(r + 68 + 4 * gp) << 16);
                            if (l == 0) scl[((slot0 * 2 + h) * NMAT + mt) * TILE_M + row0] = d[mt] * (0.5f + (float)(aux >> 28)) * 0.5f;
                            const uint32_t idx = lds_u16(r + 2 + 8 * gp + 2 * l);
                            const uint32_t code = (aux >> l7) & 127u;
                            const uint32_t sg = code | ((__popc(code) & 1u) << 7);  // bit 7 makes the number of minus signs even
                            const uint2 g1 = lutl[(idx & 0xFFu) * LUT_REP];
                            const uint2 g2 = lutl[(idx >> 8) * LUT_REP];
                            uint4 v;
                            v.x = g1.x ^ ((sg * 0x40008000u) & 0x80008000u);
                            v.y = g1.y ^ ((sg * 0x10002000u) & 0x80008000u);
                            v.z = g2.x ^ ((sg * 0x04000800u) & 0x80008000u);
                            v.w = g2.y ^ ((sg * 0x01000200u) & 0x80008000u);
                            *reinterpret_cast<uint4*>(sa + mt * A_TILE + (colb ^ (uint32_t)(h << 6))) = v;
                        }
                    }
                    fence_async_smem();  // generic-proxy stores -> visible to the tensor core's async proxy
                    __syncwarp();
                    if (lane == 0) {
                        mb_arrive(&full[st]);
                        mb_arrive(&sfull[slot0]);
                    }
                }
                fetch(kb + 1, j);
                ++g;
                if (++st == STAGES) { st = 0; ph ^= 1u; }
                if (++slot0 == SCL) slot0 = 0;
            }
        }
        cp_async_wait_all();
    } else if (warp == W_TMA) {
        // ---------------- TMA: activation tiles ----------------
        int g = 0;
        for (int k = 0; k < my_items && ok; ++k) {
            const Item it = items.get(k);
            for (int c = 0; c < nchunks; ++c, ++g) {
                const int st = g % STAGES;
                const uint32_t ph = (uint32_t)(g / STAGES) & 1u;
                if (g >= STAGES) ok = warp_all(mb_wait(&empty[st], ph ^ 1u, status, 4));
                if (!ok) break;
                uint8_t* sbp = smem + st * STAGE_BYTES + 2 * A_TILE;
                if (elect_one()) {
                    mb_expect_tx(&full[st], 2u * B_TILE);
                    tma_load_2d(sbp, &maps.hi[1], c * BK, it.prow, &full[st]);
                    tma_load_2d(sbp + B_TILE, &maps.lo[1], c * BK, it.prow, &full[st]);
                }
                __syncwarp();
            }
        }
    } else if (warp == W_MMA) {
        // ---------------- MMA issue ----------------
        const uint32_t smem_lo = desc_lo(s32(smem));
        const int total = my_items * nchunks;
        for (int g = 0; g < total && ok; ++g) {
            const int st = g % STAGES;
            const uint32_t ph = (uint32_t)(g / STAGES) & 1u;
            ok = warp_all(mb_wait(&full[st], ph, status, 5));
            if (!ok) break;
            const uint32_t a_lo = smem_lo + (uint32_t)(st * (STAGE_BYTES >> 4));
            const uint32_t bh_lo = a_lo + (uint32_t)((2 * A_TILE) >> 4), bl_lo = bh_lo + (uint32_t)(B_TILE >> 4);
            const int b = g % NBUF;  // one TMEM buffer, one commit and one hand-over to the epilogue per stage
            if (g >= NBUF) ok = warp_all(mb_wait(&tfree[b], (uint32_t)(g / NBUF - 1) & 1u, status, 6));
            if (!ok) break;
            tc_fence_after();
            if (elect_one()) {
#pragma unroll
                for (int grp = 0; grp < 2; ++grp) {
#pragma unroll
                    for (int mt = 0; mt < NMAT; ++mt) {
                        const uint32_t dcol = tmem_base + (uint32_t)(((b * 2 + grp) * NMAT + mt) * NT);
                        const uint32_t am = a_lo + (uint32_t)(mt * (A_TILE >> 4));
#pragma unroll
                        for (int ks = 0; ks < 2; ++ks) {
                            const uint32_t koff = (uint32_t)(2 * grp + ks) * 2u;  // 16 bf16 = 32 bytes, >> 4
                            const uint64_t a = desc_of(am + koff);
                            mma_bf16(dcol, a, desc_of(bh_lo + koff), ks);  // the first product of a sub-block overwrites
                            mma_bf16(dcol, a, desc_of(bl_lo + koff), 1u);
                        }
                    }
                }
                mma_commit(&tfull[b]);
                mma_commit(&empty[st]);  // the stage is free once everything issued so far has read it
            }
            __syncwarp();
        }
    } else {
        // ---------------- epilogue: TMEM lane = weight row ----------------
        // A warp owns 32 weight rows (its TMEM lane quadrant) x 16 token columns (hsel) of every matrix: the gate and
        // the up value of a (row, token) meet in one thread, and nothing is exchanged between warps.
        const int quad = warp & 3, hsel = (warp - PWARPS) >> 2;
        const int r = quad * 32 + lane;
        const uint32_t tlane = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(16 * hsel);
        // running stage counter of this warp's reads: TMEM buffer, scale slot and their phase parities
        int b = 0, slot = 0;
        uint32_t pb = 0, ps = 0;
        for (int k = 0; k < my_items && ok; ++k) {
            const Item it = items.get(k);
            float acc[NMAT][16];
#pragma unroll
            for (int mt = 0; mt < NMAT; ++mt)
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[mt][j] = 0.f;
            for (int c = 0; c < nchunks; ++c) {
                ok = mb_wait(&sfull[slot], ps, status, 3);
                if (!ok) break;
                ok = mb_wait(&tfull[b], pb, status, 3);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int grp = 0; grp < 2; ++grp) {
#pragma unroll
                    for (int mt = 0; mt < NMAT; ++mt) {
                        const float s = scl[((slot * 2 + grp) * NMAT + mt) * TILE_M + r];
                        float dv[16];
                        tmem_ld16(tlane + (uint32_t)(((b * 2 + grp) * NMAT + mt) * NT), dv);
                        tmem_ld_wait();
                        if (grp == 1 && mt == NMAT - 1) {  // the buffer has been read: hand it back before the arithmetic
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mb_arrive(&tfree[b]);
                        }
#pragma unroll
                        for (int j = 0; j < 16; ++j) acc[mt][j] = fmaf(s, dv[j], acc[mt][j]);
                    }
                }
                if (++b == NBUF) { b = 0; pb ^= 1u; }
                if (++slot == SCL) { slot = 0; ps ^= 1u; }
            }
            if (!ok) break;
            const int t0 = 16 * hsel;
            if constexpr (NMAT == 2 && !PAIR) {
                uint16_t* oh = out_hi + (size_t)(it.prow + t0) * n_out + it.r0 + r;
                uint16_t* ol = out_lo + (size_t)(it.prow + t0) * n_out + it.r0 + r;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float a = swiglu_fast(acc[0][j], acc[NMAT - 1][j]);
                    const uint16_t ah = __bfloat16_as_ushort(__float2bfloat16_rn(a));
                    const float al = a - __uint_as_float((uint32_t)ah << 16);
                    if (t0 + j < it.m_tile) {
                        oh[(size_t)j * n_out] = ah;
                        ol[(size_t)j * n_out] = (uint16_t)(__float_as_uint(al) >> 16);
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    if (t0 + j < it.m_tile) {
                        float* o = row_dst ? row_dst[it.prow + t0 + j] + it.r0 + r   // expert parallel: the owner's (token, slot) row
                                           : out_f32 + (size_t)(it.prow + t0 + j) * n_out + it.r0 + r;
#pragma unroll
                        for (int mt = 0; mt < NMAT; ++mt) o[mt * TILE_M] = acc[mt][j];
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == W_MMA) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TM_COLS) : "memory");
    }
}

}  // namespace ex

static int upload_grid(int device) {
    static bool done[64] = {false};
    if (device < 0 || device >= 64) return DNB_ERR_ARG;
    if (done[device]) return DNB_OK;
    DNB_CUDA(cudaMemcpyToSymbol(ex::c_grid, dnb_iq3xxs_grid, sizeof(ex::c_grid)));
    done[device] = true;
    return DNB_OK;
}

bool grouped_exact_handles(int type, int n_in, int n_out) {
    return type == T_IQ3_XXS && n_in % 256 == 0 && n_out % ex::TILE_M == 0;
}

// Grouped IQ3_XXS GEMM on tcgen05 with exact weights.  fused: seg[].wa/wb are gate/up, output
// silu(g)*u as hi/lo bf16 packed rows; otherwise seg[].wa, fp32 output rows.
int launch_grouped_exact(dnb_ctx* c, cudaStream_t st, bool fused, const SegDesc* seg, const int32_t* nseg_dev, int nseg_max,
                         int n_in, int n_out, const UmmaMaps* maps, uint16_t* out_hi, uint16_t* out_lo, float* out_f32,
                         float* const* row_dst) {
    static_assert(sizeof(UmmaMaps) == sizeof(ex::Maps), "UmmaMaps must mirror ex::Maps");
    if (!grouped_exact_handles(T_IQ3_XXS, n_in, n_out) || nseg_max > ex::kMaxSeg) return DNB_DECLINED;
    int rc = upload_grid(c->device);
    if (rc) return rc;
    const int rb = n_in / 256 * 98;
    const ex::Maps& M = *reinterpret_cast<const ex::Maps*>(maps);
    const dim3 grid(c->sm_count);
    const bool pair = !fused && n_out % (2 * ex::TILE_M) == 0;
    const int nmat = (fused || pair) ? 2 : 1;
    const size_t smem = (size_t)ex::STAGES * ex::STAGE_BYTES + ex::RAWS * (size_t)nmat * ex::TILE_M * ex::RAW_PITCH +
                        (size_t)ex::SCL * 2 * nmat * ex::TILE_M * 4 + 256 * ex::LUT_REP * 8 +
                        (2 * ex::STAGES + 2 * ex::NB + ex::SCL) * 8 + 16 + (ex::kMaxSeg + 1) * 4 +
                        ex::kLocalItems * sizeof(ex::Item) + 1024;
    if (fused) {
        static SmemGrant grant;
        DNB_CUDA(grant_smem(grant, c->device, ex::grouped_iq3_exact_kernel<2>, smem));
        ProfScope prof_(c, st, "exact_gate_up");
        ex::grouped_iq3_exact_kernel<2><<<grid, ex::NTHREADS, smem, st>>>(seg, nseg_dev, n_in, n_out, rb, M, out_hi, out_lo, nullptr,
                                                                         c->status, nullptr);
    } else if (pair) {
        static SmemGrant grant;
        DNB_CUDA(grant_smem(grant, c->device, ex::grouped_iq3_exact_kernel<2, true>, smem));
        ProfScope prof_(c, st, "exact_down");
        ex::grouped_iq3_exact_kernel<2, true><<<grid, ex::NTHREADS, smem, st>>>(seg, nseg_dev, n_in, n_out, rb, M, nullptr, nullptr,
                                                                               out_f32, c->status, row_dst);
    } else {
        static SmemGrant grant;
        DNB_CUDA(grant_smem(grant, c->device, ex::grouped_iq3_exact_kernel<1>, smem));
        ProfScope prof_(c, st, "exact_down");
        ex::grouped_iq3_exact_kernel<1><<<grid, ex::NTHREADS, smem, st>>>(seg, nseg_dev, n_in, n_out, rb, M, nullptr, nullptr, out_f32,
                                                                         c->status, row_dst);
    }
    c->launches++;
    DNB_CUDA(cudaGetLastError());
    return DNB_OK;
}

int launch_grouped_tc(dnb_ctx* c, cudaStream_t st, int type, bool fused, const SegDesc* seg, const int32_t* nseg_dev,
                      int nseg_max, int n_in, int n_out, const UmmaMaps* maps, int nt_max, uint16_t* out_hi,
                      uint16_t* out_lo, float* out_f32, float* const* row_dst) {
    if (type == T_IQ3_XXS)
        return launch_grouped_exact(c, st, fused, seg, nseg_dev, nseg_max, n_in, n_out, maps, out_hi, out_lo, out_f32, row_dst);
    if (type == T_Q4_K)
        return launch_grouped_umma(c, st, fused, seg, nseg_dev, nseg_max, n_in, n_out, maps, nt_max, out_hi, out_lo, out_f32, row_dst);
    return DNB_DECLINED;
}

}  // namespace dnb
