// Grouped per-expert GEMM of chunked prefill on the 5th-generation tensor cores.
//
// Reference kernels of this role: kernels_exp_iq_tc.cu:307-527 (wmma bf16, 64x64x32
// tiles, both operands rounded to bf16, "no contract"), kernels_gemm_grouped.cu:
// 134-273 (fp32 FMA), kernels_exp_k_pf.cu:188-258 (m-row fp32).  The reference has
// no tensor-core kernel for Q4_K experts at all.
//
// Design (sm_100a).  A work item is, for one expert segment, a tile of 128 weight rows
// x up to 128 token rows over the whole K:
//   D[128 rows][N tokens] (fp32, in TMEM) = W[128][K] * X[N][K]^T
// issued as tcgen05.mma (cta_group::1, kind::f16, M=128, K=16 per instruction) by
// one elected thread.  W is the A operand and the tokens are the N dimension, so N is
// only as wide as the segment needs (16/32/64/128) and a 3-token expert does not pay
// for a 128-token tile.  The kernel is persistent: one CTA per SM walks the items
// i, i + gridDim.x, ... (the segment table is sorted by token count, heavy tiles first).
//
// Precision.  The path's bar is max|err| <= 1e-3 of the output RMS, which a single
// bf16 rounding of both operands misses by several times.  Each operand is
// therefore split into two bf16 numbers (hi = the value rounded to bf16, lo = the
// exact remainder truncated to bf16), and three MMAs hi*hi + hi*lo + lo*hi
// accumulate into the same TMEM tile; the dropped lo*lo term is about 2^-18
// relative per product.  The three products are issued in the same order for every
// tile width, so a token's result does not depend on which tokens share its chunk.
//
// Operands.
//   A (weights): sixteen producer warps dequantise Q4_K bytes (each thread's next 16 qs bytes
//      per matrix arrive by cp.async in a private shared-memory slot), split to hi/lo bf16
//      and store the tiles in the K-major
//      128-byte-swizzled layout the MMA reads.
//   B (activations): a pre-pass gathers the routed token rows into the expert-major
//      packed order and splits them into hi/lo bf16 buffers once per layer; the
//      tiles then arrive by TMA (cp.async.bulk.tensor.2d, 128B swizzle), N rows x 64
//      elements, signalled on the stage's mbarrier.
// Pipeline: `full[s]` (8 producer-warp arrivals + TMA bytes) -> MMA thread ->
// tcgen05.commit -> `empty[s]`; after an item's last stage a commit on `accum[b]`.
// Epilogue: four warps read their 32 TMEM lanes (= weight rows) of accumulator buffer b
// with tcgen05.ld while the main loop fills buffer 1 - b; gate/up tiles are combined as
// silu(g)*u and written as hi/lo bf16 in packed-row order (the B operand of the down
// GEMM); down tiles are written as fp32 rows for the weighted combine.
//
// Every wait is bounded; a wait that gives up sets *status and the CTA falls
// through to the common teardown (TMEM is always freed).
#include <cuda.h>
#include <cuda_bf16.h>

#include "dnb_common.cuh"
#include "formats.cuh"
#include "tc_ptx.cuh"

namespace dnb {

namespace um {
using namespace tcp;

constexpr int BK = 64;            // K elements per stage (one 128-byte swizzle row of bf16)
constexpr int TILE_M = 128;       // weight rows per CTA
constexpr int A_TILE = TILE_M * BK * 2;   // 16 KB
constexpr int kLocalItems = 64;   // items of a CTA decoded once into shared memory
constexpr int kMaxSeg = 1055;    // segments the per-CTA tile prefix table holds
constexpr int PWARPS = 16;        // producer warps: four threads per weight row and matrix (16 elements each per stage)
constexpr int W_TMA = PWARPS;     // warp that issues the activation tile copies
constexpr int W_MMA = PWARPS + 1; // warp that issues the MMAs and owns the TMEM allocation
constexpr int NTHREADS = (PWARPS + 6) * 32;  // + TMA, MMA and four epilogue warps

__device__ __forceinline__ uint32_t make_idesc(int n) { return idesc_bf16(TILE_M, n); }

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

// One producer task: 16 elements of one Q4_K row -> hi/lo bf16 in the swizzled tiles.
// hdr = first 16 bytes of the block (d, dmin, 12 scale bytes), q = 16 qs bytes: bytes
// 16p .. 16p+15 of chunk j's 32.  nh = 0 takes the low nibbles (stage elements
// 16p .. 16p+15), nh = 1 the high nibbles (elements 32+16p ..) (kquant.rs:505-526).
__device__ __forceinline__ void dequant_q4k_task(const uint4& hdr, const uint4& q, int j, int nh, int p,
                                                 uint8_t* tile_hi, uint8_t* tile_lo, int r) {
    const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xFFFF)));
    const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
    // scale bytes 0..11 live in hdr.y, hdr.z, hdr.w
    auto sb = [&](int i) -> uint32_t {
        const uint32_t w = i < 4 ? hdr.y : (i < 8 ? hdr.z : hdr.w);
        return (w >> (8 * (i & 3))) & 0xFFu;
    };
    const int a = 2 * j + nh;  // sub-block of these 16 elements
    uint32_t sc, mn;
    if (a < 4) { sc = sb(a) & 63; mn = sb(a + 4) & 63; }
    else { sc = (sb(a + 4) & 0xF) | ((sb(a - 4) >> 6) << 4); mn = (sb(a + 4) >> 4) | ((sb(a) >> 6) << 4); }
    const float d1 = d * (float)sc;
    const float c1 = fmaf(128.0f, d1, dmin * (float)mn);
    const uint32_t rowoff = (uint32_t)(r >> 3) * 1024u + (uint32_t)(r & 7) * 128u;
    const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
    const int sh = nh * 4;
#pragma unroll
    for (int w2 = 0; w2 < 2; ++w2) {  // 8 elements = one 16-byte column of the swizzled row
        uint32_t hv[4], lv[4];
#pragma unroll
        for (int w1 = 0; w1 < 2; ++w1) {
            const uint32_t nib = (qw[2 * w2 + w1] >> sh) & 0x0F0F0F0Fu;
            // w = d1 * q - m1 evaluated as d1 * (128 + q) - (128 d1 + m1): one fma on an exact float
            const float a0 = fmaf(d1, magic128<0>(nib), -c1), a1 = fmaf(d1, magic128<1>(nib), -c1);
            const float a2 = fmaf(d1, magic128<2>(nib), -c1), a3 = fmaf(d1, magic128<3>(nib), -c1);
            split2(a0, a1, hv[2 * w1], lv[2 * w1]);
            split2(a2, a3, hv[2 * w1 + 1], lv[2 * w1 + 1]);
        }
        const uint32_t col = ((uint32_t)((4 * nh + 2 * p + w2) ^ (r & 7))) << 4;
        *reinterpret_cast<uint4*>(tile_hi + rowoff + col) = make_uint4(hv[0], hv[1], hv[2], hv[3]);
        *reinterpret_cast<uint4*>(tile_lo + rowoff + col) = make_uint4(lv[0], lv[1], lv[2], lv[3]);
    }
}

// A work item of the persistent kernel: which segment, which 128 tokens of it, which
// 128 weight rows.
struct Item {
    const uint8_t* wa;
    const uint8_t* wb;
    int prow;    // first packed row of the token tile
    int m_tile;  // tokens in the tile (1..128)
    int r0;      // first weight row
};
__device__ __forceinline__ Item decode_item(int item, int row_tiles, int nseg, const int* tile_prefix,
                                            const SegDesc* __restrict__ seg, int rows_per_item = TILE_M) {
    const int tile = item / row_tiles, rt = item - tile * row_tiles;
    int lo = 0, hi = nseg - 1;
    while (lo < hi) {  // last segment whose first tile is <= tile
        const int mid = (lo + hi + 1) >> 1;
        if (tile_prefix[mid] <= tile) lo = mid; else hi = mid - 1;
    }
    const SegDesc sd = seg[lo];
    const int t0 = (tile - tile_prefix[lo]) * 128;
    Item it;
    it.wa = sd.wa;
    it.wb = sd.wb;
    it.prow = (int)sd.row0 + t0;
    it.m_tile = min(128, (int)sd.m - t0);
    it.r0 = rt * rows_per_item;
    return it;
}
// The CTA's k-th item: from the table filled at kernel start, or decoded on the spot when
// the CTA has more items than the table holds.
struct ItemTab {
    const Item* tab;
    const SegDesc* seg;
    const int* tile_prefix;
    int nseg, row_tiles, rows_per_item;
    __device__ __forceinline__ Item get(int k) const {
        if (k < kLocalItems) return tab[k];
        return decode_item((int)blockIdx.x + k * (int)gridDim.x, row_tiles, nseg, tile_prefix, seg, rows_per_item);
    }
};
__device__ __forceinline__ int nsel_of(int m_tile) { return m_tile <= 16 ? 0 : (m_tile <= 32 ? 1 : (m_tile <= 64 ? 2 : 3)); }

// silu(g) * u with the fast exponential and reciprocal: their ~1e-6 relative error
// is far inside what the bf16 hi/lo products already carry.
__device__ __forceinline__ float swiglu_fast(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }

// What a producer warp needs from the kernel.
struct ProducerArgs {
    ItemTab items;
    uint8_t* smem;
    uint8_t* rawq;   // [16 producer warps][32 lanes][NMAT] x 16 bytes: every thread's slot for its next chunk; then
                     // [2 groups][128 rows][NMAT] x 16 bytes: the block headers
    uint64_t* full;
    uint64_t* empty;
    int* status;
    int my_items, nchunks, rb;
};

// Producer warps.  The sixteen warps form two groups of eight; group GRP dequantises the
// chunks g with g % 2 == GRP, all 128 rows of them, so the two groups fill two different
// stages at the same time and one group's waits (stage free, bytes arrived, stores
// visible) are covered by the other group's arithmetic.  Inside a group a warp owns 16
// rows x 2 qs pieces (a request covers whole 32-byte sectors) and a thread dequantises
// both nibbles of its 16 bytes: 32 elements per matrix and chunk.  Raw bytes are
// requested two of the group's chunks ahead, through item boundaries.
template <int NMAT, bool PAIR, int STAGES, int STAGE_BYTES, int GRP>
__device__ __forceinline__ bool produce(const ProducerArgs& a, int w8, int lane) {
    const int r = w8 * 16 + (lane & 15), p = lane >> 4;
    struct Raw { uint4 qa, qb; };   // one chunk's 16 qs bytes per matrix
    struct Hdr { uint4 ha, hb; };   // one block's d, dmin and scale bytes per matrix
    Raw cur;                        // the chunk being dequantised
    Hdr hdr_cur;
    // The thread's private 16 bytes per matrix in shared memory: the NEXT chunk's qs bytes arrive there by cp.async.
    uint4* slot = reinterpret_cast<uint4*>(a.rawq) + (size_t)((GRP * (PWARPS / 2) + w8) * 32 + lane) * NMAT;
    // The row's block header (16 bytes per matrix), one slot per group and row: requested by the lane with p = 0
    // together with the block's first chunk, read by both lanes of the row at the top of the block.
    uint4* hslot = reinterpret_cast<uint4*>(a.rawq) + (size_t)PWARPS * 32 * NMAT + (size_t)(GRP * TILE_M + r) * NMAT;
    int f_left = a.my_items, f_k = 0, f_c = GRP;  // fetch cursor: item (CTA-local index) and chunk
    const uint8_t* f_pa = nullptr;
    const uint8_t* f_pb = nullptr;
    // (Asking L2 for the next item's rows a full item ahead with cp.async.bulk.prefetch.L2 was measured: the same
    // kernel time with and without, and 1.9x the DRAM traffic with, because most prefetched lines were gone again
    // by the time they were needed.)
    auto f_open = [&]() {
        if (f_left > 0) {
            const Item it = a.items.get(f_k);
            f_pa = it.wa + (size_t)(it.r0 + r) * a.rb;
            if constexpr (NMAT == 2) f_pb = PAIR ? it.wa + (size_t)(it.r0 + TILE_M + r) * a.rb : it.wb + (size_t)(it.r0 + r) * a.rb;
        }
    };
    // Request the fetch cursor's chunk.  The qs bytes travel by cp.async into the thread's slot and are picked up
    // with cp.async.wait_group: with plain loads held in registers two chunks ahead, a wait for the older request
    // also waited for the younger one, and these stalls were 40 % of the kernel (measured by leaving the loads out).
    // The block header comes the same way (as a plain load a block ahead it cost 9 % of the gate/up kernel).
    auto fetch = [&]() {
        if (f_left <= 0) {
            cp_async_commit();
            return;
        }
        const int off = (f_c >> 2) * 144;
        if ((f_c & 3) == GRP && p == 0) {  // the group's first chunk of a block: fetch the block header too
            cp_async16<false>(hslot, f_pa + off);
            if constexpr (NMAT == 2) cp_async16<false>(hslot + 1, f_pb + off);
        }
        const int qoff = off + 16 + 32 * (f_c & 3) + 16 * p;
        cp_async16<false>(slot, f_pa + qoff);
        if constexpr (NMAT == 2) cp_async16<false>(slot + 1, f_pb + qoff);
        cp_async_commit();
        f_c += 2;
        if (f_c >= a.nchunks) {
            f_c = GRP;
            ++f_k;
            --f_left;
            f_open();
        }
    };
    auto take = [&]() {  // the chunk requested last has landed: into registers, and the slot is free again
        cp_async_wait_all();
        cur.qa = slot[0];
        if constexpr (NMAT == 2) cur.qb = slot[1];
    };
    // Two chunks of the group are in flight: one in `cur`, one on its way into the slot.  (A third, held in a
    // second register buffer, measured no faster.)
    f_open();
    fetch();
    take();
    fetch();
    bool ok = true;
    const int total = a.my_items * a.nchunks;  // a multiple of 4: n_in % 256 == 0
    for (int g4 = 0; g4 < total && ok; g4 += 4) {
        // Requested with the block's first chunk, which the last take() has waited for; the other lane of the row
        // sees it after the warp barrier, and both lanes have their copy before the next header is requested.
        __syncwarp();
        hdr_cur.ha = hslot[0];
        if constexpr (NMAT == 2) hdr_cur.hb = hslot[1];
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int j = GRP + 2 * i;  // chunk inside the block
            const int g = g4 + j;
            const int st = g % STAGES;
            const uint32_t ph = (uint32_t)(g / STAGES) & 1u;
            if (ok && g >= STAGES) ok = mb_wait(&a.empty[st], ph ^ 1u, a.status, 2);
            if (ok) {
                uint8_t* sa = a.smem + st * STAGE_BYTES;
#pragma unroll
                for (int nh = 0; nh < 2; ++nh) {
                    dequant_q4k_task(hdr_cur.ha, cur.qa, j, nh, p, sa, sa + A_TILE, r);
                    if constexpr (NMAT == 2) dequant_q4k_task(hdr_cur.hb, cur.qb, j, nh, p, sa + 2 * A_TILE, sa + 3 * A_TILE, r);
                }
                take();   // the group's next chunk, requested one chunk of work ago
                fetch();  // and the one after it
                fence_async_smem();   // generic-proxy stores -> visible to the tensor core's async proxy
                __syncwarp();
                if (lane == 0) mb_arrive(&a.full[st]);
            }
        }
    }
    cp_async_wait_all();
    return ok;
}

// NMAT = 2: gate and up tiles together, SwiGLU epilogue to out_hi / out_lo (bf16 packed rows).
// NMAT = 2, PAIR: two 128-row tiles of ONE matrix (rows r0.. and r0 + 128..) against the same activation tile, fp32
//   epilogue: the down GEMM (K = 512: 8 stages per item) with half the stages, hand-overs and activation copies of
// NMAT = 1: one matrix, one 128-row tile, fp32 epilogue to out_f32 (output widths that are not a multiple of 256).
//
// Persistent: grid = number of SMs (the stages fill shared memory, one CTA per SM).
// Work items are (segment, 128-token tile, 128-row tile), item i handled by CTA
// i mod gridDim.x in increasing order; every role walks the same item sequence on
// its own, coupled only through mbarriers:
//   warps 0-15   producers in two groups of eight; a group dequantises every second
//                chunk into its stage (32 elements per thread and matrix)
//   warp 16      TMA: activation tiles of the stage
//   warp 17      MMA issue (one thread); owns the TMEM allocation
//   warps 18-21  epilogue: read the finished accumulators of item i from TMEM while
//                the main loop of item i+1 fills the other accumulator buffer
// Barriers and their phases live across items: chunk counter g keeps running
// (stage g % STAGES, parity (g / STAGES) & 1); accumulator buffer = item count & 1.
template <int NMAT, bool PAIR = false>
__global__ void __launch_bounds__(NTHREADS, 1)
grouped_q4k_umma_kernel(const SegDesc* __restrict__ seg, const int32_t* __restrict__ nseg_dev, int n_in, int n_out,
                        int rb, const __grid_constant__ Maps maps, uint16_t* __restrict__ out_hi,
                        uint16_t* __restrict__ out_lo, float* __restrict__ out_f32, int* status,
                        float* const* __restrict__ row_dst) {
    constexpr int STAGES = (NMAT == 2) ? 2 : 3;
    constexpr int A_BYTES = NMAT * 2 * A_TILE;          // hi + lo per matrix
    constexpr int B_BYTES_MAX = 2 * 128 * BK * 2;       // hi + lo, N = 128
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES_MAX;
    constexpr int ACC_COLS = NMAT * 128;                // TMEM columns of one accumulator buffer
    constexpr int TM_COLS = 2 * ACC_COLS;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* accum = empty + STAGES;     // [2] accumulator buffer complete (one tcgen05.commit)
    uint64_t* drained = accum + 2;        // [2] accumulator buffer read out (4 epilogue warps)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drained + 2);
    int* tile_prefix = reinterpret_cast<int*>(tmem_slot + 2);  // [nseg + 1] token tiles before each segment
    Item* itab = reinterpret_cast<Item*>(smem + STAGES * STAGE_BYTES + 256 + (kMaxSeg + 1) * 4);  // [kLocalItems]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nchunks = n_in / BK;
    constexpr int ROWS_ITEM = PAIR ? 2 * TILE_M : TILE_M;
    const int row_tiles = n_out / ROWS_ITEM;
    const int nseg = min(*nseg_dev, kMaxSeg);

    if (tid == 0) {
        for (int i = 0; i < STAGES; ++i) {
            mb_init(&full[i], PWARPS / 2 + 1);  // one producer group + the TMA thread's expect_tx arrival
            mb_init(&empty[i], 1);          // one tcgen05.commit
        }
        for (int i = 0; i < 2; ++i) {
            mb_init(&accum[i], 1);
            mb_init(&drained[i], 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // Token tiles per segment (all threads load), then an exclusive scan by warp 0.
    for (int i = tid; i < nseg; i += NTHREADS) tile_prefix[i + 1] = ((int)seg[i].m + 127) >> 7;
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
    const int G = gridDim.x;
    const int my_items = (int)blockIdx.x < n_items ? (n_items - (int)blockIdx.x + G - 1) / G : 0;
    if (tid < min(my_items, kLocalItems)) itab[tid] = decode_item((int)blockIdx.x + tid * G, row_tiles, nseg, tile_prefix, seg, ROWS_ITEM);
    __syncthreads();
    const ItemTab items{itab, seg, tile_prefix, nseg, row_tiles, ROWS_ITEM};
    bool ok = true;

    if (warp < PWARPS) {
        // ---------------- producers ----------------
        ProducerArgs pa{items, smem, reinterpret_cast<uint8_t*>(itab + kLocalItems), full, empty, status, my_items, nchunks, rb};
        if (warp < PWARPS / 2) ok = produce<NMAT, PAIR, STAGES, STAGE_BYTES, 0>(pa, warp, lane);
        else ok = produce<NMAT, PAIR, STAGES, STAGE_BYTES, 1>(pa, warp - PWARPS / 2, lane);
    } else if (warp == W_TMA) {
        // ---------------- TMA: activation tiles ----------------
        // The whole warp walks the loop and waits; one elected lane issues.  Addresses,
        // coordinates and descriptors are then the same in every lane, which lets the
        // compiler keep them in the registers the copy and MMA instructions read.
        int g = 0;
        for (int k = 0; k < my_items && ok; ++k) {
            const Item it = items.get(k);
            const int nsel = nsel_of(it.m_tile), N = 16 << nsel;
            const CUtensorMap* mh = &maps.hi[nsel];
            const CUtensorMap* ml = &maps.lo[nsel];
            const uint32_t bbytes = (uint32_t)(2 * N * BK * 2);
            for (int c = 0; c < nchunks; ++c, ++g) {
                const int st = g % STAGES;
                const uint32_t ph = (uint32_t)(g / STAGES) & 1u;
                if (g >= STAGES) ok = warp_all(mb_wait(&empty[st], ph ^ 1u, status, 4));
                if (!ok) break;
                uint8_t* sbp = smem + st * STAGE_BYTES + A_BYTES;
                if (elect_one()) {
                    mb_expect_tx(&full[st], bbytes);
                    tma_load_2d(sbp, mh, c * BK, it.prow, &full[st]);
                    tma_load_2d(sbp + N * BK * 2, ml, c * BK, it.prow, &full[st]);
                }
                __syncwarp();
            }
        }
    } else if (warp == W_MMA) {
        // ---------------- MMA issue ----------------
        const uint32_t smem_lo = desc_lo(s32(smem));
        int g = 0;
        for (int k = 0; k < my_items && ok; ++k) {
            const Item it = items.get(k);
            const int N = 16 << nsel_of(it.m_tile);
            const uint32_t idesc = make_idesc(N);
            const int ab = k & 1;
            // the epilogue must have read this buffer's previous use (item k - 2)
            if (k >= 2) ok = warp_all(mb_wait(&drained[ab], (uint32_t)((k >> 1) - 1) & 1u, status, 6));
            if (!ok) break;
            tc_fence_after();
            const uint32_t dbase = tmem_base + (uint32_t)(ab * ACC_COLS);
            for (int c = 0; c < nchunks; ++c, ++g) {
                const int st = g % STAGES;
                const uint32_t ph = (uint32_t)(g / STAGES) & 1u;
                ok = warp_all(mb_wait(&full[st], ph, status, 5));
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_lo = smem_lo + (uint32_t)(st * (STAGE_BYTES >> 4));
                const uint32_t bh_lo = a_lo + (A_BYTES >> 4), bl_lo = bh_lo + (uint32_t)((N * BK * 2) >> 4);
                if (elect_one()) {
#pragma unroll
                    for (int ks = 0; ks < BK / 16; ++ks) {
                        const uint32_t koff = ks * 2;  // 16 bf16 = 32 bytes inside the swizzle row, >> 4
                        const uint64_t bh = desc_of(bh_lo + koff), bl = desc_of(bl_lo + koff);
#pragma unroll
                        for (int mt = 0; mt < NMAT; ++mt) {
                            const uint64_t ah = desc_of(a_lo + (uint32_t)(mt * 2 * (A_TILE >> 4)) + koff);
                            const uint64_t al = desc_of(a_lo + (uint32_t)(mt * 2 * (A_TILE >> 4) + (A_TILE >> 4)) + koff);
                            const uint32_t d = dbase + (uint32_t)(mt * 128);
                            // the same three products in the same order whatever the tile width:
                            // a token's result does not depend on who shares its chunk
                            mma_bf16(d, ah, bh, idesc, (c > 0 || ks > 0) ? 1u : 0u);
                            mma_bf16(d, ah, bl, idesc, 1u);
                            mma_bf16(d, al, bh, idesc, 1u);
                        }
                    }
                    mma_commit(&empty[st]);   // frees the stage once these MMAs have read it
                    if (c == nchunks - 1) mma_commit(&accum[ab]);  // item done -> accumulators readable
                }
                __syncwarp();
            }
        }
    } else {
        // ---------------- epilogue: TMEM lane = weight row ----------------
        const int quad = warp & 3;  // the TMEM lanes a warp may read: 32 * (warp % 4) ..
        const int r = quad * 32 + lane;
        for (int k = 0; k < my_items && ok; ++k) {
            const Item it = items.get(k);
            const int N = 16 << nsel_of(it.m_tile);
            const int ab = k & 1;
            ok = mb_wait(&accum[ab], (uint32_t)(k >> 1) & 1u, status, 3);
            tc_fence_after();
            if (!ok) break;
            const uint32_t tb = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(ab * ACC_COLS);
            for (int c0 = 0; c0 < N; c0 += 16) {
                uint32_t gq[16], uq[16];
                tmem_ld16(tb + (uint32_t)c0, gq);
                if constexpr (NMAT == 2) tmem_ld16(tb + (uint32_t)(128 + c0), uq);
                tmem_ld_wait();
                const int nv = min(16, it.m_tile - c0);
                if constexpr (NMAT == 2 && PAIR) {
                    if (row_dst) {
#pragma unroll
                        for (int j2 = 0; j2 < 16; ++j2)
                            if (j2 < nv) {
                                float* dst = row_dst[it.prow + c0 + j2] + it.r0 + r;
                                dst[0] = __uint_as_float(gq[j2]);
                                dst[TILE_M] = __uint_as_float(uq[j2]);
                            }
                    } else {
                        float* of = out_f32 + (size_t)(it.prow + c0) * n_out + it.r0 + r;
#pragma unroll
                        for (int j2 = 0; j2 < 16; ++j2)
                            if (j2 < nv) {
                                of[(size_t)j2 * n_out] = __uint_as_float(gq[j2]);
                                of[(size_t)j2 * n_out + TILE_M] = __uint_as_float(uq[j2]);
                            }
                    }
                } else if constexpr (NMAT == 2) {
                    uint16_t* oh = out_hi + (size_t)(it.prow + c0) * n_out + it.r0 + r;
                    uint16_t* ol = out_lo + (size_t)(it.prow + c0) * n_out + it.r0 + r;
#pragma unroll
                    for (int j2 = 0; j2 < 16; ++j2) {
                        const float a = swiglu_fast(__uint_as_float(gq[j2]), __uint_as_float(uq[j2]));
                        const uint16_t ah = __bfloat16_as_ushort(__float2bfloat16_rn(a));
                        const float al = a - __uint_as_float((uint32_t)ah << 16);
                        if (j2 < nv) {
                            oh[(size_t)j2 * n_out] = ah;
                            ol[(size_t)j2 * n_out] = (uint16_t)(__float_as_uint(al) >> 16);
                        }
                    }
                } else {
                    if (row_dst) {
                        // Expert parallel: packed row p's result goes where row_dst[p] points, the
                        // (token, slot) row of the GPU that owns the token -- a plain store over
                        // NVLink from this epilogue, no copy pass afterwards.
#pragma unroll
                        for (int j2 = 0; j2 < 16; ++j2)
                            if (j2 < nv) row_dst[it.prow + c0 + j2][it.r0 + r] = __uint_as_float(gq[j2]);
                    } else {
                        float* of = out_f32 + (size_t)(it.prow + c0) * n_out + it.r0 + r;
#pragma unroll
                        for (int j2 = 0; j2 < 16; ++j2)
                            if (j2 < nv) of[(size_t)j2 * n_out] = __uint_as_float(gq[j2]);
                    }
                }
            }
            tc_fence_before();  // TMEM reads ordered before the hand-back of the buffer
            __syncwarp();
            if (lane == 0) mb_arrive(&drained[ab]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == W_MMA) {
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

int tc_make_map(void* map, void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    return make_map(reinterpret_cast<CUtensorMap*>(map), base, rows, cols, box_rows);
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
                        uint16_t* out_lo, float* out_f32, float* const* row_dst) {
    if (n_in % 256 || n_out % um::TILE_M) return DNB_DECLINED;
    const int rb = n_in / 256 * 144;
    const um::Maps& M = *reinterpret_cast<const um::Maps*>(maps);
    if (nseg_max > um::kMaxSeg) return DNB_DECLINED;
    (void)nt_max;
    const dim3 grid(c->sm_count);  // persistent: one CTA per SM loops over the tiles
    if (fused) {
        const size_t smem = 2 * (2 * 2 * um::A_TILE + 2 * 128 * um::BK * 2) + 256 + (um::kMaxSeg + 1) * 4 + um::kLocalItems * sizeof(um::Item) +
                            um::PWARPS * 32 * 2 * 16 + 2 * um::TILE_M * 2 * 16 + 1024;
        static SmemGrant grant;
        DNB_CUDA(grant_smem(grant, c->device, um::grouped_q4k_umma_kernel<2>, smem));
        ProfScope prof_(c, st, "umma_gate_up");
        um::grouped_q4k_umma_kernel<2><<<grid, um::NTHREADS, smem, st>>>(seg, nseg_dev, n_in, n_out, rb, M, out_hi, out_lo,
                                                                        nullptr, c->status, nullptr);
    } else if (n_out % (2 * um::TILE_M) == 0) {
        const size_t smem = 2 * (2 * 2 * um::A_TILE + 2 * 128 * um::BK * 2) + 256 + (um::kMaxSeg + 1) * 4 + um::kLocalItems * sizeof(um::Item) +
                            um::PWARPS * 32 * 2 * 16 + 2 * um::TILE_M * 2 * 16 + 1024;
        static SmemGrant grant;
        DNB_CUDA(grant_smem(grant, c->device, um::grouped_q4k_umma_kernel<2, true>, smem));
        ProfScope prof_(c, st, "umma_down");
        um::grouped_q4k_umma_kernel<2, true><<<grid, um::NTHREADS, smem, st>>>(seg, nseg_dev, n_in, n_out, rb, M, nullptr, nullptr,
                                                                              out_f32, c->status, row_dst);
    } else {
        const size_t smem = 3 * (2 * um::A_TILE + 2 * 128 * um::BK * 2) + 256 + (um::kMaxSeg + 1) * 4 + um::kLocalItems * sizeof(um::Item) +
                            um::PWARPS * 32 * 1 * 16 + 2 * um::TILE_M * 1 * 16 + 1024;
        static SmemGrant grant;
        DNB_CUDA(grant_smem(grant, c->device, um::grouped_q4k_umma_kernel<1>, smem));
        ProfScope prof_(c, st, "umma_down");
        um::grouped_q4k_umma_kernel<1><<<grid, um::NTHREADS, smem, st>>>(seg, nseg_dev, n_in, n_out, rb, M, nullptr, nullptr,
                                                                        out_f32, c->status, row_dst);
    }
    c->launches++;
    DNB_CUDA(cudaGetLastError());
    return DNB_OK;
}

}  // namespace dnb
