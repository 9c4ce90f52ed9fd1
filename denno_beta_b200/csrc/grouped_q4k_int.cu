// Grouped per-expert Q4_K GEMM of chunked prefill on tcgen05 with INTEGER weights and block scales applied after the
// tensor-core sum.
//
// Reference kernels of this role: kernels_exp_k_pf.cu:188-258 (m-row fp32), kernels_gemm_grouped.cu:134-273 (fp32 FMA);
// block layout and arithmetic kquant.rs:505-526 (w = d * sc * q - dmin * m per 32-element sub-block).
//
// Why.  The three-product kernel of grouped_umma.cu folds d * sc and dmin * m into every weight in fp32 and splits the
// result into two bf16 numbers: about ten instructions per weight, and that dequantisation bounds it.  Here
//     W . x  =  sum over 256-blocks b of  d_b * [ sum_i (sc * q)_i * x_i ]   -   sum over sub-blocks s of (dmin * m)_s * X_s
// with X_s = the sum of the 32 activations of sub-block s.
//   * (sc * q) is an integer <= 63 * 15 = 945: EXACT in fp16.  A nibble becomes 1024 + q by a byte permute (0x6400 | q)
//     and one fma.rn.f16x2 (1024 + q) * sc - 1024 * sc gives sc * q for two weights: under two instructions per
//     weight, one 16 KB fp16 tile per matrix and stage instead of a hi and a lo tile.
//   * The bracket is accumulated by tcgen05.mma (kind::f16, fp16 x fp16 -> fp32 in TMEM) over the four 64-element
//     stages of a block; the epilogue warps then add d_b * (TMEM) to fp32 registers: one FMA per output and 256 weights.
//   * The second sum is one more "block" of the same shape, K = number of sub-blocks: A = -(dmin * m) as fp16 hi and lo
//     (two tiles of one matrix per stage), B = X.  Its scale is 1.
//   * Activations are fp16 hi + lo (22 bits) of the row scaled by a power of two so that its largest element is in
//     [256, 512) (sub-block sums stay below 65504); hi and lo rows of a tile sit one after the other in shared memory
//     and form ONE B operand of N = 2 x tokens, so a weight tile is read once per K step; the epilogue adds the two
//     halves and multiplies the row's scale back at the end.
//   Every product is exact and sums are fp32: the result is closer to the fp32 reference than the bf16 kernel's.
//   Limits: |dmin| * 63 < 65504 (fp16 range of the second sum's A operand; dmin * m is the sub-block's offset, i.e. a
//   weight magnitude), K <= 2048 (a thread builds four blocks' columns of the second sum's tiles), N out a multiple of 128 (256 for
//   the down form).
//
// Shape.  Items of 32 tokens x 128 rows x 2 "matrices" (gate and up, or rows r0.. and r0 + 128.. of the down matrix),
// persistent CTAs, item i to CTA i mod grid.  26 warps: sixteen producers in two groups that take alternate stages
// (the structure of grouped_umma.cu: a thread owns 16 qs bytes of a row per stage, fetched by cp.async one stage
// ahead), eight epilogue warps (a TMEM lane quadrant x 16 token columns each), one TMA warp (activation tiles), one
// MMA warp.  TMEM: four buffers of [2 matrices][hi | lo][32 tokens] = 128 columns, one per block in flight.
// Every wait is bounded; a wait that gives up sets *status and the CTA falls through to the teardown.
//
// Measured (B200, 512-token chunk, Zipf router bias, n_embd 2048, n_ff 512): gate/up 0.196 ms and down 0.125 ms against
// 0.174 / 0.090 ms of the three-product kernel, at a sixth of its error (1e-5 against 7e-5 of the output RMS).  Per-role
// cycle counts: the MMA warp needs ~970 cycles per 64-element stage (~480 of them with no MMA in it: barrier waits,
// fences and two commits; ~60 per 128 x 64 x 16 MMA), a producer group ~3000 per chunk of which the decode is under
// half, and with 32-token tiles the hot experts of a skewed chunk cost 2.2 times the stages of 128-token tiles.  The
// per-stage hand-over, not the arithmetic, bounds it; the block scales keep the accumulators in registers and so
// cap the tile at 32 tokens.  The library therefore uses it only on request (dnb_set_q4k_int).
#include <cuda.h>
#include <cuda_fp16.h>

#include "dnb_common.cuh"
#include "tc_ptx.cuh"

namespace dnb {
namespace qi {
using namespace tcp;

constexpr int BK = 64;                       // K per stage: one 128-byte swizzle row of fp16
constexpr int TILE_M = 128;                  // weight rows per matrix and item
constexpr int NT = 32;                       // tokens per item
constexpr int A_TILE = TILE_M * BK * 2;      // 16 KB
constexpr int B_TILE = 2 * NT * BK * 2;      // hi rows then lo rows: 8 KB
constexpr int STAGE_BYTES = 2 * A_TILE + B_TILE;
constexpr int STAGES = 3;
constexpr int NB = 4;                        // TMEM buffers (128 columns each)
constexpr int BUF_COLS = 4 * NT;
constexpr int SCL = 12;                      // ring of block scales [2][128]; a producer is at most NB + 2 blocks ahead of the epilogue
constexpr int PWARPS = 16, EWARPS = 8;
constexpr int W_TMA = PWARPS + EWARPS, W_MMA = W_TMA + 1;
constexpr int NTHREADS = (W_MMA + 1) * 32;
constexpr int kMaxSeg = 1055;
constexpr int kLocalItems = 32;
constexpr int kMaxBlocks = 8;
constexpr int RING = 2;                      // slots of a producer thread's ring of qs bytes (RING - 1 chunks on their way)

struct Maps {  // tensor maps of the B operand: box heights 16, 32, 64, 128 for hi and lo (this kernel uses 16 and 32)
    CUtensorMap hi[4];
    CUtensorMap lo[4];
};

struct Item {
    const uint8_t* pa;  // matrix 0, first row of the tile
    const uint8_t* pb;  // matrix 1
    int prow;           // first packed row of the token tile
    int m_tile;         // tokens in the tile (1..NT)
    int r0;             // first output row
    int pad;
};
template <bool PAIR>
__device__ __forceinline__ Item decode_item(int item, int row_tiles, int rb, int nseg, const int* tile_prefix,
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
    it.r0 = rt * (PAIR ? 2 * TILE_M : TILE_M);
    it.pa = sd.wa + (size_t)it.r0 * rb;
    it.pb = PAIR ? it.pa + (size_t)TILE_M * rb : sd.wb + (size_t)it.r0 * rb;
    it.prow = (int)sd.row0 + t0;
    it.m_tile = min(NT, (int)sd.m - t0);
    it.pad = 0;
    return it;
}
template <bool PAIR>
struct ItemTab {
    const Item* tab;
    const SegDesc* seg;
    const int* tile_prefix;
    int nseg, row_tiles, rb;
    __device__ __forceinline__ Item get(int k) const {
        if (k < kLocalItems) return tab[k];
        return decode_item<PAIR>((int)blockIdx.x + k * (int)gridDim.x, row_tiles, rb, nseg, tile_prefix, seg);
    }
};

__device__ __forceinline__ float swiglu_fast(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }
__device__ __forceinline__ uint32_t hfma2_bits(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t scale_byte(const uint4& hdr, int i) {  // scale bytes 0..11 live in hdr.y, hdr.z, hdr.w
    const uint32_t w = i < 4 ? hdr.y : (i < 8 ? hdr.z : hdr.w);
    return (w >> (8 * (i & 3))) & 0xFFu;
}

// 32 elements of one Q4_K row (the thread's 16 qs bytes of chunk j: both nibbles) as integers sc * q in fp16.
__device__ __forceinline__ void decode_q4k_int(const uint4& hdr, const uint4& q, int j, int p, uint8_t* tile, int r) {
    const uint32_t rowoff = (uint32_t)(r >> 3) * 1024u + (uint32_t)(r & 7) * 128u;
    const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int nh = 0; nh < 2; ++nh) {
        const int a = 2 * j + nh;  // sub-block of these 16 elements (kquant.rs:505-526: low nibbles first)
        const uint32_t sc = a < 4 ? (scale_byte(hdr, a) & 63u) : ((scale_byte(hdr, a + 4) & 0xFu) | ((scale_byte(hdr, a - 4) >> 6) << 4));
        const uint32_t s1 = (uint32_t)__half_as_ushort(__uint2half_rn(sc));
        const uint32_t c1 = (uint32_t)__half_as_ushort(__float2half_rn(-1024.0f * (float)sc));  // exact: six bits times 2^10
        const uint32_t s2 = s1 | (s1 << 16), c2 = c1 | (c1 << 16);
#pragma unroll
        for (int w2 = 0; w2 < 2; ++w2) {  // 8 elements = one 16-byte column of the swizzled row
            uint32_t v[4];
#pragma unroll
            for (int w1 = 0; w1 < 2; ++w1) {
                const uint32_t nib = (qw[2 * w2 + w1] >> (4 * nh)) & 0x0F0F0F0Fu;
                // 0x6400 | q = 1024 + q in fp16; (1024 + q) * sc - 1024 * sc rounds once, to the integer sc * q
                v[2 * w1] = hfma2_bits(__byte_perm(nib, 0x64646464u, 0x4140), s2, c2);
                v[2 * w1 + 1] = hfma2_bits(__byte_perm(nib, 0x64646464u, 0x4342), s2, c2);
            }
            const uint32_t col = ((uint32_t)((4 * nh + 2 * p + w2) ^ (r & 7))) << 4;
            *reinterpret_cast<uint4*>(tile + rowoff + col) = make_uint4(v[0], v[1], v[2], v[3]);
        }
    }
}

// The eight sub-block offsets -(dmin * m) of one block as fp16 hi and lo (one 16-byte column each).
__device__ __forceinline__ void decode_q4k_mins(const uint4& hdr, uint4& hi, uint4& lo) {
    const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
    uint32_t h[8], l[8];
#pragma unroll
    for (int s = 0; s < 8; ++s) {
        const uint32_t m = s < 4 ? (scale_byte(hdr, s + 4) & 63u) : ((scale_byte(hdr, s + 4) >> 4) | ((scale_byte(hdr, s) >> 6) << 4));
        const float v = -(dmin * (float)m);  // exact in fp32 (11 x 6 bits)
        const __half vh = __float2half_rn(v);
        h[s] = __half_as_ushort(vh);
        l[s] = __half_as_ushort(__float2half_rn(v - __half2float(vh)));
    }
    hi = make_uint4(h[0] | (h[1] << 16), h[2] | (h[3] << 16), h[4] | (h[5] << 16), h[6] | (h[7] << 16));
    lo = make_uint4(l[0] | (l[1] << 16), l[2] | (l[3] << 16), l[4] | (l[5] << 16), l[6] | (l[7] << 16));
}

template <bool PAIR>
struct ProducerArgs {
    ItemTab<PAIR> items;
    uint8_t* smem;
    uint4* rawq;   // [16 warps][32 lanes][RING][2 matrices]: every thread's ring of qs bytes on their way
    uint4* hq;     // [2 groups][128 rows][2][2 matrices]: the block headers, two blocks deep
    float* scl;    // [SCL][2][128]
    uint64_t* full;
    uint64_t* empty;
    uint64_t* sfull;
    int* status;
    int my_items, nchunks, nblk;
};

template <int N>
__device__ __forceinline__ void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Producer warps: two groups of eight; group GRP fills the stages of the chunks j with j % 2 == GRP (all 128 rows, both
// matrices) and, at the end of an item, the offsets' stage of matrix GRP.  Inside a group a warp owns 16 rows x 2 qs
// pieces; a thread decodes both nibbles of its 16 bytes per matrix: 32 elements per matrix and chunk.
// A thread keeps RING - 1 chunks of its own on their way (cp.async into a private ring, one commit group per chunk,
// wait_group RING - 2).  Three on their way measured 20 % SLOWER than one: the loop is not waiting for bytes.
template <bool PAIR, int GRP>
__device__ __forceinline__ bool produce(const ProducerArgs<PAIR>& a, int w8, int lane) {
    const int r = w8 * 16 + (lane & 15), p = lane >> 4;
    const size_t rb = (size_t)a.items.rb;
    uint4* slot = a.rawq + (size_t)((GRP * (PWARPS / 2) + w8) * 32 + lane) * (RING * 2);
    uint4* hslot = a.hq + (size_t)(GRP * TILE_M + r) * 4;
    uint4 cur_a, cur_b, hdr_a, hdr_b;
    int f_left = a.my_items, f_k = 0, f_c = GRP;  // fetch cursor: item (CTA-local index) and chunk
    int wr = 0, rd = 0;                           // ring positions of the next request and the next pick-up
    uint32_t f_hn = 0, r_hn = 0;                  // headers requested / read so far (slot = count & 1)
    const uint8_t* f_pa = nullptr;
    const uint8_t* f_pb = nullptr;
    auto f_open = [&]() {
        if (f_left > 0) {
            const Item it = a.items.get(f_k);
            f_pa = it.pa + (size_t)r * rb;
            f_pb = it.pb + (size_t)r * rb;
        }
    };
    auto fetch = [&]() {  // request the fetch cursor's chunk (and, with a block's first chunk of this group, its header)
        if (f_left > 0) {
            const int off = (f_c >> 2) * 144;
            if ((f_c & 3) == GRP) {
                if (p == 0) {
                    cp_async16(hslot + 2 * (f_hn & 1u), f_pa + off);
                    cp_async16(hslot + 2 * (f_hn & 1u) + 1, f_pb + off);
                }
                ++f_hn;
            }
            const int qoff = off + 16 + 32 * (f_c & 3) + 16 * p;
            cp_async16(slot + 2 * wr, f_pa + qoff);
            cp_async16(slot + 2 * wr + 1, f_pb + qoff);
            f_c += 2;
            if (f_c >= a.nchunks) {
                f_c = GRP;
                ++f_k;
                --f_left;
                f_open();
            }
        }
        cp_async_commit();  // also when nothing is left: the group count per chunk stays one
        if (++wr == RING) wr = 0;
    };
    auto take = [&]() {  // the oldest chunk on its way has landed: into registers, and its slot is free again
        cp_async_wait_group<RING - 2>();
        cur_a = slot[2 * rd];
        cur_b = slot[2 * rd + 1];
        if (++rd == RING) rd = 0;
    };
    f_open();
#pragma unroll
    for (int i = 0; i < RING - 1; ++i) fetch();
    bool ok = true;
    const int nch = a.nchunks + 2;
    int mblk = 0;  // running count of weight blocks: the scale ring's slot
    for (int k = 0; k < a.my_items && ok; ++k) {
        for (int blk = 0; blk < a.nblk && ok; ++blk, ++mblk) {
            const int sslot = mblk % SCL;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int j = GRP + 2 * i;  // chunk inside the block
                take();
                fetch();
                if (i == 0) {
                    // The header came with this chunk; the row's other lane sees it after the warp barrier, and both
                    // lanes have their copy before this slot's next header (two blocks on) is requested.
                    __syncwarp();
                    hdr_a = hslot[2 * (r_hn & 1u)];
                    hdr_b = hslot[2 * (r_hn & 1u) + 1];
                    ++r_hn;
                    __syncwarp();
                }
                const int g = k * nch + blk * 4 + j;
                const int st = g % STAGES;
                const uint32_t ph = (uint32_t)(g / STAGES) & 1u;
                if (ok && g >= STAGES) ok = mb_wait(&a.empty[st], ph ^ 1u, a.status, 2);
                if (ok) {
                    uint8_t* sa = a.smem + st * STAGE_BYTES;
                    decode_q4k_int(hdr_a, cur_a, j, p, sa, r);
                    decode_q4k_int(hdr_b, cur_b, j, p, sa + A_TILE, r);
                    if (j == 0 && p == 0) {  // the block's scales (the epilogue waits for sfull)
                        a.scl[(sslot * 2 + 0) * TILE_M + r] = __half2float(__ushort_as_half((unsigned short)(hdr_a.x & 0xFFFFu)));
                        a.scl[(sslot * 2 + 1) * TILE_M + r] = __half2float(__ushort_as_half((unsigned short)(hdr_b.x & 0xFFFFu)));
                    }
                    fence_async_smem();  // generic-proxy stores -> visible to the tensor core's async proxy
                    __syncwarp();
                    if (lane == 0) {
                        mb_arrive(&a.full[st]);
                        if (j == 0) mb_arrive(&a.sfull[sslot]);
                    }
                }
            }
        }
        if (!ok) break;
        {   // the offsets' stage of matrix GRP: hi tile in the first A slot, lo tile in the second.  The headers of
            // blocks 4p .. 4p+3 of the thread's row are read again (plain loads: they are in L2 since the item began).
            const Item it = a.items.get(k);
            const uint8_t* row = (GRP ? it.pb : it.pa) + (size_t)r * rb;
            uint4 hd[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
                hd[i] = 4 * p + i < a.nblk ? __ldg(reinterpret_cast<const uint4*>(row + (size_t)(4 * p + i) * 144)) : make_uint4(0u, 0u, 0u, 0u);
            const int g = k * nch + a.nchunks + GRP;
            const int st = g % STAGES;
            const uint32_t ph = (uint32_t)(g / STAGES) & 1u;
            if (g >= STAGES) ok = mb_wait(&a.empty[st], ph ^ 1u, a.status, 2);
            if (ok) {
                uint8_t* sa = a.smem + st * STAGE_BYTES;
                const uint32_t rowoff = (uint32_t)(r >> 3) * 1024u + (uint32_t)(r & 7) * 128u;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint4 hi = make_uint4(0u, 0u, 0u, 0u), lo = hi;
                    if (4 * p + i < a.nblk) decode_q4k_mins(hd[i], hi, lo);
                    const uint32_t col = ((uint32_t)((4 * p + i) ^ (r & 7))) << 4;
                    *reinterpret_cast<uint4*>(sa + rowoff + col) = hi;
                    *reinterpret_cast<uint4*>(sa + A_TILE + rowoff + col) = lo;
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mb_arrive(&a.full[st]);
            }
        }
    }
    cp_async_wait_all();
    return ok;
}

// fused (PAIR = false): seg[].wa / wb = gate / up, out = silu(g) * u as fp32 packed rows [rows][n_out].
// PAIR: seg[].wa only, two 128-row tiles per item, fp32 rows (or peer rows through row_dst).
template <bool PAIR>
__global__ void __launch_bounds__(NTHREADS, 1)
grouped_q4k_int_kernel(const SegDesc* __restrict__ seg, const int32_t* __restrict__ nseg_dev, int n_in, int n_out, int rb,
                       const __grid_constant__ Maps maps, const float* __restrict__ rowscale, float* __restrict__ out_f32,
                       int* status, float* const* __restrict__ row_dst) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint4* rawq = reinterpret_cast<uint4*>(smem + STAGES * STAGE_BYTES);
    uint4* hq = rawq + PWARPS * 32 * RING * 2;
    float* scl = reinterpret_cast<float*>(hq + 2 * TILE_M * 4);
    uint64_t* full = reinterpret_cast<uint64_t*>(scl + SCL * 2 * TILE_M);
    uint64_t* empty = full + STAGES;
    uint64_t* tfull = empty + STAGES;
    uint64_t* tfree = tfull + NB;
    uint64_t* sfull = tfree + NB;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sfull + SCL);
    int* tile_prefix = reinterpret_cast<int*>(tmem_slot + 4);         // [nseg + 1]
    Item* itab = reinterpret_cast<Item*>(tile_prefix + kMaxSeg + 1);  // [kLocalItems]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nchunks = n_in / BK, nblk = n_in / 256;
    const int nch = nchunks + 2;                    // + the two stages of the sub-block offsets
    const int kcs = (n_in / 32 + 15) / 16;          // K steps of an offsets' stage that hold sub-blocks
    const int row_tiles = n_out / (PAIR ? 2 * TILE_M : TILE_M);
    const int nseg = min(*nseg_dev, kMaxSeg);

    if (tid == 0) {
        for (int i = 0; i < STAGES; ++i) {
            mb_init(&full[i], PWARPS / 2 + 1);  // one producer group + the TMA thread's expect_tx arrival
            mb_init(&empty[i], 1);              // one tcgen05.commit
        }
        for (int i = 0; i < NB; ++i) {
            mb_init(&tfull[i], 1);
            mb_init(&tfree[i], EWARPS);
        }
        for (int i = 0; i < SCL; ++i) mb_init(&sfull[i], PWARPS / 2);
        fence_mbarrier_init();
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
    if (warp == W_MMA) tmem_alloc<NB * BUF_COLS>(tmem_slot);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int n_items = nseg > 0 ? tile_prefix[nseg] * row_tiles : 0;
    const int GR = gridDim.x;
    const int my_items = (int)blockIdx.x < n_items ? (n_items - (int)blockIdx.x + GR - 1) / GR : 0;
    if (tid < min(my_items, kLocalItems))
        itab[tid] = decode_item<PAIR>((int)blockIdx.x + tid * GR, row_tiles, rb, nseg, tile_prefix, seg);
    __syncthreads();
    const ItemTab<PAIR> items{itab, seg, tile_prefix, nseg, row_tiles, rb};
    bool ok = true;

    if (warp < PWARPS) {
        // ---------------- producers ----------------
        const ProducerArgs<PAIR> pa{items, smem, rawq, hq, scl, full, empty, sfull, status, my_items, nchunks, nblk};
        if (warp < PWARPS / 2) ok = produce<PAIR, 0>(pa, warp, lane);
        else ok = produce<PAIR, 1>(pa, warp - PWARPS / 2, lane);
    } else if (warp == W_TMA) {
        // ---------------- TMA: activation tiles (hi rows, then lo rows) ----------------
        int g = 0;
        for (int k = 0; k < my_items && ok; ++k) {
            const Item it = items.get(k);
            const int nsel = it.m_tile <= 16 ? 0 : 1, nte = 16 << nsel;
            for (int c = 0; c < nch; ++c, ++g) {
                const int st = g % STAGES;
                const uint32_t ph = (uint32_t)(g / STAGES) & 1u;
                if (g >= STAGES) ok = warp_all(mb_wait(&empty[st], ph ^ 1u, status, 4));
                if (!ok) break;
                uint8_t* sbp = smem + st * STAGE_BYTES + 2 * A_TILE;
                if (elect_one()) {
                    const int col = c < nchunks ? c * BK : n_in;  // the sub-block sums follow the row's n_in elements
                    mb_expect_tx(&full[st], (uint32_t)(2 * nte * BK * 2));
                    tma_load_2d(sbp, &maps.hi[nsel], col, it.prow, &full[st]);
                    tma_load_2d(sbp + nte * BK * 2, &maps.lo[nsel], col, it.prow, &full[st]);
                }
                __syncwarp();
            }
        }
    } else if (warp == W_MMA) {
        // ---------------- MMA issue ----------------
        const uint32_t smem_lo = desc_lo(s32(smem));
        constexpr uint32_t T = A_TILE >> 4;
        int g = 0, buf = 0;
        uint32_t blocks = 0;
        for (int k = 0; k < my_items && ok; ++k) {
            const Item it = items.get(k);
            const int nte = it.m_tile <= 16 ? 16 : 32;
            const uint32_t idesc = (1u << 4) | ((uint32_t)((2 * nte) >> 3) << 17) | ((uint32_t)(TILE_M >> 4) << 24);  // fp16 x fp16 -> fp32
            for (int c = 0; c < nch && ok; ++c, ++g) {
                const int st = g % STAGES;
                const uint32_t ph = (uint32_t)(g / STAGES) & 1u;
                ok = warp_all(mb_wait(&full[st], ph, status, 5));
                if (!ok) break;
                const bool first = c < nchunks ? (c & 3) == 0 : c == nchunks;
                const bool last = c < nchunks ? (c & 3) == 3 : c == nchunks + 1;
                if (first && blocks >= (uint32_t)NB) ok = warp_all(mb_wait(&tfree[buf], (blocks / NB - 1) & 1u, status, 6));
                if (!ok) break;
                tc_fence_after();
                if (elect_one()) {
                    const uint32_t a_lo = smem_lo + (uint32_t)(st * (STAGE_BYTES >> 4));
                    const uint32_t b_lo = a_lo + 2 * T;
                    const uint32_t d0 = tmem_base + (uint32_t)(buf * BUF_COLS);
                    if (c < nchunks) {
#pragma unroll
                        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                            for (int ks = 0; ks < BK / 16; ++ks)
                                mma_bf16(d0 + (uint32_t)(mt * 2 * NT), desc_of(a_lo + (uint32_t)mt * T + 2u * ks), desc_of(b_lo + 2u * ks),
                                         idesc, (first && ks == 0) ? 0u : 1u);
                    } else {
                        const uint32_t dm = d0 + (uint32_t)((c - nchunks) * 2 * NT);
                        for (int ks = 0; ks < kcs; ++ks) {
                            mma_bf16(dm, desc_of(a_lo + 2u * ks), desc_of(b_lo + 2u * ks), idesc, ks == 0 ? 0u : 1u);
                            mma_bf16(dm, desc_of(a_lo + T + 2u * ks), desc_of(b_lo + 2u * ks), idesc, 1u);
                        }
                    }
                    mma_commit(&empty[st]);
                    if (last) mma_commit(&tfull[buf]);
                }
                __syncwarp();
                if (last) {
                    if (++buf == NB) buf = 0;
                    ++blocks;
                }
            }
        }
    } else {
        // ---------------- epilogue: TMEM lane = weight row ----------------
        // A warp owns 32 weight rows (its TMEM lane quadrant) x 16 token columns (hsel) of both matrices.
        const int quad = warp & 3, hsel = (warp - PWARPS) >> 2;
        const int r = quad * 32 + lane;
        const uint32_t tlane = tmem_base + ((uint32_t)(quad * 32) << 16);
        int buf = 0, slot = 0;
        uint32_t pb = 0, ps = 0;
        for (int k = 0; k < my_items && ok; ++k) {
            const Item it = items.get(k);
            const int nte = it.m_tile <= 16 ? 16 : 32;
            const bool active = 16 * hsel < nte;
            float acc[2][16];
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[mt][j] = 0.f;
            for (int blk = 0; blk <= nblk; ++blk) {  // blk == nblk: the sub-block offsets, scale 1
                float s[2] = {1.f, 1.f};
                if (blk < nblk) {
                    ok = mb_wait(&sfull[slot], ps, status, 3);
                    if (!ok) break;
                    s[0] = scl[(slot * 2 + 0) * TILE_M + r];
                    s[1] = scl[(slot * 2 + 1) * TILE_M + r];
                    if (++slot == SCL) { slot = 0; ps ^= 1u; }
                }
                ok = mb_wait(&tfull[buf], pb, status, 3);
                if (!ok) break;
                tc_fence_after();
                if (active) {
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt) {
                        const uint32_t col = (uint32_t)(buf * BUF_COLS + mt * 2 * NT + 16 * hsel);
#pragma unroll
                        for (int part = 0; part < 2; ++part) {  // the products with the hi and with the lo rows
                            uint32_t v[16];
                            tmem_ld16(tlane + col + (uint32_t)(part * nte), v);
                            tmem_ld_wait();
                            if (mt == 1 && part == 1) {  // the buffer has been read: hand it back before the arithmetic
                                tc_fence_before();
                                __syncwarp();
                                if (lane == 0) mb_arrive(&tfree[buf]);
                            }
#pragma unroll
                            for (int j = 0; j < 16; ++j) acc[mt][j] = fmaf(s[mt], __uint_as_float(v[j]), acc[mt][j]);
                        }
                    }
                } else {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mb_arrive(&tfree[buf]);
                }
                if (++buf == NB) { buf = 0; pb ^= 1u; }
            }
            if (!ok) break;
            if (active) {
                const int t0 = 16 * hsel;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    if (t0 + j < it.m_tile) {
                        const float rs = rowscale[it.prow + t0 + j];  // the power of two the activation row was divided by
                        const float a0 = acc[0][j] * rs, a1 = acc[1][j] * rs;
                        if constexpr (!PAIR) {
                            out_f32[(size_t)(it.prow + t0 + j) * n_out + it.r0 + r] = swiglu_fast(a0, a1);
                        } else {
                            float* o = row_dst ? row_dst[it.prow + t0 + j] + it.r0 + r  // expert parallel: the owner's (token, slot) row
                                               : out_f32 + (size_t)(it.prow + t0 + j) * n_out + it.r0 + r;
                            o[0] = a0;
                            o[TILE_M] = a1;
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == W_MMA) {
        tc_fence_after();
        tmem_free<NB * BUF_COLS>(tmem_base);
    }
}

// Packed activation rows for the kernel above: row p of x (through row_token when given) as fp16 hi and lo of the row
// times a power of two (largest element in [256, 512)), the sums of its 32-element sub-blocks in columns K .. K + K/32
// of the same arrays, and the factor that undoes the scaling.  K % 256 == 0; row pitch of hi / lo = kp elements.
__global__ void __launch_bounds__(128)
rows_f16_kernel(const float* __restrict__ x, int ldx, const int32_t* __restrict__ row_token, int rows, int K, int kp,
                uint16_t* __restrict__ hi, uint16_t* __restrict__ lo, float* __restrict__ rowscale) {
    const int p = blockIdx.x;
    if (p >= rows) return;
    __shared__ float red[4];
    const float* xr = x + (size_t)(row_token ? row_token[p] : p) * ldx;
    const int tid = threadIdx.x, lane = tid & 31;
    float mx = 0.f;
    for (int i = tid * 2; i < K; i += 256) {
        const float2 v = *reinterpret_cast<const float2*>(xr + i);
        mx = fmaxf(mx, fmaxf(fabsf(v.x), fabsf(v.y)));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) red[tid >> 5] = mx;
    __syncthreads();
    mx = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    float up = 1.f, down = 1.f;
    if (mx > 0.f && mx <= 3.0e38f) {  // zero, infinite and NaN rows stay unscaled
        int e;
        (void)frexpf(mx, &e);         // mx = f * 2^e, f in [0.5, 1)
        e = max(e, -100);
        up = ldexpf(1.f, 9 - e);
        down = ldexpf(1.f, e - 9);
    }
    if (tid == 0) rowscale[p] = down;
    uint16_t* hr = hi + (size_t)p * kp;
    uint16_t* lr = lo + (size_t)p * kp;
    for (int i = tid * 2; i < K; i += 256) {  // a warp covers 64 consecutive elements: two sub-blocks
        const float2 v = *reinterpret_cast<const float2*>(xr + i);
        const float a = v.x * up, b = v.y * up;
        const __half2 h = __floats2half2_rn(a, b);
        const float2 hf = __half22float2(h);
        const __half2 l = __floats2half2_rn(a - hf.x, b - hf.y);
        *reinterpret_cast<__half2*>(hr + i) = h;
        *reinterpret_cast<__half2*>(lr + i) = l;
        float s = a + b;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if ((lane & 15) == 0) {
            const __half sh = __float2half_rn(s);
            hr[K + (i >> 5)] = __half_as_ushort(sh);
            lr[K + (i >> 5)] = __half_as_ushort(__float2half_rn(s - __half2float(sh)));
        }
    }
}

}  // namespace qi

bool q4k_int_handles(int n_in, int n_out, bool fused) {
    return n_in % 256 == 0 && n_in / 256 <= qi::kMaxBlocks && n_out % (fused ? qi::TILE_M : 2 * qi::TILE_M) == 0;
}

int launch_rows_f16(dnb_ctx* c, cudaStream_t st, const float* x, int ldx, const int32_t* row_token, int rows, int K,
                    uint16_t* hi, uint16_t* lo, float* rowscale, const char* name) {
    ProfScope prof_(c, st, name);
    qi::rows_f16_kernel<<<rows, 128, 0, st>>>(x, ldx, row_token, rows, K, K + kQ4kIntXcols, hi, lo, rowscale);
    c->launches++;
    DNB_CUDA(cudaGetLastError());
    return DNB_OK;
}

// fused: seg[].wa/wb = gate/up, out_f32 = silu(g) * u, fp32 packed rows; otherwise seg[].wa, fp32 rows or row_dst.
// maps: tensor maps of the fp16 hi / lo arrays made by launch_rows_f16 (row pitch n_in + kQ4kIntXcols).
int launch_grouped_q4k_int(dnb_ctx* c, cudaStream_t st, bool fused, const SegDesc* seg, const int32_t* nseg_dev, int nseg_max,
                           int n_in, int n_out, const UmmaMaps* maps, const float* rowscale, float* out_f32,
                           float* const* row_dst) {
    static_assert(sizeof(UmmaMaps) == sizeof(qi::Maps), "UmmaMaps must mirror qi::Maps");
    if (!q4k_int_handles(n_in, n_out, fused) || nseg_max > qi::kMaxSeg) return DNB_DECLINED;
    const int rb = n_in / 256 * 144;
    const qi::Maps& M = *reinterpret_cast<const qi::Maps*>(maps);
    const dim3 grid(c->sm_count);
    const size_t smem = (size_t)qi::STAGES * qi::STAGE_BYTES + (size_t)qi::PWARPS * 32 * qi::RING * 2 * 16 + 2 * qi::TILE_M * 4 * 16 +
                        (size_t)qi::SCL * 2 * qi::TILE_M * 4 + (2 * qi::STAGES + 2 * qi::NB + qi::SCL) * 8 + 16 +
                        (qi::kMaxSeg + 1) * 4 + qi::kLocalItems * sizeof(qi::Item) + 1024;
    if (fused) {
        static SmemGrant grant;
        DNB_CUDA(grant_smem(grant, c->device, qi::grouped_q4k_int_kernel<false>, smem));
        ProfScope prof_(c, st, "q4k_int_gate_up");
        qi::grouped_q4k_int_kernel<false><<<grid, qi::NTHREADS, smem, st>>>(seg, nseg_dev, n_in, n_out, rb, M, rowscale, out_f32,
                                                                           c->status, nullptr);
    } else {
        static SmemGrant grant;
        DNB_CUDA(grant_smem(grant, c->device, qi::grouped_q4k_int_kernel<true>, smem));
        ProfScope prof_(c, st, "q4k_int_down");
        qi::grouped_q4k_int_kernel<true><<<grid, qi::NTHREADS, smem, st>>>(seg, nseg_dev, n_in, n_out, rb, M, rowscale, out_f32,
                                                                          c->status, row_dst);
    }
    c->launches++;
    DNB_CUDA(cudaGetLastError());
    return DNB_OK;
}

}  // namespace dnb
