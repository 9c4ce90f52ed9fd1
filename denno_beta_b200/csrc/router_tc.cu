// Router logits of a prefill chunk on the tensor cores:  logits[t][i] = W_r[i] . x_t + bias[i]  for calls of 16 tokens or more.
//
// Reference forms of this contraction: kernels_elem.cu:1085 (dno_gemm_f32_mt, fp32 FMA) under cuda.rs:48695
// (pf_router_dev_topk); on the CPU linear_gguf.rs:836-964.  The routing decision is a comparison of these
// numbers, so the sum has to be as good as an fp32 sum.  Both operands are therefore split into THREE bf16 numbers
// (hi = the value rounded to bf16, mid = the remainder rounded, lo = what is left: 3 x 8 mantissa bits carry the 24 of
// an fp32 exactly) and six bf16 products are accumulated in fp32 by tcgen05.mma:
//     hi*hi                                         -> accumulator 0
//     hi*mid + mid*hi + hi*lo + lo*hi + mid*mid     -> accumulator 1   (the dropped terms are below 2^-24 relative)
// The small terms have their own accumulator so that they are not rounded at the magnitude of the large one.
//
// Shape.  D[128 expert rows][128 tokens] per CTA, K = n_embd split over gridDim.z CTAs (a 512 x 512 output has only 16
// tiles); the split is a constant of the model and a column's sum does not depend on what else is in its tile, so a token's
// logits do not depend on the size of its chunk (nor on how an expert-parallel group divides a chunk among its ranks).  The partial
// sums go to a scratch array; the top-k kernel (or router_reduce_kernel, where the logits themselves are wanted) adds them
// in ascending order and then the bias: deterministic, and the same bits either way.
// W_r is split once at registration; the chunk's rows are split by the RMSNorm kernel as it writes them (prep_kernel,
// moe_kernels.cu) or, for rows that come from elsewhere, by split3_kernel.  Warp 0 moves tiles by TMA (three A and
// three B tiles of 16 KB per 64-element K step, two stages), warp 1 issues the MMAs, warps 2-5 read the accumulators.
// Every wait is bounded; a wait that gives up sets *status and the CTA falls through to the teardown.
#include <cuda.h>
#include <cuda_bf16.h>

#include "dnb_common.cuh"
#include "tc_ptx.cuh"

namespace dnb {
namespace rt {
using namespace tcp;

constexpr int BK = 64;                 // K per stage: one 128-byte swizzle row of bf16
constexpr int TM = 128, TN = 128;      // expert rows x tokens per CTA
constexpr int TILE = TM * BK * 2;      // 16 KB
constexpr int STAGE_BYTES = 6 * TILE;  // W hi/mid/lo + x hi/mid/lo
constexpr int STAGES = 2;
constexpr int NTHREADS = 192;
constexpr int TM_COLS = 2 * TN;
constexpr uint32_t kIdesc = idesc_bf16(TM, TN);

struct Maps {
    CUtensorMap w[3];
    CUtensorMap x[3];
};

// n4 float4 groups of x -> three bf16 arrays of the same shape, `part` elements apart.
__global__ void __launch_bounds__(256)
split3_kernel(const float4* __restrict__ x, size_t n4, uint16_t* __restrict__ out, size_t part) {
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= n4) return;
    const float4 v = x[i];
    uint16_t h[4], m[4], l[4];
    split3_bf16(v.x, h[0], m[0], l[0]);
    split3_bf16(v.y, h[1], m[1], l[1]);
    split3_bf16(v.z, h[2], m[2], l[2]);
    split3_bf16(v.w, h[3], m[3], l[3]);
    uint2* o = reinterpret_cast<uint2*>(out) + i;
    const size_t p2 = part / 4;
    o[0] = make_uint2(h[0] | ((uint32_t)h[1] << 16), h[2] | ((uint32_t)h[3] << 16));
    o[p2] = make_uint2(m[0] | ((uint32_t)m[1] << 16), m[2] | ((uint32_t)m[3] << 16));
    o[2 * p2] = make_uint2(l[0] | ((uint32_t)l[1] << 16), l[2] | ((uint32_t)l[3] << 16));
}

// out: nsplit == 1: logits [nt][ne] (bias added here); else partial sums [nsplit][nt][ne].
__global__ void __launch_bounds__(NTHREADS, 1)
router_tc_kernel(const __grid_constant__ Maps maps, int nt, int ne, int kchunks, const float* __restrict__ bias,
                 float* __restrict__ out, int* status) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* tfull = empty + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tfull + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int m0 = blockIdx.x * TM, n0 = blockIdx.y * TN, split = blockIdx.z, nsplit = gridDim.z;
    const int c0 = split * kchunks;
    if (tid == 0) {
        for (int i = 0; i < STAGES; ++i) {
            mb_init(&full[i], 1);   // the TMA thread's expect_tx arrival
            mb_init(&empty[i], 1);  // one tcgen05.commit
        }
        mb_init(tfull, 1);
        fence_mbarrier_init();
    }
    if (warp == 1) tmem_alloc<TM_COLS>(tmem_slot);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;

    if (warp == 0) {
        // ---------------- TMA ----------------
        for (int c = 0; c < kchunks && ok; ++c) {
            const int st = c % STAGES, n = c / STAGES;
            if (n > 0) ok = warp_all(mb_wait(&empty[st], (uint32_t)(n - 1) & 1u, status, 25));
            if (!ok) break;
            if (elect_one()) {
                uint8_t* s = smem + st * STAGE_BYTES;
                mb_expect_tx(&full[st], (uint32_t)STAGE_BYTES);
#pragma unroll
                for (int p = 0; p < 3; ++p) {
                    tma_load_2d(s + p * TILE, &maps.w[p], (c0 + c) * BK, m0, &full[st]);
                    tma_load_2d(s + (3 + p) * TILE, &maps.x[p], (c0 + c) * BK, n0, &full[st]);
                }
            }
            __syncwarp();
        }
    } else if (warp == 1) {
        // ---------------- MMA issue ----------------
        const uint32_t smem_lo = desc_lo(s32(smem));
        for (int c = 0; c < kchunks && ok; ++c) {
            const int st = c % STAGES, n = c / STAGES;
            ok = warp_all(mb_wait(&full[st], (uint32_t)n & 1u, status, 25));
            if (!ok) break;
            tc_fence_after();
            if (elect_one()) {
                const uint32_t a0 = smem_lo + (uint32_t)(st * (STAGE_BYTES >> 4));
                constexpr uint32_t T = TILE >> 4;
                const uint32_t ah = a0, am = a0 + T, al = a0 + 2 * T, bh = a0 + 3 * T, bm = a0 + 4 * T, bl = a0 + 5 * T;
                const uint32_t d0 = tmem_base, d1 = tmem_base + TN;
#pragma unroll
                for (int ks = 0; ks < BK / 16; ++ks) {
                    const uint32_t ko = (uint32_t)ks * 2u;  // 16 bf16 = 32 bytes, >> 4
                    const uint32_t first = (c == 0 && ks == 0) ? 0u : 1u;
                    mma_bf16(d0, desc_of(ah + ko), desc_of(bh + ko), kIdesc, first);
                    mma_bf16(d1, desc_of(am + ko), desc_of(bm + ko), kIdesc, first);
                    mma_bf16(d1, desc_of(ah + ko), desc_of(bl + ko), kIdesc, 1u);
                    mma_bf16(d1, desc_of(al + ko), desc_of(bh + ko), kIdesc, 1u);
                    mma_bf16(d1, desc_of(ah + ko), desc_of(bm + ko), kIdesc, 1u);
                    mma_bf16(d1, desc_of(am + ko), desc_of(bh + ko), kIdesc, 1u);
                }
                mma_commit(&empty[st]);
                if (c == kchunks - 1) mma_commit(tfull);
            }
            __syncwarp();
        }
    } else {
        // ---------------- epilogue: TMEM lane = expert row, column = token ----------------
        const int quad = warp & 3;
        const int row = m0 + quad * 32 + lane;
        const uint32_t tlane = tmem_base + ((uint32_t)(quad * 32) << 16);
        ok = mb_wait(tfull, 0u, status, 25);
        if (ok) {
            tc_fence_after();
            const float b = (nsplit == 1 && bias && row < ne) ? bias[row] : 0.f;
            float* o = out + ((size_t)split * nt + n0) * ne + row;
            for (int g = 0; g < TN / 16 && n0 + 16 * g < nt; ++g) {
                uint32_t v0[16], v1[16];
                tmem_ld16(tlane + (uint32_t)(16 * g), v0);
                tmem_ld16(tlane + (uint32_t)(TN + 16 * g), v1);
                tmem_ld_wait();
                if (row < ne) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (n0 + 16 * g + j < nt) {
                            const float s = __uint_as_float(v0[j]) + __uint_as_float(v1[j]);
                            o[(size_t)(16 * g + j) * ne] = (nsplit == 1 && bias) ? s + b : s;
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_free<TM_COLS>(tmem_base);
    }
}

// logits = ((p[0] + p[1]) + p[2]) + ... (+ bias): ascending split index, one add at a time.
__global__ void __launch_bounds__(256)
router_reduce_kernel(const float4* __restrict__ part, int nsplit, size_t n4, int ne4, const float4* __restrict__ bias,
                     float4* __restrict__ logits) {
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= n4) return;
    float4 a = part[i];
    for (int s = 1; s < nsplit; ++s) {
        const float4 p = part[(size_t)s * n4 + i];
        a.x += p.x; a.y += p.y; a.z += p.z; a.w += p.w;
    }
    if (bias) {
        const float4 b = bias[i % (size_t)ne4];
        a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
    }
    logits[i] = a;
}

}  // namespace rt

static_assert(sizeof(RouterMaps) == 3 * sizeof(CUtensorMap), "RouterMaps must hold three tensor maps");

int router_tc_split(int e) {  // K splits: the largest divisor of the K steps that is at most kRouterSplitMax
    const int nchunks = e / rt::BK;
    for (int s = kRouterSplitMax; s > 1; --s)
        if (nchunks % s == 0) return s;
    return 1;
}

// Three bf16 parts of n fp32 values (n % 4 == 0), `part` elements apart.
static int launch_split3(dnb_ctx* c, cudaStream_t st, const float* x, size_t n, uint16_t* out, size_t part, const char* name) {
    ProfScope prof_(c, st, name);
    const size_t n4 = n / 4;
    rt::split3_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>(reinterpret_cast<const float4*>(x), n4, out, part);
    c->launches++;
    DNB_CUDA(cudaGetLastError());
    return DNB_OK;
}

// Once per layer, after the router matrix is resident: its three bf16 parts and their tensor maps.
int router_tc_prepare(dnb_ctx* c, Layer& L, int ne, int e) {
    L.router_tc = false;
    if (L.router_w3) cudaFree(L.router_w3);
    L.router_w3 = nullptr;
    if (e % rt::BK || ne % 4 || ne < rt::TM || !L.router_w) return DNB_OK;  // the fp32 kernel serves this shape
    const size_t part = (size_t)ne * e;
    DNB_CUDA(cudaMalloc((void**)&L.router_w3, 3 * part * sizeof(uint16_t)));
    int rc = launch_split3(c, c->stream, L.router_w, part, L.router_w3, part, "router_split_w");
    if (rc) return rc;
    DNB_CUDA(cudaStreamSynchronize(c->stream));
    CUtensorMap* m = reinterpret_cast<CUtensorMap*>(&L.rmaps);
    for (int p = 0; p < 3; ++p)
        if (tc_make_map(&m[p], L.router_w3 + p * part, (uint64_t)ne, (uint64_t)e, rt::TM) != DNB_OK) return DNB_OK;
    L.router_tc = true;
    return DNB_OK;
}

// The chunk-side buffers (inside the workspace, sized for `cap` tokens): x parts, partial sums, maps.
int router_tc_workspace(dnb_ctx* c, Workspace& w, int cap, int ne, int e) {
    w.router_tc = false;
    if (cap < kRouterTcMin || e % rt::BK || ne % 4) return DNB_OK;
    const size_t rows = (size_t)cap + rt::TN;  // a tile that starts near the end stays inside the allocation
    DNB_CUDA(cudaMalloc((void**)&w.x3, 3 * rows * e * sizeof(uint16_t)));
    DNB_CUDA(cudaMemset(w.x3, 0, 3 * rows * e * sizeof(uint16_t)));
    const int nsplit = router_tc_split(e);
    if (nsplit > 1) DNB_CUDA(cudaMalloc((void**)&w.rpart, (size_t)nsplit * cap * ne * sizeof(float)));
    CUtensorMap* m = reinterpret_cast<CUtensorMap*>(&w.xmaps);
    for (int p = 0; p < 3; ++p)
        if (tc_make_map(&m[p], w.x3 + p * rows * e, rows, (uint64_t)e, rt::TN) != DNB_OK) return DNB_OK;
    w.x3_part = rows * e;
    w.router_tc = true;
    return DNB_OK;
}

bool router_tc_eligible(const dnb_ctx* c, const Layer& L, int nt) {
    return c->router_tc && L.router_tc && c->ws.router_tc && nt >= kRouterTcMin && nt <= c->ws.nt_cap;
}

int launch_router_logits_tc(dnb_ctx* c, cudaStream_t st, const float* x, int nt, int e, const Layer& L, int ne, float* logits,
                            bool reduce, bool x_is_split) {
    Workspace& w = c->ws;
    if (!x_is_split) {  // else the kernel that produced x wrote its three parts into w.x3 as well
        int rc = launch_split3(c, st, x, (size_t)nt * e, w.x3, w.x3_part, "router_split_x");
        if (rc) return rc;
    }
    const int nsplit = router_tc_split(e);
    rt::Maps maps;
    memcpy(maps.w, &L.rmaps, sizeof(maps.w));
    memcpy(maps.x, &w.xmaps, sizeof(maps.x));
    const size_t smem = (size_t)rt::STAGES * rt::STAGE_BYTES + 64 + 1024;
    static SmemGrant grant;
    DNB_CUDA(grant_smem(grant, c->device, rt::router_tc_kernel, smem));
    const dim3 grid((ne + rt::TM - 1) / rt::TM, (nt + rt::TN - 1) / rt::TN, nsplit);
    {
        ProfScope prof_(c, st, "router_logits_tc");
        rt::router_tc_kernel<<<grid, rt::NTHREADS, smem, st>>>(maps, nt, ne, e / rt::BK / nsplit, L.router_bias,
                                                              nsplit == 1 ? logits : w.rpart, c->status);
        c->launches++;
        DNB_CUDA(cudaGetLastError());
    }
    if (nsplit > 1 && reduce) {
        ProfScope prof_(c, st, "router_reduce");
        const size_t n4 = (size_t)nt * ne / 4;
        rt::router_reduce_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>(
            reinterpret_cast<const float4*>(w.rpart), nsplit, n4, ne / 4, reinterpret_cast<const float4*>(L.router_bias),
            reinterpret_cast<float4*>(logits));
        c->launches++;
        DNB_CUDA(cudaGetLastError());
    }
    return DNB_OK;
}

}  // namespace dnb
