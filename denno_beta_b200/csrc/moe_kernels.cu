// The small kernels around the expert matmuls: RMSNorm, router logits, softmax +
// top-k + renorm, the expert-major routing tables, the weighted combine and the
// shared-expert gate coefficient.
#include "dnb_common.cuh"
#include "formats.cuh"
#include "tc_ptx.cuh"

namespace dnb {

// ---- RMSNorm (tensor.rs:1125-1135 rmsnorm_into) --------------------------------
// One CTA per token row.  ss is a fixed-order tree sum (the CPU sums left to
// right; the two differ by rounding only).  Also publishes the shared expert's
// two one-segment work descriptors for this call (m = nt, rows 0..nt-1).
// 1/rms of one row with a fixed summation order shared by every kernel that
// normalises: thread v of 128 adds x[v]^2, x[v+128]^2, ... (fma), a 32-lane xor
// tree per warp, then (w0 + w1) + (w2 + w3).
__device__ __forceinline__ float rms_inv_128(const float* __restrict__ xr, int e, float eps, float* red /*[4]*/) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < e; i += 128) ss = fmaf(xr[i], xr[i], ss);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    const float t = (red[0] + red[1]) + (red[2] + red[3]);
    return 1.0f / sqrtf(t / (float)e + eps);
}

__global__ void __launch_bounds__(128)
prep_kernel(const float* __restrict__ h, const float* __restrict__ w, float eps, int e, float* __restrict__ out,
            SegDesc* sh_gu, SegDesc* sh_dn, const uint8_t* sg, const uint8_t* su, const uint8_t* sdn, uint32_t nt,
            uint16_t* __restrict__ x3, size_t x3_part) {
    if (blockIdx.x == 0 && threadIdx.x == 0 && sh_gu) {
        sh_gu[0] = SegDesc{sg, su, nt, 0u};
        sh_dn[0] = SegDesc{sdn, nullptr, nt, 0u};
    }
    if (!w) return;
    __shared__ float red[4];
    const float* xr = h + (size_t)blockIdx.x * e;
    const float inv = rms_inv_128(xr, e, eps, red);
    float* o = out + (size_t)blockIdx.x * e;
    if (!x3) {
        for (int i = threadIdx.x; i < e; i += 128) o[i] = __fmul_rn(__fmul_rn(xr[i], inv), w[i]);
        return;
    }
    uint16_t* p3 = x3 + (size_t)blockIdx.x * e;  // the row again as three bf16 parts for the tensor-core router
    for (int i = threadIdx.x; i < e; i += 128) {
        const float v = __fmul_rn(__fmul_rn(xr[i], inv), w[i]);
        o[i] = v;
        uint16_t a, b, c;
        tcp::split3_bf16(v, a, b, c);
        p3[i] = a;
        p3[x3_part + i] = b;
        p3[2 * x3_part + i] = c;
    }
}

int launch_rmsnorm(dnb_ctx* c, cudaStream_t st, const float* h, const float* w, float eps, int nt, int e, float* out) {
    ProfScope prof_(c, st, "rmsnorm");
    prep_kernel<<<nt, 128, 0, st>>>(h, w, eps, e, out, nullptr, nullptr, nullptr, nullptr, nullptr, 0u, nullptr, 0);
    c->launches++;
    DNB_CUDA(cudaGetLastError());
    return DNB_OK;
}

int launch_prep(dnb_ctx* c, cudaStream_t st, const float* h, const float* w, float eps, int nt, int e, float* out,
                SegDesc* sh_gu, SegDesc* sh_dn, const uint8_t* sg, const uint8_t* su, const uint8_t* sdn, uint16_t* x3,
                size_t x3_part) {
    ProfScope prof_(c, st, "prep_rmsnorm");
    prep_kernel<<<nt, 128, 0, st>>>(h, w, eps, e, out, sh_gu, sh_dn, sg, su, sdn, (uint32_t)nt, w ? x3 : nullptr, x3_part);
    c->launches++;
    DNB_CUDA(cudaGetLastError());
    return DNB_OK;
}

// ---- router logits (linear_gguf.rs:836-964 f32 GEMV; kernels_elem.cu:948-1002,
// 1085 are the reference GPU forms) -------------------------------------------
// logits[t][i] = W_r[i] . x_t + bias[i].  One warp per expert row, the row read
// once as coalesced float4 and applied to up to RT tokens staged in shared memory.
constexpr int RT = 8;         // tokens per CTA (16 tokens x 16 warps measured slower: 69 us against 62 us per 512-token chunk)
constexpr int RROWS = 8;      // warps per CTA (they share the staged tokens).  Two alternating register sets for the weights
                              // instead of the copy below cost 30 registers and a CTA per SM: 76 us against 62 us.
constexpr int RW = 4;         // expert rows per warp
__global__ void __launch_bounds__(RROWS * 32)
router_logits_kernel(const float* __restrict__ x, int nt, int e, const float* __restrict__ w_r,
                     const float* __restrict__ bias, int ne, float* __restrict__ logits) {
    extern __shared__ __align__(16) float xs[];  // [RT][e]
    const int t0 = blockIdx.y * RT;
    const int ntok = min(RT, nt - t0);
    const int e4 = e >> 2;
    for (int i = threadIdx.x; i < ntok * e4; i += RROWS * 32)
        reinterpret_cast<float4*>(xs)[i] = reinterpret_cast<const float4*>(x + (size_t)t0 * e)[i];
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // a warp owns RW consecutive expert rows: every activation word read from shared
    // memory feeds RW rows (the kernel is otherwise bound by that shared-memory traffic)
    const int row0 = (blockIdx.x * RROWS + warp) * RW;
    if (row0 >= ne) return;
    const float4* wr[RW];
#pragma unroll
    for (int r = 0; r < RW; ++r) wr[r] = reinterpret_cast<const float4*>(w_r + (size_t)min(row0 + r, ne - 1) * e);
    float acc[RW][RT];
#pragma unroll
    for (int r = 0; r < RW; ++r)
#pragma unroll
        for (int t = 0; t < RT; ++t) acc[r][t] = 0.f;
    float4 wn[RW];  // the next step's weights: requested a step ahead (the rows come from L2)
#pragma unroll
    for (int r = 0; r < RW; ++r) wn[r] = lane < e4 ? __ldg(wr[r] + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
    for (int i = lane; i < e4; i += 32) {
        float4 wv[RW];
#pragma unroll
        for (int r = 0; r < RW; ++r) wv[r] = wn[r];
        if (i + 32 < e4) {
#pragma unroll
            for (int r = 0; r < RW; ++r) wn[r] = __ldg(wr[r] + i + 32);
        }
#pragma unroll
        for (int t = 0; t < RT; ++t) {
            if (t < ntok) {
                const float4 xv = reinterpret_cast<const float4*>(xs)[t * e4 + i];
#pragma unroll
                for (int r = 0; r < RW; ++r) {
                    acc[r][t] = fmaf(wv[r].x, xv.x, acc[r][t]);
                    acc[r][t] = fmaf(wv[r].y, xv.y, acc[r][t]);
                    acc[r][t] = fmaf(wv[r].z, xv.z, acc[r][t]);
                    acc[r][t] = fmaf(wv[r].w, xv.w, acc[r][t]);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < RW; ++r)
#pragma unroll
        for (int t = 0; t < RT; ++t) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc[r][t] += __shfl_xor_sync(0xffffffffu, acc[r][t], o);
        }
    if (lane == 0) {
#pragma unroll
        for (int r = 0; r < RW; ++r) {
            const int row = row0 + r;
            if (row < ne) {
                const float b = bias ? bias[row] : 0.f;
#pragma unroll
                for (int t = 0; t < RT; ++t)
                    if (t < ntok) logits[(size_t)(t0 + t) * ne + row] = bias ? acc[r][t] + b : acc[r][t];
            }
        }
    }
}

// Dynamic shared memory the router kernel has been allowed so far, per device (only raised).
static size_t g_router_smem[64] = {0};
static int router_smem_at_least(int device, size_t bytes) {
    if (device < 0 || device >= 64) return DNB_ERR_ARG;
    if (bytes <= g_router_smem[device]) return DNB_OK;
    if (bytes > 200 * 1024) {
        set_error("router: n_embd needs %zu B of shared memory", bytes);
        return DNB_DECLINED;
    }
    DNB_CUDA(cudaFuncSetAttribute(router_logits_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    g_router_smem[device] = bytes;
    return DNB_OK;
}

int launch_router_logits(dnb_ctx* c, cudaStream_t st, const float* x, int nt, int e, const float* w_r,
                         const float* bias, int ne, float* logits) {
    if (e % 4) {
        set_error("router: n_embd %d is not a multiple of 4", e);
        return DNB_DECLINED;
    }
    const size_t smem = (size_t)RT * e * sizeof(float);
    int rc = router_smem_at_least(c->device, smem);
    if (rc) return rc;
    dim3 grid((ne + RROWS * RW - 1) / (RROWS * RW), (nt + RT - 1) / RT);
    ProfScope prof_(c, st, "router_logits");
    router_logits_kernel<<<grid, RROWS * 32, smem, st>>>(x, nt, e, w_r, bias, ne, logits);
    c->launches++;
    DNB_CUDA(cudaGetLastError());
    return DNB_OK;
}

// ---- softmax + top-k + renorm (tensor.rs:1171-1183; moe.rs:188-279;
// qwen4exp.rs:11802-11821; GPU form kernels_router225.cu:36-171) -----------------
// One CTA of 128 threads per token, ne <= 1024, k <= 32.  Thread v holds entries
// v, v+128, ...  Everything that depends on evaluation order is fixed:
//   softmax denominator: per-thread partials in ascending index, then the tree
//     ((s[l]+s[l+64]) + (s[l+32]+s[l+96])) followed by a 32-lane xor tree;
//   selection: the CPU scan's rule (moe.rs:256-279) -- a strictly larger value
//     wins, ties go to the lower index, and a NaN is taken only when it is the
//     first unused entry;
//   renorm: the selected probabilities summed in ascending expert index, one add
//     at a time, as on the CPU.
// The same function serves the per-token kernel and the tail of the fused decode
// router, so a token gets the same routing bits on either path.
struct TopkSmem {
    uint32_t keys[1024];
    uint32_t cand_k[32];
    int cand_x[32];
    float red[128];
    float cand_v[4];
    int cand_i[4];
    int cand_first[4];
    float bcast;
    int ibcast;
    int sel[32];
    float pv[32];
    int ssel[32];
    float spv[32];
};

// nsplit > 1: logit_row points at the first of nsplit partial sums of the row, split_stride floats apart (the
// tensor-core router's K splits); they are added in ascending order, then the bias: the sequence of adds of
// router_reduce_kernel, so the logits are the same bits whether that kernel ran or not.
__device__ __forceinline__ void topk_block(const float* __restrict__ logit_row, int ne, int k, int norm_topk,
                                           TopkSmem& sm, int32_t* __restrict__ sels_out, float* __restrict__ wts_out,
                                           float* __restrict__ rowsum_out, int nsplit = 1, size_t split_stride = 0,
                                           const float* __restrict__ bias = nullptr) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float p[8];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int idx = j * 128 + tid;
        float v = -INFINITY;
        if (idx < ne) {
            v = __ldcg(logit_row + idx);  // L2: other CTAs of this launch may have written them
            if (nsplit > 1) {
                float part[kRouterSplitMax];  // all requested before the first is used
#pragma unroll
                for (int s = 1; s < kRouterSplitMax; ++s)
                    part[s] = s < nsplit ? __ldcg(logit_row + (size_t)s * split_stride + idx) : 0.f;
#pragma unroll
                for (int s = 1; s < kRouterSplitMax; ++s)
                    if (s < nsplit) v = __fadd_rn(v, part[s]);
                if (bias) v = __fadd_rn(v, bias[idx]);
            }
        }
        p[j] = v;
        mx = fmaxf(mx, p[j]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) sm.cand_v[warp] = mx;
    __syncthreads();
    mx = fmaxf(fmaxf(sm.cand_v[0], sm.cand_v[1]), fmaxf(sm.cand_v[2], sm.cand_v[3]));
    float part = 0.f;
    bool any_nan = false;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        if (j * 128 + tid < ne) {
            p[j] = expf(p[j] - mx);
            part += p[j];
            any_nan |= (p[j] != p[j]);
        }
    }
    sm.red[tid] = part;
    const int nan_block = __syncthreads_or(any_nan ? 1 : 0);
    if (warp == 0) {
        float a = (sm.red[lane] + sm.red[lane + 64]) + (sm.red[lane + 32] + sm.red[lane + 96]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
        if (lane == 0) sm.bcast = a;
    }
    __syncthreads();
    const float sum = sm.bcast;
    if (sum > 0.f) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (j * 128 + tid < ne) p[j] = p[j] / sum;  // (the -inf padding would take the division's slow path)
    }
    uint32_t used = 0;
    if (!nan_block) {
        // Fast path (no NaN anywhere): values map to order-preserving integer keys, the
        // warp finds the maximum and the lowest index holding it with two redux
        // instructions, and only the lane that owned the winner rescans its entries.
        // Same rule: larger value first, ties to the lower index.
        // The keys go to shared memory and warp 0 selects alone: no block barrier inside
        // the k rounds.
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t ub = __float_as_uint(p[j]);
            if (j * 128 + tid < ne) sm.keys[j * 128 + tid] = (ub & 0x80000000u) ? ~ub : (ub | 0x80000000u);
        }
        __syncthreads();
        if (warp == 0) {
            uint32_t key[32];  // entry 32 * m + lane
#pragma unroll
            for (int m = 0; m < 32; ++m) key[m] = (32 * m + lane < ne) ? sm.keys[32 * m + lane] : 0u;
            // a lane's best: maximum by a pairwise tree (depth 5, not a 32-step chain), then
            // the lowest entry holding it
            auto lane_best = [&](uint32_t& bk, int& bm) {
                uint32_t t[16];
#pragma unroll
                for (int m = 0; m < 16; ++m) t[m] = max(key[2 * m], key[2 * m + 1]);
#pragma unroll
                for (int w = 8; w > 0; w >>= 1)
#pragma unroll
                    for (int m = 0; m < w; ++m) t[m] = max(t[m], t[m + w]);
                bk = t[0];
                uint32_t hit = 0u;
#pragma unroll
                for (int m = 0; m < 32; ++m) hit |= (key[m] == bk ? 1u : 0u) << m;
                bm = bk ? __ffs((int)hit) - 1 : -1;
            };
            uint32_t bk;
            int bm;
            lane_best(bk, bm);
            // Shortcut without rounds.  t = the k-th largest of the 32 lane maxima: at least k
            // entries reach t, so every one of the top k does.  When no more than 32 entries
            // reach t (the usual case: a dozen or two), each goes to one lane, which ranks it
            // among the others by value and index; rank r < k is selection r.
            bool done = false;
            if (k <= 32) {
                int above = 0;
#pragma unroll
                for (int j = 0; j < 32; ++j) above += (__shfl_sync(0xffffffffu, bk, j) > bk) ? 1 : 0;
                const uint32_t t = __reduce_min_sync(0xffffffffu, above < k ? bk : 0xffffffffu);
                uint32_t surv = 0u;
#pragma unroll
                for (int m = 0; m < 32; ++m) surv |= ((key[m] >= t && key[m] != 0u) ? 1u : 0u) << m;
                const int mine = __popc(surv);
                int incl = mine;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int v = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) incl += v;
                }
                const int total = __shfl_sync(0xffffffffu, incl, 31);
                if (total <= 32 && total >= k) {
                    int pos = incl - mine;
                    while (surv) {
                        const int m = __ffs((int)surv) - 1;
                        surv &= surv - 1u;
                        sm.cand_k[pos] = sm.keys[32 * m + lane];
                        sm.cand_x[pos] = 32 * m + lane;
                        ++pos;
                    }
                    __syncwarp();
                    const uint32_t ck = lane < total ? sm.cand_k[lane] : 0u;
                    const int cx = lane < total ? sm.cand_x[lane] : 0x7fffffff;
                    int rank = 0;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const uint32_t ok = __shfl_sync(0xffffffffu, ck, j);
                        const int ox = __shfl_sync(0xffffffffu, cx, j);
                        rank += (ok > ck || (ok == ck && ox < cx)) ? 1 : 0;
                    }
                    if (lane < total && rank < k) {
                        sm.sel[rank] = cx;
                        sm.pv[rank] = __uint_as_float((ck & 0x80000000u) ? (ck ^ 0x80000000u) : ~ck);
                    }
                    done = true;
                }
            }
            for (int round = 0; round < k && !done; ++round) {
                const uint32_t wm = __reduce_max_sync(0xffffffffu, bk);
                const uint32_t wi = __reduce_min_sync(0xffffffffu, (bk == wm && bm >= 0) ? (uint32_t)(32 * bm + lane) : 0x7fffffffu);
                if (lane == 0) {
                    sm.sel[round] = (int)wi;
                    sm.pv[round] = __uint_as_float((wm & 0x80000000u) ? (wm ^ 0x80000000u) : ~wm);
                }
                if ((int)(wi & 31u) == lane) {  // the owner drops the winner and rescans its entries
#pragma unroll
                    for (int m = 0; m < 32; ++m)
                        if (m == (int)(wi >> 5)) key[m] = 0u;
                    lane_best(bk, bm);
                }
            }
        }
        __syncthreads();
    } else
    for (int round = 0; round < k; ++round) {
        float best = -INFINITY;
        int best_i = 0x7fffffff, first = 0x7fffffff;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int idx = j * 128 + tid;
            if (idx < ne && !((used >> j) & 1u)) {
                first = min(first, idx);
                const float v = p[j];
                if (v == v && (best_i == 0x7fffffff || v > best)) {
                    best = v;
                    best_i = idx;
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            first = min(first, __shfl_xor_sync(0xffffffffu, first, o));
            if (oi != 0x7fffffff && (best_i == 0x7fffffff || ov > best || (ov == best && oi < best_i))) {
                best = ov;
                best_i = oi;
            }
        }
        if (lane == 0) {
            sm.cand_v[warp] = best;
            sm.cand_i[warp] = best_i;
            sm.cand_first[warp] = first;
        }
        __syncthreads();
        float bv = sm.cand_v[0];
        int bi = sm.cand_i[0], gfirst = sm.cand_first[0];
#pragma unroll
        for (int w = 1; w < 4; ++w) {
            const float ov = sm.cand_v[w];
            const int oi = sm.cand_i[w];
            gfirst = min(gfirst, sm.cand_first[w]);
            if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) {
                bv = ov;
                bi = oi;
            }
        }
        int win = bi;
        if (nan_block) {  // rare path: does the scan's first unused entry hold a NaN?
            if ((gfirst & 127) == tid) {
                float fv = 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (j == (gfirst >> 7)) fv = p[j];
                sm.ibcast = (fv != fv) ? 1 : 0;
            }
            __syncthreads();
            if (sm.ibcast || bi == 0x7fffffff) win = gfirst;
        }
        if ((win & 127) == tid) {
            used |= 1u << (win >> 7);
            float wv = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (j == (win >> 7)) wv = p[j];
            sm.sel[round] = win;
            sm.pv[round] = wv;
        }
        __syncthreads();
    }
    if (tid < k) {
        const int mine = sm.sel[tid];
        int rank = 0;
        for (int j = 0; j < k; ++j) rank += (sm.sel[j] < mine) ? 1 : 0;
        sm.ssel[rank] = mine;
        sm.spv[rank] = sm.pv[tid];
    }
    __syncthreads();
    if (tid == 0) {
        float s = 0.f;
        for (int j = 0; j < k; ++j) s = __fadd_rn(s, sm.spv[j]);
        sm.bcast = s;
    }
    __syncthreads();
    const float s = sm.bcast;
    if (tid < k) {
        float w;
        if (!norm_topk) w = sm.spv[tid];
        else if (isfinite(s) && s > 0.f) w = sm.spv[tid] / s;
        else w = 1.0f / (float)k;
        sels_out[tid] = sm.ssel[tid];
        wts_out[tid] = w;
    }
    if (rowsum_out && tid == 0) *rowsum_out = s;
}

__global__ void __launch_bounds__(128)
topk_kernel(const float* __restrict__ logits, int nt, int ne, int k, int norm_topk, int32_t* __restrict__ sels,
            float* __restrict__ wts, float* __restrict__ rowsum, int nsplit, const float* __restrict__ bias) {
    __shared__ TopkSmem sm;
    const int t = blockIdx.x;
    topk_block(logits + (size_t)t * ne, ne, k, norm_topk, sm, sels + (size_t)t * k, wts + (size_t)t * k,
               rowsum ? rowsum + t : nullptr, nsplit, (size_t)nt * ne, bias);
}

// nsplit > 1: `logits` is [nsplit][nt][ne] partial sums (router_tc.cu), added here with `bias`.
int launch_topk(dnb_ctx* c, cudaStream_t st, const float* logits, int nt, int ne, int k, int norm_topk, int32_t* sels,
                float* wts, float* rowsum, int nsplit, const float* bias) {
    if (ne > 1024 || k > 32 || k < 1 || k > ne || nsplit < 1 || nsplit > kRouterSplitMax) {
        set_error("topk: n_expert %d / k %d / %d partial sums outside the kernel's range (<=1024, <=32, <=%d)", ne, k, nsplit,
                  kRouterSplitMax);
        return DNB_DECLINED;
    }
    ProfScope prof_(c, st, "router_topk");
    topk_kernel<<<nt, 128, 0, st>>>(logits, nt, ne, k, norm_topk, sels, wts, rowsum, nsplit, nsplit > 1 ? bias : nullptr);
    c->launches++;
    DNB_CUDA(cudaGetLastError());
    return DNB_OK;
}

// ---- fused decode router --------------------------------------------------------
// One token: RMSNorm + router logits + (in the CTA that finishes last) softmax,
// top-k, renorm and the work descriptors of the k routed experts and the shared
// expert.  Replaces four launches of the general path.  The "last CTA" is found
// with one atomic ticket; the values it reads were published with a fence before
// each ticket, and the arithmetic it runs has a fixed order, so the result does
// not depend on which CTA happens to be last.
//   seg_gu[s] / seg_dn[s], s < k: expert sels[s], one row each, packed row s
//   seg_gu[k] / seg_dn[k]: the shared expert (when given), packed row k
//   pos[s] = s, row_token[s] = 0
template <int NV>  // NV = n_embd / 128: float4 words of a router row per lane
__global__ void __launch_bounds__(128)
router_decode_kernel(const float* __restrict__ h, const float* __restrict__ norm_w, float eps, int e,
                     const float* __restrict__ w_r, const float* __restrict__ bias, int ne, int k, int norm_topk,
                     float* __restrict__ xn, float* __restrict__ logits, int32_t* __restrict__ sels,
                     float* __restrict__ wts, const uint8_t* gate, const uint8_t* up, const uint8_t* down, size_t eb_g,
                     size_t eb_u, size_t eb_d, const uint8_t* sg, const uint8_t* su, const uint8_t* sdn,
                     SegDesc* seg_gu, SegDesc* seg_dn, int32_t* row_token, int32_t* pos, int32_t* nseg,
                     unsigned int* ticket, float* __restrict__ xn_perm, int gate_type, int shard_first, int shard_count) {
    extern __shared__ __align__(16) float xs[];  // [e]
    __shared__ float red[4];
    __shared__ int is_last;
    __shared__ TopkSmem sm;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row = blockIdx.x * 4 + warp;
    // The router rows are constants of the layer: fetch this warp's row before
    // waiting for the kernel that produces h (it overlaps that kernel's tail).
    float4 wv[NV];
    if (row < ne) {
        const float4* wr = reinterpret_cast<const float4*>(w_r + (size_t)row * e);
#pragma unroll
        for (int j = 0; j < NV; ++j) wv[j] = __ldg(wr + lane + 32 * j);
    }
    float nw[NV];  // this thread's norm weights: layer constants as well
    if (norm_w) {
#pragma unroll
        for (int j = 0; j < NV; ++j) nw[j] = __ldg(norm_w + tid + 128 * j);
    }
    pdl_wait();
    pdl_launch_dependents();
    if (norm_w) {
        // rms_inv_128's arithmetic with the row read once and kept in registers
        float hv[NV];
#pragma unroll
        for (int j = 0; j < NV; ++j) hv[j] = h[tid + 128 * j];
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < NV; ++j) ss = fmaf(hv[j], hv[j], ss);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        const float inv = 1.0f / sqrtf(((red[0] + red[1]) + (red[2] + red[3])) / (float)e + eps);
#pragma unroll
        for (int j = 0; j < NV; ++j) xs[tid + 128 * j] = __fmul_rn(__fmul_rn(hv[j], inv), nw[j]);
    } else {
        for (int i = tid; i < e; i += 128) xs[i] = h[i];
    }
    __syncthreads();
    if (row < ne) {
        const float4* x4 = reinterpret_cast<const float4*>(xs);
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const float4 xv = x4[lane + 32 * j];
            acc = fmaf(wv[j].x, xv.x, acc);
            acc = fmaf(wv[j].y, xv.y, acc);
            acc = fmaf(wv[j].z, xv.z, acc);
            acc = fmaf(wv[j].w, xv.w, acc);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) logits[row] = bias ? acc + bias[row] : acc;
    }
    // Publish: the CTA's stores are ordered before the barrier, the ticket is taken with a
    // release-acquire atomic at device scope after it, and the last CTA's threads read the
    // logits after the barrier that follows the acquire -- no separate fences.
    __syncthreads();
    if (tid == 0) {
        unsigned int t;
        asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(t) : "l"(ticket) : "memory");
        is_last = (t == gridDim.x - 1) ? 1 : 0;
        if (is_last) *ticket = 0u;  // ready for the next launch
    }
    __syncthreads();
    // The normalised row for the next kernel, written only now: these 16 KB of stores are not what
    // the last CTA waits for, and in front of the ticket its release would have had to wait for them.
    if (blockIdx.x == 0 && xn)
        for (int i = tid; i < e; i += 128) xn[i] = xs[i];
    // every CTA holds the normalised row: the first kActRep each publish one copy in the
    // slot order of the gate/up format, for that kernel's CTAs to take with a bulk copy
    if (xn_perm && (int)blockIdx.x < kActRep) {
        float* o = xn_perm + (size_t)blockIdx.x * e;
        for (int i = tid; i < e; i += 128) o[slot_index(gate_type, i, e >> 5)] = xs[i];
    }
    if (!is_last) return;
    topk_block(logits, ne, k, norm_topk, sm, sels, wts, nullptr);
    __syncthreads();
    if (tid < k) {
        // Expert parallel: only experts [shard_first, shard_first + shard_count) are resident here (indexed from
        // 0 in the local tensors); the other slots become empty segments, which the GEMV kernels skip.
        const int li = sm.ssel[tid] - shard_first;
        const bool mine = li >= 0 && li < shard_count;
        const size_t ex = mine ? (size_t)li : 0;
        seg_gu[tid] = SegDesc{gate + ex * eb_g, up + ex * eb_u, mine ? 1u : 0u, (uint32_t)tid};
        seg_dn[tid] = SegDesc{down + ex * eb_d, nullptr, mine ? 1u : 0u, (uint32_t)tid};
        row_token[tid] = 0;
        pos[tid] = tid;
    }
    if (tid == 0) {
        if (sg) {
            seg_gu[k] = SegDesc{sg, su, 1u, (uint32_t)k};
            seg_dn[k] = SegDesc{sdn, nullptr, 1u, (uint32_t)k};
            row_token[k] = 0;
        }
        *nseg = k + (sg ? 1 : 0);
    }
}

static inline bool gridDim_ok(int ne) { return (ne + 3) / 4 >= kActRep; }  // one router CTA per replica

template <int NV>
static int launch_router_decode_t(dnb_ctx* c, cudaStream_t st, const float* h, const Model& M, const Layer& L,
                                  Workspace& w, bool fold_shared, unsigned int* ticket) {
    const size_t smem = (size_t)M.e * sizeof(float);
    // The same shared-memory carve-out as the fused gate/up + down kernel, so that this kernel's CTAs can
    // take their places beside that kernel's (an SM is not re-partitioned while CTAs run on it) and
    // fetch their router rows while it still computes.
    static SmemGrant carve;
    if (carve.got[c->device < 64 && c->device >= 0 ? c->device : 0] == 0) {
        DNB_CUDA(cudaFuncSetAttribute(router_decode_kernel<NV>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                      cudaSharedmemCarveoutMaxShared));
        carve.got[c->device < 64 && c->device >= 0 ? c->device : 0] = 1;
    }
    ProfScope prof_(c, st, "router_decode_fused");
    DNB_CUDA(launch_k(router_decode_kernel<NV>, dim3((M.ne + 3) / 4), dim3(128), smem, st, c->use_pdl, h,
                      (const float*)L.norm_w, M.eps, M.e, (const float*)L.router_w, (const float*)L.router_bias, M.ne, M.k,
                      M.norm_topk, w.xn, w.logits, w.sels, w.wts, (const uint8_t*)L.m[0].dev, (const uint8_t*)L.m[1].dev,
                      (const uint8_t*)L.m[2].dev, L.m[0].expert_bytes, L.m[1].expert_bytes, L.m[2].expert_bytes,
                      (const uint8_t*)(fold_shared ? L.m[3].dev : nullptr),
                      (const uint8_t*)(fold_shared ? L.m[4].dev : nullptr),
                      (const uint8_t*)(fold_shared ? L.m[5].dev : nullptr), w.seg_gu, w.seg_dn, w.row_token, w.pos,
                      w.nseg, ticket, (gridDim_ok(M.ne) ? w.xn_perm : nullptr), L.m[0].type, M.shard_first, M.shard_count));
    c->launches++;
    return DNB_OK;
}

int launch_router_decode(dnb_ctx* c, cudaStream_t st, const float* h, const Model& M, const Layer& L, Workspace& w,
                         bool fold_shared, unsigned int* ticket) {
    if (M.e % 128 || M.ne > 1024 || M.k > 32 || M.e > 8192) return DNB_DECLINED;
    switch (M.e / 128) {
        case 4: return launch_router_decode_t<4>(c, st, h, M, L, w, fold_shared, ticket);
        case 8: return launch_router_decode_t<8>(c, st, h, M, L, w, fold_shared, ticket);
        case 16: return launch_router_decode_t<16>(c, st, h, M, L, w, fold_shared, ticket);
        case 20: return launch_router_decode_t<20>(c, st, h, M, L, w, fold_shared, ticket);
        case 32: return launch_router_decode_t<32>(c, st, h, M, L, w, fold_shared, ticket);
        default: return DNB_DECLINED;
    }
}

// ---- router + top-k without any allocation -----------------------------------------
// The logits between the two router kernels normally live in the context's
// grow-only workspace, which is (re)allocated on demand.  Some callers must not
// allocate at all once they are running: a serving loop that has pinned its memory
// budget at start-up, a plugin host that forbids cudaMalloc on its inference thread
// (an allocation synchronises the whole device and stalls every other stream), or
// code between cudaStreamBeginCapture and EndCapture, where cudaMalloc is illegal.
// For them the same two kernels run with the logits in this fixed array, which every
// GPU that loads the library carries until the process exits (256 KiB).
constexpr int kStaticLogits = 65536;  // nt * n_expert must not exceed this
static __device__ __align__(256) float g_static_logits[kStaticLogits];
static float* g_static_logits_ptr[64] = {nullptr};  // device address of the array, per device

}  // namespace dnb

extern "C" int dnb_router_topk_static(dnb_ctx* c, int layer, const float* x_dev, int nt, int32_t* sels_dev,
                                      float* wts_dev, float* rowsum_dev) {
    using namespace dnb;
    if (!c || !x_dev || !sels_dev || !wts_dev || nt < 1) return DNB_ERR_ARG;
    const Model& M = c->model;
    if (layer < 0 || layer >= M.n_layer || !M.layers[layer].router_w) {
        set_error("router_topk_static: layer %d has no router", layer);
        return DNB_DECLINED;
    }
    if ((long)nt * M.ne > kStaticLogits) {
        set_error("router_topk_static: %d tokens x %d experts = %ld logits exceed the static scratch of %d; "
                  "use dnb_router_topk or split the call", nt, M.ne, (long)nt * M.ne, kStaticLogits);
        return DNB_ERR_ARG;
    }
    if (M.e % 4 || M.ne > 1024 || M.k > 32) {
        set_error("router_topk_static: shape outside the router kernels' range");
        return DNB_DECLINED;
    }
    if (M.k > M.ne) {
        set_error("router_topk_static: k %d exceeds the %d experts", M.k, M.ne);
        return DNB_DECLINED;
    }
    if (c->device < 0 || c->device >= 64) {
        set_error("router_topk_static: device index %d outside the per-device table (0..63)", c->device);
        return DNB_ERR_ARG;
    }
    // The calling thread's current device may be another context's: select this context's
    // device on every call (cheap, allocates nothing), not only during the set-up below.
    DNB_CUDA(cudaSetDevice(c->device));
    // One-time set-up per device: in host code the array's name is only a handle,
    // its device address has to be asked for (with that device current).
    const size_t smem = (size_t)RT * M.e * sizeof(float);
    if (!g_static_logits_ptr[c->device]) {
        float* p = nullptr;
        DNB_CUDA(cudaGetSymbolAddress((void**)&p, g_static_logits));
        const int rc = router_smem_at_least(c->device, 200 * 1024);  // the most the router kernel is ever given
        if (rc) return rc;
        g_static_logits_ptr[c->device] = p;
    }
    if (smem > g_router_smem[c->device]) {
        set_error("router_topk_static: n_embd %d needs more shared memory than the router kernel has", M.e);
        return DNB_DECLINED;
    }
    float* logits = g_static_logits_ptr[c->device];
    const Layer& L = M.layers[layer];
    const dim3 grid((M.ne + RROWS * RW - 1) / (RROWS * RW), (nt + RT - 1) / RT);
    // every logit of the [nt][n_expert] range is written before it is read, so the
    // previous call's contents need no clearing
    // (no per-kernel profiling scope here: it creates events on first use, which may allocate)
    router_logits_kernel<<<grid, RROWS * 32, smem, c->stream>>>(x_dev, nt, M.e, L.router_w, L.router_bias, M.ne, logits);
    topk_kernel<<<nt, 128, 0, c->stream>>>(logits, nt, M.ne, M.k, M.norm_topk, sels_dev, wts_dev, rowsum_dev, 1, nullptr);
    c->launches += 2;
    DNB_CUDA(cudaGetLastError());
    return DNB_OK;
}

namespace dnb {

// ---- routing tables -----------------------------------------------------------
// From sels[nt][k] build the expert-major packed row space the grouped matmuls
// work in (qwen4exp.rs:18172-18185 by_expert; moe_expert.rs:8309-8390
// build_grouped_batch; exp_pf.rs:23-31 rows[]): segments by token count descending
// (ties: expert ascending), the rows of an expert in ascending token order.
//   row_token[row] = token of the packed row       pos[t*k+slot] = packed row
//   seg_gu/seg_dn[i] = i-th active expert's matrices, m and first row; *nseg
// A grid of CTAs with RTE experts each, one per warp, dealt round-robin (expert = CTA + warp * grid: under a
// skewed router the hot experts are neighbours and would otherwise share a CTA).  Every CTA counts all
// experts and keeps, for its own, a bit per token; everything is integer work on the whole of sels, so the
// result does not depend on timing.  Phase 2: a warp ranks its expert among all (its lanes split the other
// experts), writes the two segment descriptors, scans the popcounts of its token words and lists the tokens.
// Phase 3: all threads walk sels again; a pair (token, slot) of one of this CTA's experts gets
// first row + tokens of the expert below this one.
constexpr int RTE = 8;  // experts per CTA of the routing-table kernel = warps

__global__ void __launch_bounds__(RTE * 32)
route_tables_kernel(const int32_t* __restrict__ sels, int nt, int k, int ne, const uint8_t* gate, const uint8_t* up,
                    const uint8_t* down, size_t eb_g, size_t eb_u, size_t eb_d, const uint8_t* sg, const uint8_t* su,
                    const uint8_t* sdn, SegDesc* seg_gu, SegDesc* seg_dn, int32_t* row_token, int32_t* pos,
                    int32_t* nseg, int32_t* counts_out) {
    extern __shared__ uint32_t sm[];
    const int words = (nt + 31) >> 5;
    uint32_t* bits = sm;                         // [RTE][words]: tokens of this CTA's experts
    int* before = (int*)(bits + RTE * words);    // [RTE][words]: tokens of the expert in the words below
    int* counts = before + RTE * words;          // [ne]
    __shared__ int first_row[RTE];
    __shared__ int red[RTE];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = gridDim.x, me = blockIdx.x;
    // Divisions by k and by the grid size as multiply-high with ceil(2^32 / d): exact while the dividend times d stays
    // below 2^32 (pairs: nt * k * k, experts: ne * G), which the launcher checks.  (As plain divisions they were most of
    // the kernel's instructions.)
    // A divisor of 1 has no 32-bit reciprocal: div_k / div_g pass the dividend through.
    const uint32_t rk = k > 1 ? (uint32_t)((0x100000000ull + (uint32_t)k - 1) / (uint32_t)k) : 0u;
    const uint32_t rg = G > 1 ? (uint32_t)((0x100000000ull + (uint32_t)G - 1) / (uint32_t)G) : 0u;
    auto div_k = [&](int x) { return k > 1 ? (int)__umulhi((uint32_t)x, rk) : x; };
    auto div_g = [&](int x) { return G > 1 ? (int)__umulhi((uint32_t)x, rg) : x; };
    for (int i = tid; i < RTE * words; i += RTE * 32) bits[i] = 0;
    for (int i = tid; i < ne; i += RTE * 32) counts[i] = 0;
    __syncthreads();
    constexpr int RTB = 8;  // selections a thread requests before it uses the first (the loop is bound by their latency)
    for (int i0 = tid; i0 < nt * k; i0 += RTE * 32 * RTB) {
        int ev[RTB];
#pragma unroll
        for (int u = 0; u < RTB; ++u) {
            const int i = i0 + u * RTE * 32;
            ev[u] = i < nt * k ? sels[i] : -1;
        }
#pragma unroll
        for (int u = 0; u < RTB; ++u) {
            const int e = ev[u];
            if (e >= 0 && e < ne) {
                atomicAdd(&counts[e], 1);  // integer sums: the value does not depend on the order of the adds
                const int j = div_g(e);  // e / G
                if (e - j * G == me) {
                    const int t = div_k(i0 + u * RTE * 32);  // pair index / k
                    atomicOr(&bits[j * words + (t >> 5)], 1u << (t & 31));
                }
            }
        }
    }
    __syncthreads();
    if (me == 0) {
        // number of active experts; the shared expert's segment and identity rows
        int part = 0;
        for (int i = tid; i < ne; i += RTE * 32) part += counts[i] > 0 ? 1 : 0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
        if (lane == 0) red[warp] = part;
        __syncthreads();
        if (tid == 0) {
            int n_active = 0;
            for (int w = 0; w < RTE; ++w) n_active += red[w];
            if (sg) {
                seg_gu[n_active] = SegDesc{sg, su, (uint32_t)nt, (uint32_t)(nt * k)};
                seg_dn[n_active] = SegDesc{sdn, nullptr, (uint32_t)nt, (uint32_t)(nt * k)};
                n_active++;
            }
            *nseg = n_active;
        }
        if (sg)
            for (int t = tid; t < nt; t += RTE * 32) row_token[nt * k + t] = t;
        if (counts_out)
            for (int i = tid; i < ne; i += RTE * 32) counts_out[i] = counts[i];
    }
    // Segment order: token count descending, ties by ascending expert index (moe_expert.rs:8344).
    const int e = me + warp * G;
    const int c = e < ne ? counts[e] : 0;
    if (c > 0) {  // uniform across the warp
        int rank = 0, row = 0;
        for (int o = lane; o < ne; o += 32) {
            const int co = counts[o];
            if (co > c || (co == c && o < e)) {
                rank++;
                row += co;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            rank += __shfl_xor_sync(0xffffffffu, rank, o);
            row += __shfl_xor_sync(0xffffffffu, row, o);
        }
        if (lane == 0) {
            seg_gu[rank] = SegDesc{gate + (size_t)e * eb_g, up + (size_t)e * eb_u, (uint32_t)c, (uint32_t)row};
            seg_dn[rank] = SegDesc{down + (size_t)e * eb_d, nullptr, (uint32_t)c, (uint32_t)row};
            first_row[warp] = row;
        }
        int run = 0;  // tokens of the expert in the words before this round of 32
        for (int g0 = 0; g0 < words; g0 += 32) {
            const int g = g0 + lane;
            uint32_t w = g < words ? bits[warp * words + g] : 0u;
            const int n = __popc(w);
            int incl = n;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int o = __shfl_up_sync(0xffffffffu, incl, d);
                if (lane >= d) incl += o;
            }
            int at = run + incl - n;
            if (g < words) before[warp * words + g] = at;
            while (w) {  // ascending tokens
                const int b = __ffs(w) - 1;
                w &= w - 1;
                row_token[row + at++] = g * 32 + b;
            }
            run += __shfl_sync(0xffffffffu, incl, 31);
        }
    }
    __syncthreads();
    for (int i0 = tid; i0 < nt * k; i0 += RTE * 32 * RTB) {
        int ev[RTB];
#pragma unroll
        for (int u = 0; u < RTB; ++u) {
            const int i = i0 + u * RTE * 32;
            ev[u] = i < nt * k ? sels[i] : -1;
        }
#pragma unroll
        for (int u = 0; u < RTB; ++u) {
            const int ex = ev[u], i = i0 + u * RTE * 32;
            const int j = div_g(max(ex, 0));
            if (ex >= 0 && ex < ne && ex - j * G == me) {
                const int t = div_k(i);
                const uint32_t w = bits[j * words + (t >> 5)];
                pos[i] = first_row[j] + before[j * words + (t >> 5)] + __popc(w & ((1u << (t & 31)) - 1u));
            }
        }
    }
}

int launch_route_tables(dnb_ctx* c, cudaStream_t st, const int32_t* sels, int nt, int k, int ne, const Layer& L,
                        Workspace& ws, bool fold_shared) {
    const int words = (nt + 31) >> 5;
    const size_t smem = ((size_t)2 * RTE * words + (size_t)ne) * 4;
    if (smem > 200 * 1024 || (uint64_t)nt * k * k >= (1ull << 32) || (uint64_t)ne * ((ne + RTE - 1) / RTE) >= (1ull << 32)) {
        set_error("route tables: %d tokens x %d experts exceeds the kernel's limits", nt, ne);
        return DNB_DECLINED;
    }
    static SmemGrant grant;
    DNB_CUDA(grant_smem(grant, c->device, route_tables_kernel, smem));
    ProfScope prof_(c, st, "route_tables");
    route_tables_kernel<<<(ne + RTE - 1) / RTE, RTE * 32, smem, st>>>(
        sels, nt, k, ne, L.m[0].dev, L.m[1].dev, L.m[2].dev, L.m[0].expert_bytes, L.m[1].expert_bytes,
        L.m[2].expert_bytes, fold_shared ? L.m[3].dev : nullptr, fold_shared ? L.m[4].dev : nullptr,
        fold_shared ? L.m[5].dev : nullptr, ws.seg_gu, ws.seg_dn, ws.row_token, ws.pos, ws.nseg, ws.counts);
    c->launches++;
    DNB_CUDA(cudaGetLastError());
    return DNB_OK;
}

// ---- segment tables of a decode batch --------------------------------------------------
// A few tokens (continuous batching): every (token, slot) pair is its own one-row segment,
// token-major, the shared expert as slot k -- the layout the one-token decode kernels work
// on, repeated per token.  One warp per token.
__global__ void decode_batch_tables_kernel(const int32_t* __restrict__ sels, int nt, int k, const uint8_t* gate,
                                           const uint8_t* up, const uint8_t* down, size_t eb_g, size_t eb_u, size_t eb_d,
                                           const uint8_t* sg, const uint8_t* su, const uint8_t* sdn, SegDesc* seg_gu,
                                           SegDesc* seg_dn, int32_t* row_token) {
    const int t = blockIdx.x, s = threadIdx.x, per = k + (sg ? 1 : 0);
    if (t >= nt || s >= per) return;
    const uint32_t row = (uint32_t)(t * per + s);
    if (s < k) {
        const int ex = sels[(size_t)t * k + s];
        seg_gu[row] = SegDesc{gate + (size_t)ex * eb_g, up + (size_t)ex * eb_u, 1u, row};
        seg_dn[row] = SegDesc{down + (size_t)ex * eb_d, nullptr, 1u, row};
    } else {
        seg_gu[row] = SegDesc{sg, su, 1u, row};
        seg_dn[row] = SegDesc{sdn, nullptr, 1u, row};
    }
    row_token[row] = t;
}

int launch_decode_batch_tables(dnb_ctx* c, cudaStream_t st, const int32_t* sels, int nt, int k, const Layer& L,
                               Workspace& ws, bool fold_shared) {
    ProfScope prof_(c, st, "decode_batch_tables");
    decode_batch_tables_kernel<<<nt, 64, 0, st>>>(
        sels, nt, k, (const uint8_t*)L.m[0].dev, (const uint8_t*)L.m[1].dev, (const uint8_t*)L.m[2].dev, L.m[0].expert_bytes,
        L.m[1].expert_bytes, L.m[2].expert_bytes, (const uint8_t*)(fold_shared ? L.m[3].dev : nullptr),
        (const uint8_t*)(fold_shared ? L.m[4].dev : nullptr), (const uint8_t*)(fold_shared ? L.m[5].dev : nullptr), ws.seg_gu,
        ws.seg_dn, ws.row_token);
    c->launches++;
    DNB_CUDA(cudaGetLastError());
    return DNB_OK;
}

// ---- weighted combine (kernels_dec_epi.cu:28-46 dno_dec_exp_sum;
// moe_grouped_gpu.rs:540-565 scatter; qwen4exp.rs:12126-12216) --------------------
// out[t][j] = sum over slots in ascending order of w[t][s] * h[pos[t][s]][j]
// (separate multiply and add, as on the CPU), then + coef * sh[t][j].
__global__ void __launch_bounds__(256)
combine_kernel(const float* __restrict__ hrow, const int32_t* __restrict__ pos, const float* __restrict__ wts, int k,
               int e, const float* __restrict__ sh, const float* __restrict__ shcoef, float* __restrict__ out) {
    const int t = blockIdx.x;
    __shared__ int32_t prow[32];
    __shared__ float pw[32];
    if (threadIdx.x < k) {  // pos == null: row t*k+s; wts == null: weight 1 (x * 1.0f is exact)
        prow[threadIdx.x] = pos ? pos[(size_t)t * k + threadIdx.x] : t * k + (int)threadIdx.x;
        pw[threadIdx.x] = wts ? wts[(size_t)t * k + threadIdx.x] : 1.0f;
    }
    __syncthreads();
    if ((e & 3) == 0) {
        // four columns per thread; the rows of up to eight slots are requested before the
        // first is used (the sum itself stays one slot after the other, ascending)
        for (int j = threadIdx.x * 4; j < e; j += 1024) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s0 = 0; s0 < k; s0 += 8) {
                float4 v[8];
#pragma unroll
                for (int q = 0; q < 8; ++q)
                    if (s0 + q < k) v[q] = *reinterpret_cast<const float4*>(hrow + (size_t)prow[s0 + q] * e + j);
#pragma unroll
                for (int q = 0; q < 8; ++q)
                    if (s0 + q < k) {
                        const float w = pw[s0 + q];
                        acc.x = __fadd_rn(acc.x, __fmul_rn(w, v[q].x));
                        acc.y = __fadd_rn(acc.y, __fmul_rn(w, v[q].y));
                        acc.z = __fadd_rn(acc.z, __fmul_rn(w, v[q].z));
                        acc.w = __fadd_rn(acc.w, __fmul_rn(w, v[q].w));
                    }
            }
            if (sh) {
                const float4 v = *reinterpret_cast<const float4*>(sh + (size_t)t * e + j);
                if (shcoef) {
                    const float c = shcoef[t];
                    acc.x = __fadd_rn(acc.x, __fmul_rn(v.x, c));
                    acc.y = __fadd_rn(acc.y, __fmul_rn(v.y, c));
                    acc.z = __fadd_rn(acc.z, __fmul_rn(v.z, c));
                    acc.w = __fadd_rn(acc.w, __fmul_rn(v.w, c));
                } else {
                    acc.x = __fadd_rn(acc.x, v.x);
                    acc.y = __fadd_rn(acc.y, v.y);
                    acc.z = __fadd_rn(acc.z, v.z);
                    acc.w = __fadd_rn(acc.w, v.w);
                }
            }
            *reinterpret_cast<float4*>(out + (size_t)t * e + j) = acc;
        }
        return;
    }
    for (int j = threadIdx.x; j < e; j += 256) {
        float acc = 0.f;
        for (int s = 0; s < k; ++s) acc = __fadd_rn(acc, __fmul_rn(pw[s], hrow[(size_t)prow[s] * e + j]));
        if (sh) {
            const float v = sh[(size_t)t * e + j];
            acc = __fadd_rn(acc, shcoef ? __fmul_rn(v, shcoef[t]) : v);
        }
        out[(size_t)t * e + j] = acc;
    }
}

int launch_combine(dnb_ctx* c, cudaStream_t st, const float* hrow, const int32_t* pos, const float* wts, int nt,
                   int k, int e, const float* sh, const float* shcoef, float* out) {
    ProfScope prof_(c, st, "combine");
    combine_kernel<<<nt, 256, 0, st>>>(hrow, pos, wts, k, e, sh, shcoef, out);
    c->launches++;
    DNB_CUDA(cudaGetLastError());
    return DNB_OK;
}

// coef[t] = sigmoid(row . x_t)   (hyper.rs:112-114; qwen4exp.rs:12388-12395)
__global__ void __launch_bounds__(128)
shared_coef_kernel(const float* __restrict__ x, const float* __restrict__ row, int nt, int e, float* __restrict__ coef) {
    const int t = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= nt) return;
    float acc = 0.f;
    for (int i = lane; i < e; i += 32) acc = fmaf(row[i], x[(size_t)t * e + i], acc);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) coef[t] = 1.0f / (1.0f + expf(-acc));
}

int launch_shared_coef(dnb_ctx* c, cudaStream_t st, const float* x, const float* row, int nt, int e, float* coef) {
    ProfScope prof_(c, st, "shared_coef");
    shared_coef_kernel<<<(nt + 3) / 4, 128, 0, st>>>(x, row, nt, e, coef);
    c->launches++;
    DNB_CUDA(cudaGetLastError());
    return DNB_OK;
}

// residual: h += delta
__global__ void add_inplace_kernel(float* __restrict__ h, const float* __restrict__ d, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) h[i] = __fadd_rn(h[i], d[i]);
}

int launch_add_inplace(dnb_ctx* c, cudaStream_t st, float* h, const float* d, size_t n) {
    ProfScope prof_(c, st, "residual_add");
    add_inplace_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(h, d, n);
    c->launches++;
    DNB_CUDA(cudaGetLastError());
    return DNB_OK;
}

// A few token rows from the caller's pinned host buffer into HBM, as a kernel instead of a copy
// node: the router kernel behind it is chained with programmatic dependent launch, so its
// prologue (router rows and norm weights into registers) runs while these loads cross PCIe; a
// copy node would hold the whole router launch back until the copy has ended.
__global__ void __launch_bounds__(512) stage_in_kernel(const float4* __restrict__ src, float4* __restrict__ dst, int n4) {
    pdl_launch_dependents();
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += gridDim.x * blockDim.x) dst[i] = src[i];
}

int launch_stage_in(dnb_ctx* c, cudaStream_t st, const float* host_pinned, float* dst, size_t n) {
    if (n % 4 || n / 4 > (1u << 20)) return DNB_DECLINED;
    const int n4 = (int)(n / 4);
    ProfScope prof_(c, st, "stage_in");
    DNB_CUDA(launch_k(stage_in_kernel, dim3((n4 + 511) / 512), dim3(512), 0, st, c->use_pdl,
                      reinterpret_cast<const float4*>(host_pinned), reinterpret_cast<float4*>(dst), n4));
    c->launches++;
    return DNB_OK;
}

}  // namespace dnb
