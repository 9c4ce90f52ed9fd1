// Decode GEMV (one token per segment), staged by the bulk-copy engine.
//
// The decode matmuls are tiny for a B200: 4-9 MB per launch, i.e. 30-60 KB per SM.
// What bounds them is not bandwidth but how soon every byte is in flight.  Here a
// warp owns a small group of consecutive rows (one contiguous byte range of the
// expert matrix, a multiple of 16 bytes) and its lane 0 issues ONE cp.async.bulk
// for it (two when gate and up are fused) the moment the kernel starts, completing
// on the warp's own mbarrier.  No thread spends instructions on the copy and no
// CTA-wide barrier stands between the copy and the math: a warp waits only for its
// own rows.  The grid is sized so that every CTA is resident at once, so the whole
// launch's weight bytes are requested within the first microsecond.
//
// The math is the register decode of formats.cuh (lanes split a row into
// 32-element units, fixed xor-shuffle tree), so the bits are identical run to run.
// Reference kernels of this role: kernels_seg_k.cu:201-241, kernels_exp_iq_v2.cu:
// 259-319 (one warp per row, plain loads).
#include "dnb_common.cuh"
#include "formats.cuh"
#include "bulk.cuh"
#include "dnb_iq_tables.h"

namespace dnb {

// The IQ3_XXS codebook in the replicated layout of IqLut, ready to be bulk-copied into a
// CTA's shared memory (a constant of the library: requested before any wait on other kernels).
__device__ __align__(16) uint32_t g_grid3xxs_rep[256 * kLutRep];
static bool g_tables_b[64] = {false};

static int upload_tables_b(int device) {
    if (device < 0 || device >= 64) return DNB_ERR_ARG;
    if (g_tables_b[device]) return DNB_OK;
    static uint32_t rep[256 * kLutRep];
    for (int i = 0; i < 256 * kLutRep; ++i) rep[i] = dnb_iq3xxs_grid[i / kLutRep];
    DNB_CUDA(cudaMemcpyToSymbol(g_grid3xxs_rep, rep, sizeof(rep)));
    g_tables_b[device] = true;
    return DNB_OK;
}

__device__ __forceinline__ float silu_b(float v) { return v / (1.0f + expf(-v)); }

constexpr int kWarps = 8;
constexpr int kMaxRounds = 4;  // row rounds per warp in the decode GEMV

// Stage n_in floats of x into slot order: xs4[k * nunits + u] (float4), see formats.cuh.
// The loads of a batch of eight are all issued before the first store, so a thread waits
// for memory once per batch, not once per element.
template <int T>
__device__ __forceinline__ void stage_x(float* xs, const float* xr, int n_in, int nunits, int tid, int nthr) {
    for (int i0 = tid; i0 < n_in; i0 += 8 * nthr) {
        float v[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const int i = i0 + q * nthr;
            v[q] = i < n_in ? xr[i] : 0.f;
        }
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const int i = i0 + q * nthr;
            if (i < n_in) {
                int u, sl;
                slot_of<T>(i, u, sl);
                xs[((((sl >> 2)) * nunits + u) << 2) + (sl & 3)] = v[q];
            }
        }
    }
}

// nseg activation vectors of n_in floats each, stored back to back at `act`, staged to
// nseg slot-ordered vectors at `xs` in one flat pass.
template <int T>
__device__ __forceinline__ void stage_x_multi(float* xs, const float* act, int n_in, int nunits, int nseg, int tid,
                                              int nthr) {
    const int total = nseg * n_in;
    for (int i0 = tid; i0 < total; i0 += 8 * nthr) {
        float v[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const int i = i0 + q * nthr;
            v[q] = i < total ? act[i] : 0.f;
        }
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const int i = i0 + q * nthr;
            if (i < total) {
                const int sg = i / n_in, ii = i - sg * n_in;
                int u, sl;
                slot_of<T>(ii, u, sl);
                xs[sg * n_in + ((((sl >> 2)) * nunits + u) << 2) + (sl & 3)] = v[q];
            }
        }
    }
}

// grid.x CTAs of 8 warps; warp index wi = blockIdx.x*8 + warp -> (segment wi / gps, row group wi % gps).
// Dynamic shared memory: [8 mbarriers | pad to 128][IqLut][8 x item bytes (x2 fused)][x]
template <int T, bool FUSED, int LPR, bool XSHARED, int KR /* row rounds per warp this instance can hold: 1 or kMaxRounds */>
__global__ void __launch_bounds__(kWarps * 32, (KR == 1 && FUSED) ? 5 : 4)
gemv_bulk_kernel(const SegDesc* __restrict__ seg, const int32_t* __restrict__ nseg_dev, int nseg_host, SegDesc single,
                 int n_in, int n_out, int rb, int rg, int gps, const float* __restrict__ x, int ldx,
                 const int32_t* __restrict__ row_token, float* __restrict__ out, int* status, float* out_perm,
                 int perm_type, const float* __restrict__ x_perm) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
    constexpr int lut_bytes = (T == T_IQ3_XXS) ? (int)sizeof(IqLut) : 0;
    IqLut* lut = reinterpret_cast<IqLut*>(smem + 128);
    const int item_bytes = rg * rb;  // multiple of 16 by construction
    const int per_warp = (FUSED ? 2 : 1) * item_bytes;
    uint8_t* wbase = smem + 128 + lut_bytes;
    float* xbase = reinterpret_cast<float*>(wbase + kWarps * per_warp);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint8_t* wa = wbase + warp * per_warp;
    uint8_t* wb = wa + item_bytes;
    uint64_t* bar = bars + warp;

    if (lane == 0) {
        mbar_init(bar, 1);
        if (warp == 0) {
            mbar_init(bars + kWarps, 1);      // the CTA's activation row, when it comes by bulk copy
            mbar_init(bars + kWarps + 1, 1);  // the codebook
        }
        mbar_fence_init();
        if constexpr (T == T_IQ3_XXS) {
            if (warp == 0) {
                mbar_expect_tx(bars + kWarps + 1, (uint32_t)sizeof(IqLut));
                bulk_g2s(lut, g_grid3xxs_rep, (uint32_t)sizeof(IqLut), bars + kWarps + 1);
            }
        }
    }
    // Everything above touches nothing another kernel writes.  A segment table, the token
    // count and x come from the kernel before this one; a single matrix named by the launch
    // itself does not, so its bytes are requested before the wait and stream in while the
    // previous kernel is still running (back-to-back GEMVs then overlap their fetches).
    const bool early = (seg == nullptr && nseg_dev == nullptr);
    const long wi = (long)blockIdx.x * kWarps + warp;
    const int s = (int)(wi / gps), grp = (int)(wi % gps);
    bool active = false;
    SegDesc sd = SegDesc{nullptr, nullptr, 0u, 0u};
    auto request = [&](int nseg_now) {
        active = s < nseg_now;
        if (active) sd = seg ? seg[s] : single;
        active = active && sd.m > 0;
        if (lane == 0 && active) {
            mbar_expect_tx(bar, (uint32_t)per_warp);
            bulk_g2s(wa, sd.wa + (size_t)grp * item_bytes, (uint32_t)item_bytes, bar);
            if constexpr (FUSED) bulk_g2s(wb, sd.wb + (size_t)grp * item_bytes, (uint32_t)item_bytes, bar);
        }
    };
    if (early) request(nseg_host);
    pdl_wait();
    pdl_launch_dependents();
    const int nseg = nseg_dev ? *nseg_dev : nseg_host;
    if (!early) request(nseg);
    __syncwarp();

    const int nunits = n_in >> 5;
    const float4* xs4;
    if constexpr (XSHARED) {
        if (x_perm) {
            if (tid == 0) {
                mbar_expect_tx(bars + kWarps, (uint32_t)(n_in * sizeof(float)));
                bulk_g2s(xbase, x_perm + (size_t)(blockIdx.x % kActRep) * n_in, (uint32_t)(n_in * sizeof(float)), bars + kWarps);
            }
        } else {
            // A batch of tokens: the CTA's warps all belong to one segment (the launcher
            // checks that), whose token names the row.
            const float* xr = x;
            if (row_token && seg) {
                const int s0 = (int)(((long)blockIdx.x * kWarps) / gps);
                if (s0 < nseg) xr = x + (size_t)row_token[seg[s0].row0] * ldx;
            }
            stage_x<T>(xbase, xr, n_in, nunits, tid, kWarps * 32);
        }
        xs4 = reinterpret_cast<const float4*>(xbase);
    } else {
        float* xw = xbase + (size_t)warp * n_in;
        if (active) {
            const uint32_t prow = sd.row0;
            const float* xr = x + (size_t)(row_token ? row_token[prow] : (int32_t)prow) * ldx;
            stage_x<T>(xw, xr, n_in, nunits, lane, 32);
        }
        xs4 = reinterpret_cast<const float4*>(xw);
    }
    __syncthreads();
    // Every thread waits for the CTA-wide copies (activation row, codebook) before it may leave:
    // a CTA must not end while a bulk copy into its shared memory is in flight.
    bool ready = true;
    if (XSHARED && x_perm) ready = mbar_wait_bounded(bars + kWarps, 0, status);
    if (T == T_IQ3_XXS) ready = mbar_wait_bounded(bars + kWarps + 1, 0, status) && ready;
    if (!active || !ready) return;
    if (!mbar_wait_bounded(bar, 0, status)) return;

    constexpr int GPW = 32 / LPR;
    const int sub = lane % LPR, gidx = lane / LPR;
    const int rounds = (rg + GPW - 1) / GPW;  // <= KR (launcher)
    float acc_a[KR], acc_b[KR];
#pragma unroll
    for (int it = 0; it < KR; ++it) { acc_a[it] = 0.f; acc_b[it] = 0.f; }
    for (int u = sub; u < nunits; u += LPR) {
        XUnit<T> X;
        load_x_unit<T>(xs4, nunits, u, X);
#pragma unroll
        for (int it = 0; it < KR; ++it) {
            const int rr = it * GPW + gidx;
            if (it < rounds && rr < rg) {
                acc_a[it] += unit_dot<T>(wa + rr * rb, u, lut, X);
                if constexpr (FUSED) acc_b[it] += unit_dot<T>(wb + rr * rb, u, lut, X);
            }
        }
    }
#pragma unroll
    for (int it = 0; it < KR; ++it) {
        if (it < rounds) {  // uniform across the warp
            float a = acc_a[it], bq = acc_b[it];
#pragma unroll
            for (int o = LPR / 2; o > 0; o >>= 1) {
                a += __shfl_xor_sync(0xffffffffu, a, o);
                if constexpr (FUSED) bq += __shfl_xor_sync(0xffffffffu, bq, o);
            }
            const int rr = it * GPW + gidx;
            if (rr < rg && sub == 0) {
                const int j = grp * rg + rr;
                const float v = FUSED ? silu_b(a) * bq : a;
                out[(size_t)sd.row0 * n_out + j] = v;
                if (out_perm) {  // the copies the next kernel's CTAs take whole, in its slot order
                    const size_t rep = (size_t)nseg * n_out;
                    float* o = out_perm + (size_t)sd.row0 * n_out + slot_index(perm_type, j, n_out >> 5);
#pragma unroll
                    for (int c = 0; c < kActRep; ++c) o[c * rep] = v;
                }
            }
        }
    }
}

// ---- decode down projection + weighted sum -------------------------------------
// One CTA owns R consecutive output rows for ALL segments (the k routed experts and
// the shared one): thread 0 issues one bulk copy per segment (R rows are one
// contiguous range of that expert's matrix), the CTA stages every segment's
// activation vector, each lane group computes its row for each segment in turn,
// and R threads then add the segments up in ascending order with separate multiply
// and add roundings -- the order of kernels_dec_epi.cu:28-46 / qwen4exp.rs:12126-
// 12216.  No partial results go through global memory and nothing is atomic.
constexpr int kDcWarps = 8;   // warps per CTA of the down+combine kernel
constexpr int kDcRows = 4;    // output rows per CTA

template <int T, int LPR>
__global__ void __launch_bounds__(kDcWarps * 32)
down_combine_kernel(const SegDesc* __restrict__ seg, int nseg, int k, int n_in, int n_out, int rb,
                    const float* __restrict__ act, const float* __restrict__ wts, const float* __restrict__ shcoef,
                    int has_shared, const float* __restrict__ residual, float* __restrict__ out, int* status,
                    const float* __restrict__ act_perm) {
    constexpr int GPW = 32 / LPR;
    constexpr int R = kDcRows;
    constexpr int NT = kDcWarps * 32;
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem);
    constexpr int lut_bytes = (T == T_IQ3_XXS) ? (int)sizeof(IqLut) : 0;
    IqLut* lut = reinterpret_cast<IqLut*>(smem + 128);
    const int tile_bytes = R * rb;  // multiple of 16 (checked by the launcher)
    uint8_t* wbase = smem + 128 + lut_bytes;
    float* xs = reinterpret_cast<float*>(wbase + (size_t)nseg * tile_bytes);
    float* hs = xs + (size_t)nseg * n_in;  // [nseg][R]
    float* ws = hs + nseg * R;             // [nseg] routing weights (+ shared coefficient)
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r0 = blockIdx.x * R;
    const int nunits = n_in >> 5;
    // blockIdx.y = token of a decode batch: its own nseg segments, weights, activations, rows
    const int tkn = blockIdx.y;
    seg += (size_t)tkn * nseg;
    act += (size_t)tkn * nseg * n_in;
    wts += (size_t)tkn * k;
    if (shcoef) shcoef += tkn;
    if (residual) residual += (size_t)tkn * n_out;
    out += (size_t)tkn * n_out;
    if (tid == 0) {
        mbar_init(bar, 1);
        mbar_init(bar + 1, 1);
        mbar_init(bar + 2, 1);
        mbar_fence_init();
        if constexpr (T == T_IQ3_XXS) {
            mbar_expect_tx(bar + 2, (uint32_t)sizeof(IqLut));
            bulk_g2s(lut, g_grid3xxs_rep, (uint32_t)sizeof(IqLut), bar + 2);
        }
        // The segment table was written two kernels back (the router); the kernel
        // in between waited for the router before it let this one start, so the
        // table is complete and the weights can be requested before pdl_wait().
        mbar_expect_tx(bar, (uint32_t)(nseg * tile_bytes));
        for (int s = 0; s < nseg; ++s)
            bulk_g2s(wbase + (size_t)s * tile_bytes, seg[s].wa + (size_t)r0 * rb, (uint32_t)tile_bytes, bar);
    }
    pdl_wait();               // act[] comes from the gate/up kernel
    pdl_launch_dependents();
    bool x_ok = true;
    if (act_perm) {
        // the activations arrive ready-made: one of kActRep identical copies, one bulk copy
        if (tid == 0) {
            const uint32_t bytes = (uint32_t)(nseg * n_in * sizeof(float));
            mbar_expect_tx(bar + 1, bytes);
            bulk_g2s(xs, act_perm + ((size_t)(blockIdx.x % kActRep) * gridDim.y + tkn) * nseg * n_in, bytes, bar + 1);
        }
    } else {
        stage_x_multi<T>(xs, act, n_in, nunits, nseg, tid, NT);
    }
    if (tid < nseg) ws[tid] = tid < k ? wts[tid] : (shcoef ? shcoef[0] : 1.0f);
    __syncthreads();
    if (act_perm) x_ok = mbar_wait_bounded(bar + 1, 0, status);
    if (T == T_IQ3_XXS) x_ok = mbar_wait_bounded(bar + 2, 0, status) && x_ok;
    const bool ok = mbar_wait_bounded(bar, 0, status) && x_ok;
    // (segment, row) pairs are dealt to the lane groups of all warps round-robin
    const int sub = lane % LPR;
    const int npairs = nseg * R;
    const int passes = (npairs + kDcWarps * GPW - 1) / (kDcWarps * GPW);
    for (int ps = 0; ps < passes; ++ps) {
        const int pr = (ps * kDcWarps + warp) * GPW + lane / LPR;
        const bool valid = pr < npairs;
        const int s = valid ? pr / R : 0, row = valid ? pr % R : 0;
        float acc = 0.f;
        if (ok && valid) {
            const uint8_t* ra = wbase + (size_t)s * tile_bytes + row * rb;
            const float4* xs4 = reinterpret_cast<const float4*>(xs + (size_t)s * n_in);
            for (int u = sub; u < nunits; u += LPR) {
                XUnit<T> X;
                load_x_unit<T>(xs4, nunits, u, X);
                acc += unit_dot<T>(ra, u, lut, X);
            }
        }
#pragma unroll
        for (int o = LPR / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (valid && sub == 0) hs[s * R + row] = acc;
    }
    __syncthreads();
    if (tid < R && ok) {
        float acc = 0.f;
        for (int s = 0; s < k; ++s) acc = __fadd_rn(acc, __fmul_rn(ws[s], hs[s * R + tid]));
        if (has_shared) {
            const float v = hs[k * R + tid];
            acc = __fadd_rn(acc, shcoef ? __fmul_rn(v, ws[k]) : v);
        }
        if (residual) acc = __fadd_rn(residual[r0 + tid], acc);
        out[r0 + tid] = acc;
    }
}

template <int T, int LPR>
static int launch_dc(dnb_ctx* c, cudaStream_t st, const SegDesc* seg, int nseg, int k, int n_in, int n_out,
                     const float* act, const float* wts, const float* shcoef, bool has_shared, const float* residual,
                     float* out, const float* act_perm, int ntok) {
    constexpr int R = kDcRows;
    const int rb = (int)row_bytes(T, n_in);
    if (n_out % R || (R * rb) % 16) return DNB_DECLINED;
    const size_t smem = 128 + (T == T_IQ3_XXS ? sizeof(IqLut) : 0) + (size_t)nseg * R * rb +
                        (size_t)nseg * n_in * sizeof(float) + (size_t)nseg * R * sizeof(float) + (size_t)nseg * 4 + 16;
    if (smem > 200 * 1024) return DNB_DECLINED;
    auto kern = down_combine_kernel<T, LPR>;
    static SmemGrant grant;
    DNB_CUDA(grant_smem(grant, c->device, kern, smem));
    ProfScope prof_(c, st, "gemv_down_combine");
    DNB_CUDA(launch_k(kern, dim3(n_out / R, ntok), dim3(kDcWarps * 32), smem, st, c->use_pdl, seg, nseg, k, n_in, n_out, rb, act,
                      wts, shcoef, has_shared ? 1 : 0, residual, out, c->status, act_perm));
    c->launches++;
    return DNB_OK;
}

int launch_down_combine(dnb_ctx* c, cudaStream_t st, int type, const SegDesc* seg, int nseg, int k, int n_in, int n_out,
                        const float* act, const float* wts, const float* shcoef, bool has_shared,
                        const float* residual, float* out, const float* act_perm, int ntok) {
    if (row_bytes(type, n_in) == 0 || n_in % 32 || nseg < 1 || nseg > 40 || ntok < 1 || ntok > 65535) return DNB_DECLINED;
    if ((nseg * n_in) % 4) act_perm = nullptr;  // the bulk copy moves multiples of 16 bytes
    int rc = upload_tables_b(c->device);
    if (rc != DNB_OK) return rc;
    const bool wide = (n_in / 32) >= 32;
#define DNB_DC(TT)                                                                                                      \
    case TT:                                                                                                            \
        return wide ? launch_dc<TT, 32>(c, st, seg, nseg, k, n_in, n_out, act, wts, shcoef, has_shared, residual, out, act_perm, ntok)  \
                    : launch_dc<TT, 16>(c, st, seg, nseg, k, n_in, n_out, act, wts, shcoef, has_shared, residual, out, act_perm, ntok);
    switch (type) {
        DNB_DC(T_Q4_K)
        DNB_DC(T_Q5_K)
        DNB_DC(T_Q6_K)
        DNB_DC(T_IQ3_XXS)
        DNB_DC(T_Q8_0)
        DNB_DC(T_Q5_1)
        default: return DNB_DECLINED;
    }
#undef DNB_DC
}

static int gcd_i(int a, int b) { return b ? gcd_i(b, a % b) : a; }

template <int T, bool FUSED, int LPR, bool XSHARED>
static int launch_cfg(dnb_ctx* c, cudaStream_t st, const SegDesc* seg, const int32_t* nseg_dev, int nseg_max,
                      SegDesc single, int n_in, int n_out, const float* x, int ldx, const int32_t* row_token,
                      float* out, const char* pname, PermOut perm) {
    const int rb = (int)row_bytes(T, n_in);
    constexpr int GPW = 32 / LPR;
    const int gmin = 16 / gcd_i(rb, 16);            // rows whose bytes make a multiple of 16
    int step = gmin * GPW / gcd_i(gmin, GPW);       // lcm
    if (n_out % step) return DNB_DECLINED;          // caller falls back to the tiled kernel
    int rg = step;
    // bytes per warp per matrix: short per-warp chains, many warps.  (Fatter warps for a single matrix, so that
    // a launch fills only half of every SM and the next GEMV's CTAs sit beside it, were measured: 7.6-8.7 us per
    // 4096 x 4096 GEMV at every setting -- the launch-to-launch hand-over, not the fetch, sets that time.)
    const int target = 1500;
    while (rg * 2 * rb <= target && n_out % (rg * 2) == 0 && rg * 2 <= kMaxRounds * GPW) rg *= 2;
    if (rg > kMaxRounds * GPW) return DNB_DECLINED;
    const int gps = n_out / rg;
    const int item_bytes = rg * rb;
    const size_t smem = 128 + (T == T_IQ3_XXS ? sizeof(IqLut) : 0) + (size_t)kWarps * (FUSED ? 2 : 1) * item_bytes +
                        (size_t)(XSHARED ? 1 : kWarps) * n_in * sizeof(float);
    if (smem > 200 * 1024) return DNB_DECLINED;
    // one row round per warp (the decode shapes): a leaner instance; the fused gate/up form of it
    // is built for five CTAs per SM so that the 704 CTAs of a 512-expert top-10 block are one wave
    const bool one = (rg + GPW - 1) / GPW == 1;
    auto kern = one ? gemv_bulk_kernel<T, FUSED, LPR, XSHARED, 1> : gemv_bulk_kernel<T, FUSED, LPR, XSHARED, kMaxRounds>;
    static SmemGrant grant[2];
    DNB_CUDA(grant_smem(grant[one ? 1 : 0], c->device, kern, smem));
    if (XSHARED && row_token && gps % kWarps) return DNB_DECLINED;  // a CTA must not straddle two segments' tokens
    const long warps = (long)nseg_max * gps;
    const int grid = (int)((warps + kWarps - 1) / kWarps);
    ProfScope prof_(c, st, pname);
    DNB_CUDA(launch_k(kern, dim3(grid), dim3(kWarps * 32), smem, st, c->use_pdl, seg, nseg_dev, nseg_max, single, n_in, n_out,
                      rb, rg, gps, x, ldx, row_token, out, c->status, nseg_dev ? nullptr : perm.base, perm.type,
                      (XSHARED && n_in % 4 == 0) ? perm.x_perm : nullptr));
    c->launches++;
    return DNB_OK;
}

template <int T>
static int launch_t(dnb_ctx* c, cudaStream_t st, bool fused, bool xshared, const SegDesc* seg, const int32_t* nseg_dev,
                    int nseg_max, SegDesc single, int n_in, int n_out, const float* x, int ldx,
                    const int32_t* row_token, float* out, const char* pname, PermOut perm) {
    const bool wide = (n_in / 32) >= 32;
#define DNB_B(F, L, X) \
    return launch_cfg<T, F, L, X>(c, st, seg, nseg_dev, nseg_max, single, n_in, n_out, x, ldx, row_token, out, pname, perm)
    if (fused) {
        if (wide) { if (xshared) DNB_B(true, 32, true); else DNB_B(true, 32, false); }
        else      { if (xshared) DNB_B(true, 16, true); else DNB_B(true, 16, false); }
    } else {
        if (wide) { if (xshared) DNB_B(false, 32, true); else DNB_B(false, 32, false); }
        else      { if (xshared) DNB_B(false, 16, true); else DNB_B(false, 16, false); }
    }
#undef DNB_B
}

// Every segment has exactly one token row.  xshared: all segments read the same
// activation row `x` (then x points at that row and row_token is ignored).
// Returns DNB_DECLINED when the shape does not fit this kernel (the caller then
// uses the tiled kernel of seg_matmul.cu).
int launch_seg_gemv_m1(dnb_ctx* c, cudaStream_t st, int type, bool fused, bool xshared, const SegDesc* seg,
                       const int32_t* nseg_dev, int nseg_max, int n_in, int n_out, const float* x, int ldx,
                       const int32_t* row_token, float* out, const SegDesc* single_p, const char* pname, PermOut perm) {
    const SegDesc single = single_p ? *single_p : SegDesc{nullptr, nullptr, 0u, 0u};
    if (!seg && !single_p) return DNB_ERR_ARG;
    if (row_bytes(type, n_in) == 0 || n_in % 32 || n_out <= 0 || nseg_max <= 0) return DNB_DECLINED;
    int rc;
    // The mma.sync gate/up kernel as a launch of its own is taken only on request (dnb_set_gemv_impl 4):
    // beside the register-decode down kernel it measured no faster than the register-decode gate/up.
    if (type == T_IQ3_XXS && fused && xshared && seg && !nseg_dev && !row_token && c->gemv_mma && !c->decode_fused) {
        rc = launch_gate_up_mma(c, st, seg, nseg_max, n_in, n_out, x, out, pname, perm);
        if (rc != DNB_DECLINED) return rc;
    }
    rc = upload_tables_b(c->device);
    if (rc != DNB_OK) return rc;
    switch (type) {
        case T_Q4_K: return launch_t<T_Q4_K>(c, st, fused, xshared, seg, nseg_dev, nseg_max, single, n_in, n_out, x, ldx, row_token, out, pname, perm);
        case T_Q5_K: return launch_t<T_Q5_K>(c, st, fused, xshared, seg, nseg_dev, nseg_max, single, n_in, n_out, x, ldx, row_token, out, pname, perm);
        case T_Q6_K: return launch_t<T_Q6_K>(c, st, fused, xshared, seg, nseg_dev, nseg_max, single, n_in, n_out, x, ldx, row_token, out, pname, perm);
        case T_IQ3_XXS: return launch_t<T_IQ3_XXS>(c, st, fused, xshared, seg, nseg_dev, nseg_max, single, n_in, n_out, x, ldx, row_token, out, pname, perm);
        case T_Q8_0: return launch_t<T_Q8_0>(c, st, fused, xshared, seg, nseg_dev, nseg_max, single, n_in, n_out, x, ldx, row_token, out, pname, perm);
        case T_Q5_1: return launch_t<T_Q5_1>(c, st, fused, xshared, seg, nseg_dev, nseg_max, single, n_in, n_out, x, ldx, row_token, out, pname, perm);
        default: return DNB_DECLINED;
    }
}

}  // namespace dnb
