// One-token MoE block as ONE kernel.  IQ3_XXS experts only.
//
//   ROUTED = false   the half after the router: gate/up GEMV with SwiGLU, a grid-wide
//                    barrier, down GEMV with the weighted sum over the experts; the
//                    segment tables and routing weights come from the router kernel
//   ROUTED = true    the whole block: RMSNorm, router logits, a grid-wide barrier,
//                    softmax / top-k / renorm (every CTA ranks the logits itself), then
//                    the half above -- one launch per block, no table in global memory
//
// Why one kernel: with two, the down kernel's CTAs cannot all be resident beside the
// gate/up kernel (registers, shared memory), so a good part of the down weights is
// requested only after gate/up has ended and their arrival (~1 us) plus the launch
// hand-over sits on the critical path of a 20 us block.  Here one CTA per SM requests
// ALL its weights (gate, up and down rows, ~90 KB) the moment the routing is known,
// and the down phase finds its rows already in shared memory.  With the router folded
// in as well, the last-CTA ticket, the table hand-over and one launch boundary leave the
// critical path too.
//
// Both matmul phases run on mma.sync.m16n8k16 as gemv_mma.cu describes (weights decoded
// straight into bf16 A fragments, activations as an exact three-way bf16 split in the
// B columns).  Down phase: a CTA owns up to two units of 8 output rows for all
// experts; a warp takes one unit, one PAIR of experts and half of K: rows 0-7 of the
// A tile are the unit's rows of the first expert, rows 8-15 those of the second, and
// the B columns 0-2 / 4-6 hold the two experts' activation vectors, so one mma serves
// both (the cross terms land in accumulator columns that are never read).  The
// partial sums of a row meet in shared memory and are added in a fixed order; the
// experts are then summed in ascending order with separate multiply and add roundings,
// the order of kernels_dec_epi.cu:28-46 / qwen4exp.rs:12126-12216 of the reference.
//
// Router (ROUTED): the arithmetic of the stand-alone router kernels, operation for
// operation (RMSNorm: tensor.rs:1125-1135 with the 128-thread summation tree of
// moe_kernels.cu; logits: one warp per row, float4 words lane + 32 j; softmax:
// tensor.rs:1171-1183 with the same partial-sum tree; selection rule moe.rs:256-279;
// renorm qwen4exp.rs:11802-11821), so a token gets the same routing bits on every path.
// Only the selection is organised differently: the k-th largest of the warp maxima is a
// threshold every top-k entry reaches; the few entries that reach it are ranked by
// (value, index) in parallel.
//
// Data crosses CTAs through global memory twice: the logits (ROUTED) and the SwiGLU
// outputs, which every CTA writes as bf16 triples into kActRep identical copies (so that
// the 148 readers do not all hit the same L2 lines).  Each time the CTAs arrive at a
// counter that only grows and wait (bounded) until it has reached the launch's share.  All
// CTAs are resident: one per SM, the grid never exceeds the SM count, and the kernel that
// follows in the stream is not released before every CTA of this one has started.  A wait
// that runs out sets the status word and the CTA skips the remaining phases (it still
// arrives at the later barrier, so the counter stays a multiple of the grid); nothing
// can hang.
#include <algorithm>

#include "iq3_mma.cuh"

// Optional timeline (the reference's DENNO_Q4_TLINE, cuda.rs:256-420, in kernel form): built with
// -DDNB_TIMELINE, lane 0 of every warp stamps the global timer at the phase boundaries below and
// dnb_probe_timeline copies the stamps out.  Compiled out otherwise.
#ifdef DNB_TIMELINE
__device__ unsigned long long g_dnb_tl[148][24][32];
__device__ __forceinline__ unsigned long long dnb_gtime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define DNB_STAMP(i) do { if ((threadIdx.x & 31) == 0 && blockIdx.x < 148) g_dnb_tl[blockIdx.x][threadIdx.x >> 5][i] = dnb_gtime(); } while (0)
extern "C" int dnb_probe_timeline(void* dst) { return (int)cudaMemcpyFromSymbol(dst, g_dnb_tl, sizeof(g_dnb_tl)); }
#else
#define DNB_STAMP(i) do { } while (0)
#endif

namespace dnb {

constexpr int kFdUnits = 2;                         // down units (8 output rows) per CTA
constexpr int kFdPairs = 6;                         // expert pairs per unit: up to 12 segments
constexpr int kFdWarps = kFdUnits * kFdPairs * 2;   // x2: halves of K
constexpr int kFdThreads = kFdWarps * 32;
constexpr int kFdSegs = 2 * kFdPairs;
constexpr int kFdPad = 8;                           // halves of padding per activation row (bank spread)
constexpr int kFdHeader = 256;                      // 16 mbarriers, then flags
constexpr int kFdRouterRows = 4;                    // router rows a CTA can hold (ROUTED)
constexpr int kFdCand = 64;                         // entries the parallel ranking of the top-k takes
static_assert(kFdWarps >= kGmGroups * kGmKs, "the gate/up phase needs its warps");

struct FusedArgs {
    const SegDesc* seg_gu;   // [nseg] gate/up matrices (ROUTED: unused)
    const SegDesc* seg_dn;   // [nseg] down matrices (wa)
    int nseg, k, has_shared;
    int e, ff;               // hidden width, expert width
    int rb_gu, rb_dn;        // bytes per row of the gate/up and the down matrices
    int acts_halves;         // halves of shared memory reserved for the activation triples (ROUTED: or the router rows, if larger)
    const float* x;          // normalised hidden row (natural order)   (ROUTED: unused)
    const float* x_perm;     // or: kActRep slot-ordered copies of it     (ROUTED: unused)
    float* act;              // [nseg][ff] SwiGLU outputs (fp32, for inspection)
    uint16_t* act_h;           // [kActRep][nseg][3][ff + kFdPad]
    const float* wts;        // [k] routing weights (ROUTED: unused, see wts_out)
    const float* shcoef;     // shared-expert coefficient or null (ROUTED: unused)
    const float* residual;   // or null
    float* out;              // [e]
    unsigned long long* gbar;  // arrivals of all launches so far
    int* status;
    int barrier_polls;         // acquire loads before a barrier gives up
    unsigned int barrier_bias; // test hook: added to the arrival count waited for (0 in production)
    // ---- ROUTED only ----
    const float* h;            // block input row
    const float* norm_w;       // or null
    float eps;
    const float* router_w;     // [ne][e]
    const float* router_bias;  // or null
    int ne, norm_topk;
    float* logits;             // [kActRep][ne] scratch in global memory: every CTA writes its logits into all copies and reads one
    const uint8_t *gate, *up, *down;
    size_t eb_g, eb_u, eb_d;   // bytes per expert
    const uint8_t *sg, *su, *sdn;     // shared expert (has_shared)
    const float* shared_gate_row;     // or null: coefficient 1
    int32_t* sels_out;         // [k] ascending
    float* wts_out;            // [k]
    float* xn_out;             // [e] normalised row, or null
};

// Shared memory of the routing phase (ROUTED).
struct RouteSmem {
    float probs[1024];
    uint32_t tmax[128];
    int wcnt[4];
    uint32_t cand_k[kFdCand];
    int cand_x[kFdCand];
    float red[128];
    float cmax[4];
    float bcast;
    float inv;
    int nan_any;
    int total;
    int sel[32];
    float pv[32];
    int ssel[32];
    float spv[32];
};

__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long atom_add_acq_rel(unsigned long long* p, unsigned long long v) {
    unsigned long long old;
    asm volatile("atom.acq_rel.gpu.global.add.u64 %0, [%1], %2;" : "=l"(old) : "l"(p), "l"(v) : "memory");
    return old;
}

// Grid-wide barrier, thread 0 of every CTA (the others wait at the bar.sync that follows).
// The counter only grows: every CTA adds one per barrier, a barrier is complete when the count
// reaches the next multiple of the grid size.  The release half of the atomic publishes this
// CTA's stores (the bar.sync before it ordered them), the acquire load makes the other CTAs'
// stores visible.  wait = false only arrives (a CTA that has already given up keeps the count
// whole without waiting again).  One poller per CTA: more of them (tried: four, staggered, with a
// fire-and-forget arrival) only queue on the counter's L2 line and made the barrier slower.
__device__ __forceinline__ bool grid_barrier(const FusedArgs& A, bool wait) {
    const unsigned long long ticket = atom_add_acq_rel(A.gbar, 1ull);
    if (!wait) return false;
    const unsigned long long target = (ticket / gridDim.x + 1ull) * gridDim.x + A.barrier_bias;
    bool pass = ticket + 1ull == target;
    for (int i = 0; i < A.barrier_polls && !pass; ++i) pass = ld_acquire_u64(A.gbar) >= target;  // ~0.2 s at most by default
    if (!pass) status_set(A.status, 23);
    return pass;
}

__device__ __forceinline__ uint32_t order_key(float v) {  // larger float -> larger key; never 0 for a probability
    const uint32_t ub = __float_as_uint(v);
    return (ub & 0x80000000u) ? ~ub : (ub | 0x80000000u);
}

// softmax + top-k + renorm of the ne logits in global memory (written by all CTAs before the
// barrier), by the whole CTA.  Leaves the selection ascending in R.ssel, the routing weights in
// wts_s[0..k).  Every thread of the CTA must call it (it contains CTA-wide barriers).
// Barrier of the four routing warps (named barrier 6; 1-5 belong to the gate/up groups).
__device__ __forceinline__ void route_sync() { asm volatile("bar.sync 6, 128;" ::: "memory"); }

// Softmax, top-k and renorm of one token's logits by threads 0..127 of the CTA (the other warps wait at
// the CTA barrier that follows the call).  Thread v holds entries v, v + 128, ...; every value that
// depends on evaluation order is computed as in topk_block (moe_kernels.cu), so a token gets the same
// routing bits as on the other paths.  Six 128-thread barriers: what only one warp did before (the
// sum's tree, the threshold) every warp now does for itself instead of waiting for a broadcast.
__device__ __forceinline__ void route_topk(RouteSmem& R, const float* __restrict__ logits, int ne, int k, int norm_topk,
                                           float* wts_s) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float p[8];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int idx = j * 128 + tid;
        p[j] = idx < ne ? __ldcg(logits + idx) : -INFINITY;
        mx = fmaxf(mx, p[j]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) R.cmax[warp] = mx;
    if (tid == 0) R.nan_any = 0;
    DNB_STAMP(16);
    route_sync();
    mx = fmaxf(fmaxf(R.cmax[0], R.cmax[1]), fmaxf(R.cmax[2], R.cmax[3]));
    {
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
        R.red[tid] = part;
        if (any_nan) R.nan_any = 1;
    }
    DNB_STAMP(17);
    route_sync();
    // the tree of topk_block; the xor butterfly leaves the same bits in every lane of every warp
    float sum = (R.red[lane] + R.red[lane + 64]) + (R.red[lane + 32] + R.red[lane + 96]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const bool has_nan = R.nan_any != 0;
    uint32_t key[8];
    uint32_t km = 0u;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int idx = j * 128 + tid;
        key[j] = 0u;
        if (idx < ne) {
            p[j] = sum > 0.f ? p[j] / sum : p[j];
            R.probs[idx] = p[j];
            key[j] = order_key(p[j]);
            km = max(km, key[j]);
        }
    }
    R.tmax[tid] = km;
    DNB_STAMP(18);
    route_sync();
    // ---- selection ----
    // Fast form (no NaN): the entries fall into 32 classes by index mod 32 (= lane); t = the k-th largest
    // of the class maxima.  At least k entries reach t, so every one of the top k does; the entries that
    // reach it (a dozen or two) are ranked among themselves by (value descending, index ascending) -- the
    // CPU scan's rule.
    bool fast = !has_nan && k <= 32;
    int total = 0;
    if (fast) {
        const uint32_t v = max(max(R.tmax[lane], R.tmax[lane + 32]), max(R.tmax[lane + 64], R.tmax[lane + 96]));
        int above = 0;
#pragma unroll
        for (int j = 0; j < 32; ++j) above += (__shfl_sync(0xffffffffu, v, j) > v) ? 1 : 0;
        uint32_t t = __reduce_min_sync(0xffffffffu, (above < k && v != 0u) ? v : 0xffffffffu);
        const int have = __popc(__ballot_sync(0xffffffffu, v != 0u));
        if (have < k) t = 1u;  // fewer maxima than selections: every entry is a candidate
        uint32_t smask = 0u;
#pragma unroll
        for (int j = 0; j < 8; ++j) smask |= (key[j] != 0u && key[j] >= t) ? (1u << j) : 0u;
        const int cnt = __popc(smask);
        int incl = cnt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int u = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += u;
        }
        if (lane == 31) R.wcnt[warp] = incl;
        DNB_STAMP(19);
        route_sync();
        int before = incl - cnt;
        for (int w2 = 0; w2 < 4; ++w2) {
            const int c = R.wcnt[w2];
            if (w2 < warp) before += c;
            total += c;
        }
        fast = total >= k && total <= kFdCand;
        if (fast) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if ((smask >> j) & 1u) {
                    R.cand_k[before] = key[j];
                    R.cand_x[before] = j * 128 + tid;
                    ++before;
                }
        }
        DNB_STAMP(20);
        route_sync();
        if (fast && tid < total) {
            const uint32_t ck = R.cand_k[tid];
            const int cx = R.cand_x[tid];
            int rank = 0;
            for (int j = 0; j < total; ++j) {
                const uint32_t ok = R.cand_k[j];
                const int ox = R.cand_x[j];
                rank += (ok > ck || (ok == ck && ox < cx)) ? 1 : 0;
            }
            if (rank < k) {
                R.sel[rank] = cx;
                R.pv[rank] = R.probs[cx];
            }
        }
    }
    if (!fast) {
        // General form, warp 0: k rounds of the CPU scan (moe.rs:256-279) with the entries dealt to
        // the lanes.  A strictly larger value wins, ties go to the lower index, and a NaN is taken
        // only when it is the first unused entry.
        if (warp == 0) {
            uint32_t used = 0u;  // bit m: entry 32 m + lane
            for (int round = 0; round < k; ++round) {
                float best = -INFINITY;
                int best_i = 0x7fffffff, first = 0x7fffffff;
                for (int m = 0; 32 * m + lane < ne; ++m) {
                    if ((used >> m) & 1u) continue;
                    const int idx = 32 * m + lane;
                    first = min(first, idx);
                    const float v = R.probs[idx];
                    if (v == v && (best_i == 0x7fffffff || v > best)) {
                        best = v;
                        best_i = idx;
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
                int win = best_i;
                if (has_nan || best_i == 0x7fffffff) {
                    const float fv = first != 0x7fffffff ? R.probs[first] : 0.f;
                    if (fv != fv || best_i == 0x7fffffff) win = first;
                }
                if ((win & 31) == lane) used |= 1u << (win >> 5);
                if (lane == 0) {
                    R.sel[round] = win;
                    R.pv[round] = R.probs[win];
                }
            }
        }
    }
    DNB_STAMP(21);
    route_sync();
    if (tid < k) {
        const int mine = R.sel[tid];
        int rank = 0;
        for (int j = 0; j < k; ++j) rank += (R.sel[j] < mine) ? 1 : 0;
        R.ssel[rank] = mine;
        R.spv[rank] = R.pv[tid];
    }
    route_sync();
    if (tid < k) {
        float s = 0.f;  // the selected probabilities in ascending expert index, one add at a time
        for (int j = 0; j < k; ++j) s = __fadd_rn(s, R.spv[j]);
        float w;
        if (!norm_topk) w = R.spv[tid];
        else if (isfinite(s) && s > 0.f) w = R.spv[tid] / s;
        else w = 1.0f / (float)k;
        wts_s[tid] = w;
    }
    DNB_STAMP(22);
}

// Dynamic shared memory:
// [16 mbarriers | flags, pad to 256][codebook 32 KB][gate/up rows][down rows][x fp32][x bf16 x3]
// [activations bf16 x3, all segments][gate/up K-partials][down partials][routing weights]
// ROUTED adds [segment tables][RouteSmem]; before the routing is known the down-row area holds the
// block input and the norm weights, and the activation area holds the CTA's router rows.
template <bool ROUTED>
__global__ void __maxnreg__(ROUTED ? 80 : 64) decode_fused_kernel(const FusedArgs A) {
    extern __shared__ __align__(128) uint8_t smem[];
    // [0..4] gate/up groups, [5] codebook, [6] x, [7] down rows, [8] router rows, [9] norm weights, [10] input row
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
    int* flags = reinterpret_cast<int*>(smem + 128);  // [0] second barrier passed, [1] first barrier passed (ROUTED)
    Iq3Tables* lut = reinterpret_cast<Iq3Tables*>(smem + kFdHeader);
    const int e = A.e, ff = A.ff, nseg = A.nseg;
    const int gu_bytes = kGmRows * A.rb_gu, dn_bytes = 8 * A.rb_dn;  // multiples of 16
    const int arow = ff + kFdPad;
    uint8_t* wgu = smem + kFdHeader + sizeof(Iq3Tables);
    uint8_t* wdn = wgu + (size_t)kGmGroups * 2 * gu_bytes;
    float* xf = reinterpret_cast<float*>(wdn + (size_t)kFdUnits * kFdSegs * dn_bytes);
    uint16_t* xh = reinterpret_cast<uint16_t*>(xf + e);
    uint16_t* acts = xh + (size_t)kGmSplit * e;
    float* red = reinterpret_cast<float*>(acts + (size_t)A.acts_halves);          // [group][ks][16]
    float* hp = red + kGmGroups * kGmKs * 16;                                      // [unit][half][seg][8]
    float* ws = hp + kFdUnits * 2 * kFdSegs * 8;                                   // [16]: routing weights (+ shared coefficient)
    SegDesc* sdt = reinterpret_cast<SegDesc*>(ws + 16);                            // ROUTED: [kFdSegs] gate/up, [kFdSegs] down
    RouteSmem* R = reinterpret_cast<RouteSmem*>(sdt + 2 * kFdSegs);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    // ROUTED: the CTA's router rows, the norm weights (layer constants: requested before the wait on
    // the previous kernel) and, after the wait, the block's input row
    int rrow0 = 0, nrr = 0;
    float* rrows = reinterpret_cast<float*>(acts);
    float* nwbuf = reinterpret_cast<float*>(wdn);
    float* hbuf = nwbuf + e;
    if constexpr (ROUTED) {
        const int per = (A.ne + (int)gridDim.x - 1) / (int)gridDim.x;  // <= kFdRouterRows (launcher)
        rrow0 = (int)blockIdx.x * per;
        nrr = min(per, A.ne - rrow0);
        if (nrr < 0) nrr = 0;
    }
    if (tid == 0) {
        for (int i = 0; i < 11; ++i) mbar_init(bars + i, 1);
        mbar_fence_init();
        if constexpr (ROUTED) {  // what the first phase needs goes first; the codebook is not needed before the routing is known
            if (nrr > 0) {
                mbar_expect_tx(bars + 8, (uint32_t)(nrr * e * sizeof(float)));
                bulk_g2s(rrows, A.router_w + (size_t)rrow0 * e, (uint32_t)(nrr * e * sizeof(float)), bars + 8);
            }
            if (A.norm_w) {
                mbar_expect_tx(bars + 9, (uint32_t)(e * sizeof(float)));
                bulk_g2s(nwbuf, A.norm_w, (uint32_t)(e * sizeof(float)), bars + 9);
            }
        }
        mbar_expect_tx(bars + 5, (uint32_t)(sizeof(Iq3Tables)));
        bulk_g2s(lut, &g_iq3_tables, (uint32_t)(sizeof(Iq3Tables)), bars + 5);
        flags[0] = 0;
        flags[1] = 0;
    }
    __syncthreads();
    DNB_STAMP(0);
    pdl_wait();  // the input (ROUTED) or the segment tables, routing weights and x come from the kernel before
    pdl_launch_dependents();
    DNB_STAMP(1);

    bool ready = true;
    float resid = 0.f;
    const int nunits_dn = e / 8;
    int my_units = 0;
    for (int u = 0; u < kFdUnits; ++u) my_units += (blockIdx.x + u * gridDim.x) < nunits_dn ? 1 : 0;
    if (A.residual && tid < kFdUnits * 8 && (tid >> 3) < my_units)  // fetched now, off the critical path
        resid = A.residual[(blockIdx.x + (tid >> 3) * gridDim.x) * 8 + (tid & 7)];

    if constexpr (ROUTED) {
        // ---- RMSNorm (tensor.rs:1125-1135; summation tree of rms_inv_128) ---------------------
        if (tid == 0) {
            mbar_expect_tx(bars + 10, (uint32_t)(e * sizeof(float)));
            bulk_g2s(hbuf, A.h, (uint32_t)(e * sizeof(float)), bars + 10);
        }
        ready = mbar_wait_bounded(bars + 10, 0, A.status);
        if (A.norm_w) ready = mbar_wait_bounded(bars + 9, 0, A.status) && ready;
        DNB_STAMP(2);
        if (A.norm_w && tid < 128) {
            float ss = 0.f;
            for (int i = tid; i < e; i += 128) ss = fmaf(hbuf[i], hbuf[i], ss);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (lane == 0) R->red[warp] = ss;
        }
        __syncthreads();
        {
            // every thread evaluates the same expression on the same four partial sums: no broadcast, no second barrier
            const float inv = A.norm_w ? 1.0f / sqrtf(((R->red[0] + R->red[1]) + (R->red[2] + R->red[3])) / (float)e + A.eps) : 1.0f;
            for (int i = 2 * tid; i < e; i += 2 * kFdThreads) {
                float2 v = *reinterpret_cast<const float2*>(hbuf + i);
                if (A.norm_w) {
                    const float2 nw = *reinterpret_cast<const float2*>(nwbuf + i);
                    v.x = __fmul_rn(__fmul_rn(v.x, inv), nw.x);
                    v.y = __fmul_rn(__fmul_rn(v.y, inv), nw.y);
                }
                *reinterpret_cast<float2*>(xf + i) = v;
                if (A.xn_out && blockIdx.x == 0) *reinterpret_cast<float2*>(A.xn_out + i) = v;
                uint32_t h0[kGmSplit], h1[kGmSplit];
                split3(v.x, h0);
                split3(v.y, h1);
#pragma unroll
                for (int n = 0; n < kGmSplit; ++n)
                    *reinterpret_cast<uint32_t*>(xh + (size_t)n * e + i) = h0[n] | (h1[n] << 16);
            }
        }
        __syncthreads();
        DNB_STAMP(3);
        // ---- router logits: one warp per row (linear_gguf.rs:836-964; kernels_elem.cu:948-1002) ----
        if (nrr > 0) ready = mbar_wait_bounded(bars + 8, 0, A.status) && ready;
        DNB_STAMP(4);
        if (warp < nrr && ready) {
            const float4* wr = reinterpret_cast<const float4*>(rrows + (size_t)warp * e);
            const float4* x4 = reinterpret_cast<const float4*>(xf);
            float acc = 0.f;
            for (int j = lane; j < (e >> 2); j += 32) {
                const float4 wv = wr[j], xv = x4[j];
                acc = fmaf(wv.x, xv.x, acc);
                acc = fmaf(wv.y, xv.y, acc);
                acc = fmaf(wv.z, xv.z, acc);
                acc = fmaf(wv.w, xv.w, acc);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            const float lg = A.router_bias ? acc + A.router_bias[rrow0 + warp] : acc;
            // kActRep copies: 148 CTAs reading one 2 KB vector at the same moment queue on its few L2 lines
            if (lane < kActRep) A.logits[(size_t)lane * A.ne + rrow0 + warp] = lg;
        } else if (warp == kFdRouterRows && A.has_shared) {
            // shared-expert coefficient sigmoid(row . x) (hyper.rs:112-114; qwen4exp.rs:12388-12395)
            float coef = 1.0f;
            if (A.shared_gate_row) {
                float acc = 0.f;
                for (int i = lane; i < e; i += 32) acc = fmaf(A.shared_gate_row[i], xf[i], acc);
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                coef = 1.0f / (1.0f + expf(-acc));
            }
            if (lane == 0) ws[A.k] = coef;
        }
        __syncthreads();
        DNB_STAMP(5);
        if (tid == 0) flags[1] = grid_barrier(A, true) ? 1 : 0;
        __syncthreads();
        DNB_STAMP(6);
        ready = flags[1] != 0 && ready;
        // Every CTA ranks the logits itself.  (After a failed wait the host discards the call; the
        // selection below then runs on whatever is there, and every index stays in range.)
        if (tid < 128) route_topk(*R, A.logits + (size_t)(blockIdx.x % kActRep) * A.ne, A.ne, A.k, A.norm_topk, ws);
        DNB_STAMP(7);
        if (tid < A.k) {
            int ex = R->ssel[tid];
            ex = ex < 0 ? 0 : (ex >= A.ne ? A.ne - 1 : ex);
            sdt[tid] = SegDesc{A.gate + (size_t)ex * A.eb_g, A.up + (size_t)ex * A.eb_u, 1u, (uint32_t)tid};
            sdt[kFdSegs + tid] = SegDesc{A.down + (size_t)ex * A.eb_d, nullptr, 1u, (uint32_t)tid};
            if (blockIdx.x == 0) {
                A.sels_out[tid] = ex;
                A.wts_out[tid] = ws[tid];
            }
        }
        if (tid == 32 && A.has_shared) {
            sdt[A.k] = SegDesc{A.sg, A.su, 1u, (uint32_t)A.k};
            sdt[kFdSegs + A.k] = SegDesc{A.sdn, nullptr, 1u, (uint32_t)A.k};
        }
        __syncthreads();
        DNB_STAMP(23);
    }
    const SegDesc* seg_gu = ROUTED ? sdt : A.seg_gu;
    const SegDesc* seg_dn = ROUTED ? sdt + kFdSegs : A.seg_dn;

    // ---- requests: gate/up rows per group, all down rows, x ------------------------------
    const int q = warp / kGmKs, ks = warp % kGmKs;
    const int gps = ff / kGmRows;
    const int gid = blockIdx.x + q * gridDim.x;
    const int gs = gid / gps, gr0 = (gid - gs * gps) * kGmRows;
    bool gactive = q < kGmGroups && gs < nseg;
    SegDesc sd = SegDesc{nullptr, nullptr, 0u, 0u};
    if (gactive) sd = seg_gu[gs];
    gactive = gactive && sd.m > 0;
    uint8_t* wq = wgu + (size_t)(q < kGmGroups ? q : 0) * 2 * gu_bytes;
    if (ks == 0 && lane == 0 && gactive) {
        mbar_expect_tx(bars + q, (uint32_t)(2 * gu_bytes));
        bulk_g2s(wq, sd.wa + (size_t)gr0 * A.rb_gu, (uint32_t)gu_bytes, bars + q);
        bulk_g2s(wq + gu_bytes, sd.wb + (size_t)gr0 * A.rb_gu, (uint32_t)gu_bytes, bars + q);
    }
    if constexpr (!ROUTED) {
        if (tid == 32 && A.x_perm) {
            mbar_expect_tx(bars + 6, (uint32_t)(e * sizeof(float)));
            bulk_g2s(xf, A.x_perm + (size_t)(blockIdx.x % kActRep) * e, (uint32_t)(e * sizeof(float)), bars + 6);
        }
        if (tid >= 96 && tid < 96 + nseg) {
            const int s = tid - 96;
            ws[s] = s < A.k ? A.wts[s] : (A.shcoef ? A.shcoef[0] : 1.0f);
        }
        // ---- x -> three bf16 vectors in natural element order ------------------------------------
        if (A.x_perm) ready = mbar_wait_bounded(bars + 6, 0, A.status);
        if (ready) {
            const int nunits = e >> 5;
            for (int i = 2 * tid; i < e; i += 2 * kFdThreads) {
                float2 v;
                if (A.x_perm) {
                    const int u = i >> 5, sl = i & 31;  // 32 consecutive elements per unit (slot_of of this format)
                    v = *reinterpret_cast<const float2*>(xf + ((((sl >> 2) * nunits + u) << 2) + (sl & 3)));
                } else {
                    v = *reinterpret_cast<const float2*>(A.x + i);
                }
                uint32_t h0[kGmSplit], h1[kGmSplit];
                split3(v.x, h0);
                split3(v.y, h1);
#pragma unroll
                for (int n = 0; n < kGmSplit; ++n)
                    *reinterpret_cast<uint32_t*>(xh + (size_t)n * e + i) = h0[n] | (h1[n] << 16);
            }
        }
        __syncthreads();
    }
    // The down rows are asked for only now, behind the gate/up rows: the two together are ~2 us of
    // HBM time, and the gate/up phase needs its share first.  One lane per (unit, segment), in a
    // warp that has no gate/up work.  (ROUTED: the area held the input row and the norm weights
    // until the first barrier.)
    DNB_STAMP(24);
    if (warp == kFdWarps - 1) {
        if (lane == 0) mbar_expect_tx(bars + 7, (uint32_t)(my_units * nseg * dn_bytes));
        __syncwarp();
        if (lane < my_units * nseg) {
            const int u = lane / nseg, s = lane - u * nseg;
            const size_t off = (size_t)(blockIdx.x + u * gridDim.x) * dn_bytes;
            bulk_g2s(wdn + (size_t)(u * kFdSegs + s) * dn_bytes, seg_dn[s].wa + off, (uint32_t)dn_bytes, bars + 7);
        }
    }
    ready = mbar_wait_bounded(bars + 5, 0, A.status) && ready;
    const Iq3Lane lutp(lut, lane);
    DNB_STAMP(8);

    // ---- gate/up: 8 gate + 8 up rows per group, four warps split K -----------------------------
    if (gactive) {  // all four warps of a group agree
        const bool ok = mbar_wait_bounded(bars + q, 0, A.status) && ready;
        DNB_STAMP(9);
        float accg = 0.f, accu = 0.f;
        if (ok) {
            const uint8_t* rowg = wq + g * A.rb_gu;
            const uint16_t* xb = xh + (size_t)(g < kGmSplit ? g : 0) * e + 8 * t;
            const int bpw = (e >> 8) / kGmKs;
            gate_up_warp(rowg, rowg + gu_bytes, lutp, xb, g < kGmSplit, ks * bpw, (ks + 1) * bpw, t, accg, accu);
        }
        DNB_STAMP(10);
        float* rq = red + (size_t)q * kGmKs * 16;
        if (t == 0) {
            rq[ks * 16 + g] = accg;
            rq[ks * 16 + 8 + g] = accu;
        }
        group_barrier(q);
        if (ks == 0 && ok) {
            float a = rq[g], bq = rq[8 + g];
#pragma unroll
            for (int k2 = 1; k2 < kGmKs; ++k2) {
                a += rq[k2 * 16 + g];
                bq += rq[k2 * 16 + 8 + g];
            }
            const float v = silu_m(a) * bq;
            const int j = gr0 + g;
            if (t == 0) A.act[(size_t)sd.row0 * ff + j] = v;
            uint32_t h[kGmSplit];
            split3(v, h);
            // every lane of the row writes a quarter of the kActRep copies
            for (int c2 = t; c2 < kActRep; c2 += 4) {
                uint16_t* o = A.act_h + ((size_t)(c2 * nseg + sd.row0) * kGmSplit) * arow + j;
#pragma unroll
                for (int n = 0; n < kGmSplit; ++n) o[(size_t)n * arow] = (uint16_t)h[n];
            }
        }
    }

    // ---- every CTA's activations are written: grid-wide barrier ---------------------------------
    DNB_STAMP(11);
    __syncthreads();
    if (tid == 0) flags[0] = grid_barrier(A, ROUTED ? flags[1] != 0 : true) ? 1 : 0;
    __syncthreads();
    const bool passed = flags[0] != 0;
    DNB_STAMP(12);

    // ---- all segments' activations (one of the kActRep copies) into shared memory ---------------
    if (passed) {
        const uint4* src = reinterpret_cast<const uint4*>(A.act_h + (size_t)(blockIdx.x % kActRep) * nseg * kGmSplit * arow);
        uint4* dst = reinterpret_cast<uint4*>(acts);
        const int n16 = nseg * kGmSplit * arow / 8;
        for (int i = tid; i < n16; i += kFdThreads) dst[i] = __ldcg(src + i);
    }
    __syncthreads();
    // Every thread waits for the down rows: the CTA must not end with the copies in flight.
    const bool dn_ok = mbar_wait_bounded(bars + 7, 0, A.status) && passed && ready;
    DNB_STAMP(13);

    // ---- down: warp = (unit, expert pair, half of K) -----------------------------------------------
    {
        const int u = warp / (2 * kFdPairs), rem = warp % (2 * kFdPairs), p = rem >> 1, kh = rem & 1;
        const int sa = 2 * p, sb = 2 * p + 1;
        const bool two = sb < nseg;
        if (dn_ok && u < my_units && sa < nseg) {
            const uint8_t* ra = wdn + ((size_t)(u * kFdSegs + sa) * 8 + g) * A.rb_dn;
            const uint8_t* rbp = wdn + ((size_t)(u * kFdSegs + (two ? sb : sa)) * 8 + g) * A.rb_dn;
            // B column g: columns 0-2 = the first expert's bf16 triple, 4-6 = the second's, 3 and 7 = zero
            const int n = g & 3, which = g >> 2;
            const bool has_col = n < kGmSplit && (which == 0 || two);
            const uint16_t* xb = acts + ((size_t)((which ? sb : sa) * kGmSplit + (n < kGmSplit ? n : 0))) * arow + 8 * t;
            const int nblk = ff >> 8, b0 = kh * (nblk >> 1), b1 = b0 + (nblk >> 1);
            float acc = 0.f;
            for (int b = b0; b < b1; ++b) {
                const uint8_t* ba = ra + b * 98;
                const uint8_t* bb = rbp + b * 98;
                const float da = h2f(ld16(ba)) * 0.25f, db = h2f(ld16(bb)) * 0.25f;
#pragma unroll 2
                for (int ib = 0; ib < 8; ++ib) {
                    uint4 y = make_uint4(0u, 0u, 0u, 0u);
                    if (has_col) y = *reinterpret_cast<const uint4*>(xb + (b * 8 + ib) * 32);
                    float c[4];
                    uint32_t auxa, auxb;
                    iq3_subblock_mma(ba, bb, ib, t, lutp, y, c, auxa, auxb);
                    // lanes t = 0, 1 keep the first expert's columns (rows 0-7), t = 2, 3 the second's (rows 8-15)
                    const float mine = t < 2 ? c[0] + c[1] : c[2] + c[3];
                    const float sc = t < 2 ? iq3_scale(da, auxa) : iq3_scale(db, auxb);
                    acc = fmaf(sc, mine, acc);
                }
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            float* hq = hp + (size_t)(u * 2 + kh) * kFdSegs * 8;
            if (t == 0) hq[sa * 8 + g] = acc;
            if (t == 2 && two) hq[sb * 8 + g] = acc;
        }
    }
    DNB_STAMP(14);
    __syncthreads();
    if (tid < kFdUnits * 8 && dn_ok) {
        const int u = tid >> 3, row = tid & 7;
        if (u < my_units) {
            const float* h0 = hp + (size_t)(u * 2) * kFdSegs * 8 + row;
            const float* h1 = h0 + kFdSegs * 8;
            float acc = 0.f;
            for (int s = 0; s < A.k; ++s) acc = __fadd_rn(acc, __fmul_rn(ws[s], h0[s * 8] + h1[s * 8]));
            if (A.has_shared) {
                const float v = h0[A.k * 8] + h1[A.k * 8];
                const bool scaled = ROUTED ? A.shared_gate_row != nullptr : A.shcoef != nullptr;
                acc = __fadd_rn(acc, scaled ? __fmul_rn(v, ws[A.k]) : v);
            }
            const int r = (blockIdx.x + u * gridDim.x) * 8 + row;
            if (A.residual) acc = __fadd_rn(resid, acc);
            A.out[r] = acc;
        }
    }
    DNB_STAMP(15);
}

bool decode_fused_fits(const dnb_ctx* c, int nseg, int e, int ff) {
    if (nseg < 1 || nseg > kFdSegs || e % (256 * kGmKs) || ff % 512 || e % 8) return false;
    const int grid = c->sm_count;
    if ((long)grid * kGmGroups < (long)nseg * (ff / kGmRows) || (long)grid * kFdUnits < e / 8) return false;
    return true;
}

// halves of the activation area: the bf16 triples of all segments, or (ROUTED) the CTA's router rows if they need more
static size_t fused_acts_halves(int nseg, int e, int ff, bool routed) {
    size_t h = (size_t)nseg * kGmSplit * (ff + kFdPad);
    if (routed) h = std::max(h, (size_t)kFdRouterRows * e * 2);
    return (h + 7) / 8 * 8;
}

static size_t fused_smem(int nseg, int e, int ff, bool routed) {
    const size_t rb_gu = row_bytes(T_IQ3_XXS, e), rb_dn = row_bytes(T_IQ3_XXS, ff);
    return kFdHeader + sizeof(Iq3Tables) + (size_t)kGmGroups * 2 * kGmRows * rb_gu +
           (size_t)kFdUnits * kFdSegs * 8 * rb_dn + (size_t)e * sizeof(float) + (size_t)kGmSplit * e * sizeof(uint16_t) +
           fused_acts_halves(nseg, e, ff, routed) * sizeof(uint16_t) +
           (size_t)(kGmGroups * kGmKs * 16 + kFdUnits * 2 * kFdSegs * 8 + 16) * sizeof(float) +
           (routed ? 2 * kFdSegs * sizeof(SegDesc) + sizeof(RouteSmem) + 16 : 0);
}

// halves the caller must provide at act_h
size_t decode_fused_act_halves(int nseg, int ff) { return (size_t)kActRep * nseg * kGmSplit * (ff + kFdPad); }

template <bool ROUTED>
static int launch_fused_t(dnb_ctx* c, cudaStream_t st, FusedArgs& A, size_t smem, const char* pname) {
    int rc = upload_tables_m(c->device);
    if (rc != DNB_OK) return rc;
    if (c->device < 0 || c->device >= 64) return DNB_DECLINED;
    static SmemGrant grant;
    if (grant.got[c->device] < smem)  // first use on this device: also pin the carve-out the router kernel shares
        DNB_CUDA(cudaFuncSetAttribute(decode_fused_kernel<ROUTED>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                      cudaSharedmemCarveoutMaxShared));
    DNB_CUDA(grant_smem(grant, c->device, decode_fused_kernel<ROUTED>, smem));
    // The grid barrier needs every CTA resident at once: one per SM.  Ask the runtime, once per
    // device and shared-memory size, whether a CTA of this size fits an SM at all.
    static size_t occ_ok[64] = {0};
    if (occ_ok[c->device] != smem) {
        int per_sm = 0;
        DNB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_fused_kernel<ROUTED>, kFdThreads, smem));
        if (per_sm < 1) return DNB_DECLINED;
        occ_ok[c->device] = smem;
    }
    A.status = c->status;
    A.barrier_polls = c->barrier_polls;
    A.barrier_bias = c->barrier_bias;
    ProfScope prof_(c, st, pname);
    DNB_CUDA(launch_k(decode_fused_kernel<ROUTED>, dim3(c->sm_count), dim3(kFdThreads), smem, st, c->use_pdl, A));
    c->launches++;
    return DNB_OK;
}

// Gate/up + down of a one-token block whose matrices are all IQ3_XXS.  DNB_DECLINED when the
// shape does not fit (nothing has been launched then).
int launch_decode_fused(dnb_ctx* c, cudaStream_t st, const SegDesc* seg_gu, const SegDesc* seg_dn, int nseg, int k,
                        bool has_shared, int e, int ff, const float* x, const float* x_perm, float* act, void* act_h,
                        const float* wts, const float* shcoef, const float* residual, float* out, unsigned long long* gbar) {
    if (!decode_fused_fits(c, nseg, e, ff) || !gbar || !act_h) return DNB_DECLINED;
    const size_t smem = fused_smem(nseg, e, ff, false);
    if (smem > 220 * 1024) return DNB_DECLINED;
    FusedArgs A = {};
    A.seg_gu = seg_gu; A.seg_dn = seg_dn; A.nseg = nseg; A.k = k; A.has_shared = has_shared ? 1 : 0;
    A.e = e; A.ff = ff; A.rb_gu = (int)row_bytes(T_IQ3_XXS, e); A.rb_dn = (int)row_bytes(T_IQ3_XXS, ff);
    A.acts_halves = (int)fused_acts_halves(nseg, e, ff, false);
    A.x = x; A.x_perm = x_perm; A.act = act; A.act_h = reinterpret_cast<uint16_t*>(act_h);
    A.wts = wts; A.shcoef = shcoef; A.residual = residual; A.out = out; A.gbar = gbar;
    return launch_fused_t<false>(c, st, A, smem, "decode_gate_up_down");
}

// The whole one-token block (router included) of an all-IQ3_XXS layer in one launch.
// DNB_DECLINED when the shape does not fit (nothing has been launched then).
int launch_decode_block(dnb_ctx* c, cudaStream_t st, const Model& M, const Layer& L, Workspace& w, bool fold_shared,
                        const float* h, const float* residual, float* out, unsigned long long* gbar) {
    const int nseg = M.k + (fold_shared ? 1 : 0);
    if (!decode_fused_fits(c, nseg, M.e, M.ff) || !gbar || !w.act_h || !L.router_w) return DNB_DECLINED;
    if (M.ne > 32 * kFdWarps || M.ne > 1024 || M.k > 32 || M.k >= kFdSegs + (fold_shared ? 0 : 1)) return DNB_DECLINED;
    if ((M.ne + c->sm_count - 1) / c->sm_count > kFdRouterRows) return DNB_DECLINED;
    if (M.e % 4 || (((uintptr_t)h) & 15) || (((uintptr_t)L.router_w) & 15) || (L.norm_w && (((uintptr_t)L.norm_w) & 15)))
        return DNB_DECLINED;  // bulk copies move 16-byte units
    // the down-row area, reused before the routing is known, must hold the input row and the norm weights
    if ((size_t)2 * M.e * sizeof(float) > (size_t)kFdUnits * kFdSegs * 8 * row_bytes(T_IQ3_XXS, M.ff)) return DNB_DECLINED;
    const size_t smem = fused_smem(nseg, M.e, M.ff, true);
    if (smem > 224 * 1024) return DNB_DECLINED;
    FusedArgs A = {};
    A.nseg = nseg; A.k = M.k; A.has_shared = fold_shared ? 1 : 0;
    A.e = M.e; A.ff = M.ff; A.rb_gu = (int)row_bytes(T_IQ3_XXS, M.e); A.rb_dn = (int)row_bytes(T_IQ3_XXS, M.ff);
    A.acts_halves = (int)fused_acts_halves(nseg, M.e, M.ff, true);
    A.act = w.act; A.act_h = w.act_h; A.residual = residual; A.out = out; A.gbar = gbar;
    A.h = h; A.norm_w = L.norm_w; A.eps = M.eps; A.router_w = L.router_w; A.router_bias = L.router_bias;
    A.ne = M.ne; A.norm_topk = M.norm_topk; A.logits = w.logits;
    A.gate = L.m[0].dev; A.up = L.m[1].dev; A.down = L.m[2].dev;
    A.eb_g = L.m[0].expert_bytes; A.eb_u = L.m[1].expert_bytes; A.eb_d = L.m[2].expert_bytes;
    A.sg = fold_shared ? L.m[3].dev : nullptr; A.su = fold_shared ? L.m[4].dev : nullptr; A.sdn = fold_shared ? L.m[5].dev : nullptr;
    A.shared_gate_row = fold_shared ? L.shared_gate_row : nullptr;
    A.sels_out = w.sels; A.wts_out = w.wts; A.xn_out = w.xn;
    return launch_fused_t<true>(c, st, A, smem, "decode_block");
}

}  // namespace dnb
