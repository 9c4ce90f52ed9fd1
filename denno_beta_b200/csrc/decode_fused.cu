// One-token MoE block after the router, as ONE kernel: gate/up GEMV with SwiGLU, a
// grid-wide barrier, down GEMV with the weighted sum over the experts.  IQ3_XXS only.
//
// Why one kernel: with two, the down kernel's CTAs cannot all be resident beside the
// gate/up kernel (registers, shared memory), so a good part of the down weights is
// requested only after gate/up has ended and their arrival (~1 us) plus the launch
// hand-over sits on the critical path of a 25 us block.  Here one CTA per SM requests
// ALL its weights (gate, up and down rows, ~90 KB) the moment the router has finished,
// and the down phase finds its rows already in shared memory.
//
// Both phases run on mma.sync.m16n8k16 as gemv_mma.cu describes (weights decoded
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
// The activations cross CTAs through global memory: every CTA writes its SwiGLU
// outputs as bf16 triples into kActRep identical copies (so that the 148 readers do not
// all hit the same L2 lines), arrives at a counter that only grows, and waits (bounded) until
// the counter has reached the launch's share.  All CTAs are resident: one per SM, the grid
// never exceeds the SM count, and the kernel that follows in the stream is not released
// before every CTA of this one has started.  A wait that runs out sets the status word
// and the CTA skips the down phase; nothing can hang.
#include "iq3_mma.cuh"

namespace dnb {

constexpr int kFdUnits = 2;                         // down units (8 output rows) per CTA
constexpr int kFdPairs = 6;                         // expert pairs per unit: up to 12 segments
constexpr int kFdWarps = kFdUnits * kFdPairs * 2;   // x2: halves of K
constexpr int kFdThreads = kFdWarps * 32;
constexpr int kFdSegs = 2 * kFdPairs;
constexpr int kFdPad = 8;                           // halves of padding per activation row (bank spread)
static_assert(kFdWarps >= kGmGroups * kGmKs, "the gate/up phase needs its warps");

struct FusedArgs {
    const SegDesc* seg_gu;   // [nseg] gate/up matrices
    const SegDesc* seg_dn;   // [nseg] down matrices (wa)
    int nseg, k, has_shared;
    int e, ff;               // hidden width, expert width
    int rb_gu, rb_dn;        // bytes per row of the gate/up and the down matrices
    const float* x;          // normalised hidden row (natural order)
    const float* x_perm;     // or: kActRep slot-ordered copies of it
    float* act;              // [nseg][ff] SwiGLU outputs (fp32, for inspection)
    uint16_t* act_h;           // [kActRep][nseg][3][ff + kFdPad]
    const float* wts;        // [k] routing weights
    const float* shcoef;     // shared-expert coefficient or null
    const float* residual;   // or null
    float* out;              // [e]
    unsigned long long* gbar;  // arrivals of all launches so far
    int* status;
    int barrier_polls;         // acquire loads before the barrier gives up
    unsigned int barrier_bias; // test hook: added to the arrival count waited for (0 in production)
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

// Dynamic shared memory:
// [8 mbarriers | flags, pad to 128][codebook 32 KB][gate/up rows][down rows][x fp32][x bf16 x3]
// [activations bf16 x3, all segments][gate/up K-partials][down partials][routing weights]
__global__ void __maxnreg__(64) decode_fused_kernel(const FusedArgs A) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);  // [0..4] gate/up groups, [5] codebook, [6] x, [7] down rows
    int* flags = reinterpret_cast<int*>(smem + 64);      // [0] barrier passed
    Iq3Tables* lut = reinterpret_cast<Iq3Tables*>(smem + 128);
    const int e = A.e, ff = A.ff, nseg = A.nseg;
    const int gu_bytes = kGmRows * A.rb_gu, dn_bytes = 8 * A.rb_dn;  // multiples of 16
    const int arow = ff + kFdPad;
    uint8_t* wgu = smem + 128 + sizeof(Iq3Tables);
    uint8_t* wdn = wgu + (size_t)kGmGroups * 2 * gu_bytes;
    float* xf = reinterpret_cast<float*>(wdn + (size_t)kFdUnits * kFdSegs * dn_bytes);
    uint16_t* xh = reinterpret_cast<uint16_t*>(xf + e);
    uint16_t* acts = xh + (size_t)kGmSplit * e;
    float* red = reinterpret_cast<float*>(acts + (size_t)nseg * kGmSplit * arow);  // [group][ks][16]
    float* hp = red + kGmGroups * kGmKs * 16;                                      // [unit][half][seg][8]
    float* ws = hp + kFdUnits * 2 * kFdSegs * 8;                                   // [nseg]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    if (tid == 0) {
        for (int i = 0; i < 8; ++i) mbar_init(bars + i, 1);
        mbar_fence_init();
        mbar_expect_tx(bars + 5, (uint32_t)(sizeof(Iq3Tables)));
        bulk_g2s(lut, &g_iq3_tables, (uint32_t)(sizeof(Iq3Tables)), bars + 5);
        flags[0] = 0;
    }
    __syncthreads();
    pdl_wait();  // segment tables, routing weights and x come from the router kernel
    pdl_launch_dependents();

    // ---- requests: gate/up rows per group, all down rows, x ------------------------------
    const int q = warp / kGmKs, ks = warp % kGmKs;
    const int gps = ff / kGmRows;
    const int gid = blockIdx.x + q * gridDim.x;
    const int gs = gid / gps, gr0 = (gid - gs * gps) * kGmRows;
    bool gactive = q < kGmGroups && gs < nseg;
    SegDesc sd = SegDesc{nullptr, nullptr, 0u, 0u};
    if (gactive) sd = A.seg_gu[gs];
    gactive = gactive && sd.m > 0;
    uint8_t* wq = wgu + (size_t)(q < kGmGroups ? q : 0) * 2 * gu_bytes;
    if (ks == 0 && lane == 0 && gactive) {
        mbar_expect_tx(bars + q, (uint32_t)(2 * gu_bytes));
        bulk_g2s(wq, sd.wa + (size_t)gr0 * A.rb_gu, (uint32_t)gu_bytes, bars + q);
        bulk_g2s(wq + gu_bytes, sd.wb + (size_t)gr0 * A.rb_gu, (uint32_t)gu_bytes, bars + q);
    }
    const int nunits_dn = e / 8;
    int my_units = 0;
    for (int u = 0; u < kFdUnits; ++u) my_units += (blockIdx.x + u * gridDim.x) < nunits_dn ? 1 : 0;
    if (tid == 32 && A.x_perm) {
        mbar_expect_tx(bars + 6, (uint32_t)(e * sizeof(float)));
        bulk_g2s(xf, A.x_perm + (size_t)(blockIdx.x % kActRep) * e, (uint32_t)(e * sizeof(float)), bars + 6);
    }
    float resid = 0.f;  // the combine threads fetch their residual element now, off the critical path
    if (A.residual && tid < kFdUnits * 8 && (tid >> 3) < my_units)
        resid = A.residual[(blockIdx.x + (tid >> 3) * gridDim.x) * 8 + (tid & 7)];
    if (tid >= 96 && tid < 96 + nseg) {
        const int s = tid - 96;
        ws[s] = s < A.k ? A.wts[s] : (A.shcoef ? A.shcoef[0] : 1.0f);
    }

    // ---- x -> three bf16 vectors in natural element order ------------------------------------
    bool ready = true;
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
    // The down rows are asked for only now, behind the gate/up rows: the two together are ~2 us of
    // HBM time, and the gate/up phase needs its share first.  One lane per (unit, segment), in a
    // warp that has no gate/up work.
    if (warp == kFdWarps - 1) {
        if (lane == 0) mbar_expect_tx(bars + 7, (uint32_t)(my_units * nseg * dn_bytes));
        __syncwarp();
        if (lane < my_units * nseg) {
            const int u = lane / nseg, s = lane - u * nseg;
            const size_t off = (size_t)(blockIdx.x + u * gridDim.x) * dn_bytes;
            bulk_g2s(wdn + (size_t)(u * kFdSegs + s) * dn_bytes, A.seg_dn[s].wa + off, (uint32_t)dn_bytes, bars + 7);
        }
    }
    ready = mbar_wait_bounded(bars + 5, 0, A.status) && ready;
    const Iq3Lane lutp(lut, lane);

    // ---- gate/up: 8 gate + 8 up rows per group, four warps split K -----------------------------
    if (gactive) {  // all four warps of a group agree
        const bool ok = mbar_wait_bounded(bars + q, 0, A.status) && ready;
        float accg = 0.f, accu = 0.f;
        if (ok) {
            const uint8_t* rowg = wq + g * A.rb_gu;
            const uint16_t* xb = xh + (size_t)(g < kGmSplit ? g : 0) * e + 8 * t;
            const int bpw = (e >> 8) / kGmKs;
            gate_up_warp(rowg, rowg + gu_bytes, lutp, xb, g < kGmSplit, ks * bpw, (ks + 1) * bpw, t, accg, accu);
        }
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
    __syncthreads();
    if (tid == 0) {
        // The counter only grows: launch number n of this context waits for (n + 1) * gridDim.x arrivals
        // (the grid is the SM count, the same for every launch of a context).  The release half of the
        // atomic publishes this CTA's stores (the bar.sync above ordered them before it), the acquire
        // load below makes the other CTAs' stores visible.
        const unsigned long long ticket = atom_add_acq_rel(A.gbar, 1ull);
        const unsigned long long target = (ticket / gridDim.x + 1ull) * gridDim.x + A.barrier_bias;
        bool pass = ticket + 1ull == target;
        for (int i = 0; i < A.barrier_polls && !pass; ++i) pass = ld_acquire_u64(A.gbar) >= target;  // ~0.2 s at most by default
        if (!pass) status_set(A.status, 23);
        flags[0] = pass ? 1 : 0;
    }
    __syncthreads();
    const bool passed = flags[0] != 0;

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
                acc = __fadd_rn(acc, A.shcoef ? __fmul_rn(v, ws[A.k]) : v);
            }
            const int r = (blockIdx.x + u * gridDim.x) * 8 + row;
            if (A.residual) acc = __fadd_rn(resid, acc);
            A.out[r] = acc;
        }
    }
}

bool decode_fused_fits(const dnb_ctx* c, int nseg, int e, int ff) {
    if (nseg < 1 || nseg > kFdSegs || e % (256 * kGmKs) || ff % 512 || e % 8) return false;
    const int grid = c->sm_count;
    if ((long)grid * kGmGroups < (long)nseg * (ff / kGmRows) || (long)grid * kFdUnits < e / 8) return false;
    return true;
}

static size_t fused_smem(int nseg, int e, int ff) {
    const size_t rb_gu = row_bytes(T_IQ3_XXS, e), rb_dn = row_bytes(T_IQ3_XXS, ff);
    return 128 + sizeof(Iq3Tables) + (size_t)kGmGroups * 2 * kGmRows * rb_gu +
           (size_t)kFdUnits * kFdSegs * 8 * rb_dn + (size_t)e * sizeof(float) + (size_t)kGmSplit * e * sizeof(uint16_t) +
           (size_t)nseg * kGmSplit * (ff + kFdPad) * sizeof(uint16_t) +
           (size_t)(kGmGroups * kGmKs * 16 + kFdUnits * 2 * kFdSegs * 8 + 16) * sizeof(float);
}

// halves the caller must provide at act_h
size_t decode_fused_act_halves(int nseg, int ff) { return (size_t)kActRep * nseg * kGmSplit * (ff + kFdPad); }

// Gate/up + down of a one-token block whose matrices are all IQ3_XXS.  DNB_DECLINED when the
// shape does not fit (nothing has been launched then).
int launch_decode_fused(dnb_ctx* c, cudaStream_t st, const SegDesc* seg_gu, const SegDesc* seg_dn, int nseg, int k,
                        bool has_shared, int e, int ff, const float* x, const float* x_perm, float* act, void* act_h,
                        const float* wts, const float* shcoef, const float* residual, float* out, unsigned long long* gbar) {
    if (!decode_fused_fits(c, nseg, e, ff) || !gbar || !act_h) return DNB_DECLINED;
    const size_t smem = fused_smem(nseg, e, ff);
    if (smem > 220 * 1024) return DNB_DECLINED;
    int rc = upload_tables_m(c->device);
    if (rc != DNB_OK) return rc;
    static SmemGrant grant;
    if (c->device >= 0 && c->device < 64 && grant.got[c->device] < smem)  // first use on this device: also pin the carve-out the router kernel shares
        DNB_CUDA(cudaFuncSetAttribute(decode_fused_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                      cudaSharedmemCarveoutMaxShared));
    DNB_CUDA(grant_smem(grant, c->device, decode_fused_kernel, smem));
    // The grid barrier needs every CTA resident at once: one per SM.  Ask the runtime, once per
    // device and shared-memory size, whether a CTA of this size fits an SM at all.
    static size_t occ_ok[64] = {0};
    if (occ_ok[c->device] != smem) {
        int per_sm = 0;
        DNB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_fused_kernel, kFdThreads, smem));
        if (per_sm < 1) return DNB_DECLINED;
        occ_ok[c->device] = smem;
    }
    FusedArgs A;
    A.seg_gu = seg_gu; A.seg_dn = seg_dn; A.nseg = nseg; A.k = k; A.has_shared = has_shared ? 1 : 0;
    A.e = e; A.ff = ff; A.rb_gu = (int)row_bytes(T_IQ3_XXS, e); A.rb_dn = (int)row_bytes(T_IQ3_XXS, ff);
    A.x = x; A.x_perm = x_perm; A.act = act; A.act_h = reinterpret_cast<uint16_t*>(act_h);
    A.wts = wts; A.shcoef = shcoef; A.residual = residual; A.out = out; A.gbar = gbar; A.status = c->status;
    A.barrier_polls = c->barrier_polls; A.barrier_bias = c->barrier_bias;
    ProfScope prof_(c, st, "decode_gate_up_down");
    DNB_CUDA(launch_k(decode_fused_kernel, dim3(c->sm_count), dim3(kFdThreads), smem, st, c->use_pdl, A));
    c->launches++;
    return DNB_OK;
}

}  // namespace dnb
