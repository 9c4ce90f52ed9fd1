// One-token IQ3_XXS gate/up GEMV with the dot products on the tensor cores.
//
// The register decode of gemv_bulk.cu spends about ten instructions per weight: with
// 23 M weights per launch the kernel is bound by instruction issue, not by memory.
// Here a warp decodes weights straight into the A fragment of mma.sync.m16n8k16
// (bf16 x bf16 -> f32): sixteen matrix rows (eight gate rows, eight up rows of one
// expert) against the activation vector, which occupies three of the eight B
// columns as an exact three-way bf16 split of its fp32 values (x = hi + lo + lo2: 3 x 8
// mantissa bits, fp32's exponent range, so nothing can overflow),
// so the products lose nothing against an fp32 FMA chain.  A codebook entry is four
// small integers (<= 62), exact in bf16; the lookup table holds them as two bf16 pairs,
// the sign bits are xor-ed in, and the sub-block scale multiplies the accumulator of
// the sub-block's two mma instructions in fp32.  Per weight that leaves a quarter of
// the instructions: no int-to-float conversion, no FMA, one shared-memory read of
// the activations per sixteen weights instead of one per weight.
//
// Work split: a group is 8 consecutive rows of one expert (gate and up); four warps
// share a group and split K; a CTA holds up to five groups and there is one CTA per
// SM, so the codebook and the activation split are staged once per SM.  Weights
// arrive by cp.async.bulk, one pair of copies per group, each group on its own
// mbarrier; the four K-partials of a group meet in shared memory and are added in
// a fixed order, so the result is bit-identical run to run.
//
// Block layout and decode: crates/denno-engine/src/kquant.rs:659-680 of the
// reference; kernels of this role there: kernels_exp_iq_v2.cu:259-319.
#include "iq3_mma.cuh"

namespace dnb {

// Dynamic shared memory: [8 mbarriers | pad to 128][codebook 32 KB][groups x (8 gate rows, 8 up rows)]
//                        [x fp32 (staging)][x as kGmSplit bf16 vectors][K-partials]
__global__ void __launch_bounds__(kGmThreads, 1)
gate_up_mma_kernel(const SegDesc* __restrict__ seg, int nseg, int n_in, int n_out, int rb, int ngroups,
                   const float* __restrict__ x, const float* __restrict__ x_perm, float* __restrict__ out,
                   float* __restrict__ out_perm, int perm_type, int* status) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);  // [0..4] groups, [5] codebook, [6] x
    Iq3Tables* lut = reinterpret_cast<Iq3Tables*>(smem + 128);
    const int mat_bytes = kGmRows * rb;  // 8 rows of IQ3_XXS: a multiple of 16 bytes
    uint8_t* wbase = smem + 128 + sizeof(Iq3Tables);
    float* xf = reinterpret_cast<float*>(wbase + (size_t)kGmGroups * 2 * mat_bytes);
    uint16_t* xh = reinterpret_cast<uint16_t*>(xf + n_in);
    float* red = reinterpret_cast<float*>(xh + (size_t)kGmSplit * n_in);  // [group][ks][16]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int q = warp / kGmKs, ks = warp % kGmKs;
    if (tid == 0) {
        for (int i = 0; i < kGmGroups + 2; ++i) mbar_init(bars + i, 1);
        mbar_fence_init();
        mbar_expect_tx(bars + kGmGroups, (uint32_t)(sizeof(Iq3Tables)));
        bulk_g2s(lut, &g_iq3_tables, (uint32_t)(sizeof(Iq3Tables)), bars + kGmGroups);
    }
    __syncthreads();
    pdl_wait();  // the segment table and x come from the router kernel
    pdl_launch_dependents();

    const int gps = n_out / kGmRows;
    const int gid = blockIdx.x + q * gridDim.x;
    const int s = gid / gps, r0 = (gid - s * gps) * kGmRows;
    bool active = gid < ngroups && s < nseg;
    SegDesc sd = SegDesc{nullptr, nullptr, 0u, 0u};
    if (active) sd = seg[s];
    active = active && sd.m > 0;
    uint8_t* wq = wbase + (size_t)q * 2 * mat_bytes;
    if (ks == 0 && lane == 0 && active) {
        mbar_expect_tx(bars + q, (uint32_t)(2 * mat_bytes));
        bulk_g2s(wq, sd.wa + (size_t)r0 * rb, (uint32_t)mat_bytes, bars + q);
        bulk_g2s(wq + mat_bytes, sd.wb + (size_t)r0 * rb, (uint32_t)mat_bytes, bars + q);
    }
    if (x_perm && tid == 32) {
        mbar_expect_tx(bars + kGmGroups + 1, (uint32_t)(n_in * sizeof(float)));
        bulk_g2s(xf, x_perm + (size_t)(blockIdx.x % kActRep) * n_in, (uint32_t)(n_in * sizeof(float)), bars + kGmGroups + 1);
    }
    // x -> three bf16 vectors in natural element order
    bool ready = true;
    if (x_perm) ready = mbar_wait_bounded(bars + kGmGroups + 1, 0, status);
    const int nunits = n_in >> 5;
    if (ready) {
        for (int i = 2 * tid; i < n_in; i += 2 * kGmThreads) {
            float2 v;
            if (x_perm) {
                const int u = i >> 5, sl = i & 31;  // 32 consecutive elements per unit (slot_of of this format)
                v = *reinterpret_cast<const float2*>(xf + ((((sl >> 2) * nunits + u) << 2) + (sl & 3)));
            } else {
                v = *reinterpret_cast<const float2*>(x + i);
            }
            uint32_t h0[kGmSplit], h1[kGmSplit];
            split3(v.x, h0);
            split3(v.y, h1);
#pragma unroll
            for (int n = 0; n < kGmSplit; ++n)
                *reinterpret_cast<uint32_t*>(xh + (size_t)n * n_in + i) = h0[n] | (h1[n] << 16);
        }
    }
    __syncthreads();
    // Every thread waits for the CTA-wide copies before it may leave.
    ready = mbar_wait_bounded(bars + kGmGroups, 0, status) && ready;
    if (!active) return;  // all four warps of a group agree
    const bool ok = mbar_wait_bounded(bars + q, 0, status) && ready;

    const int g = lane >> 2, t = lane & 3;
    float accg = 0.f, accu = 0.f;
    if (ok) {
        const uint8_t* rowg = wq + g * rb;
        const uint8_t* rowu = rowg + mat_bytes;
        const Iq3Lane lutp(lut, lane);
        const uint16_t* xb = xh + (size_t)(g < kGmSplit ? g : 0) * n_in + 8 * t;
        const int bpw = (n_in >> 8) / kGmKs;
        gate_up_warp(rowg, rowu, lutp, xb, g < kGmSplit, ks * bpw, (ks + 1) * bpw, t, accg, accu);
    }
    float* rq = red + (size_t)q * kGmKs * 16;
    if (t == 0) {
        rq[ks * 16 + g] = accg;
        rq[ks * 16 + 8 + g] = accu;
    }
    group_barrier(q);
    if (ks != 0 || !ok) return;
    float a = rq[g], bq = rq[8 + g];
#pragma unroll
    for (int k2 = 1; k2 < kGmKs; ++k2) {
        a += rq[k2 * 16 + g];
        bq += rq[k2 * 16 + 8 + g];
    }
    const float v = silu_m(a) * bq;
    const int j = r0 + g;
    if (t == 0) out[(size_t)sd.row0 * n_out + j] = v;
    if (out_perm) {  // the copies the next kernel's CTAs take whole, in its slot order
        const size_t rep = (size_t)nseg * n_out;
        float* o = out_perm + (size_t)sd.row0 * n_out + slot_index(perm_type, j, n_out >> 5);
#pragma unroll
        for (int c2 = t; c2 < kActRep; c2 += 4) o[c2 * rep] = v;
    }
}

// Declines (the caller then uses the register-decode kernel) unless the shape fits:
// whole 256-element blocks split evenly over the K warps, 8-row groups, at most
// kGmGroups groups per SM.
int launch_gate_up_mma(dnb_ctx* c, cudaStream_t st, const SegDesc* seg, int nseg, int n_in, int n_out, const float* x,
                       float* out, const char* pname, PermOut perm) {
    if (n_in % (256 * kGmKs) || n_out % 32 || nseg < 1) return DNB_DECLINED;
    const int rb = (int)row_bytes(T_IQ3_XXS, n_in);
    const int ngroups = nseg * (n_out / kGmRows);
    const int grid = ngroups < c->sm_count ? ngroups : c->sm_count;
    if ((long)grid * kGmGroups < ngroups) return DNB_DECLINED;
    const size_t smem = 128 + sizeof(Iq3Tables) + (size_t)kGmGroups * 2 * kGmRows * rb +
                        (size_t)n_in * sizeof(float) + (size_t)kGmSplit * n_in * sizeof(uint16_t) +
                        (size_t)kGmGroups * kGmKs * 16 * sizeof(float);
    if (smem > 200 * 1024) return DNB_DECLINED;
    int rc = upload_tables_m(c->device);
    if (rc != DNB_OK) return rc;
    static SmemGrant grant;
    DNB_CUDA(grant_smem(grant, c->device, gate_up_mma_kernel, smem));
    ProfScope prof_(c, st, pname);
    DNB_CUDA(launch_k(gate_up_mma_kernel, dim3(grid), dim3(kGmThreads), smem, st, c->use_pdl, seg, nseg, n_in, n_out, rb,
                      ngroups, x, (n_in % 4 == 0) ? perm.x_perm : nullptr, out, perm.base, perm.type, c->status));
    c->launches++;
    return DNB_OK;
}

}  // namespace dnb
