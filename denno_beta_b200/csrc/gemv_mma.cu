// One-token IQ3_XXS gate/up GEMV with the dot products on the tensor cores.
//
// The register decode of gemv_bulk.cu spends about ten instructions per weight: with
// 23 M weights per launch the kernel is bound by instruction issue, not by memory.
// Here a warp decodes weights straight into the A fragment of mma.sync.m16n8k16
// (f16 x f16 -> f32): sixteen matrix rows (eight gate rows, eight up rows of one
// expert) against the activation vector, which occupies three of the eight B
// columns as an exact three-way f16 split of its fp32 values (x = hi + lo + lo2),
// so the products lose nothing against an fp32 FMA chain.  A codebook entry is four
// small integers (<= 62), exact in f16; the lookup table holds them as two f16 pairs,
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
#include <cuda_fp16.h>

#include "dnb_common.cuh"
#include "formats.cuh"
#include "bulk.cuh"
#include "dnb_iq_tables.h"

namespace dnb {

constexpr int kGmRows = 8;     // rows of one matrix per group (x2 matrices = the 16 mma rows)
constexpr int kGmKs = 4;       // warps that split K within a group
constexpr int kGmGroups = 5;   // groups a CTA can hold
constexpr int kGmThreads = kGmGroups * kGmKs * 32;
constexpr int kGmSplit = 3;    // f16 terms per activation value

// IQ3_XXS codebook as f16 pairs: entry e of copy r at [e * kLutRep + r]; .x = elements 0,1, .y = elements 2,3
__device__ __align__(16) uint2 g_grid3xxs_h2[256 * kLutRep];
static bool g_tables_m[64] = {false};

static int upload_tables_m(int device) {
    if (device < 0 || device >= 64) return DNB_ERR_ARG;
    if (g_tables_m[device]) return DNB_OK;
    static uint2 rep[256 * kLutRep];
    for (int e = 0; e < 256; ++e) {
        const uint32_t w = dnb_iq3xxs_grid[e];
        uint32_t h[4];
        for (int j = 0; j < 4; ++j) h[j] = __half_as_ushort(__float2half((float)((w >> (8 * j)) & 0xFFu)));
        for (int r = 0; r < kLutRep; ++r) rep[e * kLutRep + r] = make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16));
    }
    DNB_CUDA(cudaMemcpyToSymbol(g_grid3xxs_h2, rep, sizeof(rep)));
    g_tables_m[device] = true;
    return DNB_OK;
}

__device__ __forceinline__ uint32_t f16_sat(float v) {
    uint16_t h;
    asm("cvt.rn.satfinite.f16.f32 %0, %1;" : "=h"(h) : "f"(v));
    return h;
}
__device__ __forceinline__ float silu_m(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float f16_val(uint32_t h) { return __half2float(__ushort_as_half((unsigned short)h)); }

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Eight weights of one IQ3_XXS sub-block as four signed f16 pairs (without the scale):
// `idx` = the two codebook indices of this lane's quarter, `code` = its 7 sign bits.
__device__ __forceinline__ void iq3_pairs(const uint2* lutp, uint32_t idx, uint32_t code, uint32_t (&p)[4]) {
    const uint32_t sg = code | ((__popc(code) & 1u) << 7);  // bit 7 makes the number of minus signs even
    const uint2 g1 = lutp[(idx & 0xFFu) * kLutRep], g2 = lutp[(idx >> 8) * kLutRep];
    p[0] = g1.x ^ ((sg * 0x40008000u) & 0x80008000u);
    p[1] = g1.y ^ ((sg * 0x10002000u) & 0x80008000u);
    p[2] = g2.x ^ ((sg * 0x04000800u) & 0x80008000u);
    p[3] = g2.y ^ ((sg * 0x01000200u) & 0x80008000u);
}

// Dynamic shared memory: [8 mbarriers | pad to 128][codebook 32 KB][groups x (8 gate rows, 8 up rows)]
//                        [x fp32 (staging)][x as kGmSplit f16 vectors][K-partials]
__global__ void __launch_bounds__(kGmThreads, 1)
gate_up_mma_kernel(const SegDesc* __restrict__ seg, int nseg, int n_in, int n_out, int rb, int ngroups,
                   const float* __restrict__ x, const float* __restrict__ x_perm, float* __restrict__ out,
                   float* __restrict__ out_perm, int perm_type, int* status) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);  // [0..4] groups, [5] codebook, [6] x
    uint2* lut = reinterpret_cast<uint2*>(smem + 128);
    const int mat_bytes = kGmRows * rb;  // 8 rows of IQ3_XXS: a multiple of 16 bytes
    uint8_t* wbase = smem + 128 + sizeof(uint2) * 256 * kLutRep;
    float* xf = reinterpret_cast<float*>(wbase + (size_t)kGmGroups * 2 * mat_bytes);
    __half* xh = reinterpret_cast<__half*>(xf + n_in);
    float* red = reinterpret_cast<float*>(xh + (size_t)kGmSplit * n_in);  // [group][ks][16]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int q = warp / kGmKs, ks = warp % kGmKs;
    if (tid == 0) {
        for (int i = 0; i < kGmGroups + 2; ++i) mbar_init(bars + i, 1);
        mbar_fence_init();
        mbar_expect_tx(bars + kGmGroups, (uint32_t)(sizeof(uint2) * 256 * kLutRep));
        bulk_g2s(lut, g_grid3xxs_h2, (uint32_t)(sizeof(uint2) * 256 * kLutRep), bars + kGmGroups);
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
    // x -> three f16 vectors in natural element order
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
            float r[2] = {v.x, v.y};
            uint32_t h[kGmSplit][2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
#pragma unroll
                for (int n = 0; n < kGmSplit; ++n) {
                    h[n][e] = f16_sat(r[e]);
                    r[e] -= f16_val(h[n][e]);
                }
            }
#pragma unroll
            for (int n = 0; n < kGmSplit; ++n)
                *reinterpret_cast<uint32_t*>(xh + (size_t)n * n_in + i) = h[n][0] | (h[n][1] << 16);
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
        const uint2* lutp = lut + (lane & (kLutRep - 1));
        const __half* xb = xh + (size_t)(g < kGmSplit ? g : 0) * n_in + 8 * t;
        const int bpw = (n_in >> 8) / kGmKs;
        for (int b = ks * bpw; b < (ks + 1) * bpw; ++b) {
            const uint8_t* bg = rowg + b * 98;
            const uint8_t* bu = rowu + b * 98;
            const float dg = h2f(ld16(bg)) * 0.25f, du = h2f(ld16(bu)) * 0.25f;
#pragma unroll 2
            for (int ib = 0; ib < 8; ++ib) {
                uint4 y = make_uint4(0u, 0u, 0u, 0u);
                if (g < kGmSplit) y = *reinterpret_cast<const uint4*>(xb + (b * 8 + ib) * 32);
                const uint32_t auxg = ld16(bg + 66 + 4 * ib) | (ld16(bg + 68 + 4 * ib) << 16);
                const uint32_t auxu = ld16(bu + 66 + 4 * ib) | (ld16(bu + 68 + 4 * ib) << 16);
                const uint32_t idg = ld16(bg + 2 + 8 * ib + 2 * t), idu = ld16(bu + 2 + 8 * ib + 2 * t);
                uint32_t p[4], u4[4];
                iq3_pairs(lutp, idg, (auxg >> (7 * t)) & 127u, p);
                iq3_pairs(lutp, idu, (auxu >> (7 * t)) & 127u, u4);
                float c[4] = {0.f, 0.f, 0.f, 0.f};
                mma_f16(c, p[0], u4[0], p[1], u4[1], y.x, y.y);
                mma_f16(c, p[2], u4[2], p[3], u4[3], y.z, y.w);
                // d * (0.5 + s) * 0.5 = (d / 4) * (2 s + 1), exact in fp32 either way (kquant.rs:667)
                const float dbg = dg * (float)(2u * (auxg >> 28) + 1u), dbu = du * (float)(2u * (auxu >> 28) + 1u);
                accg = fmaf(dbg, c[0] + c[1], accg);
                accu = fmaf(dbu, c[2] + c[3], accu);
            }
        }
        // lane t = 0 holds the hi and lo columns, t = 1 the lo2 column, t = 2, 3 nothing
        accg += __shfl_xor_sync(0xffffffffu, accg, 1);
        accu += __shfl_xor_sync(0xffffffffu, accu, 1);
    }
    float* rq = red + (size_t)q * kGmKs * 16;
    if (t == 0) {
        rq[ks * 16 + g] = accg;
        rq[ks * 16 + 8 + g] = accu;
    }
    asm volatile("bar.sync %0, %1;" ::"r"(q + 1), "r"(kGmKs * 32) : "memory");
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
    const size_t smem = 128 + sizeof(uint2) * 256 * kLutRep + (size_t)kGmGroups * 2 * kGmRows * rb +
                        (size_t)n_in * sizeof(float) + (size_t)kGmSplit * n_in * sizeof(__half) +
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
