// Hyper-connection mix and combine either side of the MoE block (model/hyper.rs of the reference;
// call sites model/qwen4exp.rs:3722-3765: hc_mix_quant -> moe_ffn_quant -> hc_combine_inplace; GPU forms
// kernels/kernels_mix_*.cu).  A layer carries hc parallel residual streams of n_embd values per token:
//
//   mix      xn[s]    = rmsnorm(res[s]) * w_norm[s]                       per stream (tensor.rs:1125-1135)
//            raw      = w_down_inject @ concat_s xn[s]                    [low_rank + hc] rows of hc*n_embd
//            lo[r]    = silu(raw[r] / hc),  r < low_rank                  silu(v) = v * (1 / (1 + exp(-v)))
//            inject[s] = raw[low_rank + s] / hc                           (no silu)
//            gate     = w_up @ lo                                         [hc*n_embd] rows of low_rank
//            mixed[d] = (1/hc) * sum_s xn[s][d] * sigmoid(gate[s][d])     ascending s, 1/hc after the sum
//   block    = MoE block (mixed)                                          no further norm
//   combine  out[s][d] = res[s][d] + block[d] * (2 * sigmoid(inject[s]))
//
// The order of operations inside an element (division by hc after the matmul, the form of silu, the
// ascending-s sum) follows hyper.rs:13-36, which states it as the numeric contract; the dot products are
// lane-split with a fixed xor tree (deterministic; the CPU's are sequential, so they differ by rounding).
// Weights are kept as fp32 (the checkpoints store them as BF16, whose expansion to fp32 is exact).
#include "dnb_common.cuh"

namespace dnb {

struct HcLayer {
    int hc = 0, low_rank = 0;
    float* w_norm = nullptr;  // [hc][e]
    float* w_down = nullptr;  // [low_rank + hc][hc*e]
    float* w_up = nullptr;    // [hc*e][low_rank]
};
struct HcState {
    std::vector<HcLayer> layers;
    Scratch xn, raw, mixed, blk, res, out;  // device scratch, grow-only
    Scratch host_in, host_out;              // pinned staging of the host-buffer entry point
};

__device__ __forceinline__ float hc_sigmoid(float v) { return 1.0f / (1.0f + expf(-v)); }

// one CTA of 128 threads per (token, stream): the summation tree of rms_inv_128 (moe_kernels.cu)
__global__ void __launch_bounds__(128)
hc_norm_kernel(const float* __restrict__ res, const float* __restrict__ w_norm, float eps, int hc, int e, float* __restrict__ xn) {
    __shared__ float red[4];
    const int s = blockIdx.x % hc;
    const float* xr = res + (size_t)blockIdx.x * e;
    float ss = 0.f;
    for (int i = threadIdx.x; i < e; i += 128) ss = fmaf(xr[i], xr[i], ss);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    const float inv = 1.0f / sqrtf(((red[0] + red[1]) + (red[2] + red[3])) / (float)e + eps);
    const float* g = w_norm + (size_t)s * e;
    float* o = xn + (size_t)blockIdx.x * e;
    for (int i = threadIdx.x; i < e; i += 128) o[i] = __fmul_rn(__fmul_rn(xr[i], inv), g[i]);
}

// raw[t][r] = w_down[r] . xn[t]; then lo / inject as above.  One warp per row, up to 4 tokens per pass.
__global__ void __launch_bounds__(128)
hc_down_kernel(const float* __restrict__ w_down, const float* __restrict__ xn, int nt, int hc_dim, int low_rank, int hc,
               float* __restrict__ raw) {
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    const int rows = low_rank + hc;
    if (row >= rows) return;
    const float4* wr = reinterpret_cast<const float4*>(w_down + (size_t)row * hc_dim);
    const float inv_hc = 1.0f / (float)hc;
    for (int t0 = blockIdx.y * 4; t0 < nt; t0 += gridDim.y * 4) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int i = lane; i < (hc_dim >> 2); i += 32) {
            const float4 wv = __ldg(wr + i);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                if (t0 + q < nt) {
                    const float4 xv = reinterpret_cast<const float4*>(xn + (size_t)(t0 + q) * hc_dim)[i];
                    acc[q] = fmaf(wv.x, xv.x, acc[q]);
                    acc[q] = fmaf(wv.y, xv.y, acc[q]);
                    acc[q] = fmaf(wv.z, xv.z, acc[q]);
                    acc[q] = fmaf(wv.w, xv.w, acc[q]);
                }
            }
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc[q] += __shfl_xor_sync(0xffffffffu, acc[q], o);
            if (lane == 0 && t0 + q < nt) {
                const float v = __fmul_rn(acc[q], inv_hc);  // 1/hc after the matmul (hyper.rs:21-22)
                raw[(size_t)(t0 + q) * rows + row] = row < low_rank ? __fmul_rn(v, hc_sigmoid(v)) : v;
            }
        }
    }
}

// gate[s][d] = w_up[s*e + d] . lo[t]; mixed[t][d] = (1/hc) * sum_s xn[t][s][d] * sigmoid(gate[s][d]).  One warp per d.
__global__ void __launch_bounds__(128)
hc_up_mixed_kernel(const float* __restrict__ w_up, const float* __restrict__ raw, const float* __restrict__ xn, int nt, int hc, int e,
                   int low_rank, float* __restrict__ mixed) {
    extern __shared__ float lo[];  // [low_rank] of the CTA's token
    const int t = blockIdx.y;
    const int rows = low_rank + hc;
    for (int i = threadIdx.x; i < low_rank; i += 128) lo[i] = raw[(size_t)t * rows + i];
    __syncthreads();
    const int d = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (d >= e) return;
    const float inv_hc = 1.0f / (float)hc;
    float m = 0.f;
    for (int s = 0; s < hc; ++s) {
        const float* wr = w_up + ((size_t)s * e + d) * low_rank;
        float acc = 0.f;
        for (int i = lane; i < low_rank; i += 32) acc = fmaf(__ldg(wr + i), lo[i], acc);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        const float term = __fmul_rn(xn[((size_t)t * hc + s) * e + d], hc_sigmoid(acc));
        m = s == 0 ? term : __fadd_rn(m, term);
    }
    if (lane == 0) mixed[(size_t)t * e + d] = __fmul_rn(m, inv_hc);
}

__global__ void hc_combine_kernel(const float* __restrict__ res, const float* __restrict__ blk, const float* __restrict__ raw, int hc, int e,
                                  int low_rank, float* __restrict__ out) {
    const int ts = blockIdx.x;  // token * hc + stream
    const int t = ts / hc, s = ts - t * hc;
    const float w = __fmul_rn(2.0f, hc_sigmoid(raw[(size_t)t * (low_rank + hc) + low_rank + s]));
    const float* r = res + (size_t)ts * e;
    const float* b = blk + (size_t)t * e;
    float* o = out + (size_t)ts * e;
    for (int d = threadIdx.x; d < e; d += blockDim.x) o[d] = __fadd_rn(r[d], __fmul_rn(b[d], w));
}

static int hc_grow(Scratch& s, size_t bytes, bool pinned = false) {
    if (bytes <= s.cap) return DNB_OK;
    if (s.p) { if (pinned) cudaFreeHost(s.p); else cudaFree(s.p); }
    s.p = nullptr;
    s.cap = 0;
    if (pinned) DNB_CUDA(cudaMallocHost(&s.p, bytes)); else DNB_CUDA(cudaMalloc(&s.p, bytes));
    s.cap = bytes;
    return DNB_OK;
}

void hc_release(dnb_ctx* c) {
    HcState* h = static_cast<HcState*>(c->hc);
    if (!h) return;
    for (auto& L : h->layers) {
        if (L.w_norm) cudaFree(L.w_norm);
        if (L.w_down) cudaFree(L.w_down);
        if (L.w_up) cudaFree(L.w_up);
    }
    for (Scratch* s : {&h->xn, &h->raw, &h->mixed, &h->blk, &h->res, &h->out})
        if (s->p) cudaFree(s->p);
    if (h->host_in.p) cudaFreeHost(h->host_in.p);
    if (h->host_out.p) cudaFreeHost(h->host_out.p);
    delete h;
    c->hc = nullptr;
}

static int hc_block_dev(dnb_ctx* c, HcState* H, int layer, const float* res, int nt, float* out) {
    const Model& M = c->model;
    const HcLayer& L = H->layers[layer];
    const int hc = L.hc, lr = L.low_rank, e = M.e, hc_dim = hc * e;
    cudaStream_t st = c->stream;
    int rc;
    if ((rc = hc_grow(H->xn, (size_t)nt * hc_dim * 4)) || (rc = hc_grow(H->raw, (size_t)nt * (lr + hc) * 4)) ||
        (rc = hc_grow(H->mixed, (size_t)nt * e * 4)) || (rc = hc_grow(H->blk, (size_t)nt * e * 4)))
        return rc;
    float* xn = (float*)H->xn.p;
    float* raw = (float*)H->raw.p;
    float* mixed = (float*)H->mixed.p;
    float* blk = (float*)H->blk.p;
    {
        ProfScope p_(c, st, "hc_norm");
        hc_norm_kernel<<<nt * hc, 128, 0, st>>>(res, L.w_norm, M.eps, hc, e, xn);
    }
    {
        ProfScope p_(c, st, "hc_down");
        const int gy = nt >= 64 ? 16 : (nt + 3) / 4;
        hc_down_kernel<<<dim3((lr + hc + 3) / 4, gy), 128, 0, st>>>(L.w_down, xn, nt, hc_dim, lr, hc, raw);
    }
    {
        ProfScope p_(c, st, "hc_up_mixed");
        hc_up_mixed_kernel<<<dim3((e + 3) / 4, nt), 128, (size_t)lr * 4, st>>>(L.w_up, raw, xn, nt, hc, e, lr, mixed);
    }
    c->launches += 3;
    DNB_CUDA(cudaGetLastError());
    if ((rc = dnb_moe_block_dev(c, layer, mixed, nt, blk))) return rc;
    {
        ProfScope p_(c, st, "hc_combine");
        hc_combine_kernel<<<nt * hc, 256, 0, st>>>(res, blk, raw, hc, e, lr, out);
    }
    c->launches++;
    DNB_CUDA(cudaGetLastError());
    return DNB_OK;
}

}  // namespace dnb

using namespace dnb;

extern "C" int dnb_register_hc(dnb_ctx* c, int layer, int hc, int low_rank, const float* w_norm, const float* w_down_inject,
                               const float* w_up) {
    if (!c || !w_norm || !w_down_inject || !w_up) return DNB_ERR_ARG;
    const Model& M = c->model;
    if (layer < 0 || layer >= M.n_layer || hc < 1 || hc > 16 || low_rank < 1 || low_rank > 8192 || M.e % 4) {
        set_error("register_hc: layer %d / hc %d / low_rank %d outside the configured model or the kernels' range", layer, hc, low_rank);
        return DNB_ERR_ARG;
    }
    DNB_CUDA(cudaSetDevice(c->device));
    if (!c->hc) c->hc = new HcState();
    HcState* H = static_cast<HcState*>(c->hc);
    H->layers.resize(M.n_layer);
    HcLayer& L = H->layers[layer];
    DNB_CUDA(cudaDeviceSynchronize());
    if (L.w_norm) cudaFree(L.w_norm);
    if (L.w_down) cudaFree(L.w_down);
    if (L.w_up) cudaFree(L.w_up);
    L = HcLayer();
    const size_t hc_dim = (size_t)hc * M.e;
    const size_t n_norm = hc_dim, n_down = (size_t)(low_rank + hc) * hc_dim, n_up = hc_dim * low_rank;
    DNB_CUDA(cudaMalloc((void**)&L.w_norm, n_norm * 4));
    DNB_CUDA(cudaMalloc((void**)&L.w_down, n_down * 4));
    DNB_CUDA(cudaMalloc((void**)&L.w_up, n_up * 4));
    DNB_CUDA(cudaMemcpy(L.w_norm, w_norm, n_norm * 4, cudaMemcpyHostToDevice));
    DNB_CUDA(cudaMemcpy(L.w_down, w_down_inject, n_down * 4, cudaMemcpyHostToDevice));
    DNB_CUDA(cudaMemcpy(L.w_up, w_up, n_up * 4, cudaMemcpyHostToDevice));
    L.hc = hc;
    L.low_rank = low_rank;
    return DNB_OK;
}

static HcState* hc_ready(dnb_ctx* c, int layer) {
    HcState* H = c ? static_cast<HcState*>(c->hc) : nullptr;
    if (!H || layer < 0 || layer >= (int)H->layers.size() || !H->layers[layer].w_norm) {
        set_error("hc_moe_block: layer %d has no hyper-connection weights registered", layer);
        return nullptr;
    }
    return H;
}

extern "C" int dnb_hc_moe_block_dev(dnb_ctx* c, int layer, const float* res_dev, int nt, float* out_dev) {
    if (!c || !res_dev || !out_dev || nt < 1) return DNB_ERR_ARG;
    HcState* H = hc_ready(c, layer);
    if (!H) return DNB_DECLINED;
    DNB_CUDA(cudaSetDevice(c->device));
    return hc_block_dev(c, H, layer, res_dev, nt, out_dev);
}

extern "C" int dnb_hc_moe_block(dnb_ctx* c, int layer, const float* res, int nt, float* out) {
    if (!c || !res || !out || nt < 1) return DNB_ERR_ARG;
    HcState* H = hc_ready(c, layer);
    if (!H) return DNB_DECLINED;
    DNB_CUDA(cudaSetDevice(c->device));
    const size_t bytes = (size_t)nt * H->layers[layer].hc * c->model.e * 4;
    int rc;
    if ((rc = hc_grow(H->res, bytes)) || (rc = hc_grow(H->out, bytes)) || (rc = hc_grow(H->host_in, bytes, true)) ||
        (rc = hc_grow(H->host_out, bytes, true)))
        return rc;
    memcpy(H->host_in.p, res, bytes);
    DNB_CUDA(cudaMemcpyAsync(H->res.p, H->host_in.p, bytes, cudaMemcpyHostToDevice, c->stream));
    if ((rc = hc_block_dev(c, H, layer, (const float*)H->res.p, nt, (float*)H->out.p))) return rc;
    DNB_CUDA(cudaMemcpyAsync(H->host_out.p, H->out.p, bytes, cudaMemcpyDeviceToHost, c->stream));
    DNB_CUDA(cudaStreamSynchronize(c->stream));
    const int st = *reinterpret_cast<volatile int*>(c->status_host);
    if (st != 0) {  // a bounded device wait gave up: nothing is written (see dnb_device_status)
        *reinterpret_cast<volatile int*>(c->status_host) = 0;
        set_error("hc_moe_block: a bounded device wait gave up (status %d); the result was discarded", st);
        return DNB_DECLINED;
    }
    memcpy(out, H->host_out.p, bytes);
    return DNB_OK;
}
