// Expert-parallel DECODE over peer memory (one process per GPU, one node).
//
// The reference is single-GPU.  With G GPUs rank g keeps experts [g*ne/G, (g+1)*ne/G) of every
// layer; router, norm and shared expert are replicated.  A decode batch is a handful of tokens
// (1, 8, 32) whose exchange is latency, not bandwidth: 10 rows of 8 KB per token.  So the residual
// stream is kept REPLICATED -- every rank holds all tokens of the batch and routes them itself (same
// arithmetic, same bits) -- and a layer needs ONE exchange instead of a dispatch and a return:
//
//   route (all tokens, every rank)                          router kernels of moe_kernels.cu
//   local experts: (token, slot) pairs whose expert lives here, gate/up + SwiGLU + down
//                                                          decode GEMV kernels (<= 16 tokens) or tiled kernels
//   push     every local result row is stored into slot (token, slot) of EVERY rank's arena
//            (plain 16-byte peer stores); the last CTA raises this rank's flag at every peer
//   combine  bounded wait for every rank's flag, then out[t] = sum_s w[t][s] * slot[t][s] in ascending
//            slot (= ascending expert) order with separate multiply and add roundings, + shared expert
//            (+ residual): the single-GPU order, so the result does not depend on G and every rank
//            ends the layer with the same bits
//
// Flags are sequence numbers that only grow; a rank writes only its own flag word at a peer and only
// the slots of its own experts, so no two ranks ever write the same word.  Slot buffers alternate by
// the call's parity: a rank can be at most one call ahead of a peer that is still reading.  Every wait
// is bounded (status 24) and nothing here uses TMA or multicast: peer traffic is ordinary stores.
#include "dnb_common.cuh"

namespace dnb {

constexpr int kEpdMaxWorld = 16;

struct EpdArena {  // head of every rank's exported allocation; the slot buffers follow at off_slots
    uint32_t flag[kEpdMaxWorld];  // [src] = seq once rank src has stored all its rows of call seq
};

struct EpdPeers {  // kernel parameter: every rank's arena as seen from this GPU
    EpdArena* arena[kEpdMaxWorld];
    float* slots[kEpdMaxWorld];  // [2][max_tokens * k][e]
};

__device__ __forceinline__ void epd_st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t epd_ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Segment tables of the decode GEMV kernels for the (token, slot) pairs of a batch: token-major one-row
// segments as in decode_batch_tables_kernel, but a pair whose expert lives on another rank gets m = 0
// (the kernels skip it).  Slot k is the shared expert, computed by every rank.
__global__ void epd_tables_kernel(const int32_t* __restrict__ sels, int nt, int k, int first, int n_local,
                                  const uint8_t* gate, const uint8_t* up, const uint8_t* down, size_t eb_g, size_t eb_u,
                                  size_t eb_d, const uint8_t* sg, const uint8_t* su, const uint8_t* sdn, SegDesc* seg_gu,
                                  SegDesc* seg_dn, int32_t* row_token) {
    const int t = blockIdx.x, s = threadIdx.x, per = k + (sg ? 1 : 0);
    if (t >= nt || s >= per) return;
    const uint32_t row = (uint32_t)(t * per + s);
    if (s < k) {
        const int ex = sels[(size_t)t * k + s] - first;
        const bool mine = ex >= 0 && ex < n_local;
        const size_t li = mine ? (size_t)ex : 0;
        seg_gu[row] = SegDesc{gate + li * eb_g, up + li * eb_u, mine ? 1u : 0u, row};
        seg_dn[row] = SegDesc{down + li * eb_d, nullptr, mine ? 1u : 0u, row};
    } else {
        seg_gu[row] = SegDesc{sg, su, 1u, row};
        seg_dn[row] = SegDesc{sdn, nullptr, 1u, row};
    }
    row_token[row] = t;
}

// sels -> local expert index, or -1 for a pair another rank computes (the routing-table kernel ignores those)
__global__ void epd_mask_kernel(const int32_t* __restrict__ sels, int n, int first, int n_local, int32_t* __restrict__ msel) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const int ex = sels[i] - first;
        msel[i] = (ex >= 0 && ex < n_local) ? ex : -1;
    }
}

// One CTA per (token, slot): a local pair's result row goes to slot t*k+s of every rank; the last CTA to
// finish raises this rank's flag everywhere.  src_row: where the pair's row is in `hrow` (pos != null: the
// packed row of the tiled path; else row t*per+s of the decode GEMV path).
__global__ void __launch_bounds__(256)
epd_push_kernel(const float* __restrict__ hrow, const int32_t* __restrict__ sels, const int32_t* __restrict__ pos, int k,
                int per, int e, int first, int n_local, int world, int me, uint32_t* seq_dev, size_t slot_stride, EpdPeers peers,
                unsigned int* ticket) {
    const int i = blockIdx.x, tid = threadIdx.x;
    // The call's sequence number lives on the device (a captured launch sequence can be replayed): this
    // kernel works with the next number and its last CTA, after every other CTA has read it, stores it back.
    const uint32_t seq = *reinterpret_cast<volatile uint32_t*>(seq_dev) + 1u;
    const int t = i / k, s = i - t * k;
    const int ex = sels[i] - first;
    if (ex >= 0 && ex < n_local) {
        const size_t src = pos ? (size_t)pos[i] : (size_t)t * per + s;
        const float4* r4 = reinterpret_cast<const float4*>(hrow + src * e);
        const size_t dst = (size_t)(seq & 1u) * slot_stride + (size_t)i * e;
        for (int c = tid; c < (e >> 2); c += 256) {
            const float4 v = r4[c];
            for (int d = 0; d < world; ++d) reinterpret_cast<float4*>(peers.slots[d] + dst)[c] = v;
        }
    }
    __threadfence_system();
    __syncthreads();
    __shared__ int last;
    if (tid == 0) {
        const unsigned int tk = atomicAdd(ticket, 1u);
        last = (tk == gridDim.x - 1) ? 1 : 0;
        if (last) *ticket = 0u;
    }
    __syncthreads();
    if (last && tid < world) epd_st_release_sys(&peers.arena[tid]->flag[me], seq);
    if (last && tid == 0) *seq_dev = seq;
}

// One CTA per token: wait (bounded) until every rank has stored its rows of this call, then the weighted
// sum in ascending slot order (kernels_dec_epi.cu:28-46; qwen4exp.rs:12126-12216), the shared expert and
// the residual.  The slots were written by peers over NVLink: read them past L1.
__global__ void __launch_bounds__(256)
epd_combine_kernel(const EpdArena* mine, const float* __restrict__ slots, const float* __restrict__ wts, int k, int e,
                   const float* __restrict__ sh, size_t sh_stride, const float* __restrict__ shcoef,
                   const float* __restrict__ residual, float* __restrict__ out, int world, const uint32_t* seq_dev,
                   size_t slot_stride, int polls, int* status) {
    const int t = blockIdx.x, tid = threadIdx.x;
    const uint32_t seq = *seq_dev;  // the push kernel before this one stored the call's number
    slots += (size_t)(seq & 1u) * slot_stride;
    __shared__ int ok_all;
    __shared__ float pw[32];
    if (tid == 0) ok_all = 1;
    if (tid < k) pw[tid] = wts[(size_t)t * k + tid];
    __syncthreads();
    if (tid < world) {
        bool ok = false;
        for (int i = 0; i < polls && !ok; ++i) {
            ok = (int32_t)(epd_ld_acquire_sys(&mine->flag[tid]) - seq) >= 0;
            if (!ok) __nanosleep(50);
        }
        if (!ok) {
            status_set(status, 24);
            ok_all = 0;
        }
    }
    __syncthreads();
    if (!ok_all) return;  // the host discards the call; out stays as it was
    const float* base = slots + (size_t)t * k * e;
    for (int j = tid * 4; j < e; j += 1024) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s = 0; s < k; ++s) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(base + (size_t)s * e + j));
            const float w = pw[s];
            acc.x = __fadd_rn(acc.x, __fmul_rn(w, v.x));
            acc.y = __fadd_rn(acc.y, __fmul_rn(w, v.y));
            acc.z = __fadd_rn(acc.z, __fmul_rn(w, v.z));
            acc.w = __fadd_rn(acc.w, __fmul_rn(w, v.w));
        }
        if (sh) {
            const float4 v = *reinterpret_cast<const float4*>(sh + (size_t)t * sh_stride + j);
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
        if (residual) {
            const float4 r = *reinterpret_cast<const float4*>(residual + (size_t)t * e + j);
            acc.x = __fadd_rn(r.x, acc.x);
            acc.y = __fadd_rn(r.y, acc.y);
            acc.z = __fadd_rn(r.z, acc.z);
            acc.w = __fadd_rn(r.w, acc.w);
        }
        *reinterpret_cast<float4*>(out + (size_t)t * e + j) = acc;
    }
}

struct EpdState {
    int rank = 0, world = 1, max_tokens = 0, n_local = 0;
    uint32_t* seq_dev = nullptr;  // calls made so far
    bool connected = false, loopback = false;
    uint8_t* arena = nullptr;
    size_t arena_bytes = 0, off_slots = 0, slot_stride = 0;  // slot_stride: floats of one parity buffer
    void* peer_base[kEpdMaxWorld] = {nullptr};
    EpdPeers peers;
    unsigned int* ticket = nullptr;
    int32_t* msel = nullptr;
};

void epd_release(dnb_ctx* c) {
    EpdState* s = static_cast<EpdState*>(c->epd);
    if (!s) return;
    for (int r = 0; r < s->world; ++r)
        if (r != s->rank && s->peer_base[r] && !s->loopback) cudaIpcCloseMemHandle(s->peer_base[r]);
    if (s->arena) cudaFree(s->arena);
    if (s->ticket) cudaFree(s->ticket);
    if (s->msel) cudaFree(s->msel);
    if (s->seq_dev) cudaFree(s->seq_dev);
    delete s;
    c->epd = nullptr;
}

static void epd_point(EpdState* s, int r, void* base) {
    s->peer_base[r] = base;
    s->peers.arena[r] = (EpdArena*)base;
    s->peers.slots[r] = (float*)((uint8_t*)base + s->off_slots);
}

// One block for all nt tokens of the batch on this rank.  residual: null, or [nt][e] added to the result
// (== out for the in-place stack).
static int epd_block(dnb_ctx* c, EpdState* s, int layer, const float* h, int nt, const float* residual, float* out) {
    const Model& M = c->model;
    const Layer& L = M.layers[layer];
    Workspace& w = c->ws;
    cudaStream_t st = c->stream;
    const bool shared = L.has_shared();
    const bool fold = shared && L.m[3].type == L.m[0].type && L.m[4].type == L.m[1].type && L.m[5].type == L.m[2].type &&
                      L.m[3].n_out == M.ff;
    if ((shared && !fold) || L.m[0].type != L.m[1].type) {
        set_error("epd_block: the shared expert must have the routed experts' formats and width");
        return DNB_DECLINED;
    }
    int rc;
    const int per = M.k + (fold ? 1 : 0);
    const int32_t* pos = nullptr;
    const float* sh = nullptr;
    size_t sh_stride = 0;
    bool done = false;
    const float* x = nullptr;
    if (nt == 1 && c->decode_fast) {
        // one token: the fused router kernel (RMSNorm, logits, top-k and the segment tables, with the other ranks'
        // slots as empty segments) and the decode GEMV kernels, chained with programmatic dependent launch
        rc = launch_router_decode(c, st, h, M, L, w, fold, c->ticket);
        if (rc == DNB_OK) {
            x = w.xn;
            rc = launch_seg_gemv_m1(c, st, L.m[0].type, true, true, w.seg_gu, nullptr, per, M.e, M.ff, w.xn, M.e, nullptr, w.act,
                                    nullptr, "gemv_gate_up", PermOut{nullptr, 0, M.ne >= 4 * kActRep ? w.xn_perm : nullptr});
            if (rc == DNB_DECLINED)
                rc = launch_seg_matmul(c, st, L.m[0].type, true, w.seg_gu, nullptr, per, M.e, M.ff, w.xn, M.e, w.row_token, w.act, 1);
            if (rc) return rc;
            rc = launch_seg_gemv_m1(c, st, L.m[2].type, false, false, w.seg_dn, nullptr, per, M.ff, M.e, w.act, M.ff, nullptr,
                                    w.hrow, nullptr, "gemv_down");
            if (rc == DNB_DECLINED)
                rc = launch_seg_matmul(c, st, L.m[2].type, false, w.seg_dn, nullptr, per, M.ff, M.e, w.act, M.ff, nullptr, w.hrow, 1);
            if (rc) return rc;
            if (fold) {
                sh = w.hrow + (size_t)M.k * M.e;
                sh_stride = (size_t)per * M.e;
            }
            done = true;
        } else if (rc != DNB_DECLINED) {
            return rc;
        }
    }
    if (!done) {
        if (L.norm_w)
            if ((rc = launch_rmsnorm(c, st, h, L.norm_w, M.eps, nt, M.e, w.xn))) return rc;
        x = L.norm_w ? w.xn : h;
        if ((rc = router_topk_dev(c, st, x, nt, L, w.sels, w.wts, nullptr))) return rc;
    }
    if (!done && nt <= kDecodeBatchMax && c->decode_fast && per <= 64) {
        // decode GEMV kernels over one-row segments; pairs of other ranks are empty segments
        epd_tables_kernel<<<nt, 64, 0, st>>>(w.sels, nt, M.k, M.shard_first, s->n_local, L.m[0].dev, L.m[1].dev, L.m[2].dev,
                                             L.m[0].expert_bytes, L.m[1].expert_bytes, L.m[2].expert_bytes,
                                             fold ? L.m[3].dev : nullptr, fold ? L.m[4].dev : nullptr,
                                             fold ? L.m[5].dev : nullptr, w.seg_gu, w.seg_dn, w.row_token);
        c->launches++;
        DNB_CUDA(cudaGetLastError());
        rc = launch_seg_gemv_m1(c, st, L.m[0].type, true, true, w.seg_gu, nullptr, nt * per, M.e, M.ff, x, M.e, w.row_token,
                                w.act, nullptr, "gemv_gate_up");
        if (rc == DNB_OK) {
            rc = launch_seg_gemv_m1(c, st, L.m[2].type, false, false, w.seg_dn, nullptr, nt * per, M.ff, M.e, w.act, M.ff,
                                    nullptr, w.hrow, nullptr, "gemv_down");
            if (rc == DNB_DECLINED)
                rc = launch_seg_matmul(c, st, L.m[2].type, false, w.seg_dn, nullptr, nt * per, M.ff, M.e, w.act, M.ff, nullptr,
                                       w.hrow, 1);
            if (rc) return rc;
            if (fold) {
                sh = w.hrow + (size_t)M.k * M.e;
                sh_stride = (size_t)per * M.e;
            }
            done = true;
        } else if (rc != DNB_DECLINED) {
            return rc;
        }
    }
    if (!done) {
        // general tiled kernels over expert-major packed rows of the local pairs (+ the shared expert's rows)
        epd_mask_kernel<<<(nt * M.k + 255) / 256, 256, 0, st>>>(w.sels, nt * M.k, M.shard_first, s->n_local, s->msel);
        c->launches++;
        DNB_CUDA(cudaGetLastError());
        if ((rc = launch_route_tables(c, st, s->msel, nt, M.k, s->n_local, L, w, fold))) return rc;
        const int nseg_max = (nt * M.k < s->n_local ? nt * M.k : s->n_local) + (fold ? 1 : 0);
        if ((rc = launch_seg_matmul(c, st, L.m[0].type, true, w.seg_gu, w.nseg, nseg_max, M.e, M.ff, x, M.e, w.row_token, w.act,
                                    nt)))
            return rc;
        if ((rc = launch_seg_matmul(c, st, L.m[2].type, false, w.seg_dn, w.nseg, nseg_max, M.ff, M.e, w.act, M.ff, nullptr,
                                    w.hrow, nt)))
            return rc;
        pos = w.pos;
        if (fold) {
            sh = w.hrow + (size_t)nt * M.k * M.e;
            sh_stride = (size_t)M.e;
        }
    }
    const float* coef = nullptr;
    if (fold && L.shared_gate_row) {
        if ((rc = launch_shared_coef(c, st, x, L.shared_gate_row, nt, M.e, w.shcoef))) return rc;
        coef = w.shcoef;
    }
    {
        ProfScope p_(c, st, "epd_push");
        epd_push_kernel<<<nt * M.k, 256, 0, st>>>(w.hrow, w.sels, pos, M.k, per, M.e, M.shard_first, s->n_local, s->world, s->rank,
                                                  s->seq_dev, s->slot_stride, s->peers, s->ticket);
    }
    {
        ProfScope p_(c, st, "epd_wait_combine");
        const float* slots = (const float*)(s->arena + s->off_slots);
        epd_combine_kernel<<<nt, 256, 0, st>>>((const EpdArena*)s->arena, slots, w.wts, M.k, M.e, sh, sh_stride, coef, residual, out,
                                               s->world, s->seq_dev, s->slot_stride, c->flag_polls, c->status);
    }
    c->launches += 2;
    DNB_CUDA(cudaGetLastError());
    return DNB_OK;
}

}  // namespace dnb

using namespace dnb;

extern "C" int dnb_epd_init(dnb_ctx* c, int rank, int world, int max_tokens, void* handle_out) {
    if (!c || !handle_out || world < 1 || world > kEpdMaxWorld || rank < 0 || rank >= world || max_tokens < 1) return DNB_ERR_ARG;
    const Model& M = c->model;
    if (M.n_layer < 1 || M.ne % world || M.shard_count != M.ne / world || M.shard_first != rank * (M.ne / world)) {
        set_error("epd_init: configure the model and call dnb_moe_set_expert_shard(rank * ne / world, ne / world) first");
        return DNB_DECLINED;
    }
    if (M.e % 4 || M.k > 32) {
        set_error("epd_init: n_embd must be a multiple of 4 and k <= 32");
        return DNB_DECLINED;
    }
    DNB_CUDA(cudaSetDevice(c->device));
    epd_release(c);
    EpdState* s = new EpdState();
    c->epd = s;
    s->rank = rank; s->world = world; s->max_tokens = max_tokens; s->n_local = M.ne / world;
    s->off_slots = 256;
    s->slot_stride = (size_t)max_tokens * M.k * M.e;
    s->arena_bytes = s->off_slots + 2 * s->slot_stride * sizeof(float);
    DNB_CUDA(cudaMalloc((void**)&s->arena, s->arena_bytes));
    DNB_CUDA(cudaMemset(s->arena, 0, s->arena_bytes));
    DNB_CUDA(cudaMalloc((void**)&s->ticket, 4));
    DNB_CUDA(cudaMemset(s->ticket, 0, 4));
    DNB_CUDA(cudaMalloc((void**)&s->msel, (size_t)max_tokens * M.k * 4));
    DNB_CUDA(cudaMalloc((void**)&s->seq_dev, 4));
    DNB_CUDA(cudaMemset(s->seq_dev, 0, 4));
    DNB_CUDA(cudaDeviceSynchronize());
    cudaIpcMemHandle_t h;
    DNB_CUDA(cudaIpcGetMemHandle(&h, s->arena));
    memcpy(handle_out, &h, sizeof(h));
    return DNB_OK;
}

extern "C" int dnb_epd_connect(dnb_ctx* c, const void* handles) {
    if (!c || !c->epd) return DNB_ERR_ARG;
    EpdState* s = static_cast<EpdState*>(c->epd);
    DNB_CUDA(cudaSetDevice(c->device));
    for (int r = 0; r < s->world; ++r) {
        if (r == s->rank || !handles) {  // handles == null: every peer is this rank's own arena (absent ranks: time-out tests)
            epd_point(s, r, s->arena);
        } else {
            cudaIpcMemHandle_t h;
            memcpy(&h, (const uint8_t*)handles + (size_t)r * 64, 64);
            void* base = nullptr;
            DNB_CUDA(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
            epd_point(s, r, base);
        }
    }
    s->loopback = handles == nullptr;
    s->connected = true;
    return DNB_OK;
}

extern "C" int dnb_epd_block_dev(dnb_ctx* c, int layer, const float* h_dev, int nt, float* out_dev) {
    if (!c || !c->epd || !h_dev || !out_dev || nt < 1) return DNB_ERR_ARG;
    EpdState* s = static_cast<EpdState*>(c->epd);
    const Model& M = c->model;
    if (!s->connected || nt > s->max_tokens || layer < 0 || layer >= M.n_layer) {
        set_error("epd_block: not connected, layer out of range, or %d tokens exceed the %d the arena was sized for", nt, s->max_tokens);
        return DNB_ERR_ARG;
    }
    const Layer& L = M.layers[layer];
    if (!L.m[0].dev || !L.m[1].dev || !L.m[2].dev || !L.router_w) {
        set_error("epd_block: layer %d is not fully registered", layer);
        return DNB_DECLINED;
    }
    DNB_CUDA(cudaSetDevice(c->device));
    int rc = ensure_workspace(c, nt);
    if (rc) return rc;
    return graphed(c, GraphKey{6, layer, nt, h_dev, out_dev}, [&]() { return epd_block(c, s, layer, h_dev, nt, nullptr, out_dev); });
}

extern "C" int dnb_epd_stack_dev(dnb_ctx* c, float* h_dev, int nt) {
    if (!c || !c->epd || !h_dev || nt < 1) return DNB_ERR_ARG;
    EpdState* s = static_cast<EpdState*>(c->epd);
    const Model& M = c->model;
    if (!s->connected || nt > s->max_tokens) {
        set_error("epd_stack: not connected, or %d tokens exceed the %d the arena was sized for", nt, s->max_tokens);
        return DNB_ERR_ARG;
    }
    for (int l = 0; l < M.n_layer; ++l) {
        const Layer& L = M.layers[l];
        if (!L.m[0].dev || !L.m[1].dev || !L.m[2].dev || !L.router_w) {
            set_error("epd_stack: layer %d is not fully registered", l);
            return DNB_DECLINED;
        }
    }
    DNB_CUDA(cudaSetDevice(c->device));
    int rc = ensure_workspace(c, nt);
    if (rc) return rc;
    // the launch sequence holds no per-call argument (the sequence number is on the device): replay it as a graph
    return graphed(c, GraphKey{5, 0, nt, h_dev, nullptr}, [&]() -> int {
        for (int l = 0; l < M.n_layer; ++l) {
            const int r = epd_block(c, s, l, h_dev, nt, h_dev, h_dev);
            if (r) return r;
        }
        return DNB_OK;
    });
}
