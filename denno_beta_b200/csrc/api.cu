// extern "C" entry points of libdnb200: context, resident tables and the
// orchestration of one MoE block (see include/dnb200.h for the contract).
#include <algorithm>
#include <chrono>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "dnb_common.cuh"

namespace dnb {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

static void drop_graphs(dnb_ctx* c);

template <typename T>
static int dev_alloc(T** p, size_t n) {
    *p = nullptr;
    if (n == 0) return DNB_OK;
    DNB_CUDA(cudaMalloc((void**)p, n * sizeof(T)));
    return DNB_OK;
}

static void free_ws(Workspace& w) {
    void* dev[] = {w.act_h, w.xn_perm, w.act_perm, w.xn, w.logits, w.wts, w.act, w.hrow, w.sact, w.sh, w.hin, w.out, w.shcoef, w.sels, w.row_token,
                   w.pos, w.nseg, w.counts, w.one, w.seg_gu, w.seg_dn, w.seg_sh_gu, w.seg_sh_dn, w.xg_hi, w.xg_lo, w.act_hi, w.act_lo,
                   w.x3, w.rpart, w.xq_hi, w.xq_lo, w.aq_hi, w.aq_lo, w.xq_scale, w.aq_scale};
    for (void* p : dev)
        if (p) cudaFree(p);
    if (w.pinned_in) cudaFreeHost(w.pinned_in);
    if (w.pinned_out) cudaFreeHost(w.pinned_out);
    if (w.pinned_sels) cudaFreeHost(w.pinned_sels);
    if (w.pinned_wts) cudaFreeHost(w.pinned_wts);
    w = Workspace();
}

// Device buffers for up to nt tokens (grow-only, like the reference's scratch,
// cuda.rs:7454-7480).
static int ensure_ws(dnb_ctx* c, int nt) {
    Workspace& w = c->ws;
    if (nt <= w.nt_cap) return DNB_OK;
    const Model& M = c->model;
    int cap = w.nt_cap ? w.nt_cap : 1;
    while (cap < nt) cap *= 2;
    DNB_CUDA(cudaDeviceSynchronize());
    drop_graphs(c);
    free_ws(w);
    const size_t rows = (size_t)cap * (M.k + 1);  // + the shared expert's row in the decode path
    const int sff = M.sff > 0 ? M.sff : M.ff;
    int rc = DNB_OK;
    if ((rc = dev_alloc(&w.xn, (size_t)cap * M.e))) return rc;
    if ((rc = dev_alloc(&w.hin, (size_t)cap * M.e))) return rc;
    if ((rc = dev_alloc(&w.out, (size_t)cap * M.e))) return rc;
    if ((rc = dev_alloc(&w.logits, std::max((size_t)cap * M.ne, (size_t)kActRep * M.ne)))) return rc;  // one-token block kernel: kActRep copies
    if ((rc = dev_alloc(&w.wts, rows))) return rc;
    if ((rc = dev_alloc(&w.sels, rows))) return rc;
    if ((rc = dev_alloc(&w.act, rows * M.ff))) return rc;
    if ((rc = dev_alloc(&w.act_perm, (size_t)kActRep * (cap < kDecodeBatchMax ? cap : kDecodeBatchMax) * (M.k + 1) * M.ff))) return rc;
    if ((rc = dev_alloc(&w.xn_perm, (size_t)kActRep * M.e))) return rc;
    if ((rc = dev_alloc(&w.act_h, decode_fused_act_halves(M.k + 1, M.ff)))) return rc;
    if ((rc = dev_alloc(&w.hrow, rows * M.e))) return rc;
    if ((rc = dev_alloc(&w.sact, (size_t)cap * sff))) return rc;
    if ((rc = dev_alloc(&w.sh, (size_t)cap * M.e))) return rc;
    if ((rc = dev_alloc(&w.shcoef, (size_t)cap))) return rc;
    if ((rc = dev_alloc(&w.row_token, rows))) return rc;
    if ((rc = dev_alloc(&w.pos, rows))) return rc;
    if ((rc = dev_alloc(&w.nseg, 1))) return rc;
    if ((rc = dev_alloc(&w.one, 1))) return rc;
    {
        const int32_t one = 1;
        DNB_CUDA(cudaMemcpy(w.one, &one, sizeof(one), cudaMemcpyHostToDevice));
    }
    if ((rc = dev_alloc(&w.counts, (size_t)M.ne))) return rc;
    // one segment per active expert (+ shared) for a chunk, or per (token, slot) for a decode batch
    const size_t nseg_cap = std::max((size_t)M.ne + 1, (size_t)kDecodeBatchMax * (M.k + 1));
    if ((rc = dev_alloc(&w.seg_gu, nseg_cap))) return rc;
    if ((rc = dev_alloc(&w.seg_dn, nseg_cap))) return rc;
    if ((rc = dev_alloc(&w.seg_sh_gu, 1))) return rc;
    if ((rc = dev_alloc(&w.seg_sh_dn, 1))) return rc;
    // bf16 hi/lo operand buffers of the tcgen05 path (a few rows of slack so that a
    // tile that starts near the end stays inside the allocation)
    const size_t rows_pad = rows + 128;
    if ((rc = dev_alloc(&w.xg_hi, rows_pad * M.e))) return rc;
    if ((rc = dev_alloc(&w.xg_lo, rows_pad * M.e))) return rc;
    if ((rc = dev_alloc(&w.act_hi, rows_pad * M.ff))) return rc;
    if ((rc = dev_alloc(&w.act_lo, rows_pad * M.ff))) return rc;
    DNB_CUDA(cudaMemset(w.xg_hi, 0, rows_pad * M.e * 2));
    DNB_CUDA(cudaMemset(w.xg_lo, 0, rows_pad * M.e * 2));
    DNB_CUDA(cudaMemset(w.act_hi, 0, rows_pad * M.ff * 2));
    DNB_CUDA(cudaMemset(w.act_lo, 0, rows_pad * M.ff * 2));
    w.maps_ok = (M.e % 64 == 0 && M.ff % 64 == 0) &&
                umma_make_maps(w.xg_hi, w.xg_lo, rows_pad, (uint64_t)M.e, &w.maps_x) == DNB_OK &&
                umma_make_maps(w.act_hi, w.act_lo, rows_pad, (uint64_t)M.ff, &w.maps_act) == DNB_OK;
    if (c->q4k_int && w.maps_ok && q4k_int_handles(M.e, M.ff, true) && q4k_int_handles(M.ff, M.e, false)) {
        const size_t xp = (size_t)M.e + kQ4kIntXcols, ap = (size_t)M.ff + kQ4kIntXcols;
        if ((rc = dev_alloc(&w.xq_hi, rows_pad * xp))) return rc;
        if ((rc = dev_alloc(&w.xq_lo, rows_pad * xp))) return rc;
        if ((rc = dev_alloc(&w.aq_hi, rows_pad * ap))) return rc;
        if ((rc = dev_alloc(&w.aq_lo, rows_pad * ap))) return rc;
        if ((rc = dev_alloc(&w.xq_scale, rows_pad))) return rc;
        if ((rc = dev_alloc(&w.aq_scale, rows_pad))) return rc;
        DNB_CUDA(cudaMemset(w.xq_hi, 0, rows_pad * xp * 2));  // the padding columns behind the sub-block sums stay zero
        DNB_CUDA(cudaMemset(w.xq_lo, 0, rows_pad * xp * 2));
        DNB_CUDA(cudaMemset(w.aq_hi, 0, rows_pad * ap * 2));
        DNB_CUDA(cudaMemset(w.aq_lo, 0, rows_pad * ap * 2));
        w.q4k_int_ok = umma_make_maps(w.xq_hi, w.xq_lo, rows_pad, xp, &w.maps_xq) == DNB_OK &&
                       umma_make_maps(w.aq_hi, w.aq_lo, rows_pad, ap, &w.maps_aq) == DNB_OK;
    }
    if ((rc = router_tc_workspace(c, w, cap, M.ne, M.e))) return rc;
    w.pinned_cap = (size_t)cap * M.e * sizeof(float);
    DNB_CUDA(cudaMallocHost((void**)&w.pinned_in, w.pinned_cap));
    DNB_CUDA(cudaMallocHost((void**)&w.pinned_out, w.pinned_cap));
    DNB_CUDA(cudaMallocHost((void**)&w.pinned_sels, rows * sizeof(int32_t)));
    DNB_CUDA(cudaMallocHost((void**)&w.pinned_wts, rows * sizeof(float)));
    w.nt_cap = cap;
    return DNB_OK;
}

int ensure_workspace(dnb_ctx* c, int nt) { return ensure_ws(c, nt); }

static int grow(Scratch& s, size_t bytes, bool pinned_host = false) {
    if (bytes <= s.cap) return DNB_OK;
    if (s.p) {
        if (pinned_host) cudaFreeHost(s.p); else cudaFree(s.p);
    }
    s.p = nullptr;
    s.cap = 0;
    if (pinned_host) DNB_CUDA(cudaMallocHost(&s.p, bytes)); else DNB_CUDA(cudaMalloc(&s.p, bytes));
    s.cap = bytes;
    return DNB_OK;
}

static void drop_graphs(dnb_ctx* c) {
    for (auto& kv : c->graphs)
        if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
    c->graphs.clear();
}

// Run `enqueue` (a sequence of launches on c->stream) directly the first time a
// key is seen, capture it into a CUDA graph the second time, replay it afterwards.
// One replay costs the host one call instead of one per kernel.
template <class F>
static int run_graphed(dnb_ctx* c, const GraphKey& key, F enqueue) {
    if (!c->use_graphs || c->prof.on) return enqueue();
    auto it = c->graphs.find(key);
    if (it == c->graphs.end()) {
        c->graphs[key] = GraphEntry();
        return enqueue();
    }
    if (!it->second.exec) {
        const uint64_t l0 = c->launches;
        DNB_CUDA(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
        const int rc = enqueue();
        cudaGraph_t g = nullptr;
        const cudaError_t e = cudaStreamEndCapture(c->stream, &g);
        const uint64_t n = c->launches - l0;
        c->launches = l0;
        if (rc != DNB_OK || e != cudaSuccess || !g) {
            if (g) cudaGraphDestroy(g);
            c->graphs.erase(it);
            cudaGetLastError();
            if (rc != DNB_OK) return rc;
            c->use_graphs = false;  // capture is not possible here: stay on direct launches
            return enqueue();
        }
        cudaGraphExec_t ex = nullptr;
        const cudaError_t e2 = cudaGraphInstantiate(&ex, g, 0);
        cudaGraphDestroy(g);
        if (e2 != cudaSuccess) {
            c->graphs.erase(it);
            cudaGetLastError();
            c->use_graphs = false;
            return enqueue();
        }
        it->second.exec = ex;
        it->second.kernels = n;
    }
    DNB_CUDA(cudaGraphLaunch(it->second.exec, c->stream));
    c->launches += it->second.kernels;
    return DNB_OK;
}

int graphed(dnb_ctx* c, const GraphKey& key, const std::function<int()>& enqueue) { return run_graphed(c, key, enqueue); }

// Wait for the stream at the end of a host-buffer call.  A decode-sized call lasts a few
// tens of microseconds, less than it takes a blocked thread to be woken, so the host polls
// the stream for up to two milliseconds before it falls back to the blocking wait.
static cudaError_t wait_short(cudaStream_t st) {
    const auto t0 = std::chrono::steady_clock::now();
    for (int i = 0;; ++i) {
        const cudaError_t e = cudaStreamQuery(st);
        if (e != cudaErrorNotReady) return e;
        if ((i & 63) == 63 && std::chrono::steady_clock::now() - t0 > std::chrono::milliseconds(2)) break;
    }
    return cudaStreamSynchronize(st);
}

// After the stream synchronisation of a host-buffer call: did a bounded wait give up on the
// device since the word was last cleared?  Then the call's result is not valid: nothing is
// copied to the caller, the word is cleared so that the next call is judged on its own, and
// the call reports DNB_DECLINED ("did not run, out untouched": cuda.rs:21024-21027,
// 8785-8788).  A grid barrier that ran out (23) also retires the one-kernel decode form
// for this context: the two-launch form has no inter-CTA wait.
static int finish_checked(dnb_ctx* c, const char* what) {
    const int st = *reinterpret_cast<volatile int*>(c->status_host);
    if (st == 0) return DNB_OK;
    *reinterpret_cast<volatile int*>(c->status_host) = 0;
    if (st == 23 && c->decode_fused) {
        c->decode_fused = false;
        drop_graphs(c);
    }
    set_error("%s: a bounded device wait gave up (status %d); the result was discarded", what, st);
    return DNB_DECLINED;
}

static bool layer_ready(const dnb_ctx* c, int layer, bool need_router) {
    const Model& M = c->model;
    if (layer < 0 || layer >= M.n_layer) return false;
    const Layer& L = M.layers[layer];
    if (!L.m[0].dev || !L.m[1].dev || !L.m[2].dev) return false;
    if (need_router && !L.router_w) return false;
    if (M.shard_count != M.ne) return false;  // only a shard is resident: use the expert-parallel entry points
    return true;
}

// The routed + shared expert half of a block on device buffers.  x: expert input
// [nt][e]; sels/wts on the device.  Writes out[nt][e].  The shared expert's
// segment descriptors must already have been published by launch_prep.
static int experts_dev(dnb_ctx* c, int layer, const float* x, int nt, const int32_t* sels, const float* wts,
                       float* out, int k = -1, int ne = -1, int with_shared = -1) {
    const Model& M = c->model;
    const Layer& L = M.layers[layer];
    Workspace& w = c->ws;
    cudaStream_t st = c->stream;
    int rc;
    if (k < 0) k = M.k;
    if (ne < 0) ne = M.ne;
    const bool shared = with_shared < 0 ? L.has_shared() : (with_shared != 0);
    if (shared) {
        // fork: the shared expert does not depend on the routing
        DNB_CUDA(cudaEventRecord(c->ev_fork, st));
        DNB_CUDA(cudaStreamWaitEvent(c->side, c->ev_fork, 0));
        const int sff = L.m[3].n_out;
        if ((rc = launch_seg_matmul(c, c->side, L.m[3].type, true, w.seg_sh_gu, nullptr, 1, M.e, sff, x, M.e, nullptr,
                                    w.sact, nt)))
            return rc;
        if ((rc = launch_seg_matmul(c, c->side, L.m[5].type, false, w.seg_sh_dn, nullptr, 1, sff, M.e, w.sact, sff,
                                    nullptr, w.sh, nt)))
            return rc;
        if (L.shared_gate_row)
            if ((rc = launch_shared_coef(c, c->side, x, L.shared_gate_row, nt, M.e, w.shcoef))) return rc;
        DNB_CUDA(cudaEventRecord(c->ev_join, c->side));
    }
    if ((rc = launch_route_tables(c, st, sels, nt, k, ne, L, w))) return rc;
    const int nseg_max = nt * k < ne ? nt * k : ne;
    if ((rc = launch_seg_matmul(c, st, L.m[0].type, true, w.seg_gu, w.nseg, nseg_max, M.e, M.ff, x, M.e, w.row_token,
                                w.act, nt)))
        return rc;
    if ((rc = launch_seg_matmul(c, st, L.m[2].type, false, w.seg_dn, w.nseg, nseg_max, M.ff, M.e, w.act, M.ff, nullptr,
                                w.hrow, nt)))
        return rc;
    if (shared) DNB_CUDA(cudaStreamWaitEvent(st, c->ev_join, 0));
    return launch_combine(c, st, w.hrow, w.pos, wts, nt, k, M.e, shared ? w.sh : nullptr,
                          (shared && L.shared_gate_row) ? w.shcoef : nullptr, out);
}

// One token: fused router kernel, gate/up GEMV over the k routed experts plus the
// shared expert as one more segment, down GEMV with the weighted sum fused in.
// Three launches.  With `residual` (== out for the in-place stack) the result is
// residual + block(h).
// Returns DNB_DECLINED when a shape or type combination is outside this path.
static int block_dev_decode(dnb_ctx* c, int layer, const float* h, float* out, const float* residual) {
    const Model& M = c->model;
    const Layer& L = M.layers[layer];
    Workspace& w = c->ws;
    cudaStream_t st = c->stream;
    const bool shared = L.has_shared();
    const bool fold = shared && L.m[3].type == L.m[0].type && L.m[4].type == L.m[1].type &&
                      L.m[5].type == L.m[2].type && L.m[3].n_out == M.ff;
    if (shared && !fold) return DNB_DECLINED;
    if (L.m[0].type != L.m[1].type) return DNB_DECLINED;
    int rc;
    if (c->gemv_mma && c->decode_fused && c->decode_routed && L.m[0].type == T_IQ3_XXS && L.m[2].type == T_IQ3_XXS) {
        // the whole block, router included, in one kernel (decode_fused.cu, ROUTED)
        rc = launch_decode_block(c, st, M, L, w, fold, h, residual, out, c->gbar);
        if (rc != DNB_DECLINED) return rc;
    }
    rc = launch_router_decode(c, st, h, M, L, w, fold, c->ticket);
    if (rc) return rc;
    const int nseg = M.k + (fold ? 1 : 0);
    const float* xperm = M.ne >= 4 * kActRep ? w.xn_perm : nullptr;
    if (c->gemv_mma && c->decode_fused && L.m[0].type == T_IQ3_XXS && L.m[2].type == T_IQ3_XXS && decode_fused_fits(c, nseg, M.e, M.ff)) {
        // gate/up, SwiGLU, down and the weighted sum in one kernel (decode_fused.cu)
        const float* fcoef = nullptr;
        if (fold && L.shared_gate_row) {
            if ((rc = launch_shared_coef(c, st, w.xn, L.shared_gate_row, 1, M.e, w.shcoef))) return rc;
            fcoef = w.shcoef;
        }
        rc = launch_decode_fused(c, st, w.seg_gu, w.seg_dn, nseg, M.k, fold, M.e, M.ff, w.xn, xperm, w.act, w.act_h, w.wts,
                                 fcoef, residual, out, c->gbar);
        if (rc != DNB_DECLINED) return rc;
    }
    rc = launch_seg_gemv_m1(c, st, L.m[0].type, true, true, w.seg_gu, nullptr, nseg, M.e, M.ff, w.xn, M.e, nullptr, w.act,
                            nullptr, "gemv_gate_up",
                            PermOut{w.act_perm, L.m[2].type, M.ne >= 4 * kActRep ? w.xn_perm : nullptr});
    const bool have_perm = rc == DNB_OK;  // the tiled fallback below writes plain rows only
    if (rc == DNB_DECLINED)
        rc = launch_seg_matmul(c, st, L.m[0].type, true, w.seg_gu, nullptr, nseg, M.e, M.ff, w.xn, M.e, w.row_token, w.act, 1);
    if (rc) return rc;
    if (fold && L.shared_gate_row)
        if ((rc = launch_shared_coef(c, st, w.xn, L.shared_gate_row, 1, M.e, w.shcoef))) return rc;
    const float* coef = (fold && L.shared_gate_row) ? w.shcoef : nullptr;
    rc = launch_down_combine(c, st, L.m[2].type, w.seg_dn, nseg, M.k, M.ff, M.e, w.act, w.wts, coef, fold, residual, out,
                             have_perm ? w.act_perm : nullptr);
    if (rc != DNB_DECLINED) return rc;
    rc = launch_seg_gemv_m1(c, st, L.m[2].type, false, false, w.seg_dn, nullptr, nseg, M.ff, M.e, w.act, M.ff, nullptr,
                            w.hrow, nullptr, "gemv_down");
    if (rc == DNB_DECLINED)
        rc = launch_seg_matmul(c, st, L.m[2].type, false, w.seg_dn, nullptr, nseg, M.ff, M.e, w.act, M.ff, nullptr, w.hrow, 1);
    if (rc) return rc;
    if ((rc = launch_combine(c, st, w.hrow, w.pos, w.wts, 1, M.k, M.e, fold ? w.hrow + (size_t)M.k * M.e : nullptr, coef,
                             residual ? w.out : out)))
        return rc;
    if (residual) return launch_add_inplace(c, st, out, w.out, (size_t)M.e);
    return DNB_OK;
}

// A decode batch (2..kDecodeBatchMax tokens, continuous batching): the one-token kernels over
// token-major one-row segments.  Router: RMSNorm, logits and top-k kernels of the general
// path, then the segment tables; gate/up GEMV with the CTA's token selecting the activation
// row; down GEMV + weighted sum with one grid row per token.  A token's arithmetic is the
// one-token path's, so its result does not depend on what else is in the batch.
static int block_dev_decode_batch(dnb_ctx* c, int layer, const float* h, int nt, float* out, const float* residual) {
    const Model& M = c->model;
    const Layer& L = M.layers[layer];
    Workspace& w = c->ws;
    cudaStream_t st = c->stream;
    const bool shared = L.has_shared();
    const bool fold = shared && L.m[3].type == L.m[0].type && L.m[4].type == L.m[1].type &&
                      L.m[5].type == L.m[2].type && L.m[3].n_out == M.ff;
    if ((shared && !fold) || L.m[0].type != L.m[1].type) return DNB_DECLINED;
    const int per = M.k + (fold ? 1 : 0), nseg = nt * per;
    if (nt < 2 || nt > kDecodeBatchMax || M.k + 1 > 64) return DNB_DECLINED;
    int rc;
    if (L.norm_w)
        if ((rc = launch_rmsnorm(c, st, h, L.norm_w, M.eps, nt, M.e, w.xn))) return rc;
    const float* x = L.norm_w ? w.xn : h;
    if ((rc = launch_router_logits(c, st, x, nt, M.e, L.router_w, L.router_bias, M.ne, w.logits))) return rc;
    if ((rc = launch_topk(c, st, w.logits, nt, M.ne, M.k, M.norm_topk, w.sels, w.wts, nullptr))) return rc;
    if ((rc = launch_decode_batch_tables(c, st, w.sels, nt, M.k, L, w, fold))) return rc;
    rc = launch_seg_gemv_m1(c, st, L.m[0].type, true, true, w.seg_gu, nullptr, nseg, M.e, M.ff, x, M.e, w.row_token, w.act,
                            nullptr, "gemv_gate_up", PermOut{w.act_perm, L.m[2].type, nullptr});
    if (rc) return rc;  // declined: nothing the later kernels depend on has been replaced, the caller runs the general path
    const float* coef = nullptr;
    if (fold && L.shared_gate_row) {
        if ((rc = launch_shared_coef(c, st, x, L.shared_gate_row, nt, M.e, w.shcoef))) return rc;
        coef = w.shcoef;
    }
    return launch_down_combine(c, st, L.m[2].type, w.seg_dn, per, M.k, M.ff, M.e, w.act, w.wts, coef, fold, residual, out,
                               w.act_perm, nt);
}

// Prefill chunks of all-Q4_K layers: expert-major packed rows as bf16 hi/lo, grouped
// GEMMs on tcgen05 (gate/up with the SwiGLU epilogue, then down), weighted combine.
// The common block format of matrices [first, last) when a tensor-core grouped GEMM takes it
// (Q4_K: three-product kernel of grouped_umma.cu; IQ3_XXS: exact-weight kernel of grouped_exact.cu), else -1.
static int tc_type(const Layer& L, int first, int last) {
    const int ty = L.m[first].type;
    if (ty != T_Q4_K && ty != T_IQ3_XXS) return -1;
    for (int i = first; i < last; ++i)
        if (!L.m[i].dev || L.m[i].type != ty) return -1;
    return ty;
}
// Tokens from which a chunk or decode batch leaves the one-token kernels for the tensor-core grouped GEMM.
static int tc_min_tokens(const dnb_ctx* c, int ty) { return ty == T_Q4_K ? 16 : c->exact_min_nt; }

static bool umma_eligible(const dnb_ctx* c, const Layer& L, int nt) {
    const Model& M = c->model;
    if (!c->use_umma || !c->ws.maps_ok) return false;
    if (M.e % 256 || M.ff % 256 || M.e % 128 || M.ff % 128) return false;
    const int ty = tc_type(L, 0, 3);
    if (ty < 0 || nt < tc_min_tokens(c, ty)) return false;
    if (L.has_shared()) {  // the shared expert rides in the same launches as one more segment
        if (tc_type(L, 3, 6) != ty || L.m[3].n_out != M.ff) return false;
    }
    return true;
}

static int experts_dev_umma(dnb_ctx* c, int layer, const float* x, int nt, const int32_t* sels, const float* wts,
                            float* out, int k = -1, int ne = -1, int with_shared = -1) {
    const Model& M = c->model;
    const Layer& L = M.layers[layer];
    Workspace& w = c->ws;
    cudaStream_t st = c->stream;
    if (k < 0) k = M.k;
    if (ne < 0) ne = M.ne;
    const bool shared = with_shared < 0 ? L.has_shared() : (with_shared != 0);
    int rc;
    if ((rc = launch_route_tables(c, st, sels, nt, k, ne, L, w, shared))) return rc;
    const int rows = nt * k + (shared ? nt : 0);
    const int nseg_max = (nt * k < ne ? nt * k : ne) + (shared ? 1 : 0);
    const int ty = L.m[0].type;
    if (ty == T_Q4_K && c->q4k_int && w.q4k_int_ok) {
        // integer weights, block scales after the tensor-core sum: fp16 rows in, fp32 activations between the two GEMMs
        if ((rc = launch_rows_f16(c, st, x, M.e, w.row_token, rows, M.e, w.xq_hi, w.xq_lo, w.xq_scale, "rows_f16_x"))) return rc;
        if ((rc = launch_grouped_q4k_int(c, st, true, w.seg_gu, w.nseg, nseg_max, M.e, M.ff, &w.maps_xq, w.xq_scale, w.act))) return rc;
        if ((rc = launch_rows_f16(c, st, w.act, M.ff, nullptr, rows, M.ff, w.aq_hi, w.aq_lo, w.aq_scale, "rows_f16_act"))) return rc;
        if ((rc = launch_grouped_q4k_int(c, st, false, w.seg_dn, w.nseg, nseg_max, M.ff, M.e, &w.maps_aq, w.aq_scale, w.hrow))) return rc;
        if (shared && L.shared_gate_row)
            if ((rc = launch_shared_coef(c, st, x, L.shared_gate_row, nt, M.e, w.shcoef))) return rc;
        return launch_combine(c, st, w.hrow, w.pos, wts, nt, k, M.e, shared ? w.hrow + (size_t)nt * k * M.e : nullptr,
                              (shared && L.shared_gate_row) ? w.shcoef : nullptr, out);
    }
    if ((rc = launch_gather_split(c, st, x, M.e, w.row_token, rows, M.e, w.xg_hi, w.xg_lo))) return rc;
    if ((rc = launch_grouped_tc(c, st, ty, true, w.seg_gu, w.nseg, nseg_max, M.e, M.ff, &w.maps_x, nt, w.act_hi, w.act_lo,
                                nullptr)))
        return rc;
    if ((rc = launch_grouped_tc(c, st, ty, false, w.seg_dn, w.nseg, nseg_max, M.ff, M.e, &w.maps_act, nt, nullptr, nullptr,
                                w.hrow)))
        return rc;
    if (shared && L.shared_gate_row)
        if ((rc = launch_shared_coef(c, st, x, L.shared_gate_row, nt, M.e, w.shcoef))) return rc;
    return launch_combine(c, st, w.hrow, w.pos, wts, nt, k, M.e, shared ? w.hrow + (size_t)nt * k * M.e : nullptr,
                          (shared && L.shared_gate_row) ? w.shcoef : nullptr, out);
}

// Router logits of nt rows: the tensor-core kernel from kRouterTcMin tokens, the fp32 kernel below.
int router_logits(dnb_ctx* c, cudaStream_t st, const float* x, int nt, const Layer& L, float* logits) {
    const Model& M = c->model;
    if (router_tc_eligible(c, L, nt)) return launch_router_logits_tc(c, st, x, nt, M.e, L, M.ne, logits);
    return launch_router_logits(c, st, x, nt, M.e, L.router_w, L.router_bias, M.ne, logits);
}

int router_topk_dev(dnb_ctx* c, cudaStream_t st, const float* x, int nt, const Layer& L, int32_t* sels, float* wts,
                    float* rowsum, bool x_is_split) {
    const Model& M = c->model;
    Workspace& w = c->ws;
    int rc;
    if (router_tc_eligible(c, L, nt)) {
        // the top-k kernel adds the K splits' partial sums itself (the reduce kernel's order: the same logits)
        if ((rc = launch_router_logits_tc(c, st, x, nt, M.e, L, M.ne, w.logits, false, x_is_split))) return rc;
        const int ns = router_tc_split(M.e);
        return launch_topk(c, st, ns > 1 ? w.rpart : w.logits, nt, M.ne, M.k, M.norm_topk, sels, wts, rowsum, ns, L.router_bias);
    }
    if ((rc = launch_router_logits(c, st, x, nt, M.e, L.router_w, L.router_bias, M.ne, w.logits))) return rc;
    return launch_topk(c, st, w.logits, nt, M.ne, M.k, M.norm_topk, sels, wts, rowsum);
}

static int block_dev(dnb_ctx* c, int layer, const float* h, int nt, float* out) {
    const Model& M = c->model;
    const Layer& L = M.layers[layer];
    Workspace& w = c->ws;
    cudaStream_t st = c->stream;
    int rc;
    if (nt == 1 && c->decode_fast) {
        rc = block_dev_decode(c, layer, h, out, nullptr);
        if (rc != DNB_DECLINED) return rc;
    }
    if (nt > 1 && nt <= kDecodeBatchMax && c->decode_fast && !umma_eligible(c, L, nt)) {
        rc = block_dev_decode_batch(c, layer, h, nt, out, nullptr);
        if (rc != DNB_DECLINED) return rc;
    }
    const bool shared = L.has_shared();
    // the RMSNorm kernel writes the router's operand (three bf16 parts of the normalised rows) in the same pass
    const bool split_in_prep = L.norm_w && router_tc_eligible(c, L, nt);
    if (L.norm_w || shared) {
        if ((rc = launch_prep(c, st, h, L.norm_w, M.eps, nt, M.e, w.xn, shared ? w.seg_sh_gu : nullptr,
                              shared ? w.seg_sh_dn : nullptr, L.m[3].dev, L.m[4].dev, L.m[5].dev,
                              split_in_prep ? w.x3 : nullptr, w.x3_part)))
            return rc;
    }
    const float* x = L.norm_w ? w.xn : h;
    if ((rc = router_topk_dev(c, st, x, nt, L, w.sels, w.wts, nullptr, split_in_prep))) return rc;
    if (umma_eligible(c, L, nt)) return experts_dev_umma(c, layer, x, nt, w.sels, w.wts, out);
    return experts_dev(c, layer, x, nt, w.sels, w.wts, out);
}

}  // namespace dnb

using namespace dnb;

extern "C" {

const char* dnb_last_error(void) { return g_err; }

int dnb_init(int device, dnb_ctx** out) {
    if (!out) return DNB_ERR_ARG;
    *out = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) {
        set_error("no CUDA device (%s); this library has no CPU path", e == cudaSuccess ? "count is 0" : cudaGetErrorString(e));
        return DNB_ERR_NO_DEVICE;
    }
    if (device < 0 || device >= n) {
        set_error("device %d out of range (0..%d)", device, n - 1);
        return DNB_ERR_ARG;
    }
    DNB_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    DNB_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) {
        set_error("device %d is sm_%d%d; the kernels are built for sm_100a only", device, prop.major, prop.minor);
        return DNB_ERR_NO_DEVICE;
    }
    dnb_ctx* c = new dnb_ctx();
    c->device = device;
    c->sm_count = prop.multiProcessorCount;
    DNB_CUDA(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
    DNB_CUDA(cudaStreamCreateWithFlags(&c->side, cudaStreamNonBlocking));
    DNB_CUDA(cudaEventCreateWithFlags(&c->ev_fork, cudaEventDisableTiming));
    DNB_CUDA(cudaEventCreateWithFlags(&c->ev_join, cudaEventDisableTiming));
    DNB_CUDA(cudaEventCreate(&c->ev_t0));
    DNB_CUDA(cudaEventCreate(&c->ev_t1));
    // The status word sits in pinned host memory the kernels can address: a wait that gave up is
    // visible to the host right after the synchronisation every host-buffer call ends with.
    DNB_CUDA(cudaHostAlloc((void**)&c->status_host, 64, cudaHostAllocMapped | cudaHostAllocPortable));
    memset(c->status_host, 0, 64);
    DNB_CUDA(cudaHostGetDevicePointer((void**)&c->status, c->status_host, 0));
    DNB_CUDA(cudaMalloc((void**)&c->ticket, sizeof(unsigned int)));
    DNB_CUDA(cudaMemset(c->ticket, 0, sizeof(unsigned int)));
    DNB_CUDA(cudaMalloc((void**)&c->gbar, sizeof(unsigned long long)));
    DNB_CUDA(cudaMemset(c->gbar, 0, sizeof(unsigned long long)));
    *out = c;
    return DNB_OK;
}

static void free_layer(Layer& L) {
    for (auto& t : L.m)
        if (t.dev && t.owned) cudaFree(t.dev);
    if (L.router_w) cudaFree(L.router_w);
    if (L.router_w3) cudaFree(L.router_w3);
    if (L.router_bias) cudaFree(L.router_bias);
    if (L.norm_w) cudaFree(L.norm_w);
    if (L.shared_gate_row) cudaFree(L.shared_gate_row);
    L = Layer();
}

void dnb_shutdown(dnb_ctx* c) {
    if (!c) return;
    cudaSetDevice(c->device);
    cudaDeviceSynchronize();
    drop_graphs(c);
    ep_release(c);
    epd_release(c);
    hc_release(c);
    for (auto& kv : c->matrices) cudaFree(kv.second.dev);
    for (auto& L : c->model.layers) free_layer(L);
    free_ws(c->ws);
    if (c->gemv_x.p) cudaFree(c->gemv_x.p);
    if (c->gemv_out.p) cudaFree(c->gemv_out.p);
    if (c->gemv_host.p) cudaFreeHost(c->gemv_host.p);
    if (c->gg_x.p) cudaFree(c->gg_x.p);
    if (c->gg_out.p) cudaFree(c->gg_out.p);
    if (c->gg_seg.p) cudaFree(c->gg_seg.p);
    if (c->status_host) cudaFreeHost(c->status_host);
    if (c->ticket) cudaFree(c->ticket);
    if (c->gbar) cudaFree(c->gbar);
    if (c->own_stream && c->stream) cudaStreamDestroy(c->stream);
    if (!c->own_stream && c->saved_stream) cudaStreamDestroy(c->saved_stream);
    if (c->flush.p) cudaFree(c->flush.p);
    if (c->side) cudaStreamDestroy(c->side);
    cudaEventDestroy(c->ev_fork);
    cudaEventDestroy(c->ev_join);
    cudaEventDestroy(c->ev_t0);
    cudaEventDestroy(c->ev_t1);
    for (auto& r : c->prof.recs) { cudaEventDestroy(r.a); cudaEventDestroy(r.b); }
    for (auto& e : c->prof.pool) cudaEventDestroy(e);
    delete c;
}

int dnb_set_stream(dnb_ctx* c, void* stream) {
    if (!c) return DNB_ERR_ARG;
    DNB_CUDA(cudaSetDevice(c->device));
    DNB_CUDA(cudaStreamSynchronize(c->stream));
    drop_graphs(c);
    if (stream) {
        if (c->own_stream) c->saved_stream = c->stream;
        c->stream = (cudaStream_t)stream;
        c->own_stream = false;
    } else if (!c->own_stream) {
        c->stream = c->saved_stream;
        c->own_stream = true;
    }
    return DNB_OK;
}

int dnb_sync(dnb_ctx* c) {
    if (!c) return DNB_ERR_ARG;
    DNB_CUDA(cudaSetDevice(c->device));
    DNB_CUDA(cudaStreamSynchronize(c->stream));
    DNB_CUDA(cudaStreamSynchronize(c->side));
    const int st = *reinterpret_cast<volatile int*>(c->status_host);
    if (st != 0) {  // sticky until dnb_clear_status: the device-pointer calls since then cannot be trusted
        set_error("sync: a bounded device wait gave up (status %d) since the status was last cleared", st);
        return DNB_DECLINED;
    }
    return DNB_OK;
}

uint64_t dnb_launch_count(dnb_ctx* c) { return c ? c->launches : 0; }

int dnb_device_status(dnb_ctx* c, int* status) {
    if (!c || !status) return DNB_ERR_ARG;
    DNB_CUDA(cudaSetDevice(c->device));
    DNB_CUDA(cudaStreamSynchronize(c->stream));
    DNB_CUDA(cudaStreamSynchronize(c->side));
    *status = *reinterpret_cast<volatile int*>(c->status_host);
    return DNB_OK;
}

int dnb_clear_status(dnb_ctx* c) {
    if (!c) return DNB_ERR_ARG;
    DNB_CUDA(cudaSetDevice(c->device));
    DNB_CUDA(cudaStreamSynchronize(c->stream));
    DNB_CUDA(cudaStreamSynchronize(c->side));
    *reinterpret_cast<volatile int*>(c->status_host) = 0;
    return DNB_OK;
}

int dnb_set_wait_limits(dnb_ctx* c, int barrier_polls, int flag_polls, int barrier_bias) {
    if (!c || barrier_polls < 1 || flag_polls < 1 || barrier_bias < 0) return DNB_ERR_ARG;
    DNB_CUDA(cudaSetDevice(c->device));
    DNB_CUDA(cudaDeviceSynchronize());
    drop_graphs(c);  // the limits are kernel arguments baked into captured launches
    c->barrier_polls = barrier_polls;
    c->flag_polls = flag_polls;
    c->barrier_bias = (unsigned int)barrier_bias;
    return DNB_OK;
}

int dnb_timer_start(dnb_ctx* c) {
    if (!c) return DNB_ERR_ARG;
    DNB_CUDA(cudaEventRecord(c->ev_t0, c->stream));
    return DNB_OK;
}

int dnb_timer_stop(dnb_ctx* c, float* ms) {
    if (!c || !ms) return DNB_ERR_ARG;
    DNB_CUDA(cudaEventRecord(c->ev_t1, c->stream));
    DNB_CUDA(cudaEventSynchronize(c->ev_t1));
    DNB_CUDA(cudaEventElapsedTime(ms, c->ev_t0, c->ev_t1));
    return DNB_OK;
}

int dnb_dev_alloc(dnb_ctx* c, size_t bytes, void** dev) {
    if (!c || !dev) return DNB_ERR_ARG;
    DNB_CUDA(cudaSetDevice(c->device));
    DNB_CUDA(cudaMalloc(dev, bytes));
    return DNB_OK;
}

int dnb_dev_free(dnb_ctx* c, void* dev) {
    if (!c) return DNB_ERR_ARG;
    DNB_CUDA(cudaSetDevice(c->device));
    DNB_CUDA(cudaFree(dev));
    return DNB_OK;
}

int dnb_dev_upload(dnb_ctx* c, void* dev, const void* host, size_t bytes) {
    if (!c) return DNB_ERR_ARG;
    DNB_CUDA(cudaMemcpyAsync(dev, host, bytes, cudaMemcpyHostToDevice, c->stream));
    DNB_CUDA(cudaStreamSynchronize(c->stream));
    return DNB_OK;
}

int dnb_dev_download(dnb_ctx* c, void* host, const void* dev, size_t bytes) {
    if (!c) return DNB_ERR_ARG;
    DNB_CUDA(cudaMemcpyAsync(host, dev, bytes, cudaMemcpyDeviceToHost, c->stream));
    DNB_CUDA(cudaStreamSynchronize(c->stream));
    return DNB_OK;
}

int dnb_dev_copy(dnb_ctx* c, void* dst, const void* src, size_t bytes) {
    if (!c) return DNB_ERR_ARG;
    DNB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, c->stream));
    return DNB_OK;
}

int dnb_flush_l2(dnb_ctx* c) {
    if (!c) return DNB_ERR_ARG;
    const size_t bytes = 256u << 20;  // > 126 MB L2
    int rc = grow(c->flush, bytes);
    if (rc) return rc;
    return launch_fill_u32(c, c->stream, (uint32_t*)c->flush.p, 0u, bytes / 4);
}

int dnb_use_graphs(dnb_ctx* c, int on) {
    if (!c) return DNB_ERR_ARG;
    DNB_CUDA(cudaDeviceSynchronize());
    drop_graphs(c);
    c->use_graphs = on != 0;
    return DNB_OK;
}

int dnb_stall(dnb_ctx* c, float ms) {
    if (!c) return DNB_ERR_ARG;
    return launch_stall(c, c->stream, ms);
}

int dnb_profile_enable(dnb_ctx* c, int on) {
    if (!c) return DNB_ERR_ARG;
    DNB_CUDA(cudaDeviceSynchronize());
    for (auto& r : c->prof.recs) { c->prof.pool.push_back(r.a); c->prof.pool.push_back(r.b); }
    c->prof.recs.clear();
    c->prof.on = on != 0;
    return DNB_OK;
}

int dnb_profile_read(dnb_ctx* c, char* buf, size_t cap) {
    if (!c || !buf || cap < 64) return DNB_ERR_ARG;
    DNB_CUDA(cudaDeviceSynchronize());
    std::map<std::string, std::pair<long, double>> acc;
    for (auto& r : c->prof.recs) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, r.a, r.b) == cudaSuccess) {
            auto& e = acc[r.name];
            e.first++;
            e.second += ms;
        }
    }
    size_t n = 0;
    n += snprintf(buf + n, cap - n, "{");
    bool first = true;
    for (auto& kv : acc) {
        if (n + 128 >= cap) break;
        n += snprintf(buf + n, cap - n, "%s\"%s\": {\"launches\": %ld, \"ms\": %.6f}", first ? "" : ", ",
                      kv.first.c_str(), kv.second.first, kv.second.second);
        first = false;
    }
    snprintf(buf + n, cap - n, "}");
    return DNB_OK;
}

// ---- single matrix ---------------------------------------------------------------

int dnb_register_matrix(dnb_ctx* c, uint64_t uid, int type, const void* blocks, size_t bytes, int k, int n) {
    if (!c || !blocks) return DNB_ERR_ARG;
    const size_t rb = row_bytes(type, k);
    if (rb == 0 || !type_supported(type)) {
        set_error("register_matrix: ggml type %d with k=%d is not handled", type, k);
        return DNB_DECLINED;
    }
    if (n <= 0 || bytes != rb * (size_t)n) {
        set_error("register_matrix: %zu bytes given, %zu expected for %d rows of %d", bytes, rb * (size_t)n, n, k);
        return DNB_ERR_ARG;
    }
    DNB_CUDA(cudaSetDevice(c->device));
    auto it = c->matrices.find(uid);
    if (it != c->matrices.end()) {
        cudaFree(it->second.dev);
        c->matrices.erase(it);
    }
    Matrix m{type, k, n, rb, nullptr};
    DNB_CUDA(cudaMalloc((void**)&m.dev, bytes));
    DNB_CUDA(cudaMemcpy(m.dev, blocks, bytes, cudaMemcpyHostToDevice));
    c->matrices[uid] = m;
    return DNB_OK;
}

int dnb_set_tc_min_tokens(dnb_ctx* c, int iq3_xxs_min_tokens) {
    if (!c || iq3_xxs_min_tokens < 1) return DNB_ERR_ARG;
    DNB_CUDA(cudaDeviceSynchronize());
    drop_graphs(c);
    c->exact_min_nt = iq3_xxs_min_tokens;
    return DNB_OK;
}

int dnb_set_q4k_int(dnb_ctx* c, int on) {
    if (!c) return DNB_ERR_ARG;
    DNB_CUDA(cudaDeviceSynchronize());
    drop_graphs(c);
    if (c->q4k_int != (on != 0)) free_ws(c->ws);  // its operand buffers exist only while it is on: the next call sizes the workspace again
    c->q4k_int = on != 0;
    return DNB_OK;
}

int dnb_set_router_tc(dnb_ctx* c, int on) {
    if (!c) return DNB_ERR_ARG;
    DNB_CUDA(cudaDeviceSynchronize());
    drop_graphs(c);
    c->router_tc = on != 0;
    return DNB_OK;
}

int dnb_set_gemv_impl(dnb_ctx* c, int impl) {
    if (!c || impl < 0 || impl > 5) return DNB_ERR_ARG;
    DNB_CUDA(cudaDeviceSynchronize());
    drop_graphs(c);
    c->gemv_impl = impl == 1 ? 1 : 0;
    c->decode_fast = impl != 2;
    c->use_umma = impl != 2;
    c->gemv_mma = impl != 3;
    c->decode_fused = impl != 3 && impl != 4;
    c->decode_routed = impl != 5;
    return DNB_OK;
}

static int gemv_dev(dnb_ctx* c, int type, const uint8_t* w, int k, int n, const float* x, float* out, int nvec) {
    if (c->gemv_impl == 1) {
        for (int v = 0; v < nvec; ++v) {
            int rc = launch_gemv_seq(c, c->stream, type, w, x + (size_t)v * k, out + (size_t)v * n, k, n);
            if (rc) return rc;
        }
        return DNB_OK;
    }
    const SegDesc sd{w, nullptr, (uint32_t)nvec, 0u};
    if (nvec == 1 && c->decode_fast && (((uintptr_t)w) & 15) == 0) {
        const int rc = launch_seg_gemv_m1(c, c->stream, type, false, true, nullptr, nullptr, 1, k, n, x, k, nullptr, out, &sd,
                                          "gemv_single");
        if (rc != DNB_DECLINED) return rc;
    }
    return launch_seg_matmul(c, c->stream, type, false, nullptr, nullptr, 1, k, n, x, k, nullptr, out, nvec, &sd);
}

int dnb_gemv_dev(dnb_ctx* c, int type, const void* w_dev, int k, int n, const float* x_dev, float* out_dev, int nvec) {
    if (!c || !w_dev || !x_dev || !out_dev || nvec < 1) return DNB_ERR_ARG;
    if (row_bytes(type, k) == 0 || !type_supported(type)) {
        set_error("gemv: ggml type %d with k=%d is not handled", type, k);
        return DNB_DECLINED;
    }
    DNB_CUDA(cudaSetDevice(c->device));
    return gemv_dev(c, type, (const uint8_t*)w_dev, k, n, x_dev, out_dev, nvec);
}

int dnb_gemv(dnb_ctx* c, uint64_t uid, const float* x, float* out) {
    if (!c || !x || !out) return DNB_ERR_ARG;
    auto it = c->matrices.find(uid);
    if (it == c->matrices.end()) {
        set_error("gemv: uid %llu is not registered", (unsigned long long)uid);
        return DNB_DECLINED;
    }
    const Matrix& m = it->second;
    DNB_CUDA(cudaSetDevice(c->device));
    int rc;
    if ((rc = grow(c->gemv_x, (size_t)m.k * 4))) return rc;
    if ((rc = grow(c->gemv_out, (size_t)m.n * 4))) return rc;
    DNB_CUDA(cudaMemcpyAsync(c->gemv_x.p, x, (size_t)m.k * 4, cudaMemcpyHostToDevice, c->stream));
    if ((rc = gemv_dev(c, m.type, m.dev, m.k, m.n, (const float*)c->gemv_x.p, (float*)c->gemv_out.p, 1))) return rc;
    if ((rc = grow(c->gemv_host, (size_t)m.n * 4, true))) return rc;
    DNB_CUDA(cudaMemcpyAsync(c->gemv_host.p, c->gemv_out.p, (size_t)m.n * 4, cudaMemcpyDeviceToHost, c->stream));
    DNB_CUDA(wait_short(c->stream));
    if ((rc = finish_checked(c, "gemv"))) return rc;
    memcpy(out, c->gemv_host.p, (size_t)m.n * 4);
    return DNB_OK;
}

// ---- model --------------------------------------------------------------------------

int dnb_moe_config(dnb_ctx* c, int n_layer, int e, int ff, int sff, int ne, int k, float eps, int norm_topk) {
    if (!c) return DNB_ERR_ARG;
    if (n_layer < 1 || e < 32 || ff < 32 || ne < 1 || k < 1 || k > ne || e % 32 || ff % 32 || (sff && sff % 32)) {
        set_error("moe_config: bad shape (layers %d, embd %d, ff %d, shared ff %d, experts %d, used %d)", n_layer, e, ff,
                  sff, ne, k);
        return DNB_ERR_ARG;
    }
    if (ne > 1024 || k > 32) {
        set_error("moe_config: the router kernels cover n_expert <= 1024 and k <= 32");
        return DNB_DECLINED;
    }
    DNB_CUDA(cudaSetDevice(c->device));
    DNB_CUDA(cudaDeviceSynchronize());
    drop_graphs(c);
    for (auto& L : c->model.layers) free_layer(L);
    free_ws(c->ws);
    hc_release(c);
    Model& M = c->model;
    M.n_layer = n_layer; M.e = e; M.ff = ff; M.sff = sff; M.ne = ne; M.k = k; M.eps = eps; M.norm_topk = norm_topk;
    M.shard_first = 0; M.shard_count = ne;
    M.layers.assign(n_layer, Layer());
    return DNB_OK;
}

static int check_expert_shape(dnb_ctx* c, int layer, int matrix, int type, int n_in, int n_out, int n_expert,
                              size_t* rb_out) {
    const Model& M = c->model;
    if (layer < 0 || layer >= M.n_layer || matrix < 0 || matrix > 5) {
        set_error("experts: layer %d / matrix %d out of range", layer, matrix);
        return DNB_ERR_ARG;
    }
    const size_t rb = row_bytes(type, n_in);
    if (rb == 0 || !type_supported(type)) {
        set_error("experts: ggml type %d with n_in=%d is not handled", type, n_in);
        return DNB_DECLINED;
    }
    const bool shared = matrix >= 3;
    const bool down = (matrix % 3) == 2;
    const int ffx = shared ? (M.sff ? M.sff : M.ff) : M.ff;
    const int want_in = down ? ffx : M.e, want_out = down ? M.e : ffx, want_ne = shared ? 1 : M.shard_count;
    if (n_in != want_in || n_out != want_out || n_expert != want_ne) {
        set_error("experts: matrix %d is [%d x %d] x %d experts, the model needs [%d x %d] x %d", matrix, n_out, n_in,
                  n_expert, want_out, want_in, want_ne);
        return DNB_ERR_ARG;
    }
    *rb_out = rb;
    return DNB_OK;
}

static int install_tensor(dnb_ctx* c, int layer, int matrix, int type, int n_in, int n_out, int n_expert, size_t rb) {
    DNB_CUDA(cudaDeviceSynchronize());
    drop_graphs(c);
    Layer& L = c->model.layers[layer];
    ExpertTensor& t = L.m[matrix];
    if (t.dev && t.owned) cudaFree(t.dev);
    t = ExpertTensor();
    t.type = type; t.n_in = n_in; t.n_out = n_out; t.n_expert = n_expert;
    t.row_bytes = rb; t.expert_bytes = rb * (size_t)n_out;
    // 256 spare bytes: the tensor-core producers fetch whole 16-byte lines around blocks that are not 16-byte sized
    DNB_CUDA(cudaMalloc((void**)&t.dev, t.expert_bytes * (size_t)n_expert + 256));
    t.owned = true;
    return DNB_OK;
}

int dnb_register_experts(dnb_ctx* c, int layer, int matrix, int type, int n_in, int n_out, int n_expert,
                         const void* blocks, size_t bytes) {
    if (!c || !blocks) return DNB_ERR_ARG;
    size_t rb;
    int rc = check_expert_shape(c, layer, matrix, type, n_in, n_out, n_expert, &rb);
    if (rc) return rc;
    if (bytes != rb * (size_t)n_out * (size_t)n_expert) {
        set_error("experts: %zu bytes given, %zu expected", bytes, rb * (size_t)n_out * (size_t)n_expert);
        return DNB_ERR_ARG;
    }
    DNB_CUDA(cudaSetDevice(c->device));
    if ((rc = install_tensor(c, layer, matrix, type, n_in, n_out, n_expert, rb))) return rc;
    DNB_CUDA(cudaMemcpy(c->model.layers[layer].m[matrix].dev, blocks, bytes, cudaMemcpyHostToDevice));
    return DNB_OK;
}

int dnb_synth_experts(dnb_ctx* c, int layer, int matrix, int type, int n_in, int n_out, int n_expert, uint64_t seed) {
    if (!c) return DNB_ERR_ARG;
    size_t rb;
    int rc = check_expert_shape(c, layer, matrix, type, n_in, n_out, n_expert, &rb);
    if (rc) return rc;
    DNB_CUDA(cudaSetDevice(c->device));
    if ((rc = install_tensor(c, layer, matrix, type, n_in, n_out, n_expert, rb))) return rc;
    const uint64_t per_expert = (uint64_t)n_out * (n_in / block_elems(type));
    const uint64_t n_blocks = (uint64_t)n_expert * per_expert;
    // an expert-parallel shard holds experts [shard_first, shard_first + n_expert) of the full tensor
    const uint64_t first = matrix < 3 ? (uint64_t)c->model.shard_first * per_expert : 0;
    return launch_synth_blocks(c, c->stream, type, seed, (uint64_t)layer * 16 + matrix,
                               c->model.layers[layer].m[matrix].dev, n_blocks, first);
}

int dnb_download_expert(dnb_ctx* c, int layer, int matrix, int expert, void* dst, size_t bytes) {
    if (!c || !dst || layer < 0 || layer >= c->model.n_layer || matrix < 0 || matrix > 5) return DNB_ERR_ARG;
    const ExpertTensor& t = c->model.layers[layer].m[matrix];
    if (!t.dev || expert < 0 || expert >= t.n_expert || bytes != t.expert_bytes) {
        set_error("download_expert: tensor missing, expert out of range or size mismatch (%zu vs %zu)", bytes,
                  t.expert_bytes);
        return DNB_ERR_ARG;
    }
    DNB_CUDA(cudaStreamSynchronize(c->stream));
    DNB_CUDA(cudaMemcpy(dst, t.dev + (size_t)expert * t.expert_bytes, bytes, cudaMemcpyDeviceToHost));
    return DNB_OK;
}

static int upload_f32(float** dst, const float* src, size_t n) {
    if (*dst) cudaFree(*dst);
    *dst = nullptr;
    if (!src) return DNB_OK;
    DNB_CUDA(cudaMalloc((void**)dst, n * sizeof(float)));
    DNB_CUDA(cudaMemcpy(*dst, src, n * sizeof(float), cudaMemcpyHostToDevice));
    return DNB_OK;
}

int dnb_register_router(dnb_ctx* c, int layer, const float* w, const float* bias, const float* norm_w,
                        const float* shared_gate_row) {
    if (!c || !w || layer < 0 || layer >= c->model.n_layer) return DNB_ERR_ARG;
    DNB_CUDA(cudaSetDevice(c->device));
    const Model& M = c->model;
    Layer& L = c->model.layers[layer];
    int rc;
    DNB_CUDA(cudaDeviceSynchronize());
    drop_graphs(c);
    if ((rc = upload_f32(&L.router_w, w, (size_t)M.ne * M.e))) return rc;
    if ((rc = upload_f32(&L.router_bias, bias, (size_t)M.ne))) return rc;
    if ((rc = upload_f32(&L.norm_w, norm_w, (size_t)M.e))) return rc;
    if ((rc = upload_f32(&L.shared_gate_row, shared_gate_row, (size_t)M.e))) return rc;
    return router_tc_prepare(c, L, M.ne, M.e);
}

// ---- block ----------------------------------------------------------------------------

int dnb_moe_block_dev(dnb_ctx* c, int layer, const float* h_dev, int nt, float* out_dev) {
    if (!c || !h_dev || !out_dev || nt < 1) return DNB_ERR_ARG;
    if (!layer_ready(c, layer, true)) {
        set_error("moe_block: layer %d is not fully registered", layer);
        return DNB_DECLINED;
    }
    DNB_CUDA(cudaSetDevice(c->device));
    int rc = ensure_ws(c, nt);
    if (rc) return rc;
    return run_graphed(c, GraphKey{1, layer, nt, h_dev, out_dev}, [&]() { return block_dev(c, layer, h_dev, nt, out_dev); });
}

int dnb_moe_block(dnb_ctx* c, int layer, const float* h, int nt, float* out, int32_t* sels_out, float* wts_out) {
    if (!c || !h || !out || nt < 1) return DNB_ERR_ARG;
    if (!layer_ready(c, layer, true)) {
        set_error("moe_block: layer %d is not fully registered", layer);
        return DNB_DECLINED;
    }
    DNB_CUDA(cudaSetDevice(c->device));
    int rc = ensure_ws(c, nt);
    if (rc) return rc;
    Workspace& w = c->ws;
    const Model& M = c->model;
    const size_t bytes = (size_t)nt * M.e * sizeof(float);
    memcpy(w.pinned_in, h, bytes);
    const bool routing = sels_out || wts_out;
    rc = run_graphed(c, GraphKey{routing ? 3 : 2, layer, nt, nullptr, nullptr}, [&]() -> int {
        // A few tokens come in through a one-CTA kernel that reads the pinned buffer (see stage_in_kernel).
        int staged = DNB_DECLINED;
        if (nt <= 8 && c->decode_fast) staged = launch_stage_in(c, c->stream, w.pinned_in, w.hin, (size_t)nt * M.e);
        if (staged != DNB_OK && staged != DNB_DECLINED) return staged;
        if (staged == DNB_DECLINED) DNB_CUDA(cudaMemcpyAsync(w.hin, w.pinned_in, bytes, cudaMemcpyHostToDevice, c->stream));
        // A few tokens: the last kernel stores the result rows straight into the pinned host
        // buffer (it is device-addressable), which saves a copy node and its dependency edge
        // on a call that lasts tens of microseconds.  Larger results go through HBM and one copy.
        const bool direct = nt <= 8;
        const int r = block_dev(c, layer, w.hin, nt, direct ? w.pinned_out : w.out);
        if (r) return r;
        if (!direct) DNB_CUDA(cudaMemcpyAsync(w.pinned_out, w.out, bytes, cudaMemcpyDeviceToHost, c->stream));
        if (routing) {
            DNB_CUDA(cudaMemcpyAsync(w.pinned_sels, w.sels, (size_t)nt * M.k * 4, cudaMemcpyDeviceToHost, c->stream));
            DNB_CUDA(cudaMemcpyAsync(w.pinned_wts, w.wts, (size_t)nt * M.k * 4, cudaMemcpyDeviceToHost, c->stream));
        }
        return DNB_OK;
    });
    if (rc) return rc;
    DNB_CUDA(nt <= 64 ? wait_short(c->stream) : cudaStreamSynchronize(c->stream));
    if ((rc = finish_checked(c, "moe_block"))) return rc;
    memcpy(out, w.pinned_out, bytes);
    if (sels_out) memcpy(sels_out, w.pinned_sels, (size_t)nt * M.k * 4);
    if (wts_out) memcpy(wts_out, w.pinned_wts, (size_t)nt * M.k * 4);
    return DNB_OK;
}

int dnb_moe_experts(dnb_ctx* c, int layer, const float* x, int nt, const int32_t* sels, const float* wts, float* out) {
    if (!c || !x || !sels || !wts || !out || nt < 1) return DNB_ERR_ARG;
    if (!layer_ready(c, layer, false)) {
        set_error("moe_experts: layer %d has no expert tensors", layer);
        return DNB_DECLINED;
    }
    const Model& M = c->model;
    for (int t = 0; t < nt; ++t)
        for (int s = 0; s < M.k; ++s) {
            const int32_t e = sels[(size_t)t * M.k + s];
            if (e < 0 || e >= M.ne || (s > 0 && e <= sels[(size_t)t * M.k + s - 1])) {
                set_error("moe_experts: token %d slot %d: expert %d out of range or not ascending", t, s, e);
                return DNB_ERR_ARG;
            }
        }
    DNB_CUDA(cudaSetDevice(c->device));
    int rc = ensure_ws(c, nt);
    if (rc) return rc;
    Workspace& w = c->ws;
    const size_t bytes = (size_t)nt * M.e * sizeof(float), rows = (size_t)nt * M.k;
    memcpy(w.pinned_in, x, bytes);
    memcpy(w.pinned_sels, sels, rows * 4);
    memcpy(w.pinned_wts, wts, rows * 4);
    DNB_CUDA(cudaMemcpyAsync(w.hin, w.pinned_in, bytes, cudaMemcpyHostToDevice, c->stream));
    DNB_CUDA(cudaMemcpyAsync(w.sels, w.pinned_sels, rows * 4, cudaMemcpyHostToDevice, c->stream));
    DNB_CUDA(cudaMemcpyAsync(w.wts, w.pinned_wts, rows * 4, cudaMemcpyHostToDevice, c->stream));
    const Layer& L = M.layers[layer];
    if (L.has_shared())
        if ((rc = launch_prep(c, c->stream, w.hin, nullptr, M.eps, nt, M.e, nullptr, w.seg_sh_gu, w.seg_sh_dn,
                              L.m[3].dev, L.m[4].dev, L.m[5].dev)))
            return rc;
    if ((rc = experts_dev(c, layer, w.hin, nt, w.sels, w.wts, w.out))) return rc;
    DNB_CUDA(cudaMemcpyAsync(w.pinned_out, w.out, bytes, cudaMemcpyDeviceToHost, c->stream));
    DNB_CUDA(nt <= 64 ? wait_short(c->stream) : cudaStreamSynchronize(c->stream));
    if ((rc = finish_checked(c, "moe_experts"))) return rc;
    memcpy(out, w.pinned_out, bytes);
    return DNB_OK;
}

int dnb_router_topk(dnb_ctx* c, int layer, const float* x, int nt, int32_t* sels, float* wts, float* rowsum) {
    if (!c || !x || !sels || !wts || nt < 1) return DNB_ERR_ARG;
    if (layer < 0 || layer >= c->model.n_layer || !c->model.layers[layer].router_w) {
        set_error("router_topk: layer %d has no router", layer);
        return DNB_DECLINED;
    }
    DNB_CUDA(cudaSetDevice(c->device));
    int rc = ensure_ws(c, nt);
    if (rc) return rc;
    Workspace& w = c->ws;
    const Model& M = c->model;
    const Layer& L = M.layers[layer];
    const size_t bytes = (size_t)nt * M.e * sizeof(float), rows = (size_t)nt * M.k;
    memcpy(w.pinned_in, x, bytes);
    DNB_CUDA(cudaMemcpyAsync(w.hin, w.pinned_in, bytes, cudaMemcpyHostToDevice, c->stream));
    if ((rc = router_topk_dev(c, c->stream, w.hin, nt, L, w.sels, w.wts, rowsum ? w.shcoef : nullptr)))
        return rc;
    DNB_CUDA(cudaMemcpyAsync(w.pinned_sels, w.sels, rows * 4, cudaMemcpyDeviceToHost, c->stream));
    DNB_CUDA(cudaMemcpyAsync(w.pinned_wts, w.wts, rows * 4, cudaMemcpyDeviceToHost, c->stream));
    if (rowsum) DNB_CUDA(cudaMemcpyAsync(w.pinned_out, w.shcoef, (size_t)nt * 4, cudaMemcpyDeviceToHost, c->stream));
    DNB_CUDA(cudaStreamSynchronize(c->stream));
    if ((rc = finish_checked(c, "router_topk"))) return rc;
    memcpy(sels, w.pinned_sels, rows * 4);
    memcpy(wts, w.pinned_wts, rows * 4);
    if (rowsum) memcpy(rowsum, w.pinned_out, (size_t)nt * 4);
    return DNB_OK;
}

int dnb_grouped_gemm(dnb_ctx* c, int layer, int matrix, const uint32_t* segs, int nseg, const float* xs, float* outs) {
    if (!c || !segs || !xs || !outs || nseg < 1) return DNB_ERR_ARG;
    if (layer < 0 || layer >= c->model.n_layer || matrix < 0 || matrix > 5 || !c->model.layers[layer].m[matrix].dev) {
        set_error("grouped_gemm: layer %d matrix %d is not registered", layer, matrix);
        return DNB_DECLINED;
    }
    const ExpertTensor& t = c->model.layers[layer].m[matrix];
    // segment table contract of moe_expert.rs:8399-8440 (check_segments): m > 0,
    // offsets contiguous from 0, experts in range
    size_t row = 0;
    uint32_t m_max = 0;
    std::vector<SegDesc> sd(nseg);
    for (int i = 0; i < nseg; ++i) {
        const uint32_t ex = segs[4 * i], m = segs[4 * i + 1], xo = segs[4 * i + 2], oo = segs[4 * i + 3];
        if (m == 0 || ex >= (uint32_t)t.n_expert || xo != row || oo != row) {
            set_error("grouped_gemm: segment %d (expert %u, m %u, x_off %u, out_off %u) breaks the table contract", i, ex,
                      m, xo, oo);
            return DNB_ERR_ARG;
        }
        sd[i] = SegDesc{t.dev + (size_t)ex * t.expert_bytes, nullptr, m, (uint32_t)row};
        row += m;
        if (m > m_max) m_max = m;
    }
    DNB_CUDA(cudaSetDevice(c->device));
    // Grow-only staging buffers of the context (no allocation per call once they are large enough).
    int rc;
    if ((rc = grow(c->gg_x, row * t.n_in * sizeof(float)))) return rc;
    if ((rc = grow(c->gg_out, row * t.n_out * sizeof(float)))) return rc;
    if ((rc = grow(c->gg_seg, (size_t)nseg * sizeof(SegDesc) + 16))) return rc;
    float* dx = (float*)c->gg_x.p;
    float* dout = (float*)c->gg_out.p;
    SegDesc* dsd = (SegDesc*)c->gg_seg.p;
    int32_t* dnseg = (int32_t*)((uint8_t*)c->gg_seg.p + (size_t)nseg * sizeof(SegDesc));
    const Model& M = c->model;
    // Q4_K matrices of the model's own shapes with enough rows go to the tcgen05 grouped GEMM
    // (the packed rows are split to bf16 hi/lo in the workspace's operand buffers first).
    const bool in_e = t.n_in == M.e, in_ff = t.n_in == M.ff;
    bool umma = c->use_umma && ((t.type == T_Q4_K && row >= 64) || (t.type == T_IQ3_XXS && row >= 16)) && (in_e || in_ff) &&
                t.n_in % 256 == 0 && t.n_out % 128 == 0;
    if (umma) {
        if ((rc = ensure_ws(c, (int)((row + M.k) / (M.k + 1))))) return rc;
        umma = c->ws.maps_ok;
    }
    DNB_CUDA(cudaMemcpyAsync(dx, xs, row * t.n_in * sizeof(float), cudaMemcpyHostToDevice, c->stream));
    DNB_CUDA(cudaMemcpyAsync(dsd, sd.data(), nseg * sizeof(SegDesc), cudaMemcpyHostToDevice, c->stream));
    if (umma) {
        Workspace& w = c->ws;
        DNB_CUDA(cudaMemcpyAsync(dnseg, &nseg, sizeof(int32_t), cudaMemcpyHostToDevice, c->stream));
        uint16_t* hi = in_e ? w.xg_hi : w.act_hi;
        uint16_t* lo = in_e ? w.xg_lo : w.act_lo;
        if ((rc = launch_gather_split(c, c->stream, dx, t.n_in, nullptr, (int)row, t.n_in, hi, lo)) == DNB_OK)
            rc = launch_grouped_tc(c, c->stream, t.type, false, dsd, dnseg, nseg, t.n_in, t.n_out, in_e ? &w.maps_x : &w.maps_act,
                                   (int)row, nullptr, nullptr, dout);
    } else {
        rc = launch_seg_matmul(c, c->stream, t.type, false, dsd, nullptr, nseg, t.n_in, t.n_out, dx, t.n_in, nullptr, dout,
                               (int)m_max);
    }
    if (rc == DNB_OK) {
        cudaError_t e = cudaMemcpyAsync(outs, dout, row * t.n_out * sizeof(float), cudaMemcpyDeviceToHost, c->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
        if (e != cudaSuccess) {
            set_error("grouped_gemm: %s", cudaGetErrorString(e));
            rc = DNB_ERR_CUDA;
        } else {
            rc = finish_checked(c, "grouped_gemm");
        }
    } else {
        cudaStreamSynchronize(c->stream);
    }
    return rc;
}

// The routing tables of a chunk as the device builds them (moe_expert.rs:8309-8390
// build_grouped_batch; exp_pf.rs:23-31 rows[]), returned to the host for inspection.
int dnb_build_grouped_batch(dnb_ctx* c, int layer, const int32_t* sels, int nt, uint32_t* segs_out, int32_t* nseg_out,
                            int32_t* row_token_out, int32_t* pos_out) {
    if (!c || !sels || !segs_out || !nseg_out || nt < 1) return DNB_ERR_ARG;
    if (!layer_ready(c, layer, false)) {
        set_error("build_grouped_batch: layer %d has no expert tensors", layer);
        return DNB_DECLINED;
    }
    const Model& M = c->model;
    const Layer& L = M.layers[layer];
    for (size_t i = 0; i < (size_t)nt * M.k; ++i)
        if (sels[i] < 0 || sels[i] >= M.ne) {
            set_error("build_grouped_batch: expert %d out of range", sels[i]);
            return DNB_ERR_ARG;
        }
    DNB_CUDA(cudaSetDevice(c->device));
    int rc = ensure_ws(c, nt);
    if (rc) return rc;
    Workspace& w = c->ws;
    const size_t rows = (size_t)nt * M.k;
    memcpy(w.pinned_sels, sels, rows * 4);
    DNB_CUDA(cudaMemcpyAsync(w.sels, w.pinned_sels, rows * 4, cudaMemcpyHostToDevice, c->stream));
    if ((rc = launch_route_tables(c, c->stream, w.sels, nt, M.k, M.ne, L, w, false))) return rc;
    int32_t nseg = 0;
    DNB_CUDA(cudaMemcpyAsync(&nseg, w.nseg, 4, cudaMemcpyDeviceToHost, c->stream));
    DNB_CUDA(cudaStreamSynchronize(c->stream));
    if (nseg < 0 || nseg > M.ne) return DNB_ERR_STATE;
    std::vector<SegDesc> sd(nseg);
    DNB_CUDA(cudaMemcpy(sd.data(), w.seg_gu, nseg * sizeof(SegDesc), cudaMemcpyDeviceToHost));
    for (int i = 0; i < nseg; ++i) {
        segs_out[4 * i] = (uint32_t)((sd[i].wa - L.m[0].dev) / L.m[0].expert_bytes);
        segs_out[4 * i + 1] = sd[i].m;
        segs_out[4 * i + 2] = sd[i].row0;
        segs_out[4 * i + 3] = sd[i].row0;
    }
    *nseg_out = nseg;
    if (row_token_out) DNB_CUDA(cudaMemcpy(row_token_out, w.row_token, rows * 4, cudaMemcpyDeviceToHost));
    if (pos_out) DNB_CUDA(cudaMemcpy(pos_out, w.pos, rows * 4, cudaMemcpyDeviceToHost));
    return DNB_OK;
}

// ---- legacy three-launch decode form and the standalone router GEMV ---------------------

// Segment table of the legacy form (expert_batch.rs:143-170; checked like seg_extents,
// expert_batch.rs:233-260): seg[i] = (expert, m, x_off, out_off), offsets in floats.
// Token j of segment i reads x[x_off + j*n_in ..] and writes out[out_off + j*n_out ..].
static int seg_gemv_run(dnb_ctx* c, const ExpertTensor& t, const uint32_t* seg, int nseg, const float* x, size_t x_len,
                        float* out, size_t out_len, const char* what) {
    std::vector<SegDesc> sd(nseg);
    size_t out_rows = 0;
    uint32_t m_max = 0;
    for (int i = 0; i < nseg; ++i) {
        const uint32_t ex = seg[4 * i], m = seg[4 * i + 1], xo = seg[4 * i + 2], oo = seg[4 * i + 3];
        if (m == 0 || ex >= (uint32_t)t.n_expert || xo % (uint32_t)t.n_in || oo % (uint32_t)t.n_out ||
            (size_t)xo + (size_t)m * t.n_in > x_len || (size_t)oo + (size_t)m * t.n_out > out_len) {
            set_error("%s: segment %d (expert %u, m %u, x_off %u, out_off %u) breaks the table contract", what, i, ex, m, xo, oo);
            return DNB_ERR_ARG;
        }
        sd[i] = SegDesc{t.dev + (size_t)ex * t.expert_bytes, nullptr, m, oo / (uint32_t)t.n_out};
        out_rows = std::max(out_rows, (size_t)(oo / t.n_out + m));
        m_max = std::max(m_max, m);
    }
    std::vector<int32_t> row_token(out_rows, 0);  // output row -> input row
    for (int i = 0; i < nseg; ++i)
        for (uint32_t j = 0; j < sd[i].m; ++j) row_token[sd[i].row0 + j] = (int32_t)(seg[4 * i + 2] / (uint32_t)t.n_in + j);
    int rc;
    if ((rc = grow(c->gg_x, x_len * sizeof(float)))) return rc;
    if ((rc = grow(c->gg_out, out_rows * t.n_out * sizeof(float)))) return rc;
    if ((rc = grow(c->gg_seg, (size_t)nseg * sizeof(SegDesc) + out_rows * sizeof(int32_t)))) return rc;
    float* dx = (float*)c->gg_x.p;
    float* dout = (float*)c->gg_out.p;
    SegDesc* dsd = (SegDesc*)c->gg_seg.p;
    int32_t* drt = (int32_t*)((uint8_t*)c->gg_seg.p + (size_t)nseg * sizeof(SegDesc));
    DNB_CUDA(cudaMemcpyAsync(dx, x, x_len * sizeof(float), cudaMemcpyHostToDevice, c->stream));
    DNB_CUDA(cudaMemcpyAsync(dsd, sd.data(), nseg * sizeof(SegDesc), cudaMemcpyHostToDevice, c->stream));
    DNB_CUDA(cudaMemcpyAsync(drt, row_token.data(), out_rows * sizeof(int32_t), cudaMemcpyHostToDevice, c->stream));
    rc = DNB_DECLINED;
    if (m_max == 1 && c->decode_fast)
        rc = launch_seg_gemv_m1(c, c->stream, t.type, false, false, dsd, nullptr, nseg, t.n_in, t.n_out, dx, t.n_in, drt, dout,
                                nullptr, "seg_gemv");
    if (rc == DNB_DECLINED)
        rc = launch_seg_matmul(c, c->stream, t.type, false, dsd, nullptr, nseg, t.n_in, t.n_out, dx, t.n_in, drt, dout,
                               (int)m_max);
    if (rc) {
        cudaStreamSynchronize(c->stream);
        return rc;
    }
    // rows no segment names keep whatever the caller had there: copy back segment by segment
    for (int i = 0; i < nseg; ++i)
        DNB_CUDA(cudaMemcpyAsync(out + seg[4 * i + 3], dout + (size_t)sd[i].row0 * t.n_out, (size_t)sd[i].m * t.n_out * sizeof(float),
                                 cudaMemcpyDeviceToHost, c->stream));
    DNB_CUDA(cudaStreamSynchronize(c->stream));
    return finish_checked(c, what);
}

static const ExpertTensor* seg_tensor(dnb_ctx* c, int layer, int matrix, const char* what) {
    if (layer < 0 || layer >= c->model.n_layer || matrix < 0 || matrix > 5 || !c->model.layers[layer].m[matrix].dev) {
        set_error("%s: layer %d matrix %d is not registered", what, layer, matrix);
        return nullptr;
    }
    return &c->model.layers[layer].m[matrix];
}

int dnb_seg_gemv(dnb_ctx* c, int layer, int matrix, const uint32_t* seg, int nseg, const float* x, size_t x_len, float* out,
                 size_t out_len) {
    if (!c || !seg || !x || !out || nseg < 1) return DNB_ERR_ARG;
    const ExpertTensor* t = seg_tensor(c, layer, matrix, "seg_gemv");
    if (!t) return DNB_DECLINED;
    DNB_CUDA(cudaSetDevice(c->device));
    return seg_gemv_run(c, *t, seg, nseg, x, x_len, out, out_len, "seg_gemv");
}

int dnb_seg_gemv_pair(dnb_ctx* c, int layer, const uint32_t* seg, int nseg, const float* x, size_t x_len, float* out_g,
                      float* out_u, size_t out_len) {
    if (!c || !seg || !x || !out_g || !out_u || nseg < 1) return DNB_ERR_ARG;
    const ExpertTensor* tg = seg_tensor(c, layer, DNB_MAT_GATE, "seg_gemv_pair");
    const ExpertTensor* tu = seg_tensor(c, layer, DNB_MAT_UP, "seg_gemv_pair");
    if (!tg || !tu) return DNB_DECLINED;
    if (tg->row_bytes != tu->row_bytes || tg->n_out != tu->n_out) {  // cuda.rs:7653-7656: rb_g != rb_u -> not run
        set_error("seg_gemv_pair: gate and up rows differ in size");
        return DNB_DECLINED;
    }
    DNB_CUDA(cudaSetDevice(c->device));
    int rc = seg_gemv_run(c, *tg, seg, nseg, x, x_len, out_g, out_len, "seg_gemv_pair");
    if (rc) return rc;
    return seg_gemv_run(c, *tu, seg, nseg, x, x_len, out_u, out_len, "seg_gemv_pair");
}

int dnb_router_gemv(dnb_ctx* c, int layer, const float* x, int nt, float* logits) {
    if (!c || !x || !logits || nt < 1) return DNB_ERR_ARG;
    const Model& M = c->model;
    if (layer < 0 || layer >= M.n_layer || !M.layers[layer].router_w) {
        set_error("router_gemv: layer %d has no router", layer);
        return DNB_DECLINED;
    }
    DNB_CUDA(cudaSetDevice(c->device));
    int rc = ensure_ws(c, nt);
    if (rc) return rc;
    Workspace& w = c->ws;
    const Layer& L = M.layers[layer];
    const size_t bytes = (size_t)nt * M.e * sizeof(float), lbytes = (size_t)nt * M.ne * sizeof(float);
    if ((rc = grow(c->gemv_host, lbytes, true))) return rc;
    memcpy(w.pinned_in, x, bytes);
    DNB_CUDA(cudaMemcpyAsync(w.hin, w.pinned_in, bytes, cudaMemcpyHostToDevice, c->stream));
    if ((rc = router_logits(c, c->stream, w.hin, nt, L, w.logits))) return rc;
    DNB_CUDA(cudaMemcpyAsync(c->gemv_host.p, w.logits, lbytes, cudaMemcpyDeviceToHost, c->stream));
    DNB_CUDA(cudaStreamSynchronize(c->stream));
    if ((rc = finish_checked(c, "router_gemv"))) return rc;
    memcpy(logits, c->gemv_host.p, lbytes);
    return DNB_OK;
}

// ---- expert-parallel building blocks ---------------------------------------------------

int dnb_moe_set_expert_shard(dnb_ctx* c, int first_expert, int n_local) {
    if (!c) return DNB_ERR_ARG;
    Model& M = c->model;
    if (M.n_layer < 1 || first_expert < 0 || n_local < 1 || first_expert + n_local > M.ne) {
        set_error("expert shard [%d, %d) does not fit the %d experts of the model", first_expert, first_expert + n_local, M.ne);
        return DNB_ERR_ARG;
    }
    for (auto& L : M.layers)
        if (L.m[0].dev || L.m[1].dev || L.m[2].dev) {
            set_error("expert shard must be set before the expert tensors are registered");
            return DNB_ERR_STATE;
        }
    M.shard_first = first_expert;
    M.shard_count = n_local;
    return DNB_OK;
}

int dnb_moe_route_dev(dnb_ctx* c, int layer, const float* h_dev, int nt, float* x_out_dev, int32_t* sels_dev,
                      float* wts_dev) {
    if (!c || !h_dev || !x_out_dev || !sels_dev || !wts_dev || nt < 1) return DNB_ERR_ARG;
    const Model& M = c->model;
    if (layer < 0 || layer >= M.n_layer || !M.layers[layer].router_w) {
        set_error("moe_route: layer %d has no router", layer);
        return DNB_DECLINED;
    }
    DNB_CUDA(cudaSetDevice(c->device));
    int rc = ensure_ws(c, nt);
    if (rc) return rc;
    const Layer& L = M.layers[layer];
    if (L.norm_w) {
        if ((rc = launch_rmsnorm(c, c->stream, h_dev, L.norm_w, M.eps, nt, M.e, x_out_dev))) return rc;
    } else if (x_out_dev != h_dev) {
        DNB_CUDA(cudaMemcpyAsync(x_out_dev, h_dev, (size_t)nt * M.e * 4, cudaMemcpyDeviceToDevice, c->stream));
    }
    return router_topk_dev(c, c->stream, x_out_dev, nt, L, sels_dev, wts_dev, nullptr);
}

int dnb_expert_rows_dev(dnb_ctx* c, int layer, const float* x_rows_dev, const int32_t* local_ids_dev, int rows,
                        int use_shared, float* h_rows_dev) {
    if (!c || !x_rows_dev || !h_rows_dev || rows < 1 || (!use_shared && !local_ids_dev)) return DNB_ERR_ARG;
    const Model& M = c->model;
    if (layer < 0 || layer >= M.n_layer) return DNB_ERR_ARG;
    const Layer& L = M.layers[layer];
    if (use_shared ? !L.has_shared() : !(L.m[0].dev && L.m[1].dev && L.m[2].dev)) {
        set_error("expert_rows: layer %d lacks the %s expert tensors", layer, use_shared ? "shared" : "routed");
        return DNB_DECLINED;
    }
    DNB_CUDA(cudaSetDevice(c->device));
    int rc = ensure_ws(c, rows);
    if (rc) return rc;
    Workspace& w = c->ws;
    cudaStream_t st = c->stream;
    const int ty_routed = use_shared ? -1 : tc_type(L, 0, 3);
    const int ty_shared = (L.has_shared() && L.m[3].n_out == M.ff) ? tc_type(L, 3, 6) : -1;
    const bool q4k_routed = ty_routed >= 0, q4k_shared = ty_shared >= 0;
    const bool umma = c->use_umma && w.maps_ok && rows >= 16 && M.e % 256 == 0 && M.ff % 256 == 0;
    if (!use_shared) {
        // every row is one (token, slot): a "chunk" of `rows` tokens with one selected expert each and weight 1
        if (umma && q4k_routed) return experts_dev_umma(c, layer, x_rows_dev, rows, local_ids_dev, nullptr, h_rows_dev, 1, M.shard_count, 0);
        return experts_dev(c, layer, x_rows_dev, rows, local_ids_dev, nullptr, h_rows_dev, 1, M.shard_count, 0);
    }
    // the shared expert on all rows: one segment, rows in place
    if ((rc = launch_prep(c, st, x_rows_dev, nullptr, M.eps, rows, M.e, nullptr, w.seg_sh_gu, w.seg_sh_dn, L.m[3].dev,
                          L.m[4].dev, L.m[5].dev)))
        return rc;
    const int sff = L.m[3].n_out;
    if (umma && q4k_shared) {
        if ((rc = launch_gather_split(c, st, x_rows_dev, M.e, nullptr, rows, M.e, w.xg_hi, w.xg_lo))) return rc;
        if ((rc = launch_grouped_tc(c, st, ty_shared, true, w.seg_sh_gu, w.one, 1, M.e, M.ff, &w.maps_x, rows, w.act_hi, w.act_lo, nullptr)))
            return rc;
        return launch_grouped_tc(c, st, ty_shared, false, w.seg_sh_dn, w.one, 1, M.ff, M.e, &w.maps_act, rows, nullptr, nullptr, h_rows_dev);
    }
    if ((rc = launch_seg_matmul(c, st, L.m[3].type, true, w.seg_sh_gu, nullptr, 1, M.e, sff, x_rows_dev, M.e, nullptr, w.sact, rows)))
        return rc;
    return launch_seg_matmul(c, st, L.m[5].type, false, w.seg_sh_dn, nullptr, 1, sff, M.e, w.sact, sff, nullptr, h_rows_dev, rows);
}

int dnb_moe_combine_dev(dnb_ctx* c, int layer, const float* h_slots_dev, const float* wts_dev, const float* shared_dev,
                        const float* x_dev, int nt, float* out_dev) {
    if (!c || !h_slots_dev || !wts_dev || !out_dev || nt < 1) return DNB_ERR_ARG;
    const Model& M = c->model;
    if (layer < 0 || layer >= M.n_layer) return DNB_ERR_ARG;
    const Layer& L = M.layers[layer];
    DNB_CUDA(cudaSetDevice(c->device));
    int rc = ensure_ws(c, nt);
    if (rc) return rc;
    const float* coef = nullptr;
    if (shared_dev && L.shared_gate_row) {
        if (!x_dev) return DNB_ERR_ARG;
        if ((rc = launch_shared_coef(c, c->stream, x_dev, L.shared_gate_row, nt, M.e, c->ws.shcoef))) return rc;
        coef = c->ws.shcoef;
    }
    return launch_combine(c, c->stream, h_slots_dev, nullptr, wts_dev, nt, M.k, M.e, shared_dev, coef, out_dev);
}

int dnb_moe_stack_dev(dnb_ctx* c, float* h_dev, int nt) {
    if (!c || !h_dev || nt < 1) return DNB_ERR_ARG;
    const Model& M = c->model;
    for (int l = 0; l < M.n_layer; ++l)
        if (!layer_ready(c, l, true)) {
            set_error("moe_stack: layer %d is not fully registered", l);
            return DNB_DECLINED;
        }
    DNB_CUDA(cudaSetDevice(c->device));
    int rc = ensure_ws(c, nt);
    if (rc) return rc;
    return run_graphed(c, GraphKey{4, 0, nt, h_dev, nullptr}, [&]() -> int {
        for (int l = 0; l < M.n_layer; ++l) {
            if (nt == 1 && c->decode_fast) {
                const int rd = block_dev_decode(c, l, h_dev, h_dev, h_dev);
                if (rd == DNB_OK) continue;
                if (rd != DNB_DECLINED) return rd;
            }
            if (nt > 1 && nt <= kDecodeBatchMax && c->decode_fast && !umma_eligible(c, M.layers[l], nt)) {
                const int rd = block_dev_decode_batch(c, l, h_dev, nt, h_dev, h_dev);
                if (rd == DNB_OK) continue;
                if (rd != DNB_DECLINED) return rd;
            }
            int r = block_dev(c, l, h_dev, nt, c->ws.out);
            if (r) return r;
            if ((r = launch_add_inplace(c, c->stream, h_dev, c->ws.out, (size_t)nt * M.e))) return r;
        }
        return DNB_OK;
    });
}

int dnb_moe_stack(dnb_ctx* c, const float* h, int nt, float* out) {
    if (!c || !h || !out || nt < 1) return DNB_ERR_ARG;
    DNB_CUDA(cudaSetDevice(c->device));
    if (c->model.n_layer < 1) {
        set_error("moe_stack: no model configured");
        return DNB_DECLINED;
    }
    int rc = ensure_ws(c, nt);
    if (rc) return rc;
    Workspace& w = c->ws;
    const size_t bytes = (size_t)nt * c->model.e * sizeof(float);
    memcpy(w.pinned_in, h, bytes);
    DNB_CUDA(cudaMemcpyAsync(w.hin, w.pinned_in, bytes, cudaMemcpyHostToDevice, c->stream));
    if ((rc = dnb_moe_stack_dev(c, w.hin, nt))) return rc;
    DNB_CUDA(cudaMemcpyAsync(w.pinned_out, w.hin, bytes, cudaMemcpyDeviceToHost, c->stream));
    DNB_CUDA(cudaStreamSynchronize(c->stream));
    if ((rc = finish_checked(c, "moe_stack"))) return rc;
    memcpy(out, w.pinned_out, bytes);
    return DNB_OK;
}

}  // extern "C"
