// Shared declarations of the CUDA library: context, layer tables, error
// plumbing and the launchers each translation unit exports to api.cu.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stddef.h>
#include <functional>
#include <map>
#include <string>
#include <vector>

#include "dnb200.h"

namespace dnb {

// ---- block formats ---------------------------------------------------------
constexpr int T_F32 = 0, T_Q5_1 = 7, T_Q8_0 = 8, T_Q4_K = 12, T_Q5_K = 13, T_Q6_K = 14, T_IQ3_XXS = 18;
// The block types of real checkpoints' remaining tensors (exp_iq.rs:390-400, cuda.rs:7364-7373):
// served by the tiled kernels and the sequential checker, not by the decode fast kernels.
constexpr int T_Q4_0 = 2, T_IQ4_NL = 20, T_IQ3_S = 21, T_IQ2_S = 22, T_IQ4_XS = 23, T_Q2_0 = 42;

__host__ __device__ constexpr int type_size(int t) {
    return t == T_Q4_K ? 144 : t == T_IQ3_XXS ? 98 : t == T_Q6_K ? 210 : t == T_Q8_0 ? 34 : t == T_Q5_K ? 176
         : t == T_Q5_1 ? 24 : t == T_F32 ? 4 : t == T_Q4_0 ? 18 : t == T_IQ4_NL ? 18 : t == T_IQ3_S ? 110
         : t == T_IQ2_S ? 82 : t == T_IQ4_XS ? 136 : t == T_Q2_0 ? 18 : 0;
}
__host__ __device__ constexpr int block_elems(int t) {
    return (t == T_Q4_K || t == T_IQ3_XXS || t == T_Q6_K || t == T_Q5_K || t == T_IQ3_S || t == T_IQ2_S || t == T_IQ4_XS) ? 256
         : (t == T_Q8_0 || t == T_Q5_1 || t == T_Q4_0 || t == T_IQ4_NL) ? 32 : t == T_Q2_0 ? 64 : t == T_F32 ? 1 : 0;
}
inline bool type_supported(int t) { return type_size(t) != 0 && t != T_F32; }
// Bytes of one row of n_in elements, or 0 when n_in is not a whole number of blocks.
inline size_t row_bytes(int t, long n_in) {
    const int be = block_elems(t);
    if (be == 0 || n_in <= 0 || n_in % be) return 0;
    return (size_t)(n_in / be) * type_size(t);
}

// ---- resident tensors --------------------------------------------------------
struct ExpertTensor {          // one of gate / up / down of a layer, expert-major
    int type = -1;
    int n_in = 0, n_out = 0, n_expert = 0;
    size_t row_bytes = 0, expert_bytes = 0;
    uint8_t* dev = nullptr;
    bool owned = false;
};

struct alignas(64) RouterMaps {  // three TMA tensor maps (bf16 hi / mid / lo parts of one fp32 matrix), opaque here
    unsigned char bytes[3 * 128];
};

struct Layer {
    ExpertTensor m[6];         // 0 gate 1 up 2 down 3 shared-gate 4 shared-up 5 shared-down
    float* router_w = nullptr;         // [ne][e]
    uint16_t* router_w3 = nullptr;     // [3][ne][e]: router_w as three bf16 parts (tensor-core router of prefill chunks)
    RouterMaps rmaps;
    bool router_tc = false;            // router_w3 and rmaps are valid
    float* router_bias = nullptr;      // [ne] or null
    float* norm_w = nullptr;           // [e] or null
    float* shared_gate_row = nullptr;  // [e] or null
    bool has_shared() const { return m[3].dev && m[4].dev && m[5].dev; }
};

struct Matrix {                // single resident matrix keyed by uid (GEMV path)
    int type; int k, n; size_t row_bytes; uint8_t* dev;
};

// One unit of grouped work: `m` token rows against one expert's matrix (or the
// gate and up matrices together).  Built on the device by the routing kernel.
struct SegDesc {
    const uint8_t* wa;
    const uint8_t* wb;
    uint32_t m;
    uint32_t row0;             // first row of the segment in the packed row space
};

struct Scratch {               // grow-only device scratch of a context
    void* p = nullptr; size_t cap = 0;
};

struct Model {
    int n_layer = 0, e = 0, ff = 0, sff = 0, ne = 0, k = 0;
    int shard_first = 0, shard_count = 0;  // routed experts resident on this GPU (expert parallel); count == ne: all
    float eps = 1e-6f;
    int norm_topk = 1;
    std::vector<Layer> layers;
};

struct alignas(64) UmmaMaps {  // eight TMA tensor maps (4 box heights x hi/lo), opaque here
    unsigned char bytes[8 * 128];
};

struct Workspace {             // device buffers of the MoE pipeline, sized for nt_cap tokens
    int nt_cap = 0;
    float *xn = nullptr, *logits = nullptr, *wts = nullptr, *act = nullptr, *hrow = nullptr, *sact = nullptr,
          *sh = nullptr, *hin = nullptr, *out = nullptr, *shcoef = nullptr,
          *act_perm = nullptr,  // [kActRep][(k + 1) * ff]: the decode gate/up result in the down format's slot order
          *xn_perm = nullptr;   // [kActRep][e]: the decode router's normalised row in the gate format's slot order
    uint16_t* act_h = nullptr;  // bf16 triples of the fused decode kernel's activations (decode_fused.cu)
    int32_t *sels = nullptr, *row_token = nullptr, *pos = nullptr, *nseg = nullptr, *counts = nullptr, *one = nullptr;
    SegDesc *seg_gu = nullptr, *seg_dn = nullptr, *seg_sh_gu = nullptr, *seg_sh_dn = nullptr;
    uint16_t *xg_hi = nullptr, *xg_lo = nullptr, *act_hi = nullptr, *act_lo = nullptr;  // bf16 hi/lo packed rows
    UmmaMaps maps_x, maps_act;
    bool maps_ok = false;
    // integer-weight Q4_K kernel (grouped_q4k_int.cu): fp16 hi / lo rows with the sub-block sums appended, row scales
    uint16_t *xq_hi = nullptr, *xq_lo = nullptr, *aq_hi = nullptr, *aq_lo = nullptr;
    float *xq_scale = nullptr, *aq_scale = nullptr;
    UmmaMaps maps_xq, maps_aq;
    bool q4k_int_ok = false;
    uint16_t* x3 = nullptr;    // [3][nt_cap + 128][e]: the chunk's rows as three bf16 parts (router_tc.cu)
    size_t x3_part = 0;        // elements between the parts
    float* rpart = nullptr;    // [K splits][nt][ne]: partial router sums
    RouterMaps xmaps;
    bool router_tc = false;    // x3, rpart and xmaps are valid
    float* pinned_in = nullptr; float* pinned_out = nullptr; size_t pinned_cap = 0;
    int32_t* pinned_sels = nullptr; float* pinned_wts = nullptr;
};

}  // namespace dnb

namespace dnb {
// Optional per-kernel timing: when enabled every launcher brackets its kernel
// with a pair of events on the launching stream.
struct ProfRec { const char* name; cudaEvent_t a, b; };
struct Profiler {
    bool on = false;
    std::vector<ProfRec> recs;      // recorded pairs, in launch order
    std::vector<cudaEvent_t> pool;  // events ready for reuse
};
}  // namespace dnb

namespace dnb {
// Captured launch sequences, replayed with one cudaGraphLaunch.  Keyed by what the
// sequence depends on: entry point, layer, token count and the device pointers.
struct GraphKey {
    int kind, layer, nt;
    const void *a, *b;
    bool operator<(const GraphKey& o) const {
        if (kind != o.kind) return kind < o.kind;
        if (layer != o.layer) return layer < o.layer;
        if (nt != o.nt) return nt < o.nt;
        if (a != o.a) return a < o.a;
        return b < o.b;
    }
};
struct GraphEntry { cudaGraphExec_t exec = nullptr; uint64_t kernels = 0; };
}  // namespace dnb

struct dnb_ctx {
    int device = 0;
    dnb::Profiler prof;
    bool use_graphs = true;
    std::map<dnb::GraphKey, dnb::GraphEntry> graphs;   // null exec = seen once, not captured yet
    cudaStream_t stream = nullptr;      // main stream (owned unless set from outside)
    cudaStream_t side = nullptr;        // shared-expert stream
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr, ev_t0 = nullptr, ev_t1 = nullptr;
    cudaStream_t saved_stream = nullptr;  // the context's own stream while an external one is set
    bool own_stream = true;
    dnb::Scratch flush;
    std::map<uint64_t, dnb::Matrix> matrices;
    dnb::Model model;
    dnb::Workspace ws;
    dnb::Scratch gemv_x, gemv_out, gemv_host;   // gemv_host: pinned host staging of dnb_gemv's result
    dnb::Scratch gg_x, gg_out, gg_seg;           // grow-only buffers of dnb_grouped_gemm
    int sm_count = 148;
    int* status = nullptr;              // status word the kernels write when a bounded wait gave up: pinned host memory, device address
    int* status_host = nullptr;         // the same word as the host reads it (valid after a stream synchronisation)
    int barrier_polls = 400000;         // polls of the fused decode kernel's grid barrier before it gives up (~0.2 s)
    int flag_polls = 1 << 21;           // polls of an expert-parallel flag wait before it gives up (~0.25 s)
    unsigned int barrier_bias = 0;      // test hook: added to the barrier's target so that it cannot be reached
    unsigned int* ticket = nullptr;     // "last CTA" counter of the fused decode router (self-resetting)
    unsigned long long* gbar = nullptr; // grid barrier of the fused decode kernel: arrivals of all launches so far
    uint64_t launches = 0;              // kernels launched by this context (bench accounting)
    int gemv_impl = 0;                  // 0 = fast (default), 1 = sequential bit-exact
    bool q4k_int = false;               // Q4_K chunks on the integer-weight tcgen05 kernel (grouped_q4k_int.cu): more exact, measured slower
    bool router_tc = true;              // router logits of large chunks on the tensor cores (router_tc.cu)
    bool decode_fast = true;            // one-token calls take the bulk-copy GEMV + fused router path
    bool use_pdl = true;                // programmatic dependent launch between the decode kernels
    bool gemv_mma = true;               // one-token IQ3_XXS kernels on mma.sync (gemv_mma.cu, decode_fused.cu) where the shape fits
    bool decode_fused = true;           // gate/up + down of a one-token IQ3_XXS block as one kernel (decode_fused.cu)
    bool decode_routed = true;          // ... with the router folded into the same kernel (one launch per block)
    int exact_min_nt = 16;              // IQ3_XXS layers: tokens from which a batch takes the exact-weight tcgen05 kernel
    bool use_umma = true;               // prefill chunks of Q4_K layers take the tcgen05 grouped GEMM
    void* ep = nullptr;                 // dnb::EpState of the peer-memory expert-parallel path (ep_p2p.cu)
    void* hc = nullptr;                 // dnb::HcState: hyper-connection mix weights and scratch (hc_mix.cu)
    void* epd = nullptr;                // dnb::EpdState of the expert-parallel decode path (ep_decode.cu)
};

namespace dnb {

void set_error(const char* fmt, ...);
void ep_release(dnb_ctx* c);  // frees the peer-memory expert-parallel state, if any (ep_p2p.cu)
void epd_release(dnb_ctx* c); // the same for the decode exchange (ep_decode.cu)
void hc_release(dnb_ctx* c);  // hyper-connection weights and scratch (hc_mix.cu)
int ensure_workspace(dnb_ctx* c, int nt);  // device buffers of the MoE pipeline for nt tokens (api.cu)
// Run a launch sequence directly the first time `key` is seen, capture it into a CUDA graph the second time,
// replay it afterwards (api.cu).
int graphed(dnb_ctx* c, const GraphKey& key, const std::function<int()>& enqueue);

struct ProfScope {
    dnb_ctx* c; cudaStream_t st; cudaEvent_t b = nullptr;
    ProfScope(dnb_ctx* c_, cudaStream_t st_, const char* name) : c(c_), st(st_) {
        if (!c->prof.on || c->prof.recs.size() >= 65536) return;
        cudaEvent_t ev[2];
        for (auto& e : ev) {
            if (!c->prof.pool.empty()) { e = c->prof.pool.back(); c->prof.pool.pop_back(); }
            else if (cudaEventCreate(&e) != cudaSuccess) return;
        }
        cudaEventRecord(ev[0], st);
        b = ev[1];
        c->prof.recs.push_back(ProfRec{name, ev[0], ev[1]});
    }
    ~ProfScope() { if (b) cudaEventRecord(b, st); }
};
#define DNB_CUDA(call)                                                                         \
    do {                                                                                       \
        cudaError_t e_ = (call);                                                               \
        if (e_ != cudaSuccess) {                                                               \
            dnb::set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, __LINE__); \
            return DNB_ERR_CUDA;                                                               \
        }                                                                                      \
    } while (0)

// Programmatic dependent launch: with pdl = true the kernel may start while the
// previous kernel on the stream is still running; it must execute pdl_wait()
// before it reads anything that kernel wrote.  Everything before pdl_wait() (weight
// prefetch of data no kernel writes) then overlaps the predecessor's tail.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl,
                            Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// Record that a bounded wait gave up.  The status word lives in pinned host memory the device can
// address, so the host reads it after its next stream synchronisation without a copy; a plain store
// is enough (several reporters may race: any of their codes will do).
__device__ __forceinline__ void status_set(int* status, int code) {
    if (status) {
        *reinterpret_cast<volatile int*>(status) = code;
        __threadfence_system();
    }
}
#endif

// ---- launchers (defined in the .cu files) -----------------------------------
// Segmented dequant matmul: for every segment s < *nseg_dev (or nseg_host when
// nseg_dev is null), rows of seg[s].wa (and wb when fused) times the segment's
// token rows.  Token i of a segment reads x + row_token[row0 + i] * ldx (or row
// row0 + i when row_token is null).  fused: out[(row0+i)*n_out + r] =
// silu(wa_r . x) * (wb_r . x); otherwise out[(row0+i)*n_out + r] = wa_r . x.
// With seg == null the single segment *single (a host struct) is passed by value.
int launch_seg_matmul(dnb_ctx* c, cudaStream_t st, int type, bool fused, const SegDesc* seg, const int32_t* nseg_dev,
                      int nseg_max, int n_in, int n_out, const float* x, int ldx, const int32_t* row_token,
                      float* out, int m_max, const SegDesc* single = nullptr);
// Bit-exact-order GEMV (one thread per row, ascending i, no FMA contraction).
int launch_gemv_seq(dnb_ctx* c, cudaStream_t st, int type, const uint8_t* w, const float* x, float* out, int n_in,
                    int n_out);

int launch_rmsnorm(dnb_ctx* c, cudaStream_t st, const float* h, const float* w, float eps, int nt, int e, float* out);
// RMSNorm (skipped when w is null) that also publishes the shared expert's two
// one-segment descriptors for this call.
// x3 (optional, needs w): the normalised rows also as three bf16 parts, x3_part elements apart (the tensor-core router's operand).
int launch_prep(dnb_ctx* c, cudaStream_t st, const float* h, const float* w, float eps, int nt, int e, float* out,
                SegDesc* sh_gu, SegDesc* sh_dn, const uint8_t* sg, const uint8_t* su, const uint8_t* sdn,
                uint16_t* x3 = nullptr, size_t x3_part = 0);
int launch_add_inplace(dnb_ctx* c, cudaStream_t st, float* h, const float* d, size_t n);
int launch_stage_in(dnb_ctx* c, cudaStream_t st, const float* host_pinned, float* dst, size_t n);  // DNB_DECLINED: use a copy
int launch_stall(dnb_ctx* c, cudaStream_t st, float ms);
int launch_fill_u32(dnb_ctx* c, cudaStream_t st, uint32_t* dst, uint32_t v, size_t n);
int launch_router_logits(dnb_ctx* c, cudaStream_t st, const float* x, int nt, int e, const float* w_r,
                         const float* bias, int ne, float* logits);
int launch_router_decode(dnb_ctx* c, cudaStream_t st, const float* h, const Model& M, const Layer& L, Workspace& w,
                         bool fold_shared, unsigned int* ticket);
// Decode down projection of all segments with the weighted sum fused in:
// out[r] = (residual ? residual[r] : 0) + sum_s wts[s] * (W_s act_s)[r] (+ coef * shared).
// DNB_DECLINED = shape not covered.
// act_perm (optional): kActRep copies of the nseg activation vectors already in the
// slot order of `type` (see PermOut); each CTA then takes one copy with a single bulk copy
// instead of staging `act` with its threads.
int launch_down_combine(dnb_ctx* c, cudaStream_t st, int type, const SegDesc* seg, int nseg, int k, int n_in, int n_out,
                        const float* act, const float* wts, const float* shcoef, bool has_shared,
                        const float* residual, float* out, const float* act_perm = nullptr, int ntok = 1);
// Hand-over of the decode gate/up result to the down kernel: besides the plain rows, the
// values are written kActRep times in the slot order the consumer's format stages its
// activations in.  Every CTA of the consumer needs all of them; with one copy they all
// hit the same few L2 lines at once, with replicas CTA b reads copy b % kActRep.
constexpr int kActRep = 16;
// Token counts up to this take the decode kernels (one-row segments); measured on the 48-layer
// stack they beat the tiled kernels at 8 tokens (6.6 vs 7.2 ms per step) and lose at 32 (20.6 vs 18.6).
constexpr int kDecodeBatchMax = 16;
struct PermOut {
    float* base = nullptr;  // [kActRep][nseg * n_out]
    int type = 0;           // format whose slot order to write
    // The same hand-over on the input side: kActRep copies of the (shared) activation row
    // already in this launch's slot order, written by the router kernel; a CTA takes one
    // with a bulk copy instead of staging x with its threads.
    const float* x_perm = nullptr;  // [kActRep][n_in]
};
// Decode GEMV staged by the bulk-copy engine (gemv_bulk.cu); DNB_DECLINED = shape not covered.
int launch_seg_gemv_m1(dnb_ctx* c, cudaStream_t st, int type, bool fused, bool xshared, const SegDesc* seg,
                       const int32_t* nseg_dev, int nseg_max, int n_in, int n_out, const float* x, int ldx,
                       const int32_t* row_token, float* out, const SegDesc* single, const char* pname,
                       PermOut perm = PermOut());
int launch_decode_batch_tables(dnb_ctx* c, cudaStream_t st, const int32_t* sels, int nt, int k, const Layer& L,
                               Workspace& ws, bool fold_shared);
int launch_topk(dnb_ctx* c, cudaStream_t st, const float* logits, int nt, int ne, int k, int norm_topk, int32_t* sels,
                float* wts, float* rowsum, int nsplit = 1, const float* bias = nullptr);
// Builds, from sels[nt][k], the expert-major row space: counts, segment
// descriptors for gate/up and down, row_token[], pos[t][slot] and *nseg.
// fold_shared: the shared expert becomes one more segment (m = nt) whose packed rows
// follow the routed rows (row nt*k + t reads token t).
int launch_route_tables(dnb_ctx* c, cudaStream_t st, const int32_t* sels, int nt, int k, int ne, const Layer& L,
                        Workspace& ws, bool fold_shared = false);
// The opt-in dynamic shared memory limit is an attribute of a kernel PER DEVICE: what was
// granted is remembered per device, so a process that drives several GPUs sets it on each.
struct SmemGrant { size_t got[64] = {0}; };
template <class K>
inline cudaError_t grant_smem(SmemGrant& g, int device, K kern, size_t bytes) {
    if (device < 0 || device >= 64) return cudaErrorInvalidDevice;
    if (bytes <= g.got[device]) return cudaSuccess;
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e == cudaSuccess) g.got[device] = bytes;
    return e;
}

// One-token IQ3_XXS gate/up GEMV on mma.sync (gemv_mma.cu); DNB_DECLINED when the shape does not fit.
int launch_gate_up_mma(dnb_ctx* c, cudaStream_t st, const SegDesc* seg, int nseg, int n_in, int n_out, const float* x,
                       float* out, const char* pname, PermOut perm);

// One-token gate/up + down of an all-IQ3_XXS block in one kernel (decode_fused.cu).
bool decode_fused_fits(const dnb_ctx* c, int nseg, int e, int ff);
size_t decode_fused_act_halves(int nseg, int ff);
int launch_decode_fused(dnb_ctx* c, cudaStream_t st, const SegDesc* seg_gu, const SegDesc* seg_dn, int nseg, int k,
                        bool has_shared, int e, int ff, const float* x, const float* x_perm, float* act, void* act_h,
                        const float* wts, const float* shcoef, const float* residual, float* out, unsigned long long* gbar);

// The whole one-token block, router included, of an all-IQ3_XXS layer in one kernel (decode_fused.cu).
int launch_decode_block(dnb_ctx* c, cudaStream_t st, const Model& M, const Layer& L, Workspace& w, bool fold_shared,
                        const float* h, const float* residual, float* out, unsigned long long* gbar);

// Router logits of chunks of kRouterTcMin tokens or more on tcgen05 (router_tc.cu)
constexpr int kRouterSplitMax = 8;  // K splits of the tensor-core router at most (the top-k kernel adds that many partial sums)
constexpr int kRouterTcMin = 16;   // the token count from which the tensor-core expert kernels take a call, too: a token's bits then do not
                                  // depend on the size of its chunk or on how an expert-parallel group split it
int router_tc_prepare(dnb_ctx* c, Layer& L, int ne, int e);
int router_tc_workspace(dnb_ctx* c, Workspace& w, int cap, int ne, int e);
bool router_tc_eligible(const dnb_ctx* c, const Layer& L, int nt);
// reduce = false leaves the K splits' partial sums in the workspace (rpart, router_tc_split(e) of them) for launch_topk
// to add; with one split the logits are complete either way.
int router_tc_split(int e);
// x_is_split: the chunk's rows are already in the workspace as three bf16 parts (written by launch_prep).
int launch_router_logits_tc(dnb_ctx* c, cudaStream_t st, const float* x, int nt, int e, const Layer& L, int ne, float* logits,
                            bool reduce = true, bool x_is_split = false);
// The router logits of a call: the tensor-core kernel where it is eligible, else the fp32 kernel (api.cu).
int router_logits(dnb_ctx* c, cudaStream_t st, const float* x, int nt, const Layer& L, float* logits);
// Router logits + softmax / top-k / renorm of a call (w.logits and, on the tensor-core path, w.rpart are its scratch).
int router_topk_dev(dnb_ctx* c, cudaStream_t st, const float* x, int nt, const Layer& L, int32_t* sels, float* wts,
                    float* rowsum, bool x_is_split = false);
// One tensor map: [rows][cols] bf16 row-major, box = 64 columns x box_rows rows, 128-byte swizzle.  map: 128 bytes.
int tc_make_map(void* map, void* base, uint64_t rows, uint64_t cols, uint32_t box_rows);

// Q4_K grouped GEMM with integer fp16 weights and block scales after the tensor-core sum (grouped_q4k_int.cu)
constexpr int kQ4kIntXcols = 64;  // sub-block sum columns appended to an activation row
bool q4k_int_handles(int n_in, int n_out, bool fused);
int launch_rows_f16(dnb_ctx* c, cudaStream_t st, const float* x, int ldx, const int32_t* row_token, int rows, int K,
                    uint16_t* hi, uint16_t* lo, float* rowscale, const char* name);
int launch_grouped_q4k_int(dnb_ctx* c, cudaStream_t st, bool fused, const SegDesc* seg, const int32_t* nseg_dev, int nseg_max,
                           int n_in, int n_out, const UmmaMaps* maps, const float* rowscale, float* out_f32,
                           float* const* row_dst = nullptr);

// tcgen05 grouped GEMM of prefill (grouped_umma.cu)
int umma_make_maps(void* hi, void* lo, uint64_t rows, uint64_t cols, UmmaMaps* out);
int launch_gather_split(dnb_ctx* c, cudaStream_t st, const float* x, int ldx, const int32_t* row_token, int rows, int e,
                        uint16_t* hi, uint16_t* lo);
int launch_grouped_umma(dnb_ctx* c, cudaStream_t st, bool fused, const SegDesc* seg, const int32_t* nseg_dev,
                        int nseg_max, int n_in, int n_out, const UmmaMaps* maps, int nt_max, uint16_t* out_hi,
                        uint16_t* out_lo, float* out_f32, float* const* row_dst = nullptr);
// grouped_exact.cu: IQ3_XXS with exact bf16 weights and the block scales applied after the tensor-core sum
int launch_grouped_exact(dnb_ctx* c, cudaStream_t st, bool fused, const SegDesc* seg, const int32_t* nseg_dev, int nseg_max,
                         int n_in, int n_out, const UmmaMaps* maps, uint16_t* out_hi, uint16_t* out_lo, float* out_f32,
                         float* const* row_dst = nullptr);
// The tensor-core grouped GEMM of a block format: Q4_K -> launch_grouped_umma, IQ3_XXS -> launch_grouped_exact.
int launch_grouped_tc(dnb_ctx* c, cudaStream_t st, int type, bool fused, const SegDesc* seg, const int32_t* nseg_dev,
                      int nseg_max, int n_in, int n_out, const UmmaMaps* maps, int nt_max, uint16_t* out_hi,
                      uint16_t* out_lo, float* out_f32, float* const* row_dst = nullptr);
int launch_combine(dnb_ctx* c, cudaStream_t st, const float* hrow, const int32_t* pos, const float* wts, int nt,
                   int k, int e, const float* sh, const float* shcoef, float* out);
int launch_shared_coef(dnb_ctx* c, cudaStream_t st, const float* x, const float* row, int nt, int e, float* coef);
int launch_synth_blocks(dnb_ctx* c, cudaStream_t st, int type, uint64_t seed, uint64_t tensor_id, uint8_t* dst,
                        uint64_t n_blocks, uint64_t first_block = 0);
int launch_synth_normal(dnb_ctx* c, cudaStream_t st, uint64_t seed, uint64_t tensor_id, float sigma, float* dst,
                        uint64_t n);

}  // namespace dnb
