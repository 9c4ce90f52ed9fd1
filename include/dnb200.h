/* dnb200 -- B200 (sm_100a) implementation of denno-beta's quantised MoE expert
 * matmul path, behind a C ABI.
 *
 * Every entry point replaces one `pub fn` of denno-engine's GPU dispatch module
 * (crates/denno-engine/src/cuda.rs) or one piece of state it keeps; the reference
 * line is cited at each declaration.  Conventions kept from the reference
 * (cuda.rs:21024-21027, 8120-8126, 8785-8788):
 *
 *   return  0  DNB_OK        the GPU computed the result
 *   return  1  DNB_DECLINED  the call did not run and wrote nothing; the caller may
 *                            take its own CPU route (unknown block type, shape the
 *                            kernels do not cover, layer not registered)
 *   return <0  misuse or a CUDA failure; dnb_last_error() has the text
 *
 * Host slices are borrowed for the duration of the call only.  Device memory is
 * owned by the library.  One context drives one device through one stream and is
 * not re-entrant; use one context per GPU.  The same inputs give the same bits on
 * every run (no order-dependent atomics anywhere).
 *
 * There is no CPU fallback inside the library: without a CUDA device dnb_init
 * fails with DNB_ERR_NO_DEVICE.
 */
#ifndef DNB200_H
#define DNB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DNB_OK 0
#define DNB_DECLINED 1
#define DNB_ERR_ARG (-1)
#define DNB_ERR_CUDA (-2)
#define DNB_ERR_NO_DEVICE (-3)
#define DNB_ERR_STATE (-4)

/* ggml type ids (kquant.rs:72-104) of the block formats the kernels decode. */
#define DNB_GGML_Q5_1 7
#define DNB_GGML_Q8_0 8
#define DNB_GGML_Q4_K 12
#define DNB_GGML_Q5_K 13
#define DNB_GGML_Q6_K 14
#define DNB_GGML_IQ3_XXS 18
/* The block types of a real checkpoint's remaining tensors (exp_iq.rs:390-400,
 * cuda.rs:7364-7373): decoded by the tiled kernels and the sequential checker; calls with
 * them take those kernels instead of the decode fast kernels. */
#define DNB_GGML_Q4_0 2
#define DNB_GGML_IQ4_NL 20
#define DNB_GGML_IQ3_S 21
#define DNB_GGML_IQ2_S 22
#define DNB_GGML_IQ4_XS 23
#define DNB_GGML_Q2_0 42

/* matrix slots of a MoE layer */
#define DNB_MAT_GATE 0
#define DNB_MAT_UP 1
#define DNB_MAT_DOWN 2
#define DNB_MAT_SHARED_GATE 3
#define DNB_MAT_SHARED_UP 4
#define DNB_MAT_SHARED_DOWN 5

typedef struct dnb_ctx dnb_ctx;

/* ---- context ----------------------------------------------------------------
 * cuda.rs:18029-18103 (cuda_enabled / shared_ctx / make_current_on_this_thread). */
int dnb_init(int device, dnb_ctx** out);
void dnb_shutdown(dnb_ctx* ctx);
const char* dnb_last_error(void);
/* Run on a stream the caller owns (e.g. the framework's current stream) instead
 * of the context's own; pass NULL to go back.  cuda.rs:100-111 (stream set-up). */
int dnb_set_stream(dnb_ctx* ctx, void* cuda_stream);
/* Waits for the context's streams.  DNB_DECLINED when a bounded device wait has given up since
 * the status word was last cleared (see dnb_device_status). */
int dnb_sync(dnb_ctx* ctx);
/* Kernels launched by this context since creation. */
uint64_t dnb_launch_count(dnb_ctx* ctx);
/* Waits inside the kernels (shared-memory barriers, the grid barrier of the one-token
 * kernel, the flags of the expert-parallel exchange) are bounded.  A wait that gives up
 * records a code in the context's status word (pinned host memory the device writes):
 *   1        a bulk copy into shared memory never completed
 *   2-6      the tcgen05 grouped GEMM (stage, accumulator or drain barrier)
 *   20-22    expert-parallel exchange: row out of range / a peer's counts or rows did not
 *            arrive / a peer's results did not arrive
 *   24       expert-parallel decode: a peer's result rows did not arrive
 *   23       grid barrier of the fused one-token kernel
 *   25       the tensor-core router GEMM of a prefill chunk (stage or accumulator barrier)
 * What the reference promises for a GPU call that did not complete -- "false: out
 * untouched, the caller recomputes" (cuda.rs:21024-21027, 8785-8788) -- holds here too:
 * every host-buffer entry point reads the word after its stream synchronisation and, when
 * it is non-zero, copies nothing to the caller, clears the word and returns DNB_DECLINED
 * (after a 23 the context also stops using the one-kernel decode form: the two-launch
 * form has no inter-CTA wait).  Device-pointer entry points are asynchronous; for them the
 * word stays set until dnb_clear_status, dnb_device_status reads it and dnb_sync returns
 * DNB_DECLINED while it is non-zero. */
int dnb_device_status(dnb_ctx* ctx, int* status);
int dnb_clear_status(dnb_ctx* ctx);
/* How long those waits last: polls of the grid barrier (default 400000, about 0.2 s) and
 * of an expert-parallel flag (default 2^21, about 0.25 s).  barrier_bias is a test hook:
 * it is added to the number of arrivals the grid barrier waits for, so any value > 0 makes
 * the barrier unreachable and the time-out path can be exercised without faulting or
 * hanging anything; 0 in production. */
int dnb_set_wait_limits(dnb_ctx* ctx, int barrier_polls, int flag_polls, int barrier_bias);
/* Device-side timing on the context's stream: start, ... calls ..., stop -> ms. */
int dnb_timer_start(dnb_ctx* ctx);
int dnb_timer_stop(dnb_ctx* ctx, float* ms);
/* Launch sequences of the block and stack entry points are captured into CUDA
 * graphs on their second use and replayed afterwards (one host call per replay
 * instead of one per kernel; the reference pays 4-5 launches and a wait per layer,
 * cuda.rs:8238-8384).  on = 0 goes back to direct launches. */
int dnb_use_graphs(dnb_ctx* ctx, int on);
/* Occupy the stream for about `ms` milliseconds (clock-bounded, at most 200), so
 * that work enqueued behind it runs without host launch gaps. */
int dnb_stall(dnb_ctx* ctx, float ms);
/* Per-kernel device timing for benchmarks (the reference's DENNO_SEG_PROF,
 * model/seg_prof.rs:1-22, cuda.rs:8417-8432): while enabled, every kernel launch is
 * bracketed by events; dnb_profile_read writes a JSON object
 * {"kernel": {"launches": n, "ms": total}, ...} into buf.  Enabling clears it. */
int dnb_profile_enable(dnb_ctx* ctx, int on);
int dnb_profile_read(dnb_ctx* ctx, char* buf, size_t cap);
/* Device memory helpers for callers that keep activations on the GPU. */
int dnb_dev_alloc(dnb_ctx* ctx, size_t bytes, void** dev);
int dnb_dev_free(dnb_ctx* ctx, void* dev);
int dnb_dev_upload(dnb_ctx* ctx, void* dev, const void* host, size_t bytes);
int dnb_dev_download(dnb_ctx* ctx, void* host, const void* dev, size_t bytes);
/* Device-to-device copy on the context's stream; does not synchronise. */
int dnb_dev_copy(dnb_ctx* ctx, void* dst, const void* src, size_t bytes);
/* Overwrite `bytes` of device scratch larger than L2 (benchmark hygiene). */
int dnb_flush_l2(dnb_ctx* ctx);

/* ---- single resident matrix: the GEMV_V3 path ---------------------------------
 * cuda.rs:21028-21111 (maybe_gpu_gguf_gemv_into): weights are uploaded once per
 * `uid` and stay resident (weights_for_gguf); the call copies x in, runs one
 * dequant-GEMV and copies out back.  out[r] = sum_i dequant(W)[r][i] * x[i]. */
int dnb_register_matrix(dnb_ctx* ctx, uint64_t uid, int ggml_type, const void* blocks, size_t bytes, int k, int n);
int dnb_gemv(dnb_ctx* ctx, uint64_t uid, const float* x, float* out);
/* The same kernel on device pointers: nvec activation vectors x[v][k] -> out[v][n]
 * (kernels_moe_v3.cu:216-266 is the reference kernel of this shape). */
int dnb_gemv_dev(dnb_ctx* ctx, int ggml_type, const void* w_dev, int k, int n, const float* x_dev, float* out_dev,
                 int nvec);
/* 0: fast lane-split kernels (default).  1: the sequential-order kernel whose fp32
 * results equal the CPU scalar path bit for bit (kernels_moe.cu contract,
 * cuda.rs:44991-45057).  2: the general tiled fp32 kernels everywhere -- one-token calls
 * skip the bulk-copy decode kernels and prefill chunks skip the tcgen05 grouped
 * GEMM (A/B checks between kernel families).  3: as 0, but one-token IQ3_XXS blocks
 * take the register-decode kernels instead of the mma.sync ones.  4: as 0, but
 * the mma.sync gate/up kernel and the down kernel run as two launches instead of
 * the fused one.  5: as 0, but the router of a one-token IQ3_XXS block runs as a
 * kernel of its own in front of the fused gate/up + down kernel instead of inside it. */
int dnb_set_gemv_impl(dnb_ctx* ctx, int impl);
/* IQ3_XXS layers: the token count from which a chunk or decode batch leaves the one-token kernels for the
 * exact-weight tcgen05 grouped GEMM (default 16, where it measured level with the one-token kernels and
 * 1.7x / 2.1x faster at 64 / 194 tokens; Q4_K layers switch to their tcgen05 kernel at 16 too).  A tuning
 * and A/B knob with no reference counterpart; results stay within the path's tolerance either way. */
int dnb_set_tc_min_tokens(dnb_ctx* ctx, int iq3_xxs_min_tokens);
/* Q4_K chunks on tcgen05: on = 0 (default) the kernel that folds the scales into bf16 hi / lo weights (three
 * products per element); on = 1 the kernel with integer fp16 weights (sc * q, exact) and the block scales d,
 * dmin * m applied after the tensor-core sum, where the shape fits (n_embd, n_ff <= 2048, multiples of 256): a
 * sixth of the error (1e-5 against 7e-5 of the output RMS) at 1.2x the time of a 512-token chunk.  Both are far
 * inside the path's tolerance of the CPU reference; an A/B knob with no reference counterpart. */
int dnb_set_q4k_int(dnb_ctx* ctx, int on);
/* Router logits of calls of 16 tokens or more (cuda.rs:48695 pf_router_dev_topk over kernels_elem.cu:1085
 * dno_gemm_f32_mt): on = 1 (default) the tcgen05 kernel -- both operands as three bf16 parts, six products,
 * fp32 accumulation: the accuracy of an fp32 sum -- on = 0 the fp32 FMA kernel that smaller calls use.  The
 * two differ by summation order only; an A/B knob.  (dnb_router_topk_static always runs the fp32 kernel: where
 * the tcgen05 kernel would take the call its weights agree within rounding, not bit for bit.) */
int dnb_set_router_tc(dnb_ctx* ctx, int on);

/* ---- MoE model: resident expert table ----------------------------------------
 * Replaces the VRAM/RAM/SSD expert tiers (expert_vram.rs:1-60; use at
 * qwen4exp.rs:12600-12629): every expert of every layer is resident. */
int dnb_moe_config(dnb_ctx* ctx, int n_layer, int n_embd, int n_ff, int n_shared_ff, int n_expert, int n_expert_used,
                   float rms_eps, int norm_topk_prob);
/* One expert tensor, expert-major as in GGUF (moe_expert.rs:49-82 ExpertSlice):
 * expert i occupies bytes [i*n_out*row_bytes, (i+1)*n_out*row_bytes).  `blocks`
 * is a host pointer, copied. */
int dnb_register_experts(dnb_ctx* ctx, int layer, int matrix, int ggml_type, int n_in, int n_out, int n_expert,
                         const void* blocks, size_t bytes);
/* Router row matrix ffn_gate_inp [n_expert][n_embd] fp32 (linear_gguf.rs:836-964),
 * optional per-expert logit bias (moe.rs:327-338), optional RMSNorm weight applied
 * to the block input (tensor.rs:1125-1135), optional shared-expert gate row
 * ffn_gate_inp_shexp (qwen4exp.rs:12388-12395; NULL = coefficient 1.0 as in
 * moe.rs:386-403).  Host pointers, copied. */
int dnb_register_router(dnb_ctx* ctx, int layer, const float* w, const float* bias, const float* norm_w,
                        const float* shared_gate_row);
/* Fill one expert tensor in place on the device from the seeded generator of
 * dnb_synth.h (tensor id = layer*16 + matrix).  For benchmarks whose expert table
 * is too large to stage through the host.  With an expert shard set
 * (dnb_moe_set_expert_shard) a routed tensor receives the bytes of experts
 * [first, first + n_expert) of the full tensor, so G ranks together hold exactly what
 * one GPU would. */
int dnb_synth_experts(dnb_ctx* ctx, int layer, int matrix, int ggml_type, int n_in, int n_out, int n_expert,
                      uint64_t seed);
/* Copy expert `expert` of a registered tensor back to the host (parity checks). */
int dnb_download_expert(dnb_ctx* ctx, int layer, int matrix, int expert, void* dst, size_t bytes);

/* ---- GGUF files -> the resident expert table ----------------------------------------
 * crates/denno-engine/src/gguf.rs:163-330 (GgufFile::open / open_split: v2/v3 containers, split
 * models as parts with split.no / split.count / split.tensors.count) and model/qwen4exp.rs:1915-1963
 * (ExpertW::load).  The reference keeps expert tensors in the file mapping and moves experts between
 * SSD, RAM and VRAM on demand (expert_vram.rs); here a layer is read from the mapping once and stays
 * in HBM.  dnb_gguf_open takes the path of one file or of all parts of a split model (any order) and
 * needs no GPU; the handle's tensor table, metadata and data pointers (into the read-only mapping,
 * valid until dnb_gguf_close) can be inspected with the getters.  DNB_DECLINED from a getter = no
 * such tensor / key.
 *   dnb_load_gguf_layer: registers blk.<gguf_layer>.{ffn_gate_exps, ffn_up_exps, ffn_down_exps}.weight
 *       (3-d, ne = [n_in, n_out, n_expert], expert-major as moe_expert.rs:49-82; with an expert shard
 *       set only this rank's contiguous byte range is copied), the shared expert ffn_{gate,up,down}
 *       _shexp.weight when present, the router ffn_gate_inp.weight (f32 [n_embd, n_expert]), and, when
 *       present, exp_probs_b.bias and ffn_gate_inp_shexp.weight (qwen4exp.rs:1018-1025) as layer
 *       `layer` of the configured model.  norm_name (may be NULL) names an f32 [n_embd] tensor of the
 *       block to use as the RMSNorm weight in front of the router. */
typedef struct dnb_gguf dnb_gguf;
int dnb_gguf_open(const char* const* paths, int n_paths, dnb_gguf** out);
void dnb_gguf_close(dnb_gguf* g);
int dnb_gguf_n_tensors(const dnb_gguf* g);
const char* dnb_gguf_tensor_name(const dnb_gguf* g, int index);
int dnb_gguf_tensor_info(const dnb_gguf* g, const char* name, int* ggml_type, int* n_dims, uint64_t dims[4], int* part,
                         uint64_t* file_offset, uint64_t* nbytes);
const void* dnb_gguf_tensor_data(const dnb_gguf* g, const char* name, uint64_t* nbytes);
int dnb_gguf_meta_u64(const dnb_gguf* g, const char* key, uint64_t* v);
int dnb_gguf_meta_f64(const dnb_gguf* g, const char* key, double* v);
int dnb_gguf_meta_str(const dnb_gguf* g, const char* key, char* buf, size_t cap);
int dnb_load_gguf_layer(dnb_ctx* ctx, const dnb_gguf* g, int layer, int gguf_layer, const char* norm_name);

/* ---- MoE block -----------------------------------------------------------------
 * One sparse-MoE block for nt tokens: (RMSNorm) -> router -> softmax -> top-k ->
 * renorm -> routed experts (gate/up GEMV, SwiGLU, down GEMV) -> weighted sum in
 * ascending expert index -> + shared expert.
 *   decode : qwen4exp.rs:11659 moe_ffn_quant_impl -> cuda.rs:8088 moe_seg_layer_sum
 *            / cuda.rs:8825 moe_experts_iq_layer_sum_overlap
 *   prefill: qwen4exp.rs:17921 moe_ffn_quant_batch_full -> cuda.rs:48695
 *            pf_router_dev_topk + cuda.rs:10919 moe_experts_iq_pf_layer /
 *            cuda.rs:7065 moe_grouped_gemm_layer + moe_grouped_gpu.rs:540 scatter
 * h, out: host [nt][n_embd].  sels_out [nt][k] / wts_out [nt][k] may be NULL. */
int dnb_moe_block(dnb_ctx* ctx, int layer, const float* h, int nt, float* out, int32_t* sels_out, float* wts_out);
/* Same with device pointers; nothing is copied and the call does not synchronise. */
int dnb_moe_block_dev(dnb_ctx* ctx, int layer, const float* h_dev, int nt, float* out_dev);
/* The routed-expert half only, with the selection given by the caller
 * (cuda.rs:8088-8107 moe_seg_layer_sum: sels ascending, routing weights w):
 * out[t] = sum_s w[t][s] * down(silu(gate x_t) * up x_t) (+ shared expert).
 * x is the expert input (already normalised), host [nt][n_embd]. */
int dnb_moe_experts(dnb_ctx* ctx, int layer, const float* x, int nt, const int32_t* sels, const float* wts,
                    float* out);
/* Router only (cuda.rs:48695-48708 pf_router_dev_topk): logits = W_r x + bias,
 * softmax, top-k (ties to the lower index, output ascending), renorm.
 * x host [nt][n_embd]; sels [nt][k], wts [nt][k], rowsum [nt] (sum of the selected
 * probabilities before renorm; may be NULL). */
int dnb_router_topk(dnb_ctx* ctx, int layer, const float* x, int nt, int32_t* sels, float* wts, float* rowsum);
/* Router + top-k for callers that must not allocate: a serving loop with a fixed
 * memory budget, a host that forbids cudaMalloc on its inference thread, or code
 * inside a stream capture.  (No counterpart in the reference: its router path grows
 * its scratch on demand, cuda.rs:7454-7480.)  Same kernels and same results as
 * dnb_router_topk, but all of x, sels [nt][k], wts [nt][k] and rowsum [nt] (may be
 * NULL) are DEVICE pointers supplied by the caller, the call runs asynchronously on
 * the context's stream, and the logits between the two kernels live in a fixed
 * 256 KiB array inside the library instead of the workspace: nt * n_expert must not
 * exceed 65536, larger calls are rejected with DNB_ERR_ARG.  The call performs no
 * cudaMalloc/cudaFree and no other allocating call.  The first call on each device
 * looks up the array's device address (cudaGetSymbolAddress) and sets a kernel
 * attribute; make that first call before any stream capture begins.  All calls on
 * a device share the one array: two calls that overlap on the GPU (different
 * streams or contexts) race; calls on one stream are ordered and safe.  Nothing in
 * the array needs to start at zero (every logit in range is rewritten per call). */
int dnb_router_topk_static(dnb_ctx* ctx, int layer, const float* x_dev, int nt, int32_t* sels_dev, float* wts_dev,
                           float* rowsum_dev);
/* Grouped per-expert GEMM on packed rows (cuda.rs:7065-7075 moe_grouped_gemm_layer,
 * moe_expert.rs:8455 grouped_expert_gemm_cpu): segs[nseg][4] = (expert, m, x_off,
 * out_off) with offsets in rows; xs host [m_total][n_in]; outs host
 * [m_total][n_out]. */
int dnb_grouped_gemm(dnb_ctx* ctx, int layer, int matrix, const uint32_t* segs, int nseg, const float* xs,
                     float* outs);
/* The expert-major row space of a chunk as the device builds it (moe_expert.rs:8309-8390
 * build_grouped_batch; Segment{expert, m, x_off, out_off} :8272-8281; exp_pf.rs:23-31 rows[]):
 * from sels host [nt][k] -> segs_out [n_expert][4] = (expert, m, first row, first row) ordered by
 * token count descending, ties by expert ascending; *nseg_out = active experts; row_token_out
 * [nt*k] = token of each packed row (ascending inside an expert); pos_out [nt*k] = packed row
 * of (token, slot).  The last two may be NULL.  For parity checks of the routing tables. */
int dnb_build_grouped_batch(dnb_ctx* ctx, int layer, const int32_t* sels, int nt, uint32_t* segs_out, int32_t* nseg_out,
                            int32_t* row_token_out, int32_t* pos_out);
/* The legacy three-launch decode form (cuda.rs:7638-7650 moe_gemv_seg_pair, 7689-7698
 * moe_gemv_seg_one): segmented GEMVs whose results return to the host, which applies
 * silu(g)*u and the weighted sum itself.  seg[nseg][4] = (expert, m, x_off, out_off) as in
 * expert_batch.rs:143-170, offsets in floats and multiples of n_in / n_out: token j of
 * segment i reads x[x_off + j*n_in ..] and writes out[out_off + j*n_out ..] (gate/up of one
 * token: x_off = 0, out_off = s*ff; down: x_off = s*ff, out_off = s*e).  Where the reference
 * passes a table of device addresses (wptrs), the expert index names the resident expert
 * of (layer, matrix).  x_len / out_len are the lengths of x / out in floats; a segment that
 * reaches beyond them is refused (expert_batch.rs:233-260 seg_extents). */
int dnb_seg_gemv(dnb_ctx* ctx, int layer, int matrix, const uint32_t* seg, int nseg, const float* x, size_t x_len,
                 float* out, size_t out_len);
int dnb_seg_gemv_pair(dnb_ctx* ctx, int layer, const uint32_t* seg, int nseg, const float* x, size_t x_len, float* out_g,
                      float* out_u, size_t out_len);
/* Router logits alone (cuda.rs:25836 maybe_gpu_router_gemv_into; kernels_elem.cu:948-1002):
 * logits[t][i] = W_r[i] . x[t] + bias[i] for nt rows, host in / host out.  Lane-split with
 * a fixed tree: deterministic, not the bits of the sequential CPU loop (the reference's
 * default dno_matvec_f32_r has the same contract). */
int dnb_router_gemv(dnb_ctx* ctx, int layer, const float* x, int nt, float* logits);
/* ---- hyper-connection mix around the block ------------------------------------------------
 * model/hyper.rs (hc_mix :369, hc_combine :384; the order of operations :13-36 is its numeric contract);
 * call sites model/qwen4exp.rs:3722-3765 (hc_mix_quant -> moe_ffn_quant -> hc_combine_inplace).  A layer
 * carries hc parallel residual streams per token; the mix turns them into the block's input (per-stream
 * RMSNorm, a low-rank gate: w_down_inject [low_rank + hc][hc*n_embd], w_up [hc*n_embd][low_rank]) and the
 * combine writes the block's output back into every stream scaled by 2*sigmoid(inject[s]).
 *   dnb_register_hc   : fp32 host tensors of layer `layer`: w_norm [hc][n_embd] (the gamma the converter
 *       folded to 1 + w), w_down_inject, w_up.  (Checkpoints store them as BF16; widen first, which is exact.)
 *   dnb_hc_moe_block  : res, out host [nt][hc][n_embd]: out = combine(res, block(mix(res)), inject).  The
 *       layer's MoE block must be registered without an RMSNorm weight of its own (the mix normalises).
 *   dnb_hc_moe_block_dev: the same on device pointers, asynchronous. */
int dnb_register_hc(dnb_ctx* ctx, int layer, int hc, int low_rank, const float* w_norm, const float* w_down_inject,
                    const float* w_up);
int dnb_hc_moe_block(dnb_ctx* ctx, int layer, const float* res, int nt, float* out);
int dnb_hc_moe_block_dev(dnb_ctx* ctx, int layer, const float* res_dev, int nt, float* out_dev);
/* ---- expert-parallel building blocks ---------------------------------------------
 * The reference runs on one GPU.  On a multi-GPU box the experts shard naturally:
 * GPU g keeps experts [g*ne/G, (g+1)*ne/G) of every layer (router, norm and shared
 * expert replicated), tokens stay data-parallel, and the routed activations are
 * exchanged with an all-to-all between the three calls below (the exchange itself
 * is the caller's: NCCL through torch.distributed in denno_beta_b200/ep.py).  All
 * pointers are device pointers; the calls are asynchronous on the context's stream.
 *   dnb_moe_set_expert_shard : which routed experts this context holds (call after
 *       dnb_moe_config and before dnb_register_experts, whose n_expert is then the
 *       shard's size).  With a proper shard the whole-block entry points decline.
 *   dnb_moe_route_dev  : (RMSNorm) + router + top-k for the caller's own tokens;
 *       writes the expert input x [nt][e], sels [nt][k] (global ids), wts [nt][k].
 *   dnb_expert_rows_dev: h[r] = down(silu(gate x[r]) * up x[r]) of LOCAL expert
 *       local_ids[r] for each of `rows` received rows; use_shared != 0 applies the
 *       shared expert to every row instead (local_ids may be NULL).
 *   dnb_moe_combine_dev: out[t] = sum_s wts[t][s] * h_slots[t*k+s] in ascending slot
 *       (= ascending expert) order, + shared[t] (times sigmoid(gate row . x[t]) when
 *       the layer has a shared gate row; x may be NULL otherwise).  The order is
 *       the single-GPU order, so the result does not depend on G. */
int dnb_moe_set_expert_shard(dnb_ctx* ctx, int first_expert, int n_local);
int dnb_moe_route_dev(dnb_ctx* ctx, int layer, const float* h_dev, int nt, float* x_out_dev, int32_t* sels_dev,
                      float* wts_dev);
int dnb_expert_rows_dev(dnb_ctx* ctx, int layer, const float* x_rows_dev, const int32_t* local_ids_dev, int rows,
                        int use_shared, float* h_rows_dev);
int dnb_moe_combine_dev(dnb_ctx* ctx, int layer, const float* h_slots_dev, const float* wts_dev, const float* shared_dev,
                        const float* x_dev, int nt, float* out_dev);
/* ---- expert-parallel block over peer memory (prefill chunks, Q4_K layers) -----------
 * No counterpart in the reference (single GPU; its multi-device plan stops at keeping
 * experts resident, src/expert_vram.rs).  One process per GPU of one node.  Instead of
 * handing the rows to a collective library between the calls above, the ranks store them
 * into each other's memory from this library's own kernels: the dispatch writes the bf16
 * operand rows straight into the owner rank's GEMM input buffers, and the epilogue of
 * the owner's down GEMM stores every result row into the (token, slot) row of the rank
 * that owns the token.  Flags in the ranks' own memory order the steps; every wait is
 * bounded and a wait that gives up shows in dnb_device_status (codes 20-22).
 *   dnb_ep_init    : after dnb_moe_config, dnb_moe_set_expert_shard(rank*ne/world,
 *       ne/world) and the expert registration.  Allocates this rank's arena for up to
 *       max_tokens own tokens per call and writes its 64-byte IPC handle to handle_out.
 *   dnb_ep_connect : handles = world x 64 bytes, rank r's handle at byte 64*r (exchange
 *       them with any host-side all-gather); maps the peers' arenas.
 *   dnb_ep_block_dev: one MoE block for this rank's nt tokens, h_dev/out_dev device
 *       [nt][n_embd].  Every rank of the group must make the same sequence of calls
 *       (same layer; nt may differ per rank).  The result equals the single-GPU block
 *       bit for bit: same operands, same accumulation order, same combine order. */
int dnb_ep_init(dnb_ctx* ctx, int rank, int world, int max_tokens, void* handle_out);
int dnb_ep_connect(dnb_ctx* ctx, const void* handles);
int dnb_ep_block_dev(dnb_ctx* ctx, int layer, const float* h_dev, int nt, float* out_dev);
/* All configured layers with identity mixers, in place: h <- h + block_l(h) for this rank's nt tokens
 * (the expert-parallel form of dnb_moe_stack_dev). */
int dnb_ep_stack_dev(dnb_ctx* ctx, float* h_dev, int nt);
/* Teardown rule of the peer-memory path: a rank's arena is memory its peers store into from
 * their kernels.  A rank must not call dnb_shutdown (or exit) before a host-side barrier
 * has shown that no peer still has a dnb_ep_block_dev in flight -- synchronise the own
 * context, then barrier, then shut down; on an error path wait at least as long as the
 * longest device wait (dnb_set_wait_limits) before leaving, so that the peers' kernels have
 * finished or given up.
 * Test hook: a group of `world` ranks of which only this one exists -- every peer pointer is
 * this rank's own arena, so the flags of the absent ranks never arrive and a block call runs
 * into its bounded waits (status 21/22) instead of a partner. */
int dnb_ep_connect_loopback(dnb_ctx* ctx);
/* ---- expert-parallel DECODE over peer memory -------------------------------------------
 * No counterpart in the reference (single GPU).  For decode batches (1 to a few dozen tokens) the
 * exchange is latency, not volume, so the residual stream is REPLICATED: every rank of the group
 * holds all tokens of the batch and routes them itself (same arithmetic, same bits); it computes
 * the (token, slot) pairs whose expert it holds and stores each result row into slot (token, slot) of
 * EVERY rank's arena with plain peer stores; after one bounded flag wait per layer every rank sums
 * the k slots in ascending expert order (+ shared expert) exactly as one GPU does.  One exchange per
 * layer, the result does not depend on the number of ranks, every rank ends with the same bits.
 *   dnb_epd_init    : after dnb_moe_config, dnb_moe_set_expert_shard(rank*ne/world, ne/world) and the
 *       registration of the rank's experts (router, norm, shared expert replicated).  Allocates the
 *       arena for batches of up to max_tokens tokens and writes its 64-byte IPC handle to handle_out.
 *   dnb_epd_connect : handles = world x 64 bytes (rank r's at byte 64*r), exchanged by any host-side
 *       all-gather.  NULL is a test hook: every peer pointer becomes this rank's own arena, so with
 *       world > 1 the absent ranks' flags never arrive and a call runs into its bounded wait (status 24).
 *   dnb_epd_block_dev / dnb_epd_stack_dev: one block, or all configured layers with identity mixers
 *       (h <- h + block_l(h), in place), for the SAME nt tokens on every rank; device pointers,
 *       asynchronous.  Every rank must make the same sequence of calls.  The teardown rule of
 *       dnb_ep_block_dev applies: barrier on the host before any rank shuts down. */
int dnb_epd_init(dnb_ctx* ctx, int rank, int world, int max_tokens, void* handle_out);
int dnb_epd_connect(dnb_ctx* ctx, const void* handles);
int dnb_epd_block_dev(dnb_ctx* ctx, int layer, const float* h_dev, int nt, float* out_dev);
int dnb_epd_stack_dev(dnb_ctx* ctx, float* h_dev, int nt);
/* A stack of the configured layers with identity mixers: h <- h + block_l(h) for
 * l = 0..n_layer-1 (device-resident between layers).  h host [nt][n_embd] in/out. */
int dnb_moe_stack(dnb_ctx* ctx, const float* h, int nt, float* out);
int dnb_moe_stack_dev(dnb_ctx* ctx, float* h_dev, int nt);

#ifdef __cplusplus
}
#endif
#endif /* DNB200_H */
