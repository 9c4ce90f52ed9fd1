/* Declarations shared by the two translation units of the CPU oracle (TEST INFRASTRUCTURE):
 * dnb_oracle.c, the sequential-order restatement that parity is checked against, and
 * dnb_cpu_fast.c, the AVX2+FMA restatement of the reference's production CPU kernels that is
 * only ever timed. */
#ifndef DNB_ORACLE_H
#define DNB_ORACLE_H
#include <stdint.h>

typedef struct {
    long e, ff, ne, k, sff;
    int norm_topk;
    int ty_gate, ty_up, ty_down;          /* routed experts */
    int ty_sgate, ty_sup, ty_sdown;       /* shared expert */
    float eps;
    const float* norm_w;                  /* [e] or NULL = no RMSNorm in front */
    const float* router_w;                /* [ne][e] fp32 */
    const float* router_bias;             /* [ne] or NULL */
    const uint8_t *gate, *up, *down;      /* [ne] experts, expert-major (ExpertSlice) */
    const uint8_t *sgate, *sup, *sdown;   /* shared expert or NULL */
    const float* shared_gate_row;         /* [e] or NULL: coefficient sigmoid(row . x), else 1.0 */
} orc_moe_layer;

/* moe_expert.rs:8272-8281 */
typedef struct {
    uint32_t expert, m, x_off, out_off;
} orc_segment;

int orc_blck_size(int type);
int orc_type_size(int type);
long orc_row_bytes(int type, long n_in);
int orc_dequant_row(int type, const uint8_t* blocks, long n, float* out);
void orc_rmsnorm(const float* x, const float* w, long rows, long cols, float eps, float* out);
void orc_softmax(float* x, long n);
float orc_silu(float v);
float orc_sigmoid(float v);
void orc_hc_mix(const float* x, const float* w_norm, const float* w_down_inject, const float* w_up, long hc, long e,
                long low_rank, float eps, float* mixed, float* inject, float* xn_out);
void orc_hc_combine(const float* residual, const float* block, const float* inject, long hc, long e, float* out);
void orc_select_topk(const float* probs, long n, long k, int32_t* out);
void orc_router_renorm(const float* probs, const int32_t* sel, long k, float* w);
long orc_build_segments(const int32_t* sels, long nt, long k, long ne, orc_segment* segs, int32_t* row_token,
                        int32_t* row_slot, long* m_total_out);
#endif
