// Expert-parallel prefill block over peer memory (one process per GPU, one node).
//
// The reference is single-GPU.  With G GPUs each rank keeps n_local = ne / G routed
// experts of every layer, owns its own tokens and runs, per layer,
//
//   route (local)                                  existing kernels
//   plan      counts per expert, row order         ep_plan_kernel      -> peers' cnt + flag
//   dispatch  x rows -> bf16 hi/lo, stored straight into the OWNER rank's operand buffers
//             (the B operand the tcgen05 kernel reads by TMA from its own memory)
//                                                  ep_dispatch_kernel  -> peers' data flag
//   build     wait for every source's counts and rows (bounded), segment table per
//             (source, expert), destination pointer of every received row
//                                                  ep_build_kernel
//   gate/up   grouped tcgen05 GEMM + SwiGLU        grouped_q4k_umma_kernel<2>
//   down      grouped tcgen05 GEMM whose epilogue stores each row into the (token, slot)
//             row of the rank that owns the token  grouped_q4k_umma_kernel<1>, row_dst
//   signal / wait   release flags to the sources, wait for every owner's flag (bounded)
//   combine   ascending slot order, as on one GPU  combine_kernel
//
// Nothing goes through the host between these launches and no library collective is
// involved: rows cross NVLink as plain stores of this library's kernels into memory the
// peers exported with cudaIpcGetMemHandle.  Every rank has one arena (EpArena header,
// then the row buffers); rank s writes only region s of a peer's buffers and slot s of
// its flag arrays, so no two ranks ever write the same word.  Flags carry the sequence
// number of the call and only grow, so they are never reset.  A source's region holds up
// to `cap` rows (all of its rows may go to one peer), sorted by (expert, token).
//
// Every wait polls a flag in the rank's own memory with a limit; when the limit runs out
// the kernel records a status and returns, the following kernels run on whatever is
// there and the host reports the status.  No load through TMA ever touches peer memory.
#include <cuda_bf16.h>

#include "dnb_common.cuh"

namespace dnb {

constexpr int kEpMaxWorld = 16;
constexpr int kEpMaxLocal = 512;

struct EpArena {                       // head of every rank's exported allocation
    uint32_t cnt_flag[kEpMaxWorld];    // [s] = seq once source s has written cnt[s][*]
    uint32_t data_flag[kEpMaxWorld];   // [s] = seq once source s has stored all its rows here
    uint32_t ret_flag[kEpMaxWorld];    // [d] = seq once owner d has stored all results for my tokens
    int32_t cnt[kEpMaxWorld][kEpMaxWorld * kEpMaxLocal / 8];  // cnt[s][e]: rows source s has for GLOBAL expert e (ne <= 1024)
};
constexpr int kEpMaxExperts = kEpMaxWorld * kEpMaxLocal / 8;

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// Poll until *p >= seq; gives up after `polls` tries (2^21 by default: about a quarter of a second).
__device__ __forceinline__ bool wait_flag(const uint32_t* p, uint32_t seq, int polls) {
    for (int i = 0; i < polls; ++i) {
        if ((int32_t)(ld_acquire_sys(p) - seq) >= 0) return true;
        __nanosleep(100);
    }
    return false;
}

// bf16 hi/lo split of a pair (hi rounded to nearest, lo = the exact remainder truncated):
// the same arithmetic as the single-GPU gather pass, so the operands are the same bits.
__device__ __forceinline__ void ep_split2(float a, float b, uint32_t& hi_pair, uint32_t& lo_pair) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    hi_pair = *reinterpret_cast<const uint32_t*>(&h);
    const float al = a - __uint_as_float(hi_pair << 16), bl = b - __uint_as_float(hi_pair & 0xFFFF0000u);
    lo_pair = __byte_perm(__float_as_uint(al), __float_as_uint(bl), 0x7632);
}

struct EpPeers {                 // kernel parameter: every rank's arena as seen from this GPU
    EpArena* arena[kEpMaxWorld];
    int32_t* recv_slot[kEpMaxWorld];
    uint16_t* xg_hi[kEpMaxWorld];
    uint16_t* xg_lo[kEpMaxWorld];
    float* h_slots[kEpMaxWorld];
};

// One CTA.  sels[nt][k] (global expert ids, ascending per token) -> send_row[i] = how many
// earlier tokens of this rank selected the same expert (the row's index among this rank's
// rows of that expert).  The per-expert counts go to EVERY rank (each needs the whole count
// matrix to place its rows), then the flag.
__global__ void __launch_bounds__(1024)
ep_plan_kernel(const int32_t* __restrict__ sels, int nt, int k, int ne, int n_local, int world, int me, uint32_t seq,
               EpPeers peers, int32_t* __restrict__ send_row) {
    extern __shared__ uint32_t sm[];
    const int words = (nt + 31) >> 5;
    uint32_t* bitmap = sm;                         // [ne][words]: token t selects expert e
    int* counts = (int*)(sm + (size_t)ne * words); // [ne]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = blockDim.x >> 5;
    for (int i = tid; i < ne * words; i += blockDim.x) bitmap[i] = 0;
    __syncthreads();
    for (int i = tid; i < nt * k; i += blockDim.x) {
        const int e = sels[i];
        if (e >= 0 && e < ne) atomicOr(&bitmap[(size_t)e * words + ((i / k) >> 5)], 1u << ((i / k) & 31));
    }
    __syncthreads();
    for (int e = warp; e < ne; e += nwarp) {
        int c = 0;
        for (int w = lane; w < words; w += 32) c += __popc(bitmap[(size_t)e * words + w]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
        if (lane == 0) counts[e] = c;
    }
    __syncthreads();
    for (int i = tid; i < nt * k; i += blockDim.x) {
        const int e = sels[i], t = i / k;
        int r = -1;
        if (e >= 0 && e < ne) {
            const uint32_t* bm = bitmap + (size_t)e * words;
            int before = __popc(bm[t >> 5] & ((1u << (t & 31)) - 1u));
            for (int w = 0; w < (t >> 5); ++w) before += __popc(bm[w]);
            r = before;
        }
        send_row[i] = r;
    }
    for (int d = 0; d < world; ++d)
        for (int i = tid; i < ne; i += blockDim.x) peers.arena[d]->cnt[me][i] = counts[i];
    __threadfence_system();
    __syncthreads();
    if (tid < world) st_release_sys(&peers.arena[tid]->cnt_flag[me], seq);
}

// One CTA.  Waits for every rank's counts, then base[e] = where this rank's rows of global
// expert e start in the owner's buffers: the owner keeps its experts in ascending order,
// inside an expert the sources in ascending rank, inside a source the tokens ascending.
__global__ void __launch_bounds__(1024)
ep_offsets_kernel(const EpArena* mine, int ne, int n_local, int world, int me, uint32_t seq, int32_t* __restrict__ base,
                  int* status, int polls) {
    __shared__ int tot[kEpMaxExperts];   // rows of expert e over all sources
    __shared__ int mine_off[kEpMaxExperts];  // rows of expert e from sources before me
    __shared__ int ok_all;
    const int tid = threadIdx.x;
    if (tid == 0) ok_all = 1;
    __syncthreads();
    if (tid < world && !wait_flag(&mine->cnt_flag[tid], seq, polls)) { status_set(status, 21); ok_all = 0; }
    __syncthreads();
    for (int e = tid; e < ne; e += blockDim.x) {
        int t = 0, b = 0;
        for (int s = 0; s < world; ++s) {
            const int c = ok_all ? mine->cnt[s][e] : 0;
            if (s < me) b += c;
            t += c;
        }
        tot[e] = t;
        mine_off[e] = b;
    }
    __syncthreads();
    if (tid < world) {  // exclusive scan of the totals inside each owner's expert range
        int run = 0;
        for (int e = tid * n_local; e < (tid + 1) * n_local; ++e) { const int t = tot[e]; tot[e] = run; run += t; }
    }
    __syncthreads();
    for (int e = tid; e < ne; e += blockDim.x) base[e] = tot[e] + mine_off[e];
}

// Rows i = t*k+slot, dealt to the CTAs round-robin: split x[t] to bf16 hi/lo and store it as row
// base[expert] + j of the owner's operand buffers; the last CTA to finish raises the data flag at every
// peer.  A CTA walks many rows and fences once at the end: the kernel runs beside the shared expert's
// GEMM, which leaves room for about one of these CTAs per SM, and with a CTA (and a system-wide fence,
// i.e. an NVLink round trip) per row the 4,096 rows of a chunk went out at a third of the link rate.
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const float* __restrict__ x, const int32_t* __restrict__ sels, const int32_t* __restrict__ send_row,
                   const int32_t* __restrict__ base, int k, int e, int n_local, int world, int me, int rows_total,
                   int n_rows, uint32_t seq, EpPeers peers, unsigned int* ticket, int* status) {
    const int tid = threadIdx.x;
    for (int i = blockIdx.x; i < n_rows; i += gridDim.x) {
        const int ex = sels[i], j = send_row[i];
        if (ex < 0 || j < 0) continue;
        const size_t r = (size_t)base[ex] + j;
        if (r >= (size_t)rows_total) {
            if (tid == 0) status_set(status, 20);
            continue;
        }
        const int d = ex / n_local;
        const float* xr = x + (size_t)(i / k) * e;
        uint16_t* hi = peers.xg_hi[d] + r * e;
        uint16_t* lo = peers.xg_lo[d] + r * e;
        for (int c = tid * 8; c < e; c += 2048) {  // 16-byte stores: the peer write is NVLink traffic
            const float4 v = *reinterpret_cast<const float4*>(xr + c);
            const float4 u = *reinterpret_cast<const float4*>(xr + c + 4);
            uint32_t h0, l0, h1, l1, h2, l2, h3, l3;
            ep_split2(v.x, v.y, h0, l0);
            ep_split2(v.z, v.w, h1, l1);
            ep_split2(u.x, u.y, h2, l2);
            ep_split2(u.z, u.w, h3, l3);
            *reinterpret_cast<uint4*>(hi + c) = make_uint4(h0, h1, h2, h3);
            *reinterpret_cast<uint4*>(lo + c) = make_uint4(l0, l1, l2, l3);
        }
        if (tid == 0) peers.recv_slot[d][r] = (me << 24) | i;  // who owns the token, and which (token, slot) row
    }
    __threadfence_system();
    __syncthreads();
    __shared__ int last;
    if (tid == 0) {
        const unsigned int t = atomicAdd(ticket, 1u);
        last = (t == gridDim.x - 1) ? 1 : 0;
        if (last) *ticket = 0u;
    }
    __syncthreads();
    if (last && tid < world) st_release_sys(&peers.arena[tid]->data_flag[me], seq);
}

// One CTA.  Waits for every source's rows, then builds the segment tables of the two grouped
// GEMMs -- one segment per local expert with rows, heaviest first (ties: expert ascending),
// rows of all sources together -- and the destination pointer of every received row.
__global__ void __launch_bounds__(1024)
ep_build_kernel(EpArena* mine, const int32_t* __restrict__ recv_slot, int world, int n_local, int me, int e, uint32_t seq,
                EpPeers peers, const uint8_t* gate, const uint8_t* up, const uint8_t* down, size_t eb_g, size_t eb_u,
                size_t eb_d, SegDesc* seg_gu, SegDesc* seg_dn, int32_t* nseg, float** row_dst, int* status, int polls) {
    __shared__ int ok_all;
    __shared__ int tot[kEpMaxLocal], first[kEpMaxLocal];
    __shared__ int n_rows;
    const int tid = threadIdx.x;
    if (tid == 0) ok_all = 1;
    __syncthreads();
    if (tid < 2 * world) {
        const uint32_t* f = tid < world ? &mine->cnt_flag[tid] : &mine->data_flag[tid - world];
        if (!wait_flag(f, seq, polls)) { status_set(status, 21); ok_all = 0; }
    }
    __syncthreads();
    if (!ok_all) {  // nothing to compute: publish an empty table
        if (tid == 0) *nseg = 0;
        return;
    }
    for (int x = tid; x < n_local; x += blockDim.x) {
        int t = 0;
        for (int s = 0; s < world; ++s) t += mine->cnt[s][me * n_local + x];
        tot[x] = t;
    }
    __syncthreads();
    if (tid == 0) {
        int run = 0, n = 0;
        for (int x = 0; x < n_local; ++x) { first[x] = run; run += tot[x]; n += tot[x] > 0 ? 1 : 0; }
        n_rows = run;
        *nseg = n;
    }
    __syncthreads();
    for (int x = tid; x < n_local; x += blockDim.x) {
        const int c = tot[x];
        if (c > 0) {
            int rank = 0;  // position in (rows descending, expert ascending) order
            for (int o = 0; o < n_local; ++o) rank += (tot[o] > c || (tot[o] == c && o < x)) ? 1 : 0;
            seg_gu[rank] = SegDesc{gate + (size_t)x * eb_g, up + (size_t)x * eb_u, (uint32_t)c, (uint32_t)first[x]};
            seg_dn[rank] = SegDesc{down + (size_t)x * eb_d, nullptr, (uint32_t)c, (uint32_t)first[x]};
        }
    }
    for (int r = tid; r < n_rows; r += blockDim.x) {
        const int v = recv_slot[r];
        row_dst[r] = peers.h_slots[v >> 24] + (size_t)(v & 0xFFFFFF) * e;
    }
}

// After the down GEMM: everything this rank stored into the owners' result rows is made
// visible, then the flag goes up at every owner.
__global__ void ep_signal_kernel(int world, int me, uint32_t seq, EpPeers peers) {
    __threadfence_system();
    if ((int)threadIdx.x < world) st_release_sys(&peers.arena[threadIdx.x]->ret_flag[me], seq);
}

__global__ void ep_wait_ret_kernel(EpArena* mine, int world, uint32_t seq, int* status, int polls) {
    if ((int)threadIdx.x < world && !wait_flag(&mine->ret_flag[threadIdx.x], seq, polls)) status_set(status, 22);
}

}  // namespace dnb

// ---- host side ---------------------------------------------------------------------------
#include "dnb200.h"

namespace dnb {

struct EpState {
    int rank = 0, world = 1, max_tokens = 0, cap = 0, rows_total = 0, n_local = 0;
    uint32_t seq = 0;
    bool connected = false;
    bool loopback = false;         // every peer pointer is the own arena (time-out test): nothing to close
    uint8_t* arena = nullptr;      // this rank's exported allocation
    size_t arena_bytes = 0;
    size_t off_slot = 0, off_hi = 0, off_lo = 0, off_h = 0;  // layout, identical on every rank
    void* peer_base[kEpMaxWorld] = {nullptr};                // every rank's arena in this process's address space
    EpPeers peers;
    // local-only buffers
    int32_t* send_row = nullptr;
    int32_t* base = nullptr;       // [ne]: where this rank's rows of each expert start at the owner
    float** row_dst = nullptr;
    uint16_t *act_hi = nullptr, *act_lo = nullptr;
    SegDesc *seg_gu = nullptr, *seg_dn = nullptr;
    int32_t* nseg = nullptr;
    unsigned int* ticket = nullptr;
    UmmaMaps maps_x, maps_act;
};

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

void ep_release(dnb_ctx* c) {
    EpState* s = static_cast<EpState*>(c->ep);
    if (!s) return;
    for (int r = 0; r < s->world; ++r)
        if (r != s->rank && s->peer_base[r] && !s->loopback) cudaIpcCloseMemHandle(s->peer_base[r]);
    void* loc[] = {s->arena, s->send_row, s->base, s->row_dst, s->act_hi, s->act_lo, s->seg_gu, s->seg_dn, s->nseg, s->ticket};
    for (void* p : loc)
        if (p) cudaFree(p);
    delete s;
    c->ep = nullptr;
}

}  // namespace dnb

using namespace dnb;

extern "C" int dnb_ep_init(dnb_ctx* c, int rank, int world, int max_tokens, void* handle_out) {
    if (!c || !handle_out || world < 1 || world > kEpMaxWorld || rank < 0 || rank >= world || max_tokens < 1)
        return DNB_ERR_ARG;
    const Model& M = c->model;
    if (M.n_layer < 1 || M.ne % world || M.shard_count != M.ne / world || M.shard_first != rank * (M.ne / world)) {
        set_error("ep_init: configure the model and call dnb_moe_set_expert_shard(rank * ne / world, ne / world) first");
        return DNB_DECLINED;
    }
    if (M.ne / world > kEpMaxLocal || M.ne > kEpMaxExperts || M.e % 256 || M.ff % 256 || M.k > 32) {
        set_error("ep_init: shape outside the peer-memory path (e, ff multiples of 256; at most %d local experts)", kEpMaxLocal);
        return DNB_DECLINED;
    }
    if ((long)max_tokens * M.k >= (1L << 24)) {
        set_error("ep_init: max_tokens * k = %ld does not fit the 24-bit row field of a receive slot", (long)max_tokens * M.k);
        return DNB_ERR_ARG;
    }
    DNB_CUDA(cudaSetDevice(c->device));
    ep_release(c);
    EpState* s = new EpState();
    c->ep = s;
    s->rank = rank; s->world = world; s->max_tokens = max_tokens; s->n_local = M.ne / world;
    s->cap = max_tokens * M.k;                 // all of a source's rows may go to one owner
    s->rows_total = world * s->cap;
    const size_t rows_pad = (size_t)s->rows_total + 128;  // a tile that starts near the end stays inside
    s->off_slot = align_up(sizeof(EpArena), 256);
    s->off_hi = align_up(s->off_slot + (size_t)s->rows_total * 4, 256);
    s->off_lo = align_up(s->off_hi + rows_pad * M.e * 2, 256);
    s->off_h = align_up(s->off_lo + rows_pad * M.e * 2, 256);
    s->arena_bytes = align_up(s->off_h + (size_t)s->cap * M.e * 4, 256);
    DNB_CUDA(cudaMalloc((void**)&s->arena, s->arena_bytes));
    DNB_CUDA(cudaMemset(s->arena, 0, s->arena_bytes));
    DNB_CUDA(cudaMalloc((void**)&s->send_row, (size_t)s->cap * 4));
    DNB_CUDA(cudaMalloc((void**)&s->base, (size_t)M.ne * 4));
    DNB_CUDA(cudaMalloc((void**)&s->row_dst, (size_t)s->rows_total * sizeof(float*)));
    DNB_CUDA(cudaMalloc((void**)&s->act_hi, rows_pad * M.ff * 2));
    DNB_CUDA(cudaMalloc((void**)&s->act_lo, rows_pad * M.ff * 2));
    DNB_CUDA(cudaMemset(s->act_hi, 0, rows_pad * M.ff * 2));
    DNB_CUDA(cudaMemset(s->act_lo, 0, rows_pad * M.ff * 2));
    DNB_CUDA(cudaMalloc((void**)&s->seg_gu, ((size_t)world * s->n_local + 1) * sizeof(SegDesc)));
    DNB_CUDA(cudaMalloc((void**)&s->seg_dn, ((size_t)world * s->n_local + 1) * sizeof(SegDesc)));
    DNB_CUDA(cudaMalloc((void**)&s->nseg, 4));
    DNB_CUDA(cudaMalloc((void**)&s->ticket, 4));
    DNB_CUDA(cudaMemset(s->ticket, 0, 4));
    if (umma_make_maps(s->arena + s->off_hi, s->arena + s->off_lo, rows_pad, (uint64_t)M.e, &s->maps_x) != DNB_OK ||
        umma_make_maps(s->act_hi, s->act_lo, rows_pad, (uint64_t)M.ff, &s->maps_act) != DNB_OK) {
        set_error("ep_init: tensor maps of the operand buffers could not be made");
        return DNB_DECLINED;
    }
    DNB_CUDA(cudaDeviceSynchronize());
    cudaIpcMemHandle_t h;
    DNB_CUDA(cudaIpcGetMemHandle(&h, s->arena));
    static_assert(sizeof(h) == 64, "cudaIpcMemHandle_t is 64 bytes");
    memcpy(handle_out, &h, sizeof(h));
    return DNB_OK;
}

extern "C" int dnb_ep_connect(dnb_ctx* c, const void* handles) {
    if (!c || !c->ep || !handles) return DNB_ERR_ARG;
    EpState* s = static_cast<EpState*>(c->ep);
    DNB_CUDA(cudaSetDevice(c->device));
    for (int r = 0; r < s->world; ++r) {
        if (r == s->rank) {
            s->peer_base[r] = s->arena;
        } else {
            cudaIpcMemHandle_t h;
            memcpy(&h, (const uint8_t*)handles + (size_t)r * 64, 64);
            DNB_CUDA(cudaIpcOpenMemHandle(&s->peer_base[r], h, cudaIpcMemLazyEnablePeerAccess));
        }
        uint8_t* b = (uint8_t*)s->peer_base[r];
        s->peers.arena[r] = (EpArena*)b;
        s->peers.recv_slot[r] = (int32_t*)(b + s->off_slot);
        s->peers.xg_hi[r] = (uint16_t*)(b + s->off_hi);
        s->peers.xg_lo[r] = (uint16_t*)(b + s->off_lo);
        s->peers.h_slots[r] = (float*)(b + s->off_h);
    }
    s->connected = true;
    return DNB_OK;
}

// Test hook: a group of `world` ranks in which only this one exists.  Every peer pointer is
// this rank's own arena, so all stores stay on this GPU, and the flags the missing ranks would
// raise never arrive: a block call then runs into its bounded waits (status 21) instead of a
// partner.  Used to check that a wait that runs out is reported and does not hang.
extern "C" int dnb_ep_connect_loopback(dnb_ctx* c) {
    if (!c || !c->ep) return DNB_ERR_ARG;
    EpState* s = static_cast<EpState*>(c->ep);
    for (int r = 0; r < s->world; ++r) {
        uint8_t* b = s->arena;
        s->peer_base[r] = s->arena;
        s->peers.arena[r] = (EpArena*)b;
        s->peers.recv_slot[r] = (int32_t*)(b + s->off_slot);
        s->peers.xg_hi[r] = (uint16_t*)(b + s->off_hi);
        s->peers.xg_lo[r] = (uint16_t*)(b + s->off_lo);
        s->peers.h_slots[r] = (float*)(b + s->off_h);
    }
    s->connected = true;
    s->loopback = true;
    return DNB_OK;
}

extern "C" int dnb_ep_block_dev(dnb_ctx* c, int layer, const float* h_dev, int nt, float* out_dev) {
    if (!c || !c->ep || !h_dev || !out_dev || nt < 1) return DNB_ERR_ARG;
    EpState* s = static_cast<EpState*>(c->ep);
    const Model& M = c->model;
    if (!s->connected || nt > s->max_tokens || layer < 0 || layer >= M.n_layer) {
        set_error("ep_block: not connected, layer out of range, or %d tokens exceed the %d the arena was sized for", nt, s->max_tokens);
        return DNB_ERR_ARG;
    }
    const Layer& L = M.layers[layer];
    for (int i = 0; i < 3; ++i)
        if (!L.m[i].dev || L.m[i].type != L.m[0].type || (L.m[i].type != T_Q4_K && L.m[i].type != T_IQ3_XXS)) {
            set_error("ep_block: the peer-memory path runs Q4_K or IQ3_XXS expert layers (tcgen05 grouped GEMMs)");
            return DNB_DECLINED;
        }
    DNB_CUDA(cudaSetDevice(c->device));
    int rc;
    // 1. route the rank's own tokens
    if ((rc = ensure_workspace(c, nt))) return rc;
    Workspace& w = c->ws;
    if ((rc = dnb_moe_route_dev(c, layer, h_dev, nt, w.xn, w.sels, w.wts))) return rc;
    cudaStream_t st = c->stream;
    const uint32_t seq = ++s->seq;
    const int words = (nt + 31) >> 5;
    const size_t plan_smem = ((size_t)M.ne * words + (size_t)M.ne) * 4;
    static SmemGrant plan_grant;
    if (plan_smem > 200 * 1024) return DNB_DECLINED;
    DNB_CUDA(grant_smem(plan_grant, c->device, ep_plan_kernel, plan_smem));
    {
        ProfScope p_(c, st, "ep_plan");
        ep_plan_kernel<<<1, 1024, plan_smem, st>>>(w.sels, nt, M.k, M.ne, s->n_local, s->world, s->rank, seq, s->peers, s->send_row);
    }
    {
        ProfScope p_(c, st, "ep_offsets");
        ep_offsets_kernel<<<1, 1024, 0, st>>>((const EpArena*)s->arena, M.ne, s->n_local, s->world, s->rank, seq, s->base, c->status, c->flag_polls);
    }
    // The dispatch stores run on the side stream, beside the shared expert of the own tokens
    // on the main one: peer stores over NVLink and a local GEMM do not compete for much.
    DNB_CUDA(cudaEventRecord(c->ev_fork, st));
    DNB_CUDA(cudaStreamWaitEvent(c->side, c->ev_fork, 0));
    {
        ProfScope p_(c, c->side, "ep_dispatch");
        const int n_rows = nt * M.k;
        const int ctas = n_rows < 4 * c->sm_count ? n_rows : 4 * c->sm_count;
        ep_dispatch_kernel<<<ctas, 256, 0, c->side>>>(w.xn, w.sels, s->send_row, s->base, M.k, M.e, s->n_local, s->world,
                                                     s->rank, s->rows_total, n_rows, seq, s->peers, s->ticket, c->status);
    }
    DNB_CUDA(cudaEventRecord(c->ev_join, c->side));
    c->launches += 3;
    DNB_CUDA(cudaGetLastError());
    // 2. the shared expert of the own tokens while the rows travel
    const bool shared = L.has_shared();
    if (shared)
        if ((rc = dnb_expert_rows_dev(c, layer, w.xn, nullptr, nt, 1, w.sh))) return rc;
    DNB_CUDA(cudaStreamWaitEvent(st, c->ev_join, 0));
    // 3. the rows this rank owns: tables, the two grouped GEMMs, results stored at the token owners
    {
        ProfScope p_(c, st, "ep_build");
        ep_build_kernel<<<1, 1024, 0, st>>>((EpArena*)s->arena, (const int32_t*)(s->arena + s->off_slot), s->world, s->n_local,
                                            s->rank, M.e, seq, s->peers, (const uint8_t*)L.m[0].dev, (const uint8_t*)L.m[1].dev,
                                            (const uint8_t*)L.m[2].dev, L.m[0].expert_bytes, L.m[1].expert_bytes,
                                            L.m[2].expert_bytes, s->seg_gu, s->seg_dn, s->nseg, s->row_dst, c->status, c->flag_polls);
    }
    c->launches++;
    DNB_CUDA(cudaGetLastError());
    const int nseg_max = s->n_local;
    if ((rc = launch_grouped_tc(c, st, L.m[0].type, true, s->seg_gu, s->nseg, nseg_max, M.e, M.ff, &s->maps_x, s->rows_total, s->act_hi,
                                s->act_lo, nullptr)))
        return rc;
    if ((rc = launch_grouped_tc(c, st, L.m[0].type, false, s->seg_dn, s->nseg, nseg_max, M.ff, M.e, &s->maps_act, s->rows_total, nullptr,
                                nullptr, nullptr, s->row_dst)))
        return rc;
    {
        ProfScope p_(c, st, "ep_signal_wait");
        ep_signal_kernel<<<1, 32, 0, st>>>(s->world, s->rank, seq, s->peers);
        ep_wait_ret_kernel<<<1, 32, 0, st>>>((EpArena*)s->arena, s->world, seq, c->status, c->flag_polls);
    }
    c->launches += 2;
    DNB_CUDA(cudaGetLastError());
    // 4. weighted sum in ascending slot order, as on one GPU
    const float* coef = nullptr;
    if (shared && L.shared_gate_row) {
        if ((rc = launch_shared_coef(c, st, w.xn, L.shared_gate_row, nt, M.e, w.shcoef))) return rc;
        coef = w.shcoef;
    }
    return launch_combine(c, st, (const float*)(s->arena + s->off_h), nullptr, w.wts, nt, M.k, M.e, shared ? w.sh : nullptr, coef,
                          out_dev);
}

// All configured layers with identity mixers for this rank's nt tokens: h <- h + block_l(h), in place
// (the expert-parallel form of dnb_moe_stack_dev; the residual add is the same separate-rounding add).
extern "C" int dnb_ep_stack_dev(dnb_ctx* c, float* h_dev, int nt) {
    if (!c || !c->ep || !h_dev || nt < 1) return DNB_ERR_ARG;
    const Model& M = c->model;
    int rc = ensure_workspace(c, nt);
    if (rc) return rc;
    for (int l = 0; l < M.n_layer; ++l) {
        if ((rc = dnb_ep_block_dev(c, l, h_dev, nt, c->ws.out))) return rc;
        if ((rc = launch_add_inplace(c, c->stream, h_dev, c->ws.out, (size_t)nt * M.e))) return rc;
    }
    return DNB_OK;
}
