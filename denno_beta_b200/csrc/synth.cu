// Device-side fills from the seeded generator of dnb_synth.h, so that expert
// tables of tens of GB can be created in HBM without staging through the host.
#include "dnb_common.cuh"
#include "dnb_synth.h"

namespace dnb {

// word0 / byte0 / block0: where `dst` starts inside the whole tensor (a rank's shard of an expert
// tensor is generated with the indices of the full tensor, so every rank holds the same bytes a
// single GPU would).
__global__ void synth_payload_kernel(uint64_t key, uint64_t* dst, uint64_t n_words, uint64_t word0) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n_words) dst[i] = dnb_synth_draw(key, word0 + i);
}

__global__ void synth_tail_kernel(uint64_t key, uint8_t* dst, uint64_t first, uint64_t bytes, uint64_t byte0) {
    const uint64_t j = first + threadIdx.x;
    if (j < bytes) dst[j] = dnb_synth_byte(key, byte0 + j);
}

__global__ void synth_fix_kernel(int type, uint64_t key, uint8_t* dst, uint64_t n_blocks, int ts, uint64_t block0) {
    const uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b < n_blocks) dnb_synth_fix_block(type, key, block0 + b, dst + b * ts);
}

__global__ void synth_normal_kernel(uint64_t key, float sigma, float* dst, uint64_t n) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = (float)(dnb_synth_normal(key, i) * (double)sigma);
}

__global__ void fill_u32_kernel(uint32_t* dst, uint32_t v, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = v;
}

int launch_synth_blocks(dnb_ctx* c, cudaStream_t st, int type, uint64_t seed, uint64_t tensor_id, uint8_t* dst,
                        uint64_t n_blocks, uint64_t first_block) {
    const int ts = dnb_synth_type_size(type);
    if (ts == 0 || ((uintptr_t)dst & 7)) {
        set_error("synth: unsupported type %d or unaligned destination", type);
        return DNB_ERR_ARG;
    }
    const uint64_t key = dnb_synth_key(seed, tensor_id);
    const uint64_t bytes = n_blocks * (uint64_t)ts;
    const uint64_t words = bytes / 8;
    const uint64_t byte0 = first_block * (uint64_t)ts;
    if (byte0 % 8) {
        set_error("synth: the shard starts at byte %llu of the tensor, not on an 8-byte word", (unsigned long long)byte0);
        return DNB_ERR_ARG;
    }
    if (words) synth_payload_kernel<<<(unsigned)((words + 255) / 256), 256, 0, st>>>(key, (uint64_t*)dst, words, byte0 / 8);
    if (bytes % 8) synth_tail_kernel<<<1, 8, 0, st>>>(key, dst, words * 8, bytes, byte0);
    synth_fix_kernel<<<(unsigned)((n_blocks + 255) / 256), 256, 0, st>>>(type, key, dst, n_blocks, ts, first_block);
    c->launches += 2;
    DNB_CUDA(cudaGetLastError());
    return DNB_OK;
}

int launch_synth_normal(dnb_ctx* c, cudaStream_t st, uint64_t seed, uint64_t tensor_id, float sigma, float* dst,
                        uint64_t n) {
    const uint64_t key = dnb_synth_key(seed, tensor_id);
    synth_normal_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(key, sigma, dst, n);
    c->launches++;
    DNB_CUDA(cudaGetLastError());
    return DNB_OK;
}

// Keeps the stream busy for about `ms` milliseconds (bounded by the clock, it
// always ends): work enqueued behind it then runs back to back, which is how the
// per-kernel timing pass removes host launch gaps from its event intervals.
__global__ void stall_kernel(long long cycles) {
    const long long t0 = clock64();
    while (clock64() - t0 < cycles) {
    }
}

int launch_stall(dnb_ctx* c, cudaStream_t st, float ms) {
    if (ms < 0.f) ms = 0.f;
    if (ms > 200.f) ms = 200.f;
    int khz = 1900000;
    cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, c->device);
    stall_kernel<<<1, 1, 0, st>>>((long long)((double)ms * (double)khz));
    c->launches++;
    DNB_CUDA(cudaGetLastError());
    return DNB_OK;
}

int launch_fill_u32(dnb_ctx* c, cudaStream_t st, uint32_t* dst, uint32_t v, size_t n) {
    fill_u32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(dst, v, n);
    c->launches++;
    DNB_CUDA(cudaGetLastError());
    return DNB_OK;
}

}  // namespace dnb
