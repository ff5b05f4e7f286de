// Allocation-free variant of the routing-count kernels; see noalloc.h for the contract.
#include "noalloc.h"

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <mutex>

namespace {

constexpr int kChunkTokens = 128;
constexpr int kMaxChunks = 512;    // 65536 tokens
constexpr int kMaxCols = 1088;     // E + N + 2
constexpr int kMaxDevices = 64;

// Per-chunk histograms.  File scope, so it exists once per device that loads this library.
static __device__ __align__(256) int g_chunk_hist[kMaxChunks * kMaxCols];

__device__ __forceinline__ long long load_idx(const void* idx, int is64, long i) {
    return is64 ? reinterpret_cast<const long long*>(idx)[i] : (long long) reinterpret_cast<const int*>(idx)[i];
}

// One block per 128-token chunk: histogram in shared memory, then the whole row is written out, so
// no column of a row that the sum kernel reads is left over from an earlier call.
__global__ void __launch_bounds__(kChunkTokens)
noalloc_hist_kernel(const void* topk_idx, int is64, int T, int K, int E, int N, int* chunk_hist) {
    extern __shared__ int sh[];
    const int C = E + N + 2;
    const int e_local = E / N;
    for (int i = threadIdx.x; i < C; i += blockDim.x) sh[i] = 0;
    __syncthreads();
    const int t = blockIdx.x * kChunkTokens + threadIdx.x;
    if (t < T) {
        unsigned mask = 0;
        for (int k = 0; k < K; ++k) {
            const long long e = load_idx(topk_idx, is64, (long)t * K + k);
            if (e >= 0 && e < E) {
                atomicAdd(&sh[(int)e], 1);
                mask |= 1u << ((int)e / e_local);
            }
        }
        for (int d = 0; d < N; ++d)
            if (mask >> d & 1u) atomicAdd(&sh[E + d], 1);
        atomicAdd(&sh[E + N], __popc(mask));
        atomicAdd(&sh[E + N + 1], 1);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < C; i += blockDim.x) chunk_hist[(long)blockIdx.x * C + i] = sh[i];
}

__global__ void __launch_bounds__(256) noalloc_sum_kernel(const int* chunk_hist, int num_chunks, int C, int* counts_out) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    int s = 0;
    for (int ch = 0; ch < num_chunks; ++ch) s += chunk_hist[(long)ch * C + c];
    counts_out[c] = s;
}

std::mutex g_mutex;
int* g_scratch_dev[kMaxDevices] = {nullptr};

int fail(int code, char* err, size_t err_len, const char* msg) {
    if (err != nullptr && err_len > 0) snprintf(err, err_len, "%s", msg);
    return code;
}

}  // namespace

extern "C" __attribute__((visibility("default"))) int tmoe_route_counts_noalloc(const void* topk_idx, int idx_is_64bit, int num_tokens,
                                                                                 int top_k, int num_experts, int num_ranks,
                                                                                 int* counts_out, void* stream, char* err,
                                                                                 size_t err_len) {
    if (topk_idx == nullptr && num_tokens > 0) return fail(TMOE_NOALLOC_BAD_ARGUMENT, err, err_len, "topk_idx is null");
    if (counts_out == nullptr) return fail(TMOE_NOALLOC_BAD_ARGUMENT, err, err_len, "counts_out is null");
    if (num_tokens < 0 || top_k <= 0 || num_experts <= 0 || num_ranks <= 0 || num_experts % num_ranks != 0)
        return fail(TMOE_NOALLOC_BAD_ARGUMENT, err, err_len, "need T >= 0, K > 0, E > 0, N > 0 and E divisible by N");
    const int C = num_experts + num_ranks + 2;
    // compare the token count itself: rounding it up to chunks first could overflow an int near INT_MAX
    if (num_tokens > kMaxChunks * kChunkTokens || C > kMaxCols || top_k > 32 || num_ranks > 32) {
        char msg[200];
        snprintf(msg, sizeof(msg), "size beyond the built-in scratch: limits are T <= %d, K <= 32, N <= 32, E + N + 2 <= %d (got T=%d K=%d N=%d E=%d)",
                 kMaxChunks * kChunkTokens, kMaxCols, num_tokens, top_k, num_ranks, num_experts);
        return fail(TMOE_NOALLOC_TOO_LARGE, err, err_len, msg);
    }
    const int chunks = (num_tokens + kChunkTokens - 1) / kChunkTokens;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(TMOE_NOALLOC_CUDA_ERROR, err, err_len, cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return fail(TMOE_NOALLOC_BAD_ARGUMENT, err, err_len, "device index out of range");
    int* scratch = nullptr;
    {
        // First call on this device: resolve the device address of the scratch array.  In host code the
        // array's name is only a stand-in; a kernel must be given the address looked up here.
        std::lock_guard<std::mutex> lock(g_mutex);
        if (g_scratch_dev[dev] == nullptr) {
            int* p = nullptr;
            e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_chunk_hist);
            if (e != cudaSuccess || p == nullptr)
                return fail(TMOE_NOALLOC_CUDA_ERROR, err, err_len, e != cudaSuccess ? cudaGetErrorString(e) : "scratch symbol has no address");
            g_scratch_dev[dev] = p;
        }
        scratch = g_scratch_dev[dev];
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (chunks > 0) {
        noalloc_hist_kernel<<<chunks, kChunkTokens, C * sizeof(int), s>>>(topk_idx, idx_is_64bit, num_tokens, top_k, num_experts, num_ranks,
                                                                          scratch);
        e = cudaGetLastError();
        if (e != cudaSuccess) return fail(TMOE_NOALLOC_CUDA_ERROR, err, err_len, cudaGetErrorString(e));
    }
    noalloc_sum_kernel<<<(C + 255) / 256, 256, 0, s>>>(scratch, chunks, C, counts_out);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(TMOE_NOALLOC_CUDA_ERROR, err, err_len, cudaGetErrorString(e));
    return TMOE_NOALLOC_OK;
}
