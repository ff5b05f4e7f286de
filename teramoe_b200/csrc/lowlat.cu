// Low-latency dispatch / combine kernels; see lowlat.h for the protocol and the reference counterparts.
//
//   ll_dispatch_send  one block per GLOBAL expert: finds this rank's tokens for the expert in token order (so slots are
//                     deterministic, no atomics), casts each token in flight (bf16 -> e4m3 with one scale per 128
//                     channels, optionally power-of-two / UE8M0 scales), stores the message into its window on the
//                     expert's rank and finally publishes the window's row count with one release store.
//   ll_dispatch_recv  per local expert: waits (bounded) for every source's count, packs the windows back to back,
//                     writes the scales column-major, the source token of every row, the per-source ranges and counts;
//                     adds the wait time per source and the received rows per expert to the caller's statistics.
//   ll_combine_send   one block per (local expert, source rank): sends that source's rows home, plain bf16 or LogFMT-10
//                     (sign + 9-bit logarithmic code per value where a 128-channel group qualifies), then one flag.
//   ll_combine_recv   one warp per token: waits for the flags of its experts, decodes and forms the weighted sum.
//
// A wait that runs out either reports through the status block or, in shrink mode, masks the silent rank; masked ranks
// are neither written to nor waited for.  No kernel here traps or spins without a limit.
#include "lowlat.h"

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "ptx.cuh"

namespace tmoe {

namespace {

constexpr int kSendThreads = 256;
constexpr int kRecvSplit = 4;
constexpr float kFp8Max = 448.f;
constexpr float kFp8Margin = 1e-4f;

__device__ __forceinline__ long long ld_acquire_sys_b64(const long long* p) {
    long long v;
    asm volatile("ld.acquire.sys.global.b64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys_b64(long long* p, long long v) {
    asm volatile("st.release.sys.global.b64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ long long load_idx(const void* idx, int is64, long i) {
    return is64 ? reinterpret_cast<const long long*>(idx)[i] : (long long) reinterpret_cast<const int*>(idx)[i];
}

// Wait until the flag carries this call's number.  Returns the low word, or -1 when the wait ran out (then either the
// rank gets masked or the status block gets the report) or the rank is masked already.
__device__ __forceinline__ int wait_call_flag(const long long* flag, long long call_seq, int src, int* mask, int shrink, uint64_t limit_ns,
                                              int* status, int site, unsigned long long* waited_ns) {
    if (mask != nullptr && mask[src] != 0) return -1;
    const uint64_t t0 = globaltimer_ns();
    long long v = ld_acquire_sys_b64(flag);
    while ((v >> 32) != call_seq) {
        if (globaltimer_ns() - t0 > limit_ns) {
            if (shrink && mask != nullptr) atomicExch(mask + src, 1);
            else report_status(status, kStatusFlagTimeout, site, src);
            if (waited_ns != nullptr) *waited_ns = globaltimer_ns() - t0;
            return -1;
        }
        if (!shrink && status != nullptr && ld_relaxed_sys(status) != 0) return -1;      // someone else already gave up
        __nanosleep(100);
        v = ld_acquire_sys_b64(flag);
    }
    if (waited_ns != nullptr) *waited_ns = globaltimer_ns() - t0;
    return (int)(v & 0xffffffffll);
}

// scale (what the receiver multiplies by) for a 128-channel group with the given amax
__device__ __forceinline__ float fp8_scale(float amax, int round_scale) {
    float s = amax / kFp8Max;
    if (round_scale) {
        // 2^ceil(log2 s): exact on the bit pattern
        const uint32_t bits = __float_as_uint(s);
        const int e = (int)((bits >> 23) & 0xff) - 127 + ((bits & 0x7fffffu) != 0u ? 1 : 0);
        s = __uint_as_float((uint32_t)(e + 127) << 23);
    }
    return s;
}

__global__ void __launch_bounds__(kSendThreads)
ll_dispatch_send_kernel(LowLatLayout lay, const __nv_bfloat16* x, const void* topk_idx, int is64, int T, int K, const uint64_t* arena_ptrs,
                        long long call_seq, const int* mask) {
    extern __shared__ int list[];                  // tokens of this rank for the block's expert, in token order
    __shared__ int warp_cnt[kSendThreads / 32];
    __shared__ int base;
    const int e = blockIdx.x;
    const int El = lay.num_experts / lay.num_ranks;
    const int d = e / El, le = e - d * El;
    if (mask != nullptr && mask[d] != 0) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) base = 0;
    __syncthreads();
    const int entries = T * K;
    for (int start = 0; start < entries; start += kSendThreads) {
        const int i = start + tid;
        const bool match = i < entries && load_idx(topk_idx, is64, i) == (long long)e;
        const uint32_t b = __ballot_sync(0xffffffffu, match);
        if (lane == 0) warp_cnt[warp] = __popc(b);
        __syncthreads();
        int off = base;
        for (int w2 = 0; w2 < warp; ++w2) off += warp_cnt[w2];
        if (match) {
            const int pos = off + __popc(b & ((1u << lane) - 1u));
            if (pos < lay.max_tokens) list[pos] = i / K;
        }
        __syncthreads();
        if (tid == 0) {
            int tot = 0;
            for (int w2 = 0; w2 < kSendThreads / 32; ++w2) tot += warp_cnt[w2];
            base += tot;
        }
        __syncthreads();
    }
    const int count = min(base, lay.max_tokens);
    const int H = lay.hidden;
    uint8_t* window = reinterpret_cast<uint8_t*>(arena_ptrs[d] + lay.off_d_stage) +
                      ((size_t)(le * lay.num_ranks + lay.rank) * lay.max_tokens) * lay.d_msg_bytes;
    for (int j = warp; j < count; j += kSendThreads / 32) {
        const int t = list[j];
        uint8_t* msg = window + (size_t)j * lay.d_msg_bytes;
        if (lane == 0) *reinterpret_cast<int4*>(msg) = make_int4(t, 0, 0, 0);
        const __nv_bfloat16* row = x + (size_t)t * H;
        if (lay.use_fp8) {
            uint32_t* payload = reinterpret_cast<uint32_t*>(msg + 16);
            uint8_t* scales = msg + 16 + H;
            for (int g = 0; g < H / 128; ++g) {
                const uint2 raw = *reinterpret_cast<const uint2*>(row + g * 128 + lane * 4);
                const float2 v01 = unpack_bf16x2(raw.x), v23 = unpack_bf16x2(raw.y);
                float amax = fmaxf(fmaxf(fabsf(v01.x), fabsf(v01.y)), fmaxf(fabsf(v23.x), fabsf(v23.y)));
                for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                amax = fmaxf(amax, kFp8Margin);
                const float s = fp8_scale(amax, lay.round_scale);
                const float q[4] = {fminf(fmaxf(__fdiv_rn(v01.x, s), -kFp8Max), kFp8Max), fminf(fmaxf(__fdiv_rn(v01.y, s), -kFp8Max), kFp8Max),
                                    fminf(fmaxf(__fdiv_rn(v23.x, s), -kFp8Max), kFp8Max), fminf(fmaxf(__fdiv_rn(v23.y, s), -kFp8Max), kFp8Max)};
                uint32_t word = 0;
#pragma unroll
                for (int c = 0; c < 4; ++c) word |= (uint32_t)__nv_cvt_float_to_fp8(q[c], __NV_SATFINITE, __NV_E4M3) << (8 * c);
                payload[g * 32 + lane] = word;
                if (lane == 0) {
                    if (lay.use_ue8m0) scales[g] = (uint8_t)(__float_as_uint(s) >> 23);
                    else reinterpret_cast<float*>(scales)[g] = s;
                }
            }
        } else {
            int4* dst = reinterpret_cast<int4*>(msg + 16);
            const int4* src = reinterpret_cast<const int4*>(row);
            for (int i = lane; i < H / 8; i += 32) st_na_v4(dst + i, src[i]);
        }
    }
    __syncthreads();
    if (tid == 0) {
        __threadfence_system();
        long long* flag = reinterpret_cast<long long*>(arena_ptrs[d] + lay.off_d_flags) + (le * lay.num_ranks + lay.rank);
        st_release_sys_b64(flag, (call_seq << 32) | (long long)(count + 1));
    }
}

__global__ void __launch_bounds__(256)
ll_dispatch_recv_kernel(LowLatLayout lay, const uint8_t* arena, uint8_t* recv_x, uint8_t* recv_scales, int* src_info, long long* layout_range,
                        int* recv_count, int* expert_stats, long long* wait_stats, long long call_seq, int* mask, int shrink, uint64_t limit_ns,
                        int* status) {
    __shared__ int cnt[32];
    __shared__ int beg[33];
    const int le = blockIdx.x / kRecvSplit, part = blockIdx.x % kRecvSplit;
    const int N = lay.num_ranks, M = lay.max_tokens, H = lay.hidden;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid < N) {
        unsigned long long waited = 0;
        const long long* flag = reinterpret_cast<const long long*>(arena + lay.off_d_flags) + (le * N + tid);
        const int v = wait_call_flag(flag, call_seq, tid, mask, shrink, limit_ns, status, 700 + tid, &waited);
        cnt[tid] = v > 0 ? min(v - 1, M) : 0;
        if (part == 0 && le == 0 && wait_stats != nullptr) atomicAdd(reinterpret_cast<unsigned long long*>(wait_stats) + tid, waited);
    }
    __syncthreads();
    if (tid == 0) {
        int run = 0;
        for (int s = 0; s < N; ++s) {
            beg[s] = run;
            run += cnt[s];
        }
        beg[N] = run;
        if (part == 0) {
            recv_count[le] = run;
            if (expert_stats != nullptr) atomicAdd(expert_stats + le, run);
        }
    }
    __syncthreads();
    if (part == 0 && tid < N) layout_range[le * N + tid] = ((long long)cnt[tid] << 32) | (long long)beg[tid];
    const int total = beg[N];
    const long NM = (long)N * M;
    const int G = H / 128;
    for (int r = part * 8 + warp; r < total; r += kRecvSplit * 8) {
        int s = 0;
        while (s + 1 < N && r >= beg[s + 1]) ++s;
        const uint8_t* msg = arena + lay.off_d_stage + ((size_t)(le * N + s) * M + (r - beg[s])) * lay.d_msg_bytes;
        const long out_row = (long)le * NM + r;
        if (lane == 0) src_info[out_row] = __ldcg(reinterpret_cast<const int*>(msg));
        if (lay.use_fp8) {
            const int4* src = reinterpret_cast<const int4*>(msg + 16);
            int4* dst = reinterpret_cast<int4*>(recv_x + out_row * H);
            for (int i = lane; i < H / 16; i += 32) dst[i] = __ldcg(src + i);
            // scales of expert le: [G (or G/4 words), ranks*max_tokens], i.e. column-major, as the reference hands them out
            if (lay.use_ue8m0) {
                const uint32_t* sw = reinterpret_cast<const uint32_t*>(msg + 16 + H);
                uint32_t* so = reinterpret_cast<uint32_t*>(recv_scales);
                for (int g = lane; g < G / 4; g += 32) so[((long)le * (G / 4) + g) * NM + r] = __ldcg(sw + g);
            } else {
                const float* sf = reinterpret_cast<const float*>(msg + 16 + H);
                float* so = reinterpret_cast<float*>(recv_scales);
                for (int g = lane; g < G; g += 32) so[((long)le * G + g) * NM + r] = __ldcg(sf + g);
            }
        } else {
            const int4* src = reinterpret_cast<const int4*>(msg + 16);
            int4* dst = reinterpret_cast<int4*>(recv_x + out_row * H * 2);
            for (int i = lane; i < H / 8; i += 32) dst[i] = __ldcg(src + i);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// LogFMT-10 (reference: csrc/kernels/internode_ll.cu:557-713).  A group is 128 channels, handled by 16 lanes with 8
// channels each.  If log2(amax) < 0 and the group has a range, every value becomes a sign bit and a 9-bit code of
// log2|x| on a grid of 510 steps between max(log2 amin, log2 amax - 32) and log2 amax (code 0 = zero); 8 values pack into
// 80 bits.  Otherwise the group travels as plain bf16.  Header: two floats (amax, amin; amax == 0 marks a plain group).
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void logfmt_params(float amax, float amin, float& log_amin, float& step, bool& use) {
    const float log_amax = log2f(fmaxf(amax, 1e-38f));
    log_amin = fmaxf(log2f(fmaxf(amin, 1e-38f)), log_amax - 32.f);
    use = (log_amax < 0.f) && (log_amin < log_amax) && isfinite(amin);
    step = (log_amax - log_amin) / 510.f;
}

// 16 lanes (half a warp) encode one group: lane j of the half holds channels 8j .. 8j+7 in v[8]
__device__ __forceinline__ void logfmt_encode_group(const float (&v)[8], uint8_t* group, int j) {
    float amax = 0.f, amin = INFINITY;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        const float a = fabsf(v[c]);
        amax = fmaxf(amax, a);
        if (a > 0.f) amin = fminf(amin, a);
    }
    for (int o = 8; o > 0; o >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        amin = fminf(amin, __shfl_xor_sync(0xffffffffu, amin, o));
    }
    float log_amin, step;
    bool use;
    logfmt_params(amax, amin, log_amin, step, use);
    if (j == 0) *reinterpret_cast<float2*>(group) = make_float2(use ? amax : 0.f, amin);
    if (!use) {
        uint4 raw;
        raw.x = pack_bf16x2(v[0], v[1]); raw.y = pack_bf16x2(v[2], v[3]); raw.z = pack_bf16x2(v[4], v[5]); raw.w = pack_bf16x2(v[6], v[7]);
        *reinterpret_cast<uint4*>(group + 16 + j * 16) = raw;
        return;
    }
    const float inv_step = 1.f / fmaxf(step, 1e-30f);
    unsigned long long lo = 0;      // bits 0..63 of the 80
    uint32_t hi = 0;                // bits 64..79
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        const float a = fabsf(v[c]);
        uint32_t code = 0;
        if (a > 0.f) {
            const float f = floorf((log2f(fmaxf(a, 1e-38f)) - log_amin) * inv_step + 0.5f) + 1.f;
            code = (uint32_t)fminf(fmaxf(f, 1.f), 511.f);
            if (v[c] < 0.f) code |= 512u;
        }
        const int bit = 10 * c;
        if (bit < 64) lo |= (unsigned long long)code << bit;
        if (bit + 10 > 64) hi |= bit >= 64 ? code << (bit - 64) : code >> (64 - bit);
    }
    uint16_t* out = reinterpret_cast<uint16_t*>(group + 16 + j * 10);
    out[0] = (uint16_t)lo; out[1] = (uint16_t)(lo >> 16); out[2] = (uint16_t)(lo >> 32); out[3] = (uint16_t)(lo >> 48); out[4] = (uint16_t)hi;
}

__device__ __forceinline__ void logfmt_decode_group(const uint8_t* group, int j, float (&v)[8]) {
    const float2 hdr = __ldcg(reinterpret_cast<const float2*>(group));
    if (hdr.x == 0.f) {
        const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(group + 16 + j * 16));
        const float2 a = unpack_bf16x2(raw.x), b = unpack_bf16x2(raw.y), c = unpack_bf16x2(raw.z), d = unpack_bf16x2(raw.w);
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
        return;
    }
    float log_amin, step;
    bool use;
    logfmt_params(hdr.x, hdr.y, log_amin, step, use);
    const uint16_t* in = reinterpret_cast<const uint16_t*>(group + 16 + j * 10);
    const unsigned long long lo = (unsigned long long)__ldcg(in) | ((unsigned long long)__ldcg(in + 1) << 16) |
                                  ((unsigned long long)__ldcg(in + 2) << 32) | ((unsigned long long)__ldcg(in + 3) << 48);
    const uint32_t hi = __ldcg(in + 4);
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        const int bit = 10 * c;
        uint32_t code = bit < 64 ? (uint32_t)(lo >> bit) : 0u;
        if (bit + 10 > 64) code |= bit >= 64 ? hi >> (bit - 64) : hi << (64 - bit);
        code &= 1023u;
        const uint32_t mag = code & 511u;
        const float a = mag == 0u ? 0.f : exp2f((float)(mag - 1u) * step + log_amin);
        v[c] = (code & 512u) ? -a : a;
    }
}

__global__ void __launch_bounds__(256)
ll_combine_send_kernel(LowLatLayout lay, const __nv_bfloat16* x, const int* src_info, const long long* layout_range, const uint64_t* arena_ptrs,
                       long long call_seq, const int* mask) {
    const int N = lay.num_ranks, M = lay.max_tokens, H = lay.hidden;
    const int El = lay.num_experts / N;
    const int le = blockIdx.x / N, s = blockIdx.x % N;
    if (mask != nullptr && mask[s] != 0) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const long long range = layout_range[le * N + s];
    const int count = (int)(range >> 32), begin = (int)(range & 0xffffffffll);
    const int ge = lay.rank * El + le;
    uint8_t* window = reinterpret_cast<uint8_t*>(arena_ptrs[s] + lay.off_c_stage) + (size_t)ge * M * lay.c_row_bytes;
    const long NM = (long)N * M;
    for (int i = warp; i < count; i += 8) {
        const long in_row = (long)le * NM + begin + i;
        const int t = src_info[in_row];
        if (t < 0 || t >= M) continue;                 // never store outside the window
        const __nv_bfloat16* row = x + in_row * H;
        uint8_t* dst = window + (size_t)t * lay.c_row_bytes;
        if (!lay.use_logfmt) {
            const int4* src = reinterpret_cast<const int4*>(row);
            int4* d4 = reinterpret_cast<int4*>(dst);
            for (int c = lane; c < H / 8; c += 32) st_na_v4(d4 + c, src[c]);
        } else {
            // a warp covers two groups (256 channels) per step, lanes 0-15 the first and 16-31 the second (hidden % 256 == 0)
            for (int c0 = 0; c0 < H; c0 += 256) {
                const int g = c0 / 128 + (lane >> 4), j = lane & 15;
                const uint4 raw = *reinterpret_cast<const uint4*>(row + g * 128 + j * 8);
                const float2 a = unpack_bf16x2(raw.x), b = unpack_bf16x2(raw.y), c = unpack_bf16x2(raw.z), d = unpack_bf16x2(raw.w);
                const float v[8] = {a.x, a.y, b.x, b.y, c.x, c.y, d.x, d.y};
                logfmt_encode_group(v, dst + (size_t)g * kLogfmtGroupBytes, j);
            }
        }
    }
    __syncthreads();
    if (tid == 0) {
        __threadfence_system();
        long long* flag = reinterpret_cast<long long*>(arena_ptrs[s] + lay.off_c_flags) + ge;
        st_release_sys_b64(flag, (call_seq << 32) | 1ll);
    }
}

__global__ void __launch_bounds__(256)
ll_combine_recv_kernel(LowLatLayout lay, const uint8_t* arena, const void* topk_idx, int is64, const float* topk_w, int T, int K,
                       __nv_bfloat16* out, long long* wait_stats, long long call_seq, int* mask, int shrink, uint64_t limit_ns, int* status) {
    const int lane = threadIdx.x & 31;
    const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (t >= T) return;
    const int N = lay.num_ranks, M = lay.max_tokens, H = lay.hidden;
    const int El = lay.num_experts / N;
    long long e = -1;
    float w = 0.f;
    if (lane < K) {
        e = load_idx(topk_idx, is64, (long)t * K + lane);
        if (e < 0 || e >= lay.num_experts) e = -1;
        else w = topk_w[(long)t * K + lane];
    }
    // every lane with an entry waits for its expert's flag (each expert's rank sets one flag per token owner)
    bool okk = e >= 0;
    if (e >= 0) {
        unsigned long long waited = 0;
        const int src = (int)e / El;
        const long long* flag = reinterpret_cast<const long long*>(arena + lay.off_c_flags) + e;
        okk = wait_call_flag(flag, call_seq, src, mask, shrink, limit_ns, status, 750 + src, &waited) > 0;
        if (wait_stats != nullptr && waited > 0) atomicAdd(reinterpret_cast<unsigned long long*>(wait_stats) + src, waited);
    }
    const uint32_t valid = __ballot_sync(0xffffffffu, okk);
    const uint8_t* stage = arena + lay.off_c_stage;
    for (int c0 = 0; c0 < H; c0 += 256) {
        const int col = c0 + lane * 8;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (uint32_t m = valid; m != 0; m &= m - 1) {
            const int k = __ffs(m) - 1;
            const long long ek = __shfl_sync(0xffffffffu, e, k);
            const float wk = __shfl_sync(0xffffffffu, w, k);
            const uint8_t* row = stage + ((size_t)ek * M + t) * lay.c_row_bytes;
            float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (col < H) {
                if (!lay.use_logfmt) {
                    const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(row + (size_t)col * 2));
                    const float2 a = unpack_bf16x2(raw.x), b = unpack_bf16x2(raw.y), c = unpack_bf16x2(raw.z), d = unpack_bf16x2(raw.w);
                    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
                } else {
                    logfmt_decode_group(row + (size_t)(col / 128) * kLogfmtGroupBytes, lane & 15, v);
                }
            }
#pragma unroll
            for (int c = 0; c < 8; ++c) acc[c] += wk * v[c];
        }
        if (col < H) {
            uint4 o;
            o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]); o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
            *reinterpret_cast<uint4*>(out + (size_t)t * H + col) = o;
        }
    }
}

__global__ void ll_mask_update_kernel(int* mask, int num_ranks, int rank, int value) {
    if (threadIdx.x == 0 && rank >= 0 && rank < num_ranks) atomicExch(mask + rank, value);
}
__global__ void ll_mask_query_kernel(const int* mask, int num_ranks, int* out) {
    if ((int)threadIdx.x < num_ranks) out[threadIdx.x] = mask[threadIdx.x];
}
__global__ void ll_mask_clean_kernel(int* mask, int num_ranks) {
    if ((int)threadIdx.x < num_ranks) mask[threadIdx.x] = 0;
}

bool layout_ok(const LowLatLayout& lay) {
    return lay.num_ranks >= 1 && lay.num_ranks <= 32 && lay.num_experts % lay.num_ranks == 0 && lay.hidden % 256 == 0 && lay.max_tokens > 0 &&
           lay.d_msg_bytes % 16 == 0 && lay.c_row_bytes % 16 == 0 && (!lay.use_ue8m0 || (lay.use_fp8 && lay.hidden % 512 == 0));
}

}  // namespace

cudaError_t ll_dispatch_send(const LowLatLayout& lay, const void* x, const void* topk_idx, int idx_is64, int T, int K, const uint64_t* arena_ptrs,
                             long long call_seq, const int* mask, cudaStream_t stream) {
    if (!layout_ok(lay) || T > lay.max_tokens || K > 32) return cudaErrorInvalidValue;
    const size_t smem = (size_t)lay.max_tokens * sizeof(int);
    if (smem > 48 * 1024) return cudaErrorInvalidValue;      // at most 12288 tokens per rank and call
    ll_dispatch_send_kernel<<<lay.num_experts, kSendThreads, smem, stream>>>(lay, static_cast<const __nv_bfloat16*>(x), topk_idx, idx_is64, T, K,
                                                                           arena_ptrs, call_seq, mask);
    return cudaGetLastError();
}

cudaError_t ll_dispatch_recv(const LowLatLayout& lay, const void* arena_local, void* recv_x, void* recv_scales, int* src_info,
                             long long* layout_range, int* recv_count, int* expert_stats, long long* wait_stats, long long call_seq, int* mask,
                             int shrink, uint64_t limit_ns, int* status, cudaStream_t stream) {
    if (!layout_ok(lay)) return cudaErrorInvalidValue;
    const int El = lay.num_experts / lay.num_ranks;
    ll_dispatch_recv_kernel<<<El * kRecvSplit, 256, 0, stream>>>(lay, static_cast<const uint8_t*>(arena_local), static_cast<uint8_t*>(recv_x),
                                                                static_cast<uint8_t*>(recv_scales), src_info, layout_range, recv_count,
                                                                expert_stats, wait_stats, call_seq, mask, shrink, limit_ns, status);
    return cudaGetLastError();
}

cudaError_t ll_combine_send(const LowLatLayout& lay, const void* x, const int* src_info, const long long* layout_range,
                            const uint64_t* arena_ptrs, long long call_seq, const int* mask, cudaStream_t stream) {
    if (!layout_ok(lay)) return cudaErrorInvalidValue;
    const int El = lay.num_experts / lay.num_ranks;
    ll_combine_send_kernel<<<El * lay.num_ranks, 256, 0, stream>>>(lay, static_cast<const __nv_bfloat16*>(x), src_info, layout_range, arena_ptrs,
                                                                  call_seq, mask);
    return cudaGetLastError();
}

cudaError_t ll_combine_recv(const LowLatLayout& lay, const void* arena_local, const void* topk_idx, int idx_is64, const float* topk_weights, int T,
                            int K, void* out, long long* wait_stats, long long call_seq, int* mask, int shrink, uint64_t limit_ns, int* status,
                            cudaStream_t stream) {
    if (!layout_ok(lay) || T > lay.max_tokens || K > 32) return cudaErrorInvalidValue;
    if (T == 0) return cudaSuccess;
    ll_combine_recv_kernel<<<(T + 7) / 8, 256, 0, stream>>>(lay, static_cast<const uint8_t*>(arena_local), topk_idx, idx_is64, topk_weights, T, K,
                                                           static_cast<__nv_bfloat16*>(out), wait_stats, call_seq, mask, shrink, limit_ns, status);
    return cudaGetLastError();
}

cudaError_t ll_mask_update(int* mask, int num_ranks, int rank, int value, cudaStream_t stream) {
    ll_mask_update_kernel<<<1, 32, 0, stream>>>(mask, num_ranks, rank, value);
    return cudaGetLastError();
}
cudaError_t ll_mask_query(const int* mask, int num_ranks, int* out, cudaStream_t stream) {
    ll_mask_query_kernel<<<1, 32, 0, stream>>>(mask, num_ranks, out);
    return cudaGetLastError();
}
cudaError_t ll_mask_clean(int* mask, int num_ranks, cudaStream_t stream) {
    ll_mask_clean_kernel<<<1, 32, 0, stream>>>(mask, num_ranks);
    return cudaGetLastError();
}

}  // namespace tmoe
