// Small memory-bound helper kernels: gating, chunk-local cumulative sum, MN-major transpose.
// They stand in for gdn_gating_kernel, chunk_local_cumsum_kernel_{headfirst,seqfirst}
// (gdn_cuda/include/gdn_cuda/kernels/gdn_helpers.cuh:41-256) and transpose_fp32_sf /
// transpose_generic (kernels/sm90_layout.cuh:10-87) of the reference.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace gdn {

template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16(x); }

// beta = sigmoid(b); gate = -exp(A_log[h]) * softplus(a + dt_bias[h]).  One thread per element.
template <typename TIn, typename TGate>
__global__ void __launch_bounds__(256) gdn_gating_kernel(const TIn* __restrict__ A_log,
                                                         const TIn* __restrict__ dt_bias,
                                                         const TIn* __restrict__ a,
                                                         const TIn* __restrict__ b,
                                                         TIn* __restrict__ beta,
                                                         TGate* __restrict__ gate, long long total,
                                                         int vh) {
    for (long long i = blockIdx.x * 256ll + threadIdx.x; i < total; i += 256ll * gridDim.x) {
        const int h = static_cast<int>(i % vh);
        const float x = to_f32(a[i]) + to_f32(dt_bias[h]);
        const float sp = x <= 20.f ? log1pf(expf(x)) : x;
        gate[i] = from_f32<TGate>(-expf(to_f32(A_log[h])) * sp);
        beta[i] = from_f32<TIn>(1.f / (1.f + expf(-to_f32(b[i]))));
    }
}

// Chunk-local inclusive cumsum, token-major (tokens, H): one thread per (chunk, head), heads
// on consecutive threads so each step of the 64-token walk is a coalesced row access.
template <typename TIn>
__global__ void __launch_bounds__(128) gdn_cumsum_token_major_kernel(
    const TIn* __restrict__ in, float* __restrict__ out, int num_chunks_total, int chunks_per_seq,
    long long seq_len, int H, const int* __restrict__ cu_seqlens,
    const int* __restrict__ chunk_indices) {
    const long long gid = blockIdx.x * 128ll + threadIdx.x;
    if (gid >= static_cast<long long>(num_chunks_total) * H) return;
    const int h = static_cast<int>(gid % H);
    const int chunk = static_cast<int>(gid / H);
    long long bos, eos, c;
    if (cu_seqlens) {
        const int s = chunk_indices[2 * chunk];
        c = chunk_indices[2 * chunk + 1];
        bos = cu_seqlens[s];
        eos = cu_seqlens[s + 1];
    } else {
        const int s = chunk / chunks_per_seq;
        c = chunk % chunks_per_seq;
        bos = s * seq_len;
        eos = bos + seq_len;
    }
    const long long t0 = bos + c * 64;
    const long long t1 = t0 + 64 < eos ? t0 + 64 : eos;
    float acc = 0.f;
    for (long long t = t0; t < t1; ++t) {
        acc += to_f32(in[t * H + h]);
        out[t * H + h] = acc;
    }
}

// Chunk-local inclusive cumsum, time-contiguous (rows, T): one warp per (row, chunk).
// Padded: rows = batch*H, row length seq_len.  Packed: rows = H, row length = total tokens.
template <typename TIn>
__global__ void __launch_bounds__(128) gdn_cumsum_time_major_kernel(
    const TIn* __restrict__ in, float* __restrict__ out, int num_chunks_total, int chunks_per_seq,
    long long seq_len, int H, int batch, const int* __restrict__ cu_seqlens,
    const int* __restrict__ chunk_indices) {
    const long long wid = (blockIdx.x * 128ll + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= static_cast<long long>(num_chunks_total) * H) return;
    const int h = static_cast<int>(wid % H);
    const int chunk = static_cast<int>(wid / H);
    long long base, t0, t1;
    if (cu_seqlens) {
        const int s = chunk_indices[2 * chunk];
        const long long c = chunk_indices[2 * chunk + 1];
        t0 = cu_seqlens[s] + c * 64;
        const long long eos = cu_seqlens[s + 1];
        t1 = t0 + 64 < eos ? t0 + 64 : eos;
        base = static_cast<long long>(h) * seq_len;  // seq_len = total tokens here
    } else {
        const int s = chunk / chunks_per_seq;
        const long long c = chunk % chunks_per_seq;
        t0 = c * 64;
        t1 = t0 + 64 < seq_len ? t0 + 64 : seq_len;
        base = (static_cast<long long>(s) * H + h) * seq_len;
    }
    const long long ta = t0 + lane, tb = t0 + 32 + lane;
    float x0 = ta < t1 ? to_f32(in[base + ta]) : 0.f;
    float x1 = tb < t1 ? to_f32(in[base + tb]) : 0.f;
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {
        const float y0 = __shfl_up_sync(0xffffffffu, x0, m);
        const float y1 = __shfl_up_sync(0xffffffffu, x1, m);
        if (lane >= m) {
            x0 += y0;
            x1 += y1;
        }
    }
    x1 += __shfl_sync(0xffffffffu, x0, 31);
    if (ta < t1) out[base + ta] = x0;
    if (tb < t1) out[base + tb] = x1;
}

// (G, mn, k) row-major -> (G, k, mn_aligned) row-major; columns mn..mn_aligned-1 are zero.
template <typename T>
__global__ void __launch_bounds__(256) gdn_transpose_kernel(const T* __restrict__ in,
                                                            T* __restrict__ out, long long mn,
                                                            long long k, long long mn_al) {
    __shared__ T tile[32][33];
    const long long g = blockIdx.z;
    const long long mn0 = blockIdx.x * 32ll, k0 = blockIdx.y * 32ll;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
    const T* src = in + g * mn * k;
    T* dst = out + g * k * mn_al;
    for (int r = ty; r < 32; r += 8) {
        const long long m = mn0 + r, kk = k0 + tx;
        tile[r][tx] = (m < mn && kk < k) ? src[m * k + kk] : T(0);
    }
    __syncthreads();
    for (int r = ty; r < 32; r += 8) {
        const long long kk = k0 + r, m = mn0 + tx;
        if (kk < k && m < mn_al) dst[kk * mn_al + m] = tile[tx][r];
    }
}

}  // namespace gdn
