// The two memory-bound steps that sit on either side of Gated DeltaNet in Qwen3-Next-style blocks and
// that the reference leaves to its callers: the short causal depthwise convolution (+ SiLU) applied to
// the q/k/v projections before the layer, and the gated RMS norm  y = rmsnorm(o) * w * silu(z)  applied
// to its output.  Plain coalesced CUDA: 16-byte accesses, every input element read once.
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

#include <type_traits>

namespace gdn {

constexpr int kConvTokBlock = 32;  // tokens per thread along the sequence
constexpr int kConvMaxWidth = 4;
constexpr int kConvRing = 8;       // tokens requested ahead per thread

struct ConvParams {
    const __nv_bfloat16* x;   // (batch, seq_len, C) through strides, or packed (tokens, C)
    __nv_bfloat16* y;
    const __nv_bfloat16* w;   // (C, width), row per channel
    const __nv_bfloat16* bias;  // (C) or NULL
    const __nv_bfloat16* state_in;   // (sequences, width - 1, C) or NULL: the inputs before the first token
    __nv_bfloat16* state_out;        // (sequences, width - 1, C) or NULL: the last width - 1 inputs
    long long x_sb, x_st, y_sb, y_st;
    const int* cu_seqlens;  // packed mode or NULL
    int batch, seq_len, channels, width, silu;
    long long total_tokens;
};

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + __expf(-v)); }

__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        f[2 * e] = __uint_as_float(w[e] << 16);
        f[2 * e + 1] = __uint_as_float(w[e] & 0xFFFF0000u);
    }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
    uint32_t w[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        __nv_bfloat162 v = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
        w[e] = *reinterpret_cast<uint32_t*>(&v);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// One thread: 8 adjacent channels, kConvTokBlock consecutive tokens; the last width - 1 inputs slide
// along in registers, so every input is loaded once (plus width - 1 tokens of halo per block).
// blockIdx.x: channel groups, blockIdx.y: token blocks, blockIdx.z: batch entry (padded mode).
template <int W>
__global__ void __launch_bounds__(128) gdn_causal_conv1d_kernel(const ConvParams p) {
    static_assert(W >= 2 && W <= kConvMaxWidth, "filter widths 2 .. 4");
    const int cg = blockIdx.x * blockDim.x + threadIdx.x;
    if (cg * 8 >= p.channels) return;
    const int c0 = cg * 8;
    float wt[W][8], bs[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        bs[e] = p.bias ? __bfloat162float(p.bias[c0 + e]) : 0.f;
#pragma unroll
        for (int i = 0; i < W; ++i) wt[i][e] = __bfloat162float(p.w[static_cast<long long>(c0 + e) * W + i]);
    }
    // token range of this thread and the sequence it starts in
    long long t0, t_end;   // global token positions (packed) or positions inside the batch entry (padded)
    int seq;
    long long bos, eos;
    const __nv_bfloat16* xb;
    __nv_bfloat16* yb;
    if (p.cu_seqlens) {
        t0 = static_cast<long long>(blockIdx.y) * kConvTokBlock;
        if (t0 >= p.total_tokens) return;
        t_end = min(t0 + kConvTokBlock, p.total_tokens);
        int lo = 0, hi = p.batch;  // last sequence whose start is <= t0
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (p.cu_seqlens[mid] <= t0) lo = mid; else hi = mid;
        }
        seq = lo;
        bos = p.cu_seqlens[seq];
        eos = p.cu_seqlens[seq + 1];
        xb = p.x;
        yb = p.y;
    } else {
        seq = blockIdx.z;
        t0 = static_cast<long long>(blockIdx.y) * kConvTokBlock;
        if (t0 >= p.seq_len) return;
        t_end = min(t0 + kConvTokBlock, static_cast<long long>(p.seq_len));
        bos = 0;
        eos = p.seq_len;
        xb = p.x + seq * p.x_sb;
        yb = p.y + seq * p.y_sb;
    }
    // the input at position t of the current sequence; positions before its start come from the state, or are zero
    auto load_input = [&](long long t) {
        if (t >= bos) return *reinterpret_cast<const uint4*>(xb + t * p.x_st + c0);
        if (p.state_in && bos - t <= W - 1) {
            const long long row = (W - 1) - (bos - t);  // state row W-2 is the input right before the sequence
            return *reinterpret_cast<const uint4*>(p.state_in + (static_cast<long long>(seq) * (W - 1) + row) * p.channels + c0);
        }
        return make_uint4(0u, 0u, 0u, 0u);
    };
    auto store_state = [&](long long last) {  // the sequence's final width - 1 inputs, `last` = its last token
        if (!p.state_out) return;
#pragma unroll
        for (int r = 0; r < W - 1; ++r) {
            const uint4 v = load_input(last - (W - 2) + r);
            *reinterpret_cast<uint4*>(p.state_out + (static_cast<long long>(seq) * (W - 1) + r) * p.channels + c0) = v;
        }
    };
    // The inputs of the thread's tokens travel through a private ring of kConvRing 16-byte slots in shared
    // memory, filled by asynchronous copies issued kConvRing tokens ahead: that many loads per thread are in
    // flight without costing registers (a thread with one load in flight at a time cannot keep HBM busy).
    __shared__ uint4 ring[kConvRing][128];
    auto request = [&](long long t) {
        if (t < t_end) {
            const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(&ring[static_cast<int>(t - t0) % kConvRing][threadIdx.x]));
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(xb + t * p.x_st + c0) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");  // one group per token, empty past the end
    };
#pragma unroll
    for (int u = 0; u < kConvRing; ++u) request(t0 + u);
    // The last W inputs are kept unpacked in W register sets used as a ring: step R of every W consecutive
    // tokens finds tap i in set (R + i) % W and puts the new token into set (R + W - 1) % W, so nothing is
    // ever moved or unpacked twice.
    float win[W][8];
    auto step = [&](auto rot, long long t) {
        constexpr int R = decltype(rot)::value;
        bool refill = t == t0;
        if (t >= eos) {  // packed mode: the block runs into the next sequence(s); empty ones are skipped
            do {
                ++seq;
                bos = p.cu_seqlens[seq];
                eos = p.cu_seqlens[seq + 1];
            } while (t >= eos);
            refill = true;
        }
        if (refill) {
#pragma unroll
            for (int i = 0; i < W - 1; ++i) unpack8(load_input(t - (W - 1) + i), win[(R + i) % W]);
        }
        asm volatile("cp.async.wait_group %0;" ::"n"(kConvRing - 1) : "memory");  // the oldest request has landed
        unpack8(ring[static_cast<int>(t - t0) % kConvRing][threadIdx.x], win[(R + W - 1) % W]);
        request(t + kConvRing);  // (the slot's value is in registers: it may be handed to the next copy)
        float acc[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = bs[e];
#pragma unroll
        for (int i = 0; i < W; ++i) {
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] = fmaf(wt[i][e], win[(R + i) % W][e], acc[e]);
        }
        if (p.silu) {
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] = __fdividef(acc[e], 1.f + __expf(-acc[e]));
        }
        *reinterpret_cast<uint4*>(yb + t * p.y_st + c0) = pack8(acc);
        if (t == eos - 1) store_state(t);
    };
    for (long long t = t0; t < t_end; t += W) {
        step(std::integral_constant<int, 0>{}, t);
        if (t + 1 < t_end) step(std::integral_constant<int, 1 % W>{}, t + 1);
        if (W > 2 && t + 2 < t_end) step(std::integral_constant<int, 2 % W>{}, t + 2);
        if (W > 3 && t + 3 < t_end) step(std::integral_constant<int, 3 % W>{}, t + 3);
    }
}

// Sequences without tokens keep their state: copied through when the output state is another buffer.
__global__ void gdn_conv_state_passthrough_kernel(const ConvParams p) {
    const int seq = blockIdx.x;
    if (!p.cu_seqlens || !p.state_out || !p.state_in || p.state_out == p.state_in) return;
    if (p.cu_seqlens[seq + 1] != p.cu_seqlens[seq]) return;
    const long long n = static_cast<long long>(p.width - 1) * p.channels;
    for (long long i = threadIdx.x; i < n; i += blockDim.x) p.state_out[seq * n + i] = p.state_in[seq * n + i];
}

struct NormParams {
    const __nv_bfloat16* x;
    const __nv_bfloat16* z;   // gate, same shape as x
    __nv_bfloat16* y;
    const __nv_bfloat16* w;   // (D)
    long long rows, x_sr, z_sr, y_sr;  // row strides in elements
    int dim;
    float eps;
};

// y = x * rsqrt(mean(x^2) + eps) * w * silu(z), one row per (token, head).  A row is handled by LPR lanes
// (8 elements = 16 bytes per lane and pass), so a warp takes 32 / LPR rows at a time and every lane has two
// rows in flight; rows longer than 8 * LPR elements take several passes.
template <int LPR>
__global__ void __launch_bounds__(256) gdn_gated_rmsnorm_kernel(const NormParams p) {
    constexpr int kRowsPerWarp = 32 / LPR;
    constexpr int kMaxPass = LPR == 32 ? 4 : 1;  // dims up to 1024
    constexpr int kUnroll = LPR == 32 ? 1 : 2;   // rows in flight per lane group (four: more registers, slower)
    const int lane = threadIdx.x & 31;
    const int sub = lane / LPR, l = lane % LPR;
    const long long warp_id = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long row0 = warp_id * (kRowsPerWarp * kUnroll) + sub;
    float xv[kUnroll][kMaxPass][8];
    uint4 zraw[kUnroll][kMaxPass];  // the gate is requested with x, not after the reduction
    float ss[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        const long long row = row0 + u * kRowsPerWarp;
        ss[u] = 0.f;
#pragma unroll
        for (int it = 0; it < kMaxPass; ++it) {
            const int c = (it * LPR + l) * 8;
            if (row < p.rows && c < p.dim) {
                unpack8(*reinterpret_cast<const uint4*>(p.x + row * p.x_sr + c), xv[u][it]);
                zraw[u][it] = *reinterpret_cast<const uint4*>(p.z + row * p.z_sr + c);
#pragma unroll
                for (int e = 0; e < 8; ++e) ss[u] = fmaf(xv[u][it][e], xv[u][it][e], ss[u]);
            }
        }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
#pragma unroll
        for (int m = LPR / 2; m > 0; m >>= 1) ss[u] += __shfl_xor_sync(0xffffffffu, ss[u], m);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        const long long row = row0 + u * kRowsPerWarp;
        const float rstd = rsqrtf(ss[u] / static_cast<float>(p.dim) + p.eps);
#pragma unroll
        for (int it = 0; it < kMaxPass; ++it) {
            const int c = (it * LPR + l) * 8;
            if (row < p.rows && c < p.dim) {
                float zv[8], wv[8], o[8];
                unpack8(zraw[u][it], zv);
                unpack8(*reinterpret_cast<const uint4*>(p.w + c), wv);
#pragma unroll
                for (int e = 0; e < 8; ++e) o[e] = xv[u][it][e] * rstd * wv[e] * silu_f(zv[e]);
                *reinterpret_cast<uint4*>(p.y + row * p.y_sr + c) = pack8(o);
            }
        }
    }
}

}  // namespace gdn
