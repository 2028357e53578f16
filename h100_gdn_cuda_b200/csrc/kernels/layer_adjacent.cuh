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

// Both kernels are bound by instruction issue before they are bound by HBM, so the arithmetic runs on
// packed pairs of fp32 values (one 64-bit register pair, f32x2 instructions) and SiLU costs one approximate
// special-function operation per element.
namespace la {
// Both kernels are launched as programmatic dependents of the preceding work in the stream and wait here before
// their first access to global memory (a no-op for an ordinary launch).
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
using f2 = unsigned long long;
__device__ __forceinline__ f2 pk(float a, float b) {
    f2 d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(a), "f"(b));
    return d;
}
__device__ __forceinline__ void unpk(f2 v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ f2 fma2(f2 a, f2 b, f2 c) {
    f2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ f2 mul2(f2 a, f2 b) {
    f2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f2 add2(f2 a, f2 b) {
    f2 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float tanh_approx(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// v -> silu(v) = v * sigmoid(v) = v * (0.5 + 0.5 tanh(v / 2)) on a pair: ONE special-function operation per
// element (the exp + reciprocal form takes two, and the special-function unit, 4 lanes per cycle and scheduler,
// was the busiest pipe of both kernels).  tanh.approx is good to about 2^-11, well inside bf16.
__device__ __forceinline__ f2 silu2(f2 v) {
    float a, b;
    unpk(mul2(v, pk(0.5f, 0.5f)), a, b);
    return mul2(v, fma2(pk(tanh_approx(a), tanh_approx(b)), pk(0.5f, 0.5f), pk(0.5f, 0.5f)));
}
// eight bf16 values (16 bytes) <-> four packed fp32 pairs
__device__ __forceinline__ void unpack8(const uint4& u, f2* f) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) f[e] = pk(__uint_as_float(w[e] << 16), __uint_as_float(w[e] & 0xFFFF0000u));
}
__device__ __forceinline__ uint4 pack8(const f2* f) {
    uint32_t w[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        float a, b;
        unpk(f[e], a, b);
        __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
        w[e] = *reinterpret_cast<uint32_t*>(&v);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}
}  // namespace la

// One thread: 8 adjacent channels, kConvTokBlock consecutive tokens; the last width - 1 inputs slide
// along in registers, so every input is loaded once (plus width - 1 tokens of halo per block).
// blockIdx.x: channel groups, blockIdx.y: token blocks, blockIdx.z: batch entry (padded mode).
// Token positions inside the kernel are 32-bit offsets from the block's first token and addresses advance
// by pointer increments: the kernel is bound by instruction issue, and 64-bit index arithmetic per token was a
// good part of it.  (Unrolling all 32 tokens, which makes ring slots constants, is slower: 3 k instructions
// per thread no longer sit in the instruction cache.)
template <int W>
__global__ void __launch_bounds__(128, 5) gdn_causal_conv1d_kernel(const ConvParams p) {
    static_assert(W >= 2 && W <= kConvMaxWidth, "filter widths 2 .. 4");
    using namespace la;
    grid_dep_wait();
    const int cg = blockIdx.x * blockDim.x + threadIdx.x;
    if (cg * 8 >= p.channels) return;
    const int c0 = cg * 8;
    f2 wt[W][4], bs[4];  // channel pairs
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        bs[e] = p.bias ? pk(__bfloat162float(p.bias[c0 + 2 * e]), __bfloat162float(p.bias[c0 + 2 * e + 1])) : pk(0.f, 0.f);
#pragma unroll
        for (int i = 0; i < W; ++i)
            wt[i][e] = pk(__bfloat162float(p.w[static_cast<long long>(c0 + 2 * e) * W + i]),
                          __bfloat162float(p.w[static_cast<long long>(c0 + 2 * e + 1) * W + i]));
    }
    // the thread's token block [t0, t0 + n_tok) and the sequence it starts in
    const bool packed = p.cu_seqlens != nullptr;
    const long long t0 = static_cast<long long>(blockIdx.y) * kConvTokBlock;
    const long long limit = packed ? p.total_tokens : static_cast<long long>(p.seq_len);
    if (t0 >= limit) return;
    const int n_tok = static_cast<int>(min(static_cast<long long>(kConvTokBlock), limit - t0));
    int seq;
    const __nv_bfloat16* xb;
    __nv_bfloat16* yb;
    constexpr int kFar = 1 << 20;
    int bos_rel, eos_rel;  // start and end of the current sequence relative to t0 (clipped far away)
    auto set_sequence = [&](int s_) {
        seq = s_;
        const long long b = packed ? p.cu_seqlens[s_] : 0, e = packed ? p.cu_seqlens[s_ + 1] : p.seq_len;
        bos_rel = static_cast<int>(max(b - t0, static_cast<long long>(-kFar)));
        eos_rel = static_cast<int>(min(e - t0, static_cast<long long>(kFar)));
    };
    if (packed) {
        int lo = 0, hi = p.batch;  // last sequence whose start is <= t0
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (p.cu_seqlens[mid] <= t0) lo = mid; else hi = mid;
        }
        set_sequence(lo);
        xb = p.x;
        yb = p.y;
    } else {
        set_sequence(static_cast<int>(blockIdx.z));
        xb = p.x + seq * p.x_sb;
        yb = p.y + seq * p.y_sb;
    }
    const __nv_bfloat16* const x0 = xb + t0 * p.x_st + c0;  // this thread's channels of token t0
    // the input at offset j (from t0) of the current sequence; positions before its start come from the state, or are zero
    auto load_input = [&](int j) {
        if (j >= bos_rel) return *reinterpret_cast<const uint4*>(x0 + j * p.x_st);
        if (p.state_in && bos_rel - j <= W - 1) {
            const int row = (W - 1) - (bos_rel - j);  // state row W-2 is the input right before the sequence
            return *reinterpret_cast<const uint4*>(p.state_in + (static_cast<long long>(seq) * (W - 1) + row) * p.channels + c0);
        }
        return make_uint4(0u, 0u, 0u, 0u);
    };
    auto store_state = [&](int last) {  // the sequence's final width - 1 inputs, `last` = offset of its last token
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
    const uint32_t ring0 = static_cast<uint32_t>(__cvta_generic_to_shared(&ring[0][threadIdx.x]));
    constexpr uint32_t kSlotBytes = 128 * sizeof(uint4);
    const __nv_bfloat16* xreq = x0;  // source of the next request
    auto request = [&](int j) {      // j: offset of the token
        if (j < n_tok)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ring0 + (j % kConvRing) * kSlotBytes), "l"(xreq) : "memory");
        xreq += p.x_st;
        asm volatile("cp.async.commit_group;" ::: "memory");  // one group per token, empty past the end
    };
#pragma unroll
    for (int u = 0; u < kConvRing; ++u) request(u);
    // The last W inputs are kept unpacked in W register sets used as a ring: step R of every W consecutive
    // tokens finds tap i in set (R + i) % W and puts the new token into set (R + W - 1) % W, so nothing is
    // ever moved or unpacked twice.
    f2 win[W][4];
#pragma unroll
    for (int i = 0; i < W - 1; ++i) unpack8(load_input(i - (W - 1)), win[i]);
    __nv_bfloat16* yp = yb + t0 * p.y_st + c0;
    auto step = [&](auto rot, int j) {
        constexpr int R = decltype(rot)::value;
        if (j >= eos_rel) {  // packed mode: the block runs into the next sequence(s); empty ones are skipped
            int s_ = seq;
            do {
                ++s_;
                set_sequence(s_);
            } while (j >= eos_rel);
#pragma unroll
            for (int i = 0; i < W - 1; ++i) unpack8(load_input(j - (W - 1) + i), win[(R + i) % W]);
        }
        asm volatile("cp.async.wait_group %0;" ::"n"(kConvRing - 1) : "memory");  // the oldest request has landed
        uint4 raw;
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(raw.x), "=r"(raw.y), "=r"(raw.z), "=r"(raw.w)
                     : "r"(ring0 + (j % kConvRing) * kSlotBytes)
                     : "memory");
        unpack8(raw, win[(R + W - 1) % W]);
        request(j + kConvRing);  // (the slot's value is in registers: it may be handed to the next copy)
        f2 acc[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[e] = bs[e];
#pragma unroll
        for (int i = 0; i < W; ++i) {
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[e] = fma2(wt[i][e], win[(R + i) % W][e], acc[e]);
        }
        if (p.silu) {
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[e] = silu2(acc[e]);
        }
        *reinterpret_cast<uint4*>(yp) = pack8(acc);
        yp += p.y_st;
        if (j == eos_rel - 1) store_state(j);
    };
#pragma unroll 1
    for (int j = 0; j < n_tok; j += W) {
        step(std::integral_constant<int, 0>{}, j);
        if (j + 1 < n_tok && j + 1 < kConvTokBlock) step(std::integral_constant<int, 1 % W>{}, j + 1);
        if (W > 2 && j + 2 < n_tok && j + 2 < kConvTokBlock) step(std::integral_constant<int, 2 % W>{}, j + 2);
        if (W > 3 && j + 3 < n_tok && j + 3 < kConvTokBlock) step(std::integral_constant<int, 3 % W>{}, j + 3);
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
    using namespace la;
    grid_dep_wait();
    f2 xv[kUnroll][kMaxPass][4];
    uint4 zraw[kUnroll][kMaxPass];  // the gate is requested with x, not after the reduction
    float ss[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        const long long row = row0 + u * kRowsPerWarp;
        f2 sq = pk(0.f, 0.f);
#pragma unroll
        for (int it = 0; it < kMaxPass; ++it) {
            const int c = (it * LPR + l) * 8;
            if (row < p.rows && c < p.dim) {
                unpack8(*reinterpret_cast<const uint4*>(p.x + row * p.x_sr + c), xv[u][it]);
                zraw[u][it] = *reinterpret_cast<const uint4*>(p.z + row * p.z_sr + c);
#pragma unroll
                for (int e = 0; e < 4; ++e) sq = fma2(xv[u][it][e], xv[u][it][e], sq);
            }
        }
        float s0, s1;
        unpk(sq, s0, s1);
        ss[u] = s0 + s1;
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
                f2 zv[4], wv[4], o[4];
                unpack8(zraw[u][it], zv);
                unpack8(*reinterpret_cast<const uint4*>(p.w + c), wv);
                const f2 r2 = pk(rstd, rstd);
#pragma unroll
                for (int e = 0; e < 4; ++e) o[e] = mul2(mul2(mul2(xv[u][it][e], r2), wv[e]), silu2(zv[e]));
                *reinterpret_cast<uint4*>(p.y + row * p.y_sr + c) = pack8(o);
            }
        }
    }
}

}  // namespace gdn
