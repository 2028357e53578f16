// State propagation + output of chunked Gated DeltaNet prefill, warp-specialised.
// One CTA of 448 threads walks the chunks of one (sequence, v-head):
//     U_new = U - W S^T
//     O     = scale * ( e^{g} .* (Q S^T) + P U_new ),   P = tril(Q K^T .* e^{g_i - g_j}) (precomputed)
//     S    <- e^{g_L} S + U_new^T (K .* e^{g_L - g})
// This is the path gdn_chunked_forward uses; it stands in for the reference's
// sm90_bf16_chunked_seq_state_update and sm90_bf16_gdn_chunked_compute_O
// (kernels/sm90_bf16_chunked_seq_state_update2.cuh, sm90_bf16_gdn_chunked_compute_O.cuh:23-530)
// and never writes per-chunk states.
//
// The only serial dependence between chunks runs through the state:
//     S_bf(c) -> [MMA] D1 = U^T I - S_bf W^T -> [pass] Un_a, Un_b -> [MMA] dS = Un_b K -> [pass] S, S_bf(c+1)
// Roles keep everything else off that chain:
//   warps 0-7   state warps: own the fp32 state in registers (row = TMEM lane, 64 columns each),
//               run the two passes of the chain
//   warps 8-11  output warps: O epilogue (scale, transpose through shared memory, coalesced stores)
//   warp 12     producer: chunk-local gate cumsum; per chunk one bulk copy of its U, W, P block of
//               the scratch and tensor copies of Q and K, into a two-stage ring
//   warp 13     one thread issues every tcgen05.mma and commits completion onto mbarriers
// All operands are transposed so that the 128 state rows are the MMA M dimension; S_bf, Un_a,
// Un_b are bf16 A operands in tensor memory; Q, K, W, U, P tiles are used as TMA delivered them.
#pragma once
#include <cuda.h>

#include "prefill_common.cuh"

namespace gdn {

struct FusedParams {
    ChunkMap map;
    ScalarView gate;  // raw per-token log-decay; ptr == NULL: no decay
    TokenView out;
    const __nv_bfloat16* state_in;
    long long si_ss, si_sh;
    __nv_bfloat16* state_out;  // final state or NULL
    long long so_ss, so_sh;
    int kh, vh;
    float scale;
    int* status;
    const uint8_t* blocks;  // U, W, P of every (global chunk, v-head): kUnitBlockBytes each
    // Segmented runs (padded mode, few long sequences; see gdn_chunked_forward).  The state obeys
    // S' = S M_c + N_c per chunk, so a segment of chunks has a composite (M, N) as well.
    //   mode 0: one CTA walks the whole sequence (blockIdx.z = 0).
    //   mode 1: blockIdx.z = 2 * segment + kind; no output.  kind 0 starts from S = 0 and ends with
    //           N of the segment; kind 1 starts from S = I with U taken as 0 and ends with M.
    //           Both are written in fp32 to seg_mn[((chain * num_segments + segment) * 2 + kind)].
    //   mode 2: blockIdx.z = segment; starts from seg_start[chain * num_segments + segment] (fp32),
    //           writes the output of its chunks; the last segment writes the final state.
    int mode, seg_chunks, num_segments;
    float* seg_mn;
    const float* seg_start;
    // Packed mode with more CTAs than SMs: sequences sorted by length, longest first (written by
    // gdn_seq_order_kernel).  Then blockIdx.x = head and blockIdx.y = rank of the sequence, so the
    // longest chains are dispatched first and the short ones fill the tail.  NULL: blockIdx.x =
    // sequence, blockIdx.y = head.
    const int* seq_order;
};

struct FusedSmem {
    static constexpr int D = 128;
    static constexpr int kTile = kChunk * D * 2;  // 16 KB
    // U, W, P in the order of a unit block of the scratch, so that one bulk copy fills all three
    static constexpr int kOffQ = 0, kOffK = kTile, kOffU = 2 * kTile, kOffW = 3 * kTile, kOffP = 4 * kTile;
    static constexpr int kStage = 2 * kTile + kUnitBlockBytes;  // Q, K, U, W, P
    static constexpr int kOffO = 2 * kStage;         // two output staging tiles
    static constexpr int kOffGate = kOffO + 2 * kTile;  // 3 x { e^g[64], e^{gL-g}[64], e^{gL} }
    static constexpr int kGateStride = (2 * 64 + 4) * 4;
    static constexpr int kOffBar = kOffGate + 3 * kGateStride;
    static constexpr int kBytes = kOffBar + 128 + 1024;
};

namespace fused {
constexpr int kThreads = 512;  // 16 warps = 4 warpgroups (the last holds the producer, the issuer and 2 idle warps)
constexpr uint32_t kTmSbf = 0;    // bf16 state, 64 columns
constexpr uint32_t kTmUnA = 64;   // bf16 U_new^T, 32 columns
constexpr uint32_t kTmUnB = 96;   // bf16 U_new^T .* decay, 32 columns
constexpr uint32_t kTmD1 = 128;   // fp32 U_new^T, 64 columns
constexpr uint32_t kTmO1a = 192;  // fp32 S Q^T, even chunks
constexpr uint32_t kTmDS = 256;   // fp32 state increment, 128 columns
constexpr uint32_t kTmO1b = 384;  // fp32 S Q^T, odd chunks
constexpr uint32_t kTmO2 = 448;   // fp32 U_new^T P^T

// Register re-allocation between warpgroups (every warp of the warpgroup executes it).
template <int N>
__device__ __forceinline__ void reg_inc() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_dec() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
// two fp32 values in one 64-bit register pair, and the two-wide fp32 instructions on them
using f2 = unsigned long long;
__device__ __forceinline__ f2 pk(float lo, float hi) {
    f2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpk(f2 v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f2 fma2(f2 a, f2 b, f2 c) {
    f2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ f2 add2(f2 a, f2 b) {
    f2 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f2 mul2(f2 a, f2 b) {
    f2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
}  // namespace fused

__global__ void __launch_bounds__(fused::kThreads, 1)
    gdn_fused_seq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                         const __grid_constant__ CUtensorMap tmO, const FusedParams p) {
    using namespace ptx;
    using namespace fused;
    using L = FusedSmem;
    constexpr int D = 128;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kOffBar);
    uint64_t* bar_full = bars;        // [2]
    uint64_t* bar_empty = bars + 2;   // [2]
    uint64_t* bar_sbf = bars + 4;
    uint64_t* bar_d1 = bars + 5;
    uint64_t* bar_un = bars + 6;
    uint64_t* bar_ds = bars + 7;
    uint64_t* bar_o = bars + 8;
    uint64_t* bar_ofree = bars + 9;
    uint64_t* bar_full2 = bars + 10;  // [2]: P, K, Q of a stage (bar_full: U, W and the gate vectors)
    uint64_t* bar_go = bars + 12;     // state warps are past their chunk-boundary work: the epilogue may run
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
    int* abort_flag = reinterpret_cast<int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int seq = p.seq_order ? p.seq_order[blockIdx.y] : static_cast<int>(blockIdx.x);
    const int head = p.seq_order ? static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.y);
    const int khead = head / (p.vh / p.kh);

    int batch, gchunk0;
    long long seq_tok0, seq_tokens;
    if (p.map.cu_seqlens) {
        const int bos = p.map.cu_seqlens[seq], eos = p.map.cu_seqlens[seq + 1];
        seq_tok0 = bos;
        seq_tokens = eos - bos;
        batch = 0;
        gchunk0 = p.map.cu_chunks[seq];
    } else {
        seq_tok0 = 0;
        seq_tokens = p.map.seq_len;
        batch = seq;
        gchunk0 = seq * p.map.chunks_per_seq;
    }
    int nchunks = static_cast<int>((seq_tokens + kChunk - 1) / kChunk);
    // A segment is handled as a sequence of its own: shift the token and chunk origins.
    const int segment = p.mode == 1 ? static_cast<int>(blockIdx.z >> 1) : (p.mode == 2 ? static_cast<int>(blockIdx.z) : 0);
    const int seg_kind = p.mode == 1 ? static_cast<int>(blockIdx.z & 1) : 0;
    const bool emit_o = p.mode != 1;
    const bool zero_u = p.mode == 1 && seg_kind == 1;
    if (p.mode != 0) {
        const int c0 = min(segment * p.seg_chunks, nchunks);
        const int c1 = min(c0 + p.seg_chunks, nchunks);
        seq_tok0 += static_cast<long long>(c0) * kChunk;
        seq_tokens = min(seq_tokens - static_cast<long long>(c0) * kChunk, static_cast<long long>(c1 - c0) * kChunk);
        gchunk0 += c0;
        nchunks = c1 - c0;
    }
    const long long chain = static_cast<long long>(seq) * p.vh + head;
    auto chunk_n = [&](int c) {
        const long long rem = seq_tokens - static_cast<long long>(c) * kChunk;
        return rem < kChunk ? static_cast<int>(rem) : kChunk;
    };
    auto gate_buf = [&](int c) { return reinterpret_cast<float*>(smem + L::kOffGate + (c % 3) * L::kGateStride); };

    if (tid == 0) {
        *abort_flag = 0;
        mbar_init(&bar_full[0], 1);
        mbar_init(&bar_full[1], 1);
        mbar_init(&bar_empty[0], 1);
        mbar_init(&bar_empty[1], 1);
        mbar_init(&bar_full2[0], 1);
        mbar_init(&bar_full2[1], 1);
        mbar_init(bar_go, 8);
        mbar_init(bar_sbf, 8);
        mbar_init(bar_d1, 1);
        mbar_init(bar_un, 8);
        mbar_init(bar_ds, 1);
        mbar_init(bar_o, 1);
        mbar_init(bar_ofree, 4);
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(tmem_slot, 512);
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp < 8) {
        // =============================================================== state warps
        reg_inc<168>();
        const int lq = warp & 3, hf = warp >> 2;
        const int row = 32 * lq + lane;
        const uint32_t tm_lane = static_cast<uint32_t>(32 * lq) << 16;
        // element (token i, this row) of a swizzled 64 x 128 tile: i * 128 + uoff8[i & 7]
        uint32_t uoff8[8];
#pragma unroll
        for (int k = 0; k < 8; ++k)
            uoff8[k] = static_cast<uint32_t>((row >> 6) * 8192 + ((((row & 63) >> 3) ^ k) << 4) + (row & 7) * 2);
        float S[64];
        if (p.mode == 2) {
            const float4* src = reinterpret_cast<const float4*>(p.seg_start + (chain * p.num_segments + segment) * (D * D) +
                                                                static_cast<long long>(row) * D + 64 * hf);
#pragma unroll
            for (int q = 0; q < 16; ++q) {
                const float4 v = __ldg(src + q);
                S[4 * q] = v.x; S[4 * q + 1] = v.y; S[4 * q + 2] = v.z; S[4 * q + 3] = v.w;
            }
        } else if (p.mode == 1) {
#pragma unroll
            for (int q = 0; q < 64; ++q) S[q] = (seg_kind == 1 && row == 64 * hf + q) ? 1.f : 0.f;
        } else if (p.state_in) {
            const uint4* src = reinterpret_cast<const uint4*>(p.state_in + seq * p.si_ss + head * p.si_sh +
                                                              static_cast<long long>(row) * D + 64 * hf);
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const uint4 v = __ldg(src + q);
                S[q * 8 + 0] = bf16_lo(v.x); S[q * 8 + 1] = bf16_hi(v.x);
                S[q * 8 + 2] = bf16_lo(v.y); S[q * 8 + 3] = bf16_hi(v.y);
                S[q * 8 + 4] = bf16_lo(v.z); S[q * 8 + 5] = bf16_hi(v.z);
                S[q * 8 + 6] = bf16_lo(v.w); S[q * 8 + 7] = bf16_hi(v.w);
            }
        } else {
#pragma unroll
            for (int q = 0; q < 64; ++q) S[q] = 0.f;
        }
        auto publish_state = [&]() {
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                uint32_t w[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) w[e] = pack_bf16(S[q * 32 + 2 * e], S[q * 32 + 2 * e + 1]);
                tmem_st16(tmem + kTmSbf + tm_lane + 32 * hf + 16 * q, w);
            }
            tmem_wait_st();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_sbf);
        };
        publish_state();

        for (int c = 0; c < nchunks; ++c) {
            const uint32_t par = static_cast<uint32_t>(c & 1);
            const int n = chunk_n(c);
            const float* gb = gate_buf(c);
            mbar_wait(&bar_full[c & 1], static_cast<uint32_t>((c >> 1) & 1), abort_flag);  // gate values visible
            // ---- U_new^T = U^T - S W^T -> two bf16 operand copies (rows past the end zeroed)
            // This thread's 32 values of U^T come straight from the TMA tile (element (token, row)
            // of the swizzled layout), packed two tokens per register while the MMA is running.
            const uint8_t* sU = smem + (c & 1) * L::kStage + L::kOffU;
            uint32_t upk[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) {
                const int i0 = 32 * hf + 2 * e;
                const uint32_t lo = *reinterpret_cast<const uint16_t*>(sU + i0 * 128 + uoff8[i0 & 7]);
                const uint32_t hi = *reinterpret_cast<const uint16_t*>(sU + (i0 + 1) * 128 + uoff8[(i0 + 1) & 7]);
                upk[e] = zero_u ? 0u : (lo | (hi << 16));
            }
            const int nloc = n - 32 * hf;  // tokens of this half that exist
            // The state warps now idle until D1 arrives: the window in which the output warps (which
            // share the schedulers) run the previous chunk's epilogue without slowing the chain down.
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_go);
            mbar_wait(bar_d1, par, abort_flag);
            tc_fence_after_sync();
            if (c == 40 && tid == 0) GDN_STAMP_ANY(40);
            {
                uint32_t r[32];
                tmem_ld32(tmem + kTmD1 + tm_lane + 32 * hf, r);  // -(S W^T)
                float dec[32];
#pragma unroll
                for (int e4 = 0; e4 < 8; ++e4) {
                    const float4 t = *reinterpret_cast<const float4*>(gb + 64 + 32 * hf + 4 * e4);
                    dec[4 * e4] = t.x; dec[4 * e4 + 1] = t.y; dec[4 * e4 + 2] = t.z; dec[4 * e4 + 3] = t.w;
                }
                tmem_wait_ld();
                uint32_t wa[16], wb[16];
                if (nloc >= 32) {  // every token of this half exists (all chunks but a ragged last one)
#pragma unroll
                    // the plain copy is on its way to tensor memory while the scaled one is computed
                    f2 u2[16];
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        u2[e] = add2(pk(bf16_lo(upk[e]), bf16_hi(upk[e])),
                                     pk(__uint_as_float(r[2 * e]), __uint_as_float(r[2 * e + 1])));
                        float u0, u1;
                        unpk(u2[e], u0, u1);
                        wa[e] = pack_bf16(u0, u1);
                    }
                    tmem_st16(tmem + kTmUnA + tm_lane + 16 * hf, wa);
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        float d0, d1;
                        unpk(mul2(u2[e], pk(dec[2 * e], dec[2 * e + 1])), d0, d1);
                        wb[e] = pack_bf16(d0, d1);
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        const float u0 = 2 * e < nloc ? bf16_lo(upk[e]) + __uint_as_float(r[2 * e]) : 0.f;
                        const float u1 = 2 * e + 1 < nloc ? bf16_hi(upk[e]) + __uint_as_float(r[2 * e + 1]) : 0.f;
                        wa[e] = pack_bf16(u0, u1);
                        wb[e] = pack_bf16(u0 * dec[2 * e], u1 * dec[2 * e + 1]);
                    }
                }
                if (nloc < 32) tmem_st16(tmem + kTmUnA + tm_lane + 16 * hf, wa);
                tmem_st16(tmem + kTmUnB + tm_lane + 16 * hf, wb);
            }
            tmem_wait_st();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_un);
            if (c == 40 && tid == 0) GDN_STAMP_ANY(41);
            // ---- S <- e^{g_L} S + dS
            const float eg_last = gb[128];
            const f2 eg2 = pk(eg_last, eg_last);
            mbar_wait(bar_ds, par, abort_flag);
            tc_fence_after_sync();
            if (c == 40 && tid == 0) GDN_STAMP_ANY(42);
            {
                // both halves of this thread's 64 increments are requested at once; the new bf16
                // state of a half is on its way to tensor memory while the other half is computed
                uint32_t r0[32], r1[32];
                tmem_ld32(tmem + kTmDS + tm_lane + 64 * hf, r0);
                tmem_ld32(tmem + kTmDS + tm_lane + 64 * hf + 32, r1);
                tmem_wait_ld();
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    const uint32_t* r = q ? r1 : r0;
                    uint32_t w[16];
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        const f2 s2 = fma2(pk(S[q * 32 + 2 * e], S[q * 32 + 2 * e + 1]), eg2,
                                           pk(__uint_as_float(r[2 * e]), __uint_as_float(r[2 * e + 1])));
                        unpk(s2, S[q * 32 + 2 * e], S[q * 32 + 2 * e + 1]);
                        w[e] = pack_bf16(S[q * 32 + 2 * e], S[q * 32 + 2 * e + 1]);
                    }
                    tmem_st16(tmem + kTmSbf + tm_lane + 32 * hf + 16 * q, w);
                }
                tmem_wait_st();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_sbf);
            }
            if (c == 40 && tid == 0) GDN_STAMP_ANY(43);
        }
        if (lane == 0) mbar_arrive(bar_go);  // releases the last chunk's epilogue
        if (p.mode == 1) {
            float4* d4 = reinterpret_cast<float4*>(p.seg_mn + ((chain * p.num_segments + segment) * 2 + seg_kind) * (D * D) +
                                                   static_cast<long long>(row) * D + 64 * hf);
#pragma unroll
            for (int q = 0; q < 16; ++q) d4[q] = make_float4(S[4 * q], S[4 * q + 1], S[4 * q + 2], S[4 * q + 3]);
        } else if (p.state_out && (p.mode == 0 || segment == p.num_segments - 1)) {
            uint4* d4 = reinterpret_cast<uint4*>(p.state_out + seq * p.so_ss + head * p.so_sh +
                                                 static_cast<long long>(row) * D + 64 * hf);
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                uint4 v;
                v.x = pack_bf16(S[q * 8 + 0], S[q * 8 + 1]);
                v.y = pack_bf16(S[q * 8 + 2], S[q * 8 + 3]);
                v.z = pack_bf16(S[q * 8 + 4], S[q * 8 + 5]);
                v.w = pack_bf16(S[q * 8 + 6], S[q * 8 + 7]);
                d4[q] = v;
            }
        }
    } else if (warp < 12) {
        // =============================================================== output warps
        reg_dec<88>();
        const int lq = warp & 3;
        const int row = 32 * lq + lane;  // dv index = TMEM lane
        const int otid = tid - 256;
        const uint32_t tm_lane = static_cast<uint32_t>(32 * lq) << 16;
        // element (token i, dv row) of the swizzled staging tile: i * 128 + off8[i & 7]
        uint32_t off8[8];
#pragma unroll
        for (int k = 0; k < 8; ++k)
            off8[k] = static_cast<uint32_t>((row >> 6) * 8192 + ((((row & 63) >> 3) ^ k) << 4) + (row & 7) * 2);
        const bool packed = p.map.cu_seqlens != nullptr;
        for (int c = 0; c < (emit_o ? nchunks : 0); ++c) {
            const uint32_t par = static_cast<uint32_t>(c & 1);
            const int n = chunk_n(c);
            const float* gb = gate_buf(c);
            uint8_t* sO = smem + L::kOffO + (c & 1) * L::kTile;
            const uint32_t tO1 = tmem + ((c & 1) ? kTmO1b : kTmO1a) + tm_lane;
            const uint32_t tO2 = tmem + kTmO2 + tm_lane;
            mbar_wait_relaxed<200>(&bar_full[c & 1], static_cast<uint32_t>((c >> 1) & 1), abort_flag);
            if (c == 40 && otid == 0) GDN_STAMP_ANY(49);
            mbar_wait_relaxed<100>(bar_o, par, abort_flag);
            mbar_wait_relaxed<50>(bar_go, static_cast<uint32_t>((c + 1) & 1), abort_flag);
            tc_fence_after_sync();
            if (c == 40 && otid == 0) GDN_STAMP_ANY(50);
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                uint32_t r1[16], r2[16];
                tmem_ld16(tO1 + 16 * b, r1);
                tmem_ld16(tO2 + 16 * b, r2);
                // the gate factors of this batch are read before any store to the staging tile, so
                // that the loads do not queue up behind the stores they might alias
                float gv[16];
#pragma unroll
                for (int e4 = 0; e4 < 4; ++e4) {
                    const float4 t = *reinterpret_cast<const float4*>(gb + 16 * b + 4 * e4);
                    gv[4 * e4] = t.x; gv[4 * e4 + 1] = t.y; gv[4 * e4 + 2] = t.z; gv[4 * e4 + 3] = t.w;
                }
                tmem_wait_ld();
                if (c == 40 && otid == 0) GDN_STAMP_ANY(53 + 2 * b);
                if (b == 3) {
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_ofree);  // accumulators consumed
                }
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    const int i = 16 * b + e;
                    const float o = fmaf(gv[e], __uint_as_float(r1[e]), __uint_as_float(r2[e]));
                    *reinterpret_cast<__nv_bfloat16*>(sO + i * 128 + off8[i & 7]) = __float2bfloat16(o);
                }
                if (c == 40 && otid == 0) GDN_STAMP_ANY(54 + 2 * b);
            }
            if (c == 40 && otid == 0) GDN_STAMP_ANY(51);
            const long long tok0 = seq_tok0 + static_cast<long long>(c) * kChunk;
            const bool ragged = packed && n < kChunk;  // a full-box store would spill into the next sequence
            fence_proxy_async_smem();
            if (otid == 0) bulk_wait_read<0>();  // earlier stores have finished reading their staging tiles
            named_bar_sync(1, 128);
            if (!ragged) {
                if (otid == 0) {
                    tma_store_4d(&tmO, sO, 0, head, static_cast<int>(tok0), batch);
                    tma_store_4d(&tmO, sO + 8192, 64, head, static_cast<int>(tok0), batch);
                    bulk_commit();
                }
            } else {
                store_tile_rows<128>(sO, p.out, batch, tok0, head, n, otid);
            }
            if (c == 40 && otid == 0) GDN_STAMP_ANY(52);
        }
        if (otid == 0) bulk_wait_read<0>();
    } else {
        reg_dec<40>();
    }
    if (warp == 12) {
        // =============================================================== producer
        // Raw gate values are fetched two chunks ahead into registers (lane l holds tokens l and
        // l + 32), so that when a stage frees up only the TMA issue remains to be done.
        auto load_raw = [&](int c, float& a0, float& a1) {
            a0 = 0.f;
            a1 = 0.f;
            if (p.gate.ptr && c < nchunks) {
                const long long t0 = static_cast<long long>(c) * kChunk + lane;
                if (t0 < seq_tokens) a0 = p.gate.load(batch, seq_tok0 + t0, head);
                if (t0 + 32 < seq_tokens) a1 = p.gate.load(batch, seq_tok0 + t0 + 32, head);
            }
        };
        float ra0, ra1, rb0, rb1;  // raw gates of chunks c and c + 1
        load_raw(0, ra0, ra1);
        load_raw(1, rb0, rb1);
        for (int c = 0; c < nchunks; ++c) {
            const int s = c & 1;
            const int n = chunk_n(c);
            float g0 = ra0, g1 = ra1;
            ra0 = rb0;
            ra1 = rb1;
            load_raw(c + 2, rb0, rb1);
            // chunk-local cumulative gate
#pragma unroll
            for (int m = 1; m < 32; m <<= 1) {
                const float y0 = __shfl_up_sync(0xffffffffu, g0, m);
                const float y1 = __shfl_up_sync(0xffffffffu, g1, m);
                if (lane >= m) {
                    g0 += y0;
                    g1 += y1;
                }
            }
            g1 += __shfl_sync(0xffffffffu, g0, 31);
            // tokens past the end carry the last valid value (their raw gate was taken as 0)
            const float g_last = __shfl_sync(0xffffffffu, (n - 1 < 32) ? g0 : g1, (n - 1) & 31);
            const float e0 = p.scale * __expf(g0), e1 = p.scale * __expf(g1);  // epilogue factor for S q
            const float d0 = __expf(g_last - g0), d1 = __expf(g_last - g1);
            const float el = __expf(g_last);
            if (c == 40 && lane == 0) GDN_STAMP_ANY(20);
            mbar_wait_relaxed<200>(&bar_empty[s], static_cast<uint32_t>(((c >> 1) + 1) & 1), abort_flag);
            if (c == 40 && lane == 0) GDN_STAMP_ANY(21);
            if (c == 40 && lane == 0) GDN_STAMP_ANY(23);
            float* gb = gate_buf(c);
            gb[lane] = e0;
            gb[lane + 32] = e1;
            gb[64 + lane] = d0;
            gb[64 + lane + 32] = d1;
            if (lane == 0) gb[128] = el;
            __syncwarp();
            {
                // warp-uniform issue: one elected lane arms the barrier and launches the loads
                uint8_t* st = smem + s * L::kStage;
                const int tok = static_cast<int>(seq_tok0 + static_cast<long long>(c) * kChunk);
                const uint8_t* blk = p.blocks + (static_cast<size_t>(gchunk0 + c) * p.vh + head) * kUnitBlockBytes;
                // what the serial chain needs first (W for the first MMA, U for the pass that follows)
                // goes first and on its own barrier; P, K, Q are not needed before the second MMA group
                mbar_arrive_expect_tx_w(&bar_full[s], 2 * L::kTile);
                bulk_load_w(st + L::kOffU, blk, 2 * L::kTile, &bar_full[s]);
                if (emit_o) {
                    mbar_arrive_expect_tx_w(&bar_full2[s], L::kStage - 2 * L::kTile);
#pragma unroll
                    for (int a = 0; a < 2; ++a) tma_load_4d_w(st + L::kOffQ + a * 8192, &tmQ, &bar_full2[s], a * 64, khead, tok, batch);
                } else {
                    mbar_arrive_expect_tx_w(&bar_full2[s], L::kTile);  // no output: K is all the second group needs
                }
#pragma unroll
                for (int a = 0; a < 2; ++a) tma_load_4d_w(st + L::kOffK + a * 8192, &tmK, &bar_full2[s], a * 64, khead, tok, batch);
                if (emit_o) bulk_load_w(st + L::kOffP, blk + 2 * L::kTile, kChunk * kChunk * 2, &bar_full2[s]);
                if (c == 40 && lane == 0) GDN_STAMP_ANY(22);
            }
        }
    } else if (warp == 13) {
        // =============================================================== MMA issuer
        // The whole warp runs this loop with warp-uniform values; one elected lane issues.
        {
            constexpr uint32_t id_sw = make_idesc_bf16(128, 64, false, false, true);
            constexpr uint32_t id_sq = make_idesc_bf16(128, 64, false, false);
            constexpr uint32_t id_ds = make_idesc_bf16(128, 128, false, true);
            // one base descriptor per tile and stage; K-steps are constant offsets from them
            uint64_t dW[2], dQ[2], dK[2], dP[2];
#pragma unroll
            for (int s = 0; s < 2; ++s) {
                const uint32_t st = smem_u32(smem + s * L::kStage);
                dW[s] = make_smem_desc_sw128(st + L::kOffW, 0, 1024);     // K-major B
                dQ[s] = make_smem_desc_sw128(st + L::kOffQ, 0, 1024);     // K-major B
                dK[s] = make_smem_desc_sw128(st + L::kOffK, 8192, 1024);  // MN-major B
                dP[s] = make_smem_desc_sw128(st + L::kOffP, 0, 1024);     // K-major B
            }
            const uint32_t tS = tmem + kTmSbf, tD1 = tmem + kTmD1, tDS = tmem + kTmDS, tO2 = tmem + kTmO2;
            const uint32_t tUa = tmem + kTmUnA, tUb = tmem + kTmUnB;
            for (int c = 0; c < nchunks; ++c) {
                const int s = c & 1;
                const uint32_t par = static_cast<uint32_t>(c & 1);
                const uint64_t w = dW[s], q = dQ[s], k = dK[s], pp = dP[s];
                if (c == 40) GDN_STAMP_ANY(29);
                mbar_wait(&bar_full[s], static_cast<uint32_t>((c >> 1) & 1), abort_flag);
                tc_fence_after_sync();
                if (c == 40) GDN_STAMP_ANY(30);
                if (c == 40) GDN_STAMP_ANY(31);
                mbar_wait(bar_sbf, par, abort_flag);
                tc_fence_after_sync();
                if (c == 40) GDN_STAMP_ANY(32);
                // D1 = -(S_bf W^T)
                mma_ts_k128_w<false>(tD1, tS, w, id_sw);
                mma_commit_w(bar_d1);
                if (c == 40) GDN_STAMP_ANY(33);
                // O1 = S_bf Q^T
                mbar_wait(&bar_full2[s], static_cast<uint32_t>((c >> 1) & 1), abort_flag);
                tc_fence_after_sync();
                if (emit_o) {
                    const uint32_t tO1 = tmem + ((c & 1) ? kTmO1b : kTmO1a);
                    mma_ts_k128_w<false>(tO1, tS, q, id_sq);
                }
                if (c == 40) GDN_STAMP_ANY(34);
                mbar_wait(bar_un, par, abort_flag);
                tc_fence_after_sync();
                if (c == 40) GDN_STAMP_ANY(35);
                // dS = Un_b K
                mma_ts_k64_w<false, 128>(tDS, tUb, k, id_ds);
                mma_commit_w(bar_ds);
                if (c == 40) GDN_STAMP_ANY(36);
                // O2 = Un_a P^T (its accumulator must have been drained by the previous epilogue)
                if (emit_o) {
                    if (c > 0) {
                        mbar_wait(bar_ofree, static_cast<uint32_t>((c - 1) & 1), abort_flag);
                        tc_fence_after_sync();
                    }
                    mma_ts_k64_w<false, 2>(tO2, tUa, pp, id_sq);
                    mma_commit_w(bar_o);
                }
                mma_commit_w(&bar_empty[s]);
                if (c == 40) GDN_STAMP_ANY(37);
                if (c == 41) GDN_STAMP_ANY(38);
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 512);
    if (tid == 0 && *abort_flag && p.status) atomicExch(p.status, 4);
}

// order[r] = the sequence with the r-th largest token count (ties: lower index first), for up to
// kMaxOrderedSeqs sequences.  One thread per sequence counts the sequences that go before its own.
constexpr int kMaxOrderedSeqs = 2048;

__global__ void __launch_bounds__(128) gdn_seq_order_kernel(const int* __restrict__ cu_seqlens, int num_seqs,
                                                            int* __restrict__ order) {
    __shared__ int len[kMaxOrderedSeqs];
    for (int j = threadIdx.x; j < num_seqs; j += blockDim.x) len[j] = cu_seqlens[j + 1] - cu_seqlens[j];
    __syncthreads();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= num_seqs) return;
    const int mine = len[i];
    int rank = 0;
    for (int j = 0; j < num_seqs; ++j) rank += (len[j] > mine) || (len[j] == mine && j < i);
    order[rank] = i;
}

}  // namespace gdn
