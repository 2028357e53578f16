// State propagation + output of chunked Gated DeltaNet prefill, warp-specialised.
// One CTA of 512 threads walks the chunks of one (sequence, v-head).  With T = (I + A)^-1 diag(beta) of
// the WY/UT transform folded into two precomputed matrices per chunk (prefill_zp.cuh),
//     Z = T^T diag(e^{g_L - g}) K   and   PT = scale tril(Q K^T .* e^{g_i - g_j}) T,
// the chunk step is
//     R  = V - e^{g} .* (K S^T)            (U_new = T R is never formed)
//     O  = scale * e^{g} .* (Q S^T) + PT R
//     S <- e^{g_L} S + R^T Z
// This is the path gdn_chunked_forward uses; it stands in for the reference's
// sm90_bf16_chunked_seq_state_update and sm90_bf16_gdn_chunked_compute_O
// (kernels/sm90_bf16_chunked_seq_state_update2.cuh, sm90_bf16_gdn_chunked_compute_O.cuh:23-530)
// and never writes per-chunk states.
//
// The only serial dependence between chunks runs through the state:
//     S_bf(c) -> [MMA] D1 = S_bf K^T -> [pass] R = V^T - e^g D1 -> [MMA] dS = R Z -> [pass] S, S_bf(c+1)
// Roles keep everything else off that chain:
//   warps 0-7   state warps: own the fp32 state in registers (row = TMEM lane, 64 columns each),
//               run the two passes of the chain
//   warps 8-11  output warps: O epilogue (scale, transpose through shared memory, coalesced stores)
//   warp 12     producer: chunk-local gate cumsum; per chunk one bulk copy of its Z, PT block of
//               the scratch and tensor copies of Q, K and V, into a two-stage ring
//   warp 13     one thread issues every tcgen05.mma and commits completion onto mbarriers
// All operands are transposed so that the 128 state rows are the MMA M dimension; S_bf and R are
// bf16 A operands in tensor memory; Q, K, Z, PT tiles are used as the copies delivered them.
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
    int d;  // head dim of the caller's tensors and states (a multiple of 8, at most 128); the kernel computes on 128
            // columns, the tensor maps fill the rest with zeros, states are read and written with a predicate
    float scale;
    int* status;
    const uint8_t* blocks;  // Z, PT of every (global chunk, v-head): kZPBlockBytes each
    // q/k L2 normalisation: NULL, or per (global chunk, k-head) 64 inverse key norms then 64 inverse query
    // norms (written by gdn_zp_kernel); they enter through the two per-token factors of a chunk
    const float* norms;
    // Segmented runs (few long sequences; see gdn_chunked_forward).  The state obeys
    // S' = S M_c + N_c per chunk, so a segment of chunks has a composite (M, N) as well.
    //   mode 0: one CTA walks the whole sequence (grid = sequences x heads, or heads x ranks with seq_order).
    //   mode 1: grid = (slots, heads, 2); blockIdx.x = slot of a (sequence, segment) pair (locate_segment),
    //           blockIdx.z = kind; no output.  kind 0 starts from S = 0 and ends with N of the segment;
    //           kind 1 starts from S = I with V taken as 0 and ends with M.
    //           Both are written in fp32 to seg_mn[(slot * vh + head) * 2 + kind].
    //   mode 2: grid = (slots, heads); starts from seg_start[slot * vh + head] (fp32), writes the
    //           output of its chunks; the last segment of a sequence writes the final state.
    int mode, seg_chunks, num_segments, num_seqs;
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
    // Z, PT in the order of a unit block of the scratch, so that one bulk copy fills both
    static constexpr int kOffQ = 0, kOffK = kTile, kOffV = 2 * kTile, kOffZ = 3 * kTile, kOffPT = 4 * kTile;
    static constexpr int kStage = 3 * kTile + kZPBlockBytes;  // Q, K, V, Z, PT
    static constexpr int kOffO = 2 * kStage;         // two output staging tiles
    static constexpr int kOffGate = kOffO + 2 * kTile;  // 3 x { scale e^g[64], -e^g[64], e^{gL} }
    static constexpr int kGateStride = (2 * 64 + 4) * 4;
    static constexpr int kOffBar = kOffGate + 3 * kGateStride;
    static constexpr int kBytes = kOffBar + 128 + 1024;
};

namespace fused {
constexpr int kThreads = 512;  // 16 warps = 4 warpgroups (the last holds the producer, the issuer and 2 idle warps)
constexpr uint32_t kTmSbf = 0;    // bf16 state, 64 columns
constexpr uint32_t kTmR = 64;     // bf16 R = V^T - e^g .* (S K^T), 32 columns
constexpr uint32_t kTmD1 = 128;   // fp32 S K^T, 64 columns
constexpr uint32_t kTmO1a = 192;  // fp32 S Q^T, even chunks
constexpr uint32_t kTmDS = 256;   // fp32 state increment, 128 columns
constexpr uint32_t kTmO1b = 384;  // fp32 S Q^T, odd chunks
constexpr uint32_t kTmO2 = 448;   // fp32 R PT^T

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
                         const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                         const FusedParams p) {
    using namespace ptx;
    using namespace fused;
    using L = FusedSmem;
    constexpr int D = 128;
    extern __shared__ uint8_t smem_raw[];
    // aligned by an offset from the array itself, so that the compiler still knows the pointer is shared memory
    uint8_t* smem = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kOffBar);
    uint64_t* bar_full = bars;        // [2]
    uint64_t* bar_empty = bars + 2;   // [2]
    uint64_t* bar_sbf = bars + 4;
    uint64_t* bar_d1 = bars + 5;
    uint64_t* bar_un = bars + 6;
    uint64_t* bar_ds = bars + 7;
    uint64_t* bar_o = bars + 8;
    uint64_t* bar_ofree = bars + 9;
    uint64_t* bar_full2 = bars + 10;  // [2]: Z, PT, Q of a stage (bar_full: K, V and the gate vectors)
    uint64_t* bar_go = bars + 12;     // state warps are past their chunk-boundary work: the epilogue may run
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
    int* abort_flag = reinterpret_cast<int*>(tmem_slot + 1);
    volatile int* issued = abort_flag + 1;  // chunks whose loads the producer has issued (read by the L2 prefetcher)

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    SegPos sp{0, 0, 1, 0};
    if (p.mode != 0) {
        sp = locate_segment(p.map, static_cast<int>(blockIdx.x), p.seg_chunks, p.num_segments, p.num_seqs);
        if (sp.seq < 0) return;  // packed mode launches an upper bound of slots
    }
    const int seq = p.mode != 0 ? sp.seq : (p.seq_order ? p.seq_order[blockIdx.y] : static_cast<int>(blockIdx.x));
    const int head = p.mode == 0 && p.seq_order ? static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.y);
    const int segment = sp.segment, seq_nseg = sp.nseg;
    const int seg_kind = p.mode == 1 ? static_cast<int>(blockIdx.z) : 0;
    const long long seg_idx = static_cast<long long>(blockIdx.x) * p.vh + head;  // modes 1, 2
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
    auto chunk_n = [&](int c) {
        const long long rem = seq_tokens - static_cast<long long>(c) * kChunk;
        return rem < kChunk ? static_cast<int>(rem) : kChunk;
    };
    auto gate_buf = [&](int c) { return reinterpret_cast<float*>(smem + L::kOffGate + (c % 3) * L::kGateStride); };

    if (tid == 0) {
        *abort_flag = 0;
        *issued = 0;
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
        // setmaxnreg moves registers inside the CTA's own pool (threads x the kernel's register count = 512 x 128);
        // a request the pool cannot serve blocks for ever: 8 state warps at 168, 4 output warps at 88, 4 others at 40.
        static_assert(32 * (8 * 168 + 4 * 88 + 4 * 40) <= kThreads * 128, "register pool of the CTA");
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
            grid_dep_wait();  // the start states come from the kernel launched just before this one
            const float4* src = reinterpret_cast<const float4*>(p.seg_start + seg_idx * (D * D) +
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
                                                              static_cast<long long>(row) * p.d + 64 * hf);
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const uint4 v = (row < p.d && 64 * hf + 8 * q < p.d) ? __ldg(src + q) : make_uint4(0u, 0u, 0u, 0u);
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
            // ---- R = V^T - e^g .* (S K^T) -> bf16 operand copy in tensor memory
            // This thread's 32 values of V^T come straight from the TMA tile (element (token, row)
            // of the swizzled layout), packed two tokens per register while the MMA is running.
            const uint8_t* sV = smem + (c & 1) * L::kStage + L::kOffV;
            uint32_t vpk[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) {
                const int i0 = 32 * hf + 2 * e;
                const uint32_t lo = *reinterpret_cast<const uint16_t*>(sV + i0 * 128 + uoff8[i0 & 7]);
                const uint32_t hi = *reinterpret_cast<const uint16_t*>(sV + (i0 + 1) * 128 + uoff8[(i0 + 1) & 7]);
                vpk[e] = zero_u ? 0u : (lo | (hi << 16));
            }
            const int nloc = n - 32 * hf;  // tokens of this half that exist
            // The state warps now idle until D1 arrives: the window in which the output warps (which
            // share the schedulers) run the previous chunk's epilogue without slowing the chain down.
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_go);
            mbar_wait(bar_d1, par, abort_flag);
            tc_fence_after_sync();
            {
                uint32_t r[32];
                tmem_ld32(tmem + kTmD1 + tm_lane + 32 * hf, r);  // S K^T
                float neg[32];                                    // -e^{g} of this half's tokens
#pragma unroll
                for (int e4 = 0; e4 < 8; ++e4) {
                    const float4 t = *reinterpret_cast<const float4*>(gb + 64 + 32 * hf + 4 * e4);
                    neg[4 * e4] = t.x; neg[4 * e4 + 1] = t.y; neg[4 * e4 + 2] = t.z; neg[4 * e4 + 3] = t.w;
                }
                tmem_wait_ld();
                uint32_t wa[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    float r0, r1;
                    unpk(fma2(pk(neg[2 * e], neg[2 * e + 1]), pk(__uint_as_float(r[2 * e]), __uint_as_float(r[2 * e + 1])),
                              pk(bf16_lo(vpk[e]), bf16_hi(vpk[e]))),
                         r0, r1);
                    // rows past the end of a sequence meet zero rows of Z and zero columns of PT; they are
                    // cleared all the same so that no stray Inf/NaN of a neighbouring sequence can enter
                    if (nloc < 32) {
                        if (2 * e >= nloc) r0 = 0.f;
                        if (2 * e + 1 >= nloc) r1 = 0.f;
                    }
                    wa[e] = pack_bf16(r0, r1);
                }
                tmem_st16(tmem + kTmR + tm_lane + 16 * hf, wa);
            }
            tmem_wait_st();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_un);
            // ---- S <- e^{g_L} S + dS
            const float eg_last = gb[128];
            const f2 eg2 = pk(eg_last, eg_last);
            mbar_wait(bar_ds, par, abort_flag);
            tc_fence_after_sync();
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
        }
        if (lane == 0) mbar_arrive(bar_go);  // releases the last chunk's epilogue
        // nothing is written once a wait of this CTA has given up (the results would be garbage)
        const bool healthy = *abort_flag == 0;
        if (!healthy) {
        } else if (p.mode == 1) {
            float4* d4 = reinterpret_cast<float4*>(p.seg_mn + (seg_idx * 2 + seg_kind) * (D * D) +
                                                   static_cast<long long>(row) * D + 64 * hf);
#pragma unroll
            for (int q = 0; q < 16; ++q) d4[q] = make_float4(S[4 * q], S[4 * q + 1], S[4 * q + 2], S[4 * q + 3]);
        } else if (p.state_out && (p.mode == 0 || segment == seq_nseg - 1)) {
            uint4* d4 = reinterpret_cast<uint4*>(p.state_out + seq * p.so_ss + head * p.so_sh +
                                                 static_cast<long long>(row) * p.d + 64 * hf);
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                uint4 v;
                v.x = pack_bf16(S[q * 8 + 0], S[q * 8 + 1]);
                v.y = pack_bf16(S[q * 8 + 2], S[q * 8 + 3]);
                v.z = pack_bf16(S[q * 8 + 4], S[q * 8 + 5]);
                v.w = pack_bf16(S[q * 8 + 6], S[q * 8 + 7]);
                if (row < p.d && 64 * hf + 8 * q < p.d) d4[q] = v;
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
            mbar_wait_relaxed<100>(bar_o, par, abort_flag);
            mbar_wait_relaxed<50>(bar_go, static_cast<uint32_t>((c + 1) & 1), abort_flag);
            tc_fence_after_sync();
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
            }
            const long long tok0 = seq_tok0 + static_cast<long long>(c) * kChunk;
            const bool ragged = packed && n < kChunk;  // a full-box store would spill into the next sequence
            fence_proxy_async_smem();
            if (otid == 0) bulk_wait_read<0>();  // earlier stores have finished reading their staging tiles
            named_bar_sync(1, 128);
            if (*abort_flag != 0) {
                // a wait has given up: the tile is garbage and stays on chip
            } else if (!ragged) {
                if (otid == 0) {
                    tma_store_4d(&tmO, sO, 0, head, static_cast<int>(tok0), batch);  // columns past the head dim are clipped
                    if (p.d > 64) tma_store_4d(&tmO, sO + 8192, 64, head, static_cast<int>(tok0), batch);
                    bulk_commit();
                }
            } else {
                store_tile_rows<128>(sO, p.out, batch, tok0, head, n, otid, p.d >> 3);
            }
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
        // the Z, PT blocks and the V tiles are read exactly once: first in line for eviction from L2
        const uint64_t once = l2_policy_evict_first();
        float ra0, ra1, rb0, rb1;  // raw gates of chunks c and c + 1
        load_raw(0, ra0, ra1);
        load_raw(1, rb0, rb1);
        // Everything up to here (and the state warps' load of the initial state) touches only the caller's
        // inputs and may run while the chunk-parallel kernel drains; its blocks and norm factors are read below.
        grid_dep_wait();
        for (int c = 0; c < nchunks; ++c) {
            const int s = c & 1;
            const int n = chunk_n(c);
            float g0 = ra0, g1 = ra1;
            ra0 = rb0;
            ra1 = rb1;
            load_raw(c + 2, rb0, rb1);
            float rk0 = 1.f, rk1 = 1.f, rq0 = 1.f, rq1 = 1.f;
            if (p.norms) {  // requested here, used after the wait for a free stage
                const float* nr = p.norms + (static_cast<size_t>(gchunk0 + c) * p.kh + khead) * 128;
                rk0 = __ldg(nr + lane);
                rk1 = __ldg(nr + 32 + lane);
                rq0 = __ldg(nr + 64 + lane);
                rq1 = __ldg(nr + 96 + lane);
            }
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
            const float d0 = -__expf(g0), d1 = -__expf(g1);  // factor of S k in R = v - e^g (S k)
            const float el = __expf(g_last);
            mbar_wait_relaxed<200>(&bar_empty[s], static_cast<uint32_t>(((c >> 1) + 1) & 1), abort_flag);
            float* gb = gate_buf(c);
            gb[lane] = e0 * rq0;
            gb[lane + 32] = e1 * rq1;
            gb[64 + lane] = d0 * rk0;
            gb[64 + lane + 32] = d1 * rk1;
            if (lane == 0) gb[128] = el;
            __syncwarp();
            {
                // warp-uniform issue: one elected lane arms the barrier and launches the loads
                uint8_t* st = smem + s * L::kStage;
                const int tok = static_cast<int>(seq_tok0 + static_cast<long long>(c) * kChunk);
                const uint8_t* blk = p.blocks + (static_cast<size_t>(gchunk0 + c) * p.vh + head) * kZPBlockBytes;
                // what the serial chain needs first (K for the first MMA, V for the pass that follows)
                // goes first and on its own barrier; Z, PT, Q are not needed before the second MMA group
                mbar_arrive_expect_tx_w(&bar_full[s], 2 * L::kTile);
#pragma unroll
                for (int a = 0; a < 2; ++a) tma_load_4d_w(st + L::kOffK + a * 8192, &tmK, &bar_full[s], a * 64, khead, tok, batch);
#pragma unroll
                for (int a = 0; a < 2; ++a) tma_load_4d_hint_w(st + L::kOffV + a * 8192, &tmV, &bar_full[s], a * 64, head, tok, batch, once);
                if (emit_o) {
                    mbar_arrive_expect_tx_w(&bar_full2[s], L::kTile + kZPBlockBytes);
                    bulk_load_hint_w(st + L::kOffZ, blk, kZPBlockBytes, &bar_full2[s], once);
#pragma unroll
                    for (int a = 0; a < 2; ++a) tma_load_4d_w(st + L::kOffQ + a * 8192, &tmQ, &bar_full2[s], a * 64, khead, tok, batch);
                } else {
                    mbar_arrive_expect_tx_w(&bar_full2[s], L::kTile);  // no output: Z is all the second group needs
                    bulk_load_hint_w(st + L::kOffZ, blk, L::kTile, &bar_full2[s], once);
                }
                if (lane == 0) *issued = c + 1;
            }
        }
    } else if (warp == 14) {
        // =============================================================== L2 prefetcher
        // With every SM running a chain, a stage's loads (requested one chunk time before they are needed)
        // take longer than that to arrive from DRAM.  This otherwise idle warp pulls the tiles of the chunk
        // kLead positions after the one the producer has just requested into L2, so that the producer's own
        // loads find them there.  A hint only: when its bounded wait runs out it simply stops.
        constexpr int kLead = 3;
        grid_dep_wait();
        if (lane == 0) {
            for (int c = kLead; c < nchunks; ++c) {
                int spins = 0;
                while (*issued < c - kLead + 1 && *abort_flag == 0 && ++spins < (1 << 22)) __nanosleep(256);
                if (*issued < c - kLead + 1) break;
                const int tok = static_cast<int>(seq_tok0 + static_cast<long long>(c) * kChunk);
                const uint8_t* blk = p.blocks + (static_cast<size_t>(gchunk0 + c) * p.vh + head) * kZPBlockBytes;
#pragma unroll
                for (int a = 0; a < 2; ++a) {
                    if (a * 64 >= p.d) break;  // nothing in memory behind the second half of a small head
                    tma_prefetch_4d(&tmK, a * 64, khead, tok, batch);
                    tma_prefetch_4d(&tmV, a * 64, head, tok, batch);
                    if (emit_o) tma_prefetch_4d(&tmQ, a * 64, khead, tok, batch);
                }
                bulk_prefetch_l2(blk, emit_o ? kZPBlockBytes : L::kTile);
            }
        }
    } else if (warp == 13) {
        // =============================================================== MMA issuer
        // The whole warp runs this loop with warp-uniform values; one elected lane issues.
        {
            constexpr uint32_t id_sq = make_idesc_bf16(128, 64, false, false);
            constexpr uint32_t id_ds = make_idesc_bf16(128, 128, false, true);
            // one base descriptor per tile and stage; K-steps are constant offsets from them
            uint64_t dK[2], dQ[2], dZ[2], dP[2];
#pragma unroll
            for (int s = 0; s < 2; ++s) {
                const uint32_t st = smem_u32(smem + s * L::kStage);
                dK[s] = make_smem_desc_sw128(st + L::kOffK, 0, 1024);     // K-major B
                dQ[s] = make_smem_desc_sw128(st + L::kOffQ, 0, 1024);     // K-major B
                dZ[s] = make_smem_desc_sw128(st + L::kOffZ, 8192, 1024);  // MN-major B
                dP[s] = make_smem_desc_sw128(st + L::kOffPT, 0, 1024);    // K-major B
            }
            const uint32_t tS = tmem + kTmSbf, tD1 = tmem + kTmD1, tDS = tmem + kTmDS, tO2 = tmem + kTmO2;
            const uint32_t tR = tmem + kTmR;
            for (int c = 0; c < nchunks; ++c) {
                const int s = c & 1;
                const uint32_t par = static_cast<uint32_t>(c & 1);
                const uint64_t k = dK[s], q = dQ[s], z = dZ[s], pp = dP[s];
                mbar_wait(&bar_full[s], static_cast<uint32_t>((c >> 1) & 1), abort_flag);
                tc_fence_after_sync();
                mbar_wait(bar_sbf, par, abort_flag);
                tc_fence_after_sync();
                // D1 = S_bf K^T
                mma_ts_k128_w<false>(tD1, tS, k, id_sq);
                mma_commit_w(bar_d1);
                // O1 = S_bf Q^T
                mbar_wait(&bar_full2[s], static_cast<uint32_t>((c >> 1) & 1), abort_flag);
                tc_fence_after_sync();
                if (emit_o) {
                    const uint32_t tO1 = tmem + ((c & 1) ? kTmO1b : kTmO1a);
                    mma_ts_k128_w<false>(tO1, tS, q, id_sq);
                }
                mbar_wait(bar_un, par, abort_flag);
                tc_fence_after_sync();
                // dS = R Z
                mma_ts_k64_w<false, 128>(tDS, tR, z, id_ds);
                mma_commit_w(bar_ds);
                // O2 = R PT^T (its accumulator must have been drained by the previous epilogue)
                if (emit_o) {
                    if (c > 0) {
                        mbar_wait(bar_ofree, static_cast<uint32_t>((c - 1) & 1), abort_flag);
                        tc_fence_after_sync();
                    }
                    mma_ts_k64_w<false, 2>(tO2, tR, pp, id_sq);
                    mma_commit_w(bar_o);
                }
                mma_commit_w(&bar_empty[s]);
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
