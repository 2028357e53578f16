// Chunk-to-chunk state propagation of chunked Gated DeltaNet prefill, optionally fused with
// the output computation.  One CTA of 256 threads walks the chunks of one (sequence, v-head):
//     U_new = U - W S^T                                  (h[c] = S is the state entering chunk c)
//     O     = scale * ( e^{g} .* (Q S^T) + tril(Q K^T .* e^{g_i - g_j}) U_new )
//     S    <- e^{g_L} S + U_new^T (K .* e^{g_L - g})
// Stands in for the reference's sm90_bf16_chunked_seq_state_update
// (kernels/sm90_bf16_chunked_seq_state_update2.cuh) and, when kComputeO is set, also for
// sm90_bf16_gdn_chunked_compute_O (kernels/sm90_bf16_gdn_chunked_compute_O.cuh:23-530) without
// ever writing the per-chunk states to memory.
//
// Everything is computed transposed so that the 128 state rows (dv) are the M dimension of
// the tcgen05 MMAs and map one-to-one onto the 128 tensor-memory lanes:
//   D1^T (dv x 64)  = U^T I  -  S_bf W^T     A = U tile read MN-major / S_bf in tensor memory
//   O1^T (dv x 64)  = S_bf Q^T
//   QK   (64 x 64)  = Q K^T                  -> P = masked, decayed, bf16, in shared memory
//   dS   (dv x dk)  = Un_b K                 A = bf16(U_new^T .* e^{g_L-g_j}) in tensor memory, B = K tile MN-major
//   O2^T (dv x 64)  = Un_a P^T               A = bf16(U_new^T) in tensor memory
// Q, K, W, U tiles arrive by TMA (128-byte swizzle) into a two-stage ring and are used
// as they are: every decay factor is folded into a small operand (P, Un_b) or into an
// epilogue.  The running state stays in fp32 registers (64 per thread); a bf16 copy in
// tensor memory is the A operand of the next chunk.
#pragma once
#include <cuda.h>

#include "prefill_common.cuh"

namespace gdn {

struct SeqParams {
    ChunkMap map;
    ScalarView gate;   // ptr == NULL: no decay
    int gate_is_raw;   // 1: per-token log-decay; 0: chunk-local cumsum
    TokenView u_out;   // kEmitUnew: where U_new goes (normally the U tensor itself)
    TokenView out;     // kComputeO
    const __nv_bfloat16* state_in;
    long long si_ss, si_sh;
    __nv_bfloat16* state_out;  // final state or NULL
    long long so_ss, so_sh;
    __nv_bfloat16* chunk_states;  // kEmitH: (global chunk, vh, dv, dk) contiguous
    int kh, vh;
    float scale;
    int* status;
};

struct SeqSmem {
    static constexpr int D = 128;
    static constexpr int kTile = kChunk * D * 2;  // 16 KB
    static constexpr int kStage = 4 * kTile;      // Q, K, W, U
    static constexpr int kOffQ = 0, kOffK = kTile, kOffW = 2 * kTile, kOffU = 3 * kTile;
    static constexpr int kOffP = 2 * kStage;      // 64x64 bf16 K-major
    static constexpr int kOffI = kOffP + 8192;    // identity 64x64 bf16 K-major
    static constexpr int kOffO = kOffI + 8192;    // output staging 64 x 128 bf16
    static constexpr int kOffVec = kOffO + kTile; // g[64], e^g[64], e^{gL-g}[64], scratch[80]
    static constexpr int kBytes = kOffVec + (3 * 64 + 80) * 4 + 1024;
};

// tensor-memory columns (512 allocated)
constexpr uint32_t kTmSbf = 0;     // bf16 state, 64 columns
constexpr uint32_t kTmUnA = 64;    // bf16 U_new^T, 32 columns
constexpr uint32_t kTmUnB = 96;    // bf16 U_new^T .* decay, 32 columns
constexpr uint32_t kTmD1 = 128;    // fp32 U_new^T, 64 columns
constexpr uint32_t kTmQK = 192;    // fp32 Q K^T (M=64 layout), 64 columns
constexpr uint32_t kTmDS = 256;    // fp32 state increment, 128 columns
constexpr uint32_t kTmO1 = 384;    // 64 columns
constexpr uint32_t kTmO2 = 448;    // 64 columns

template <bool kComputeO, bool kEmitH, bool kEmitUnew>
__global__ void __launch_bounds__(256, 1) gdn_seq_kernel(const __grid_constant__ CUtensorMap tmQ,
                                                         const __grid_constant__ CUtensorMap tmK,
                                                         const __grid_constant__ CUtensorMap tmW,
                                                         const __grid_constant__ CUtensorMap tmU,
                                                         const SeqParams p) {
    using namespace ptx;
    using L = SeqSmem;
    constexpr int D = 128;
    extern __shared__ uint8_t smem_raw[];
    // aligned by an offset from the array itself, so that the compiler still knows the pointer is shared memory
    uint8_t* smem = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* sP = smem + L::kOffP;
    uint8_t* sI = smem + L::kOffI;
    uint8_t* sO = smem + L::kOffO;
    float* sG = reinterpret_cast<float*>(smem + L::kOffVec);
    float* sEg = sG + 64;
    float* sDec = sEg + 64;
    float* sScr = sDec + 64;
    __shared__ uint64_t bar_full[2], bar_a, bar_b, bar_c, bar_d;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int lq = warp & 3, hf = warp >> 2;
    const int row = 32 * lq + lane;  // state row (dv index) = tensor-memory lane
    const uint32_t tm_lane = static_cast<uint32_t>(32 * lq) << 16;
    const int seq = blockIdx.x, head = blockIdx.y;
    const int khead = head / (p.vh / p.kh);

    // chunks of this sequence
    int nchunks, batch, gchunk0;
    long long seq_tok0, seq_tokens;
    if (p.map.cu_seqlens) {
        const int bos = p.map.cu_seqlens[seq], eos = p.map.cu_seqlens[seq + 1];
        seq_tok0 = bos;
        seq_tokens = eos - bos;
        batch = 0;
        gchunk0 = p.map.cu_chunks ? p.map.cu_chunks[seq] : 0;
    } else {
        seq_tok0 = 0;
        seq_tokens = p.map.seq_len;
        batch = seq;
        gchunk0 = seq * p.map.chunks_per_seq;
    }
    nchunks = static_cast<int>((seq_tokens + kChunk - 1) / kChunk);

    if (tid == 0) {
        abort_flag = 0;
        mbar_init(&bar_full[0], 1);
        mbar_init(&bar_full[1], 1);
        mbar_init(&bar_a, 1);
        mbar_init(&bar_b, 1);
        mbar_init(&bar_c, 1);
        mbar_init(&bar_d, 1);
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(&tmem_slot, 512);

    auto issue_loads = [&](int c) {
        uint8_t* st = smem + (c & 1) * L::kStage;
        const int tok = static_cast<int>(seq_tok0 + static_cast<long long>(c) * kChunk);
        mbar_arrive_expect_tx(&bar_full[c & 1], (kComputeO ? 4 : 3) * L::kTile);
#pragma unroll
        for (int a = 0; a < 2; ++a) {
            if (kComputeO) tma_load_4d(st + L::kOffQ + a * 8192, &tmQ, &bar_full[c & 1], a * 64, khead, tok, batch);
            tma_load_4d(st + L::kOffK + a * 8192, &tmK, &bar_full[c & 1], a * 64, khead, tok, batch);
            tma_load_4d(st + L::kOffW + a * 8192, &tmW, &bar_full[c & 1], a * 64, head, tok, batch);
            tma_load_4d(st + L::kOffU + a * 8192, &tmU, &bar_full[c & 1], a * 64, head, tok, batch);
        }
    };
    __syncthreads();  // barriers initialised
    if (tid == 0 && nchunks > 0) issue_loads(0);

    // identity tile (bf16 1.0 = 0x3F80)
    for (int idx = tid; idx < 64 * 8; idx += 256) {
        const int r = idx >> 3, ch = idx & 7;
        uint32_t w[4] = {0, 0, 0, 0};
        if ((r >> 3) == ch) w[(r & 7) >> 1] = (r & 1) ? 0x3F800000u : 0x00003F80u;
        *reinterpret_cast<uint4*>(sI + sw128_offset(r, ch * 8)) = make_uint4(w[0], w[1], w[2], w[3]);
    }
    // running state: thread owns row `row`, columns [64*hf, 64*hf + 64)
    float S[64];
    if (p.state_in) {
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
    tc_fence_before_sync();
    __syncthreads();  // tensor-memory address visible
    tc_fence_after_sync();
    const uint32_t tmem = tmem_slot;

    auto store_state_operand = [&]() {
        // bf16 copy of S -> tensor memory columns [32*hf, 32*hf + 32) of the A operand
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            uint32_t w[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) w[e] = pack_bf16(S[q * 32 + 2 * e], S[q * 32 + 2 * e + 1]);
            tmem_st16(tmem + kTmSbf + tm_lane + 32 * hf + 16 * q, w);
        }
    };
    auto store_state_global = [&](__nv_bfloat16* dst) {
        uint4* d4 = reinterpret_cast<uint4*>(dst + static_cast<long long>(row) * D + 64 * hf);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            uint4 v;
            v.x = pack_bf16(S[q * 8 + 0], S[q * 8 + 1]);
            v.y = pack_bf16(S[q * 8 + 2], S[q * 8 + 3]);
            v.z = pack_bf16(S[q * 8 + 4], S[q * 8 + 5]);
            v.w = pack_bf16(S[q * 8 + 6], S[q * 8 + 7]);
            d4[q] = v;
        }
    };
    store_state_operand();
    tmem_wait_st();

    // gate values of chunk 0, one token per thread of warps 0-1
    auto load_gate = [&](int c) -> float {
        if (tid >= 64 || !p.gate.ptr || c >= nchunks) return 0.f;
        const long long t = static_cast<long long>(c) * kChunk + tid;
        return t < seq_tokens ? p.gate.load(batch, seq_tok0 + t, head) : 0.f;
    };
    float g_mine = load_gate(0);
    fence_proxy_async_smem();  // identity tile
    tc_fence_before_sync();
    __syncthreads();

    for (int c = 0; c < nchunks; ++c) {
        const int stage = c & 1;
        uint8_t* st = smem + stage * L::kStage;
        const uint32_t par = static_cast<uint32_t>(c & 1);
        const long long tok0 = seq_tok0 + static_cast<long long>(c) * kChunk;
        const long long rem = seq_tokens - static_cast<long long>(c) * kChunk;
        const int n = rem < kChunk ? static_cast<int>(rem) : kChunk;

        if (tid == 0 && c + 1 < nchunks) issue_loads(c + 1);
        if (kEmitH) {
            store_state_global(p.chunk_states + (static_cast<long long>(gchunk0 + c) * p.vh + head) * D * D);
        }
        // ---- chunk-local cumulative gate
        if (tid < 64) {
            float g = g_mine;  // zero past the end of the sequence
            if (p.gate_is_raw) {
#pragma unroll
                for (int m = 1; m < 32; m <<= 1) {
                    const float y = __shfl_up_sync(0xffffffffu, g, m);
                    if (lane >= m) g += y;
                }
                if (tid == 31) sScr[0] = g;
            } else if (tid < n) {
                sScr[1 + tid] = g;  // needed to extend the last valid value
            }
            g_mine = g;
        }
        __syncthreads();
        if (tid < 64) {
            float g = g_mine;
            if (p.gate_is_raw) {
                if (tid >= 32) g += sScr[0];
            } else {
                if (tid >= n) g = p.gate.ptr ? sScr[1 + n - 1] : 0.f;
            }
            sG[tid] = g;
            sEg[tid] = __expf(g);
        }
        __syncthreads();
        if (tid < 64) sDec[tid] = __expf(sG[n - 1] - sG[tid]);
        g_mine = load_gate(c + 1);
        const float eg_last = sEg[n - 1];
        __syncthreads();

        // ---- first wave of MMAs
        mbar_wait(&bar_full[stage], static_cast<uint32_t>((c >> 1) & 1), &abort_flag);
        if (tid == 0) {
            tc_fence_after_sync();
            if (kComputeO) {
                constexpr uint32_t id_qk = make_idesc_bf16(64, 64, false, false);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t off = (ks / 4) * 8192 + (ks % 4) * 32;
                    mma_ss(tmem + kTmQK, make_smem_desc_sw128(smem_u32(st + L::kOffQ) + off, 0, 1024),
                           make_smem_desc_sw128(smem_u32(st + L::kOffK) + off, 0, 1024), id_qk, ks > 0);
                }
                mma_commit(&bar_a);
            }
            constexpr uint32_t id_ui = make_idesc_bf16(128, 64, true, false);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                mma_ss(tmem + kTmD1, make_smem_desc_sw128(smem_u32(st + L::kOffU) + ks * 2048, 8192, 1024),
                       make_smem_desc_sw128(smem_u32(sI) + ks * 32, 0, 1024), id_ui, ks > 0);
            }
            constexpr uint32_t id_sw = make_idesc_bf16(128, 64, false, false, true);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const uint32_t off = (ks / 4) * 8192 + (ks % 4) * 32;
                mma_ts(tmem + kTmD1, tmem + kTmSbf + ks * 8,
                       make_smem_desc_sw128(smem_u32(st + L::kOffW) + off, 0, 1024), id_sw, 1);
            }
            mma_commit(&bar_b);
            if (kComputeO) {
                constexpr uint32_t id_sq = make_idesc_bf16(128, 64, false, false);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t off = (ks / 4) * 8192 + (ks % 4) * 32;
                    mma_ts(tmem + kTmO1, tmem + kTmSbf + ks * 8,
                           make_smem_desc_sw128(smem_u32(st + L::kOffQ) + off, 0, 1024), id_sq, ks > 0);
                }
            }
        }
        __syncwarp();

        // ---- P = tril(Q K^T .* e^{g_i - g_j}) -> bf16 K-major tile
        if (kComputeO) {
            mbar_wait(&bar_a, par, &abort_flag);
            tc_fence_after_sync();
            uint32_t r[32];
            tmem_ld32(tmem + kTmQK + tm_lane + 32 * hf, r);
            tmem_wait_ld();
            if (lane < 16) {
                const int i = 16 * lq + lane;
                const float gi = sG[i];
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    uint32_t w[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        float v[2];
#pragma unroll
                        for (int q = 0; q < 2; ++q) {
                            const int j = 32 * hf + ch * 8 + e * 2 + q;
                            v[q] = (j <= i && i < n) ? __uint_as_float(r[ch * 8 + e * 2 + q]) * __expf(gi - sG[j]) : 0.f;
                        }
                        w[e] = pack_bf16(v[0], v[1]);
                    }
                    *reinterpret_cast<uint4*>(sP + sw128_offset(i, 32 * hf + ch * 8)) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
            fence_proxy_async_smem();
        }

        // ---- U_new^T: mask rows past the end, make the two bf16 operand copies
        mbar_wait(&bar_b, par, &abort_flag);
        tc_fence_after_sync();
        {
            uint32_t r[32];
            tmem_ld32(tmem + kTmD1 + tm_lane + 32 * hf, r);
            tmem_wait_ld();
            uint32_t wa[16], wb[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) {
                const int i0 = 32 * hf + 2 * e;
                const float u0 = i0 < n ? __uint_as_float(r[2 * e]) : 0.f;
                const float u1 = i0 + 1 < n ? __uint_as_float(r[2 * e + 1]) : 0.f;
                wa[e] = pack_bf16(u0, u1);
                wb[e] = pack_bf16(u0 * sDec[i0], u1 * sDec[i0 + 1]);
            }
            tmem_st16(tmem + kTmUnA + tm_lane + 16 * hf, wa);
            tmem_st16(tmem + kTmUnB + tm_lane + 16 * hf, wb);
            if (kEmitUnew) {
                __nv_bfloat16* ub = p.u_out.ptr + batch * p.u_out.sb + tok0 * p.u_out.st +
                                    static_cast<long long>(head) * p.u_out.sh + row;
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    const int i0 = 32 * hf + 2 * e;
                    if (i0 < n) ub[i0 * p.u_out.st] = __ushort_as_bfloat16(static_cast<unsigned short>(wa[e] & 0xFFFFu));
                    if (i0 + 1 < n) ub[(i0 + 1) * p.u_out.st] = __ushort_as_bfloat16(static_cast<unsigned short>(wa[e] >> 16));
                }
            }
            tmem_wait_st();
        }
        tc_fence_before_sync();
        __syncthreads();

        // ---- second wave of MMAs
        if (tid == 0) {
            tc_fence_after_sync();
            constexpr uint32_t id_ds = make_idesc_bf16(128, 128, false, true);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                mma_ts(tmem + kTmDS, tmem + kTmUnB + ks * 8,
                       make_smem_desc_sw128(smem_u32(st + L::kOffK) + ks * 2048, 8192, 1024), id_ds, ks > 0);
            }
            mma_commit(&bar_c);
            if (kComputeO) {
                constexpr uint32_t id_o2 = make_idesc_bf16(128, 64, false, false);
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    mma_ts(tmem + kTmO2, tmem + kTmUnA + ks * 8,
                           make_smem_desc_sw128(smem_u32(sP) + ks * 32, 0, 1024), id_o2, ks > 0);
                }
                mma_commit(&bar_d);
            }
        }
        __syncwarp();

        // ---- S <- e^{g_L} S + dS ; refresh the bf16 operand copy
        mbar_wait(&bar_c, par, &abort_flag);
        tc_fence_after_sync();
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            uint32_t r[32];
            tmem_ld32(tmem + kTmDS + tm_lane + 64 * hf + 32 * q, r);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) S[q * 32 + e] = fmaf(S[q * 32 + e], eg_last, __uint_as_float(r[e]));
        }
        store_state_operand();

        // ---- O = scale (e^{g_i} O1 + O2), transposed through shared memory
        if (kComputeO) {
            mbar_wait(&bar_d, par, &abort_flag);
            tc_fence_after_sync();
            uint32_t r1[32], r2[32];
            tmem_ld32(tmem + kTmO1 + tm_lane + 32 * hf, r1);
            tmem_ld32(tmem + kTmO2 + tm_lane + 32 * hf, r2);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) {
                const int i = 32 * hf + e;
                const float o = p.scale * fmaf(sEg[i], __uint_as_float(r1[e]), __uint_as_float(r2[e]));
                *reinterpret_cast<__nv_bfloat16*>(sO + stage_off<D>(i, row >> 3) + (row & 7) * 2) = __float2bfloat16(o);
            }
            __syncthreads();
            store_staged_tile<D, 256>(sO, p.out, batch, tok0, head, n, tid);
        }
        tmem_wait_st();
        tc_fence_before_sync();
        __syncthreads();
    }

    if (p.state_out) store_state_global(p.state_out + seq * p.so_ss + head * p.so_sh);
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 512);
    if (tid == 0 && abort_flag && p.status) atomicExch(p.status, 3);
}

}  // namespace gdn
