// Recurrent Gated DeltaNet step (decode, speculative verify, short prefill).
//
// Replaces the reference's fused_recurrent_gated_delta_rule_bf16
// (gdn_cuda/include/gdn_cuda/kernels/sm90_bf16_gdn_recurrent.cuh:20-440) with the
// canonical update order  S <- exp(g) S ;  S <- S + beta (v - S k) k^T ;  o = scale S q.
//
// The kernel is bound by HBM traffic: per (sequence, v-head) it must read and write the
// dv x dk bf16 state once.  Work unit = a tile of 32 state rows (32 x DK bf16, 8 KB at
// DK = 128).  A persistent CTA of 128 threads walks tiles round-robin; tiles are fetched
// ahead into a ring of shared-memory buffers by bulk asynchronous copies (one elected
// thread issues them, completion is signalled on an mbarrier), so several tiles per CTA
// are in flight while the current one is processed.  Each thread keeps 4 rows x DK/16
// columns of the tile in fp32 registers; the two products S.k and S.q are row sums reduced
// over 16 lanes with shuffles, both taken from the same pass over the old state:
//     r = v - e^g (S k),   S' = e^g S + beta r k^T,   o = scale (e^g (S q) + beta r (k.q)).
// New states leave through coalesced 8-byte stores straight from registers.
#pragma once
#include "sm100_ptx.cuh"

namespace gdn {

struct RecurrentParams {
    const __nv_bfloat16* q;
    const __nv_bfloat16* k;
    const __nv_bfloat16* v;
    __nv_bfloat16* out;
    int64_t q_sb, q_st, q_sh;
    int64_t k_sb, k_st, k_sh;
    int64_t v_sb, v_st, v_sh;
    int64_t o_sb, o_st, o_sh;
    const void* beta;
    const void* gate;
    int beta_f32, gate_f32;
    int64_t beta_sb, beta_st, beta_sh;
    int64_t gate_sb, gate_st, gate_sh;
    const __nv_bfloat16* state_in;
    __nv_bfloat16* state_out;
    int64_t si_ss, si_sh, so_ss, so_sh;
    const int* cu_seqlens;
    const int* num_accepted;
    int batch, seq_len, kh, vh, dv;
    float scale;
    int is_qk_norm, store_step;
    long long num_tiles;
    int* status;
};

constexpr int kRecTileRows = 32;
constexpr int kRecStages = 4;
constexpr int kRecThreads = 128;

template <int DK>
constexpr int recurrent_smem_bytes() {
    return kRecStages * kRecTileRows * DK * 2 + 128;
}

template <int DK>
__global__ void __launch_bounds__(kRecThreads, (DK <= 128 ? 4 : 2)) gdn_recurrent_kernel(const RecurrentParams p) {
    using namespace ptx;
    constexpr int NP = DK / 64;  // 64-column pieces; each lane owns 4 columns of every piece
    constexpr int TILE_BYTES = kRecTileRows * DK * 2;
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + kRecStages * TILE_BYTES);
    __shared__ int abort_flag;

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int half = lane >> 4, l16 = lane & 15;
    const int rblocks = p.dv / kRecTileRows;
    const bool has_in = p.state_in != nullptr;
    const int rep = p.vh / p.kh;

    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < kRecStages; ++s) mbar_init(&full[s], 1);
        mbar_fence_init();
    }
    __syncthreads();

    auto tile_src = [&](long long tile) -> const __nv_bfloat16* {
        const int rb = static_cast<int>(tile % rblocks);
        const long long sh = tile / rblocks;
        const int head = static_cast<int>(sh % p.vh);
        const long long seq = sh / p.vh;
        return p.state_in + seq * p.si_ss + head * p.si_sh + static_cast<long long>(rb) * kRecTileRows * DK;
    };

    // prologue: fill the ring
    if (has_in && tid == 0) {
        long long t = blockIdx.x;
        for (int s = 0; s < kRecStages - 1 && t < p.num_tiles; ++s, t += gridDim.x) {
            mbar_arrive_expect_tx(&full[s], TILE_BYTES);
            bulk_load(smem + s * TILE_BYTES, tile_src(t), TILE_BYTES, &full[s]);
        }
    }

    long long it = 0;
    for (long long tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++it) {
        const int stage = static_cast<int>(it % kRecStages);
        const uint32_t parity = static_cast<uint32_t>((it / kRecStages) & 1);
        if (has_in && tid == 0) {
            // the stage consumed in the previous iteration is free (block-wide barrier below)
            const long long nt = tile + static_cast<long long>(kRecStages - 1) * gridDim.x;
            if (nt < p.num_tiles) {
                const int ns = static_cast<int>((it + kRecStages - 1) % kRecStages);
                mbar_arrive_expect_tx(&full[ns], TILE_BYTES);
                bulk_load(smem + ns * TILE_BYTES, tile_src(nt), TILE_BYTES, &full[ns]);
            }
        }
        const int rb = static_cast<int>(tile % rblocks);
        const long long sh = tile / rblocks;
        const int head = static_cast<int>(sh % p.vh);
        const int seq = static_cast<int>(sh / p.vh);
        const int khead = head / rep;

        long long tok0;
        int ntok;
        if (p.cu_seqlens) {
            tok0 = p.cu_seqlens[seq];
            ntok = p.cu_seqlens[seq + 1] - static_cast<int>(tok0);
        } else {
            tok0 = 0;
            ntok = p.seq_len;
        }
        if (p.num_accepted) ntok = min(ntok, p.num_accepted[seq]);
        const long long bidx = p.cu_seqlens ? 0 : seq;

        // ---- state tile -> registers
        float S[4][NP * 4];
        if (has_in) {
            mbar_wait(&full[stage], parity, &abort_flag);
            const uint8_t* tile_s = smem + stage * TILE_BYTES;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int row = warp * 8 + 2 * j + half;
#pragma unroll
                for (int pc = 0; pc < NP; ++pc) {
                    const uint2 w = *reinterpret_cast<const uint2*>(tile_s + (row * DK + pc * 64 + l16 * 4) * 2);
                    S[j][pc * 4 + 0] = bf16_lo(w.x);
                    S[j][pc * 4 + 1] = bf16_hi(w.x);
                    S[j][pc * 4 + 2] = bf16_lo(w.y);
                    S[j][pc * 4 + 3] = bf16_hi(w.y);
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int c = 0; c < NP * 4; ++c) S[j][c] = 0.f;
        }
        __syncthreads();  // every thread has read this stage: it may be refilled

        // ---- token loop (inputs of token t+1 are fetched while token t is computed)
        uint2 kw[NP], qw[NP];
        float vr[4], beta_t = 0.f, g_t = 0.f;
        auto load_token = [&](int t, uint2* kk, uint2* qq, float* vv, float& bt, float& gt) {
            const long long tok = tok0 + t;
            const __nv_bfloat16* kp = p.k + bidx * p.k_sb + tok * p.k_st + khead * p.k_sh;
            const __nv_bfloat16* qp = p.q + bidx * p.q_sb + tok * p.q_st + khead * p.q_sh;
#pragma unroll
            for (int pc = 0; pc < NP; ++pc) {
                kk[pc] = __ldg(reinterpret_cast<const uint2*>(kp + pc * 64 + l16 * 4));
                qq[pc] = __ldg(reinterpret_cast<const uint2*>(qp + pc * 64 + l16 * 4));
            }
            const __nv_bfloat16* vp = p.v + bidx * p.v_sb + tok * p.v_st + head * p.v_sh + rb * kRecTileRows;
#pragma unroll
            for (int j = 0; j < 4; ++j) vv[j] = __bfloat162float(vp[warp * 8 + 2 * j + half]);
            const long long bo = bidx * p.beta_sb + tok * p.beta_st + head * p.beta_sh;
            bt = p.beta_f32 ? reinterpret_cast<const float*>(p.beta)[bo]
                            : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.beta)[bo]);
            if (p.gate) {
                const long long go = bidx * p.gate_sb + tok * p.gate_st + head * p.gate_sh;
                gt = p.gate_f32 ? reinterpret_cast<const float*>(p.gate)[go]
                                : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.gate)[go]);
            } else {
                gt = 0.f;
            }
        };
        if (ntok > 0) load_token(0, kw, qw, vr, beta_t, g_t);

        for (int t = 0; t < ntok; ++t) {
            float kc[NP * 4], qc[NP * 4];
#pragma unroll
            for (int pc = 0; pc < NP; ++pc) {
                kc[pc * 4 + 0] = bf16_lo(kw[pc].x); kc[pc * 4 + 1] = bf16_hi(kw[pc].x);
                kc[pc * 4 + 2] = bf16_lo(kw[pc].y); kc[pc * 4 + 3] = bf16_hi(kw[pc].y);
                qc[pc * 4 + 0] = bf16_lo(qw[pc].x); qc[pc * 4 + 1] = bf16_hi(qw[pc].x);
                qc[pc * 4 + 2] = bf16_lo(qw[pc].y); qc[pc * 4 + 3] = bf16_hi(qw[pc].y);
            }
            uint2 kn[NP], qn[NP];
            float vn[4], beta_n = 0.f, g_n = 0.f;
            if (t + 1 < ntok) load_token(t + 1, kn, qn, vn, beta_n, g_n);

            float kq = 0.f;
            float inv_k = 1.f, inv_q = 1.f;
            if (p.is_qk_norm) {
                float sk = 0.f, sq = 0.f;
#pragma unroll
                for (int c = 0; c < NP * 4; ++c) {
                    sk = fmaf(kc[c], kc[c], sk);
                    sq = fmaf(qc[c], qc[c], sq);
                }
#pragma unroll
                for (int m = 1; m < 16; m <<= 1) {
                    sk += __shfl_xor_sync(0xffffffffu, sk, m);
                    sq += __shfl_xor_sync(0xffffffffu, sq, m);
                }
                inv_k = rsqrtf(sk + 1e-6f);
                inv_q = rsqrtf(sq + 1e-6f);
#pragma unroll
                for (int c = 0; c < NP * 4; ++c) {
                    kc[c] *= inv_k;
                    qc[c] *= inv_q;
                }
            }
            float dk_[4], dq_[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                dk_[j] = 0.f;
                dq_[j] = 0.f;
            }
#pragma unroll
            for (int c = 0; c < NP * 4; ++c) {
                kq = fmaf(kc[c], qc[c], kq);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    dk_[j] = fmaf(S[j][c], kc[c], dk_[j]);
                    dq_[j] = fmaf(S[j][c], qc[c], dq_[j]);
                }
            }
#pragma unroll
            for (int m = 1; m < 16; m <<= 1) {
                kq += __shfl_xor_sync(0xffffffffu, kq, m);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    dk_[j] += __shfl_xor_sync(0xffffffffu, dk_[j], m);
                    dq_[j] += __shfl_xor_sync(0xffffffffu, dq_[j], m);
                }
            }
            const float eg = __expf(g_t);
            float o_mine = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float r = vr[j] - eg * dk_[j];
                const float br = beta_t * r;
                const float o = p.scale * fmaf(eg, dq_[j], br * kq);
                if (l16 == j) o_mine = o;
#pragma unroll
                for (int c = 0; c < NP * 4; ++c) S[j][c] = fmaf(eg, S[j][c], br * kc[c]);
            }
            const long long tok = tok0 + t;
            if (l16 < 4) {
                __nv_bfloat16* op = p.out + bidx * p.o_sb + tok * p.o_st + head * p.o_sh + rb * kRecTileRows;
                op[warp * 8 + 2 * l16 + half] = __float2bfloat16(o_mine);
            }
            if (p.store_step) {
                const long long sidx = p.cu_seqlens ? tok : (static_cast<long long>(seq) * p.seq_len + t);
                __nv_bfloat16* sp = p.state_out + sidx * p.so_ss + head * p.so_sh +
                                    static_cast<long long>(rb) * kRecTileRows * DK;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int row = warp * 8 + 2 * j + half;
#pragma unroll
                    for (int pc = 0; pc < NP; ++pc) {
                        uint2 w;
                        w.x = pack_bf16(S[j][pc * 4 + 0], S[j][pc * 4 + 1]);
                        w.y = pack_bf16(S[j][pc * 4 + 2], S[j][pc * 4 + 3]);
                        *reinterpret_cast<uint2*>(sp + row * DK + pc * 64 + l16 * 4) = w;
                    }
                }
            }
#pragma unroll
            for (int pc = 0; pc < NP; ++pc) {
                kw[pc] = kn[pc];
                qw[pc] = qn[pc];
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) vr[j] = vn[j];
            beta_t = beta_n;
            g_t = g_n;
        }

        if (!p.store_step) {
            __nv_bfloat16* sp = p.state_out + static_cast<long long>(seq) * p.so_ss + head * p.so_sh +
                                static_cast<long long>(rb) * kRecTileRows * DK;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int row = warp * 8 + 2 * j + half;
#pragma unroll
                for (int pc = 0; pc < NP; ++pc) {
                    uint2 w;
                    w.x = pack_bf16(S[j][pc * 4 + 0], S[j][pc * 4 + 1]);
                    w.y = pack_bf16(S[j][pc * 4 + 2], S[j][pc * 4 + 3]);
                    *reinterpret_cast<uint2*>(sp + row * DK + pc * 64 + l16 * 4) = w;
                }
            }
        }
    }
    if (tid == 0 && abort_flag && p.status) atomicExch(p.status, 1);
}

}  // namespace gdn
