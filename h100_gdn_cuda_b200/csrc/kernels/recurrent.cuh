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

// One ring stage: the 32 x DK state tile, then k and q of the sequence's first token
// (DK bf16 each) and the 32 entries of v that belong to the tile's rows.
template <int DK>
struct RecStage {
    static constexpr int kTileBytes = kRecTileRows * DK * 2;
    static constexpr int kOffK = kTileBytes;
    static constexpr int kOffQ = kOffK + DK * 2;
    static constexpr int kOffV = kOffQ + DK * 2;
    static constexpr int kBytes = (kOffV + kRecTileRows * 2 + 127) / 128 * 128;
};

template <int DK>
constexpr int recurrent_smem_bytes() {
    return kRecStages * RecStage<DK>::kBytes + 128;
}

template <int DK>
__global__ void __launch_bounds__(kRecThreads, (DK <= 128 ? 4 : 2)) gdn_recurrent_kernel(const RecurrentParams p) {
    using namespace ptx;
    using Stage = RecStage<DK>;
    constexpr int NP = DK / 64;  // 64-column pieces; each lane owns 4 columns of every piece
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + kRecStages * Stage::kBytes);
    __shared__ int abort_flag;

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int half = lane >> 4, l16 = lane & 15;
    const int rblocks = p.dv / kRecTileRows;
    const bool has_in = p.state_in != nullptr;
    const int rep = p.vh / p.kh;
    const int num_tiles = static_cast<int>(p.num_tiles);
    const int stride = static_cast<int>(gridDim.x);

    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < kRecStages; ++s) mbar_init(&full[s], 1);
        mbar_fence_init();
    }
    __syncthreads();

    struct Tile {
        int seq, head, rb, khead, ntok;
        long long tok0, bidx;
    };
    auto decode = [&](int tile) {
        Tile t;
        t.rb = tile % rblocks;
        const int sh = tile / rblocks;
        t.head = sh % p.vh;
        t.seq = sh / p.vh;
        t.khead = t.head / rep;
        if (p.cu_seqlens) {
            t.tok0 = p.cu_seqlens[t.seq];
            t.ntok = p.cu_seqlens[t.seq + 1] - static_cast<int>(t.tok0);
            t.bidx = 0;
        } else {
            t.tok0 = 0;
            t.ntok = p.seq_len;
            t.bidx = t.seq;
        }
        if (p.num_accepted) t.ntok = min(t.ntok, p.num_accepted[t.seq]);
        return t;
    };
    // Producer (one thread): everything the tile needs for its first token, on one barrier.
    auto issue = [&](int tile, int stage) {
        const Tile t = decode(tile);
        uint8_t* dst = smem + stage * Stage::kBytes;
        uint32_t bytes = (has_in ? Stage::kTileBytes : 0) + (t.ntok > 0 ? 4 * DK + kRecTileRows * 2 : 0);
        mbar_arrive_expect_tx(&full[stage], bytes);
        if (has_in) {
            const __nv_bfloat16* src = p.state_in + t.seq * p.si_ss + t.head * p.si_sh +
                                       static_cast<long long>(t.rb) * kRecTileRows * DK;
            bulk_load(dst, src, Stage::kTileBytes, &full[stage]);
        }
        if (t.ntok > 0) {
            bulk_load(dst + Stage::kOffK, p.k + t.bidx * p.k_sb + t.tok0 * p.k_st + t.khead * p.k_sh, DK * 2, &full[stage]);
            bulk_load(dst + Stage::kOffQ, p.q + t.bidx * p.q_sb + t.tok0 * p.q_st + t.khead * p.q_sh, DK * 2, &full[stage]);
            bulk_load(dst + Stage::kOffV, p.v + t.bidx * p.v_sb + t.tok0 * p.v_st + t.head * p.v_sh + t.rb * kRecTileRows,
                      kRecTileRows * 2, &full[stage]);
        }
    };
    auto load_scalars = [&](const Tile& t, int tk, float& bt, float& gt) {
        const long long tok = t.tok0 + tk;
        const long long bo = t.bidx * p.beta_sb + tok * p.beta_st + t.head * p.beta_sh;
        bt = p.beta_f32 ? __ldg(reinterpret_cast<const float*>(p.beta) + bo)
                        : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.beta)[bo]);
        if (p.gate) {
            const long long go = t.bidx * p.gate_sb + tok * p.gate_st + t.head * p.gate_sh;
            gt = p.gate_f32 ? __ldg(reinterpret_cast<const float*>(p.gate) + go)
                            : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.gate)[go]);
        } else {
            gt = 0.f;
        }
    };

    // prologue: fill the ring
    if (tid == 0) {
        int t = blockIdx.x;
        for (int s = 0; s < kRecStages - 1 && t < num_tiles; ++s, t += stride) issue(t, s);
    }
    float beta_first = 0.f, g_first = 0.f;  // scalars of the first token of the *current* tile
    if (static_cast<int>(blockIdx.x) < num_tiles) {
        const Tile t0 = decode(blockIdx.x);
        if (t0.ntok > 0) load_scalars(t0, 0, beta_first, g_first);
    }

    int it = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += stride, ++it) {
        const int stage = it % kRecStages;
        const uint32_t parity = static_cast<uint32_t>((it / kRecStages) & 1);
        if (tid == 0) {
            // the stage consumed in the previous iteration is free (block-wide barrier below)
            const int nt = tile + (kRecStages - 1) * stride;
            if (nt < num_tiles) issue(nt, (it + kRecStages - 1) % kRecStages);
        }
        const Tile T = decode(tile);
        // scalars of the next tile's first token: requested now, used next iteration
        float beta_next = 0.f, g_next = 0.f;
        if (tile + stride < num_tiles) {
            const Tile tn = decode(tile + stride);
            if (tn.ntok > 0) load_scalars(tn, 0, beta_next, g_next);
        }

        // ---- staged data -> registers
        float S[4][NP * 4];
        uint2 kw[NP], qw[NP];
        float vr[4];
        mbar_wait(&full[stage], parity, &abort_flag);
        const uint8_t* st = smem + stage * Stage::kBytes;
        if (has_in) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int row = warp * 8 + 2 * j + half;
#pragma unroll
                for (int pc = 0; pc < NP; ++pc) {
                    const uint2 w = *reinterpret_cast<const uint2*>(st + (row * DK + pc * 64 + l16 * 4) * 2);
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
        if (T.ntok > 0) {
#pragma unroll
            for (int pc = 0; pc < NP; ++pc) {
                kw[pc] = *reinterpret_cast<const uint2*>(st + Stage::kOffK + (pc * 64 + l16 * 4) * 2);
                qw[pc] = *reinterpret_cast<const uint2*>(st + Stage::kOffQ + (pc * 64 + l16 * 4) * 2);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j)
                vr[j] = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(st + Stage::kOffV)[warp * 8 + 2 * j + half]);
        }
        __syncthreads();  // every thread has read this stage: it may be refilled

        // ---- token loop (inputs of token t+1 are fetched from global while token t is computed)
        float beta_t = beta_first, g_t = g_first;
        auto load_token = [&](int t, uint2* kk, uint2* qq, float* vv, float& bt, float& gt) {
            const long long tok = T.tok0 + t;
            const __nv_bfloat16* kp = p.k + T.bidx * p.k_sb + tok * p.k_st + T.khead * p.k_sh;
            const __nv_bfloat16* qp = p.q + T.bidx * p.q_sb + tok * p.q_st + T.khead * p.q_sh;
#pragma unroll
            for (int pc = 0; pc < NP; ++pc) {
                kk[pc] = __ldg(reinterpret_cast<const uint2*>(kp + pc * 64 + l16 * 4));
                qq[pc] = __ldg(reinterpret_cast<const uint2*>(qp + pc * 64 + l16 * 4));
            }
            const __nv_bfloat16* vp = p.v + T.bidx * p.v_sb + tok * p.v_st + T.head * p.v_sh + T.rb * kRecTileRows;
#pragma unroll
            for (int j = 0; j < 4; ++j) vv[j] = __bfloat162float(vp[warp * 8 + 2 * j + half]);
            load_scalars(T, t, bt, gt);
        };

        for (int t = 0; t < T.ntok; ++t) {
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
            if (t + 1 < T.ntok) load_token(t + 1, kn, qn, vn, beta_n, g_n);

            float kq = 0.f;
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
                const float inv_k = rsqrtf(sk + 1e-6f);
                const float inv_q = rsqrtf(sq + 1e-6f);
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
            const long long tok = T.tok0 + t;
            if (l16 < 4) {
                __nv_bfloat16* op = p.out + T.bidx * p.o_sb + tok * p.o_st + T.head * p.o_sh + T.rb * kRecTileRows;
                op[warp * 8 + 2 * l16 + half] = __float2bfloat16(o_mine);
            }
            if (p.store_step) {
                const long long sidx = p.cu_seqlens ? tok : (static_cast<long long>(T.seq) * p.seq_len + t);
                __nv_bfloat16* sp = p.state_out + sidx * p.so_ss + T.head * p.so_sh +
                                    static_cast<long long>(T.rb) * kRecTileRows * DK;
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
            __nv_bfloat16* sp = p.state_out + static_cast<long long>(T.seq) * p.so_ss + T.head * p.so_sh +
                                static_cast<long long>(T.rb) * kRecTileRows * DK;
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
        beta_first = beta_next;
        g_first = g_next;
    }
    if (tid == 0 && abort_flag && p.status) atomicExch(p.status, 1);
}

}  // namespace gdn
