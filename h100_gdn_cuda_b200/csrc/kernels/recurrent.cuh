// Recurrent Gated DeltaNet step (decode, speculative verify, short prefill).
//
// Replaces the reference's fused_recurrent_gated_delta_rule_bf16
// (gdn_cuda/include/gdn_cuda/kernels/sm90_bf16_gdn_recurrent.cuh:20-440) with the
// canonical update order  S <- exp(g) S ;  S <- S + beta (v - S k) k^T ;  o = scale S q.
//
// The kernel is bound by HBM traffic: per (sequence, v-head) it must read and write the
// dv x dk bf16 state once.  A persistent CTA of 128 threads takes (sequence, v-head) units
// round-robin and walks each unit's tiles of 32 state rows (32 x DK bf16, 8 KB at DK = 128).
// Tiles are fetched ahead into a ring of shared-memory buffers by bulk asynchronous copies
// (one elected thread issues them together with the first token's k, q and v slice,
// completion is signalled on an mbarrier), so several tiles per CTA are in flight while the
// current one is processed.  Each thread keeps 4 rows x DK/16 columns of the tile as packed
// fp32 pairs and works on them with two-wide fp32 FMAs; the two products S.k and S.q come
// from the same pass over the old state:
//     r = v - e^g (S k),   S' = e^g S + beta r k^T,   o = scale (e^g (S q) + beta r (k.q)).
// The eight row sums are reduced over 16 lanes with a transposing butterfly (8 shuffles
// instead of 32).  For single-token decode q/k normalisation and k.q are computed once per
// unit, not per tile.  New states leave through coalesced 8-byte stores from registers.
// Long runs of tokens (short prefill, head dims the chunked kernels do not cover) take a second
// instance of the kernel (kRing), chosen by the host when the sequences average more than
// kRecTokRingMin tokens: every tile is a work unit of its own, so that a few long sequences
// still spread over all CTAs, and k, q, v arrive 8 tokens at a time by bulk copies: the first
// block with the tile's stage, the others through a two-slot ring.  (With one token fetched ahead
// of the one in work, as the decode instance does for its few tokens, every token paid the whole
// load latency, about a microsecond.)
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
    const void* state_in;   // bf16, or fp32 in the kF32 instances; strides in elements of that type
    void* state_out;
    int64_t si_ss, si_sh, so_ss, so_sh;
    const int* cu_seqlens;
    const int* num_accepted;
    const int* state_idx;  // indexed state pool: slot of every sequence (negative: padding sequence), or NULL
    int batch, seq_len, kh, vh, dv;
    float scale;
    int is_qk_norm, store_step;
    // Fused gating: `beta` / `gate` then hold the layer's raw projections b / a and the kernel computes
    // beta = sigmoid(b), g = -exp(A_log[h]) softplus(a + dt_bias[h]) itself (fp32, nothing rounded to bf16).
    int fused_gating, gating_param_f32;
    const void* A_log;
    const void* dt_bias;
    int split_tiles;  // 1: every 32-row tile is a work unit (multi-token runs of the ring instance); 0: a unit = all tiles of a (sequence, v-head)
    long long num_tiles;
    int* status;
};

constexpr int kRecTileRows = 32;
constexpr int kRecStages = 4;      // state tiles in flight per CTA (decode)
constexpr int kRecStagesRing = 2;  // in the multi-token instance a tile lasts for many tokens: two are enough
constexpr int kRecThreads = 128;
constexpr int kRecTokBlock = 8;     // tokens per slot of the multi-token ring
constexpr int kRecTokRingMin = 16;  // sequences longer than this use it

// One ring stage: the 32 x DK state tile, then k and q (DK bf16 each) and the 32 entries of v that
// belong to the tile's rows, for the unit's first token (decode instance) or its first
// kRecTokBlock tokens (multi-token instance; same layout as a slot of the token ring).
template <int DK, bool kRing = false, bool kF32 = false>
struct RecStage {
    static constexpr int kTok = kRing ? kRecTokBlock : 1;
    static constexpr int kTileBytes = kRecTileRows * DK * (kF32 ? 4 : 2);
    static constexpr int kOffK = kTileBytes;
    static constexpr int kOffQ = kOffK + kTok * DK * 2;
    static constexpr int kOffV = kOffQ + kTok * DK * 2;
    static constexpr int kBytes = (kOffV + kTok * kRecTileRows * 2 + 127) / 128 * 128;
};

// One slot of the multi-token ring: k, q (DK bf16 each) and the tile's 32 entries of v for 8 tokens.
template <int DK>
struct RecTokSlot {
    static constexpr int kOffK = 0;
    static constexpr int kOffQ = kRecTokBlock * DK * 2;
    static constexpr int kOffV = 2 * kRecTokBlock * DK * 2;
    static constexpr int kBytes = kOffV + kRecTokBlock * kRecTileRows * 2;
};

// fp32 states double the tile: the decode instance then keeps two tiles in flight instead of four
template <bool kRing, bool kF32>
constexpr int recurrent_stages() {
    return kRing ? kRecStagesRing : (kF32 ? 2 : kRecStages);
}
template <int DK, bool kRing = true, bool kF32 = false>
constexpr int recurrent_smem_bytes() {
    return recurrent_stages<kRing, kF32>() * RecStage<DK, kRing, kF32>::kBytes + 128 + (kRing ? 2 * RecTokSlot<DK>::kBytes : 0);
}

// Multi-token units of the decode instance (speculative verify, short runs): the per-token inputs that every
// 32-row tile of a (sequence, v-head) unit needs - the normalised k and q, k.q, beta, the gate and the head's v -
// are prepared ONCE per unit by the CTA's warps (one token each) and kept here for the unit's tiles; without it every
// tile, and in it every warp, reloaded and re-normalised every token (a third of the instructions of such a step).
constexpr int kRecPrepTok = 8;     // units with 2 .. 8 tokens use the buffer, longer ones the per-tile path
constexpr int kRecPrepRows = 256;  // v rows of a unit that fit (dv <= 256)
template <int DK, bool kEnable>
struct RecPrepBuf {
    float k[kRecPrepTok][DK];
    float q[kRecPrepTok][DK];
    float sc[kRecPrepTok][4];  // beta, gate, k.q
    __nv_bfloat16 v[kRecPrepTok][kRecPrepRows];
};
template <int DK>
struct RecPrepBuf<DK, false> {
    int unused;
};

namespace rec {
using f2 = unsigned long long;  // two packed fp32 values
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
__device__ __forceinline__ f2 mul2(f2 a, f2 b) {
    f2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f2 bf2_to_f2(uint32_t w) {  // bf16 pair -> fp32 pair
    return pk(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
}
__device__ __forceinline__ float hsum(f2 v) {
    float a, b;
    unpk(v, a, b);
    return a + b;
}
}  // namespace rec

// Body of the kernel as a device function: the ahead-of-time entry points below and the
// entry point the run-time compiler generates (csrc/gdn_jit.cu) both instantiate it.
// kRing: with the multi-token ring (long runs of tokens); without it the kernel is the lean decode
// kernel (its registers are at the limit of four CTAs per SM at DK = 128).
// kLean (decode instance only): the launch is plain single-token decode from a given state - padded
// inputs with one token per sequence, an initial state, one state per sequence out.  The host
// promises that, and the corresponding run-time tests compile away.
// kF32: the state is kept in fp32 in memory (read, updated and written as such; serving engines that run
// many decode steps on one state use it to avoid a bf16 rounding per step).
namespace rec {
template <bool kF32>
struct StateElem {
    typedef __nv_bfloat16 type;
};
template <>
struct StateElem<true> {
    typedef float type;
};
}  // namespace rec
template <int DK, bool kRing = true, bool kLean = false, bool kF32 = false>
__device__ __forceinline__ void gdn_recurrent_body(const RecurrentParams& p) {
    static_assert(!(kRing && kLean), "the lean instance is a decode instance");
    using namespace ptx;
    using namespace rec;
    using Stage = RecStage<DK, kRing, kF32>;
    using ST = typename StateElem<kF32>::type;
    const ST* const state_in = static_cast<const ST*>(p.state_in);
    ST* const state_out = static_cast<ST*>(p.state_out);
    constexpr int NQ = DK / 32;  // packed pairs per row per lane (lane owns 4 columns of every 64)
    extern __shared__ __align__(128) uint8_t smem[];
    using TokSlot = RecTokSlot<DK>;
    constexpr int kStages = recurrent_stages<kRing, kF32>();
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStages * Stage::kBytes);
    uint64_t* tokfull = full + kStages;  // [2]
    uint8_t* tokbase = smem + kStages * Stage::kBytes + 128;
    __shared__ int abort_flag;
    // Fused gating: load_scalars returns the raw projections b and a (fetched a unit ahead like beta and the
    // gate); the transform is applied where they are consumed, with the per-head parameters A_log and
    // dt_bias staged here once per CTA (heads beyond the table are read from global memory).
    constexpr int kGateTable = 128;
    __shared__ float s_alog[kGateTable], s_dtb[kGateTable];
    constexpr bool kPrep = !kRing && !kLean;
    __shared__ __align__(16) RecPrepBuf<DK, kPrep> prep;

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int half = lane >> 4, l16 = lane & 15;
    const int rblocks = p.dv / kRecTileRows;
    const bool has_in = kLean || p.state_in != nullptr;
    const bool store_step = !kLean && p.store_step != 0;
    const int rep = p.vh / p.kh;
    const int tpu = (kRing && p.split_tiles) ? 1 : rblocks;  // tiles per work unit
    const int upg = rblocks / tpu;                // work units per (sequence, v-head)
    const int num_units = static_cast<int>(p.num_tiles / tpu);
    const int stride = static_cast<int>(gridDim.x);

    // The kernel is launched as a programmatic dependent of the preceding work in the stream: its CTAs are placed
    // while that work drains and wait here, before the first access to global memory (a no-op for an ordinary launch).
    grid_dep_wait();
    if (p.fused_gating) {
        for (int h = threadIdx.x; h < min(p.vh, kGateTable); h += blockDim.x) {
            s_alog[h] = p.gating_param_f32 ? __ldg(reinterpret_cast<const float*>(p.A_log) + h)
                                           : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.A_log)[h]);
            s_dtb[h] = p.gating_param_f32 ? __ldg(reinterpret_cast<const float*>(p.dt_bias) + h)
                                          : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.dt_bias)[h]);
        }
    }
    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < kStages; ++s) mbar_init(&full[s], 1);
        mbar_init(&tokfull[0], 1);
        mbar_init(&tokfull[1], 1);
        mbar_fence_init();
    }
    __syncthreads();

    struct Unit {
        int seq, head, khead, ntok, rb0;
        int slot;  // where the sequence's state lives (its index, or its slot of an indexed pool; negative: skip)
        long long tok0, bidx;
    };
    // head counts are almost always powers of two: shifts instead of integer divisions then
    const int vh_shift = (p.vh & (p.vh - 1)) == 0 ? __ffs(p.vh) - 1 : -1;
    const int rep_shift = (rep & (rep - 1)) == 0 ? __ffs(rep) - 1 : -1;
    auto decode = [&](int unit) {
        Unit t;
        int sh = unit;
        t.rb0 = 0;
        if (upg != 1) {
            sh = unit / upg;
            t.rb0 = (unit - sh * upg) * tpu;
        }
        if (vh_shift >= 0) {
            t.seq = sh >> vh_shift;
            t.head = sh & (p.vh - 1);
        } else {
            t.seq = sh / p.vh;
            t.head = sh - t.seq * p.vh;
        }
        t.khead = rep_shift >= 0 ? (t.head >> rep_shift) : (t.head / rep);
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
        t.slot = t.seq;
        if (!kLean && p.state_idx) {
            t.slot = p.state_idx[t.seq];
            if (t.slot < 0) t.ntok = 0;
        }
        return t;
    };
    // Producer (one thread): everything tile `rb` of `unit` needs for its first token.
    // source addresses of the producer's current unit (its first token), computed when the unit changes
    const ST* prod_s = nullptr;
    const __nv_bfloat16* prod_k = nullptr;
    const __nv_bfloat16* prod_q = nullptr;
    const __nv_bfloat16* prod_v = nullptr;
    auto producer_bases = [&](const Unit& t) {
        prod_s = has_in ? state_in + static_cast<long long>(max(t.slot, 0)) * p.si_ss + t.head * p.si_sh : nullptr;
        prod_k = p.k + t.bidx * p.k_sb + t.tok0 * p.k_st + t.khead * p.k_sh;
        prod_q = p.q + t.bidx * p.q_sb + t.tok0 * p.q_st + t.khead * p.q_sh;
        prod_v = p.v + t.bidx * p.v_sb + t.tok0 * p.v_st + t.head * p.v_sh;
    };
    auto issue = [&](const Unit& t, int rb, int stage) {
        uint8_t* dst = smem + stage * Stage::kBytes;
        const int nt0 = min(t.ntok, Stage::kTok);  // tokens whose k, q, v travel with the tile
        const uint32_t bytes = (has_in ? Stage::kTileBytes : 0) + static_cast<uint32_t>(nt0) * (4 * DK + kRecTileRows * 2);
        mbar_arrive_expect_tx(&full[stage], bytes);
        if (has_in) bulk_load(dst, prod_s + rb * (kRecTileRows * DK), Stage::kTileBytes, &full[stage]);
        for (int i = 0; i < nt0; ++i) {
            bulk_load(dst + Stage::kOffK + i * DK * 2, prod_k + i * p.k_st, DK * 2, &full[stage]);
            bulk_load(dst + Stage::kOffQ + i * DK * 2, prod_q + i * p.q_st, DK * 2, &full[stage]);
            bulk_load(dst + Stage::kOffV + i * kRecTileRows * 2, prod_v + i * p.v_st + rb * kRecTileRows, kRecTileRows * 2,
                      &full[stage]);
        }
    };
    auto load_scalars = [&](const Unit& t, int tk, float& bt, float& gt) {
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

    // raw projections (b, a) of a token of v-head `head` -> (beta, gate)
    auto apply_gating = [&](int head, float& bt, float& gt) {
        float al, db;
        if (head < kGateTable) {
            al = s_alog[head];
            db = s_dtb[head];
        } else {
            al = p.gating_param_f32 ? __ldg(reinterpret_cast<const float*>(p.A_log) + head)
                                    : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.A_log)[head]);
            db = p.gating_param_f32 ? __ldg(reinterpret_cast<const float*>(p.dt_bias) + head)
                                    : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.dt_bias)[head]);
        }
        // softplus and sigmoid on the fast exponential, logarithm and reciprocal (a few ulp, far inside what a bf16
        // beta or an e^gate can show); log(1 + e) switches to e where 1 + e would round to 1
        const float x = gt + db;
        const float e = __expf(x);
        const float sp = x > 20.f ? x : (x < -15.f ? e : __logf(1.f + e));
        gt = -__expf(al) * sp;
        bt = __fdividef(1.f, 1.f + __expf(-bt));
    };

    // The producer walks (unit, rb) pairs kStages-1 iterations ahead of the consumers.
    int prod_unit = blockIdx.x, prod_rb = 0, prod_it = 0;
    Unit prod_u{};
    if (tid == 0 && prod_unit < num_units) {
        prod_u = decode(prod_unit);
        producer_bases(prod_u);
    }
    auto produce_one = [&]() {
        if (prod_unit >= num_units) return;
        issue(prod_u, prod_u.rb0 + prod_rb, prod_it % kStages);
        ++prod_it;
        if (++prod_rb == tpu) {
            prod_rb = 0;
            prod_unit += stride;
            if (prod_unit < num_units) {
                prod_u = decode(prod_unit);
                producer_bases(prod_u);
            }
        }
    };
    if (tid == 0) {
        for (int s = 0; s < kStages - 1; ++s) produce_one();
    }

    float beta_first = 0.f, g_first = 0.f;  // scalars of the first token of the current unit
    if (static_cast<int>(blockIdx.x) < num_units) {
        const Unit t0 = decode(blockIdx.x);
        const int tk = kRing ? lane : 0;  // multi-token instance: lane l holds the scalars of token l
        if (tk < t0.ntok) load_scalars(t0, tk, beta_first, g_first);
    }

    int it = 0;
    int tb_it = 0;  // blocks that have gone through the multi-token ring (slot and parity bookkeeping)
    Unit T_carry{};
    if (static_cast<int>(blockIdx.x) < num_units) T_carry = decode(blockIdx.x);
    for (int unit = blockIdx.x; unit < num_units; unit += stride) {
        const Unit T = T_carry;
        float beta_next = 0.f, g_next = 0.f;
        if (unit + stride < num_units) {
            T_carry = decode(unit + stride);
            const int tk = kRing ? lane : 0;
            if (tk < T_carry.ntok) load_scalars(T_carry, tk, beta_next, g_next);
        }
        // where this unit's outputs go: computed once per unit, not per tile or token
        __nv_bfloat16* const out_unit = p.out + T.bidx * p.o_sb + T.tok0 * p.o_st + T.head * p.o_sh;
        ST* const sout_unit = state_out + T.head * p.so_sh + (store_step ? 0 : static_cast<long long>(max(T.slot, 0)) * p.so_ss);
        // fused gating: the first token's (the ring instance: the first 32 tokens') raw projections become
        // beta and the gate once per unit, not once per tile
        if (p.fused_gating) apply_gating(T.head, beta_first, g_first);
        // per-unit values of the first token (kept across the unit's tiles when ntok == 1)
        f2 k2[NQ], q2[NQ];
        float kq = 0.f;

        auto prep_kq = [&](const uint2* kw_, const uint2* qw_) {
                // unpack, optional L2 normalisation, k.q
#pragma unroll
                for (int pc = 0; pc < NQ / 2; ++pc) {
                    k2[2 * pc] = bf2_to_f2(kw_[pc].x);
                    k2[2 * pc + 1] = bf2_to_f2(kw_[pc].y);
                    q2[2 * pc] = bf2_to_f2(qw_[pc].x);
                    q2[2 * pc + 1] = bf2_to_f2(qw_[pc].y);
                }
                f2 akk = 0ull, aqq = 0ull, akq = 0ull;
#pragma unroll
                for (int c = 0; c < NQ; ++c) {
                    akk = fma2(k2[c], k2[c], akk);
                    aqq = fma2(q2[c], q2[c], aqq);
                    akq = fma2(k2[c], q2[c], akq);
                }
                float skk = hsum(akk), sqq = hsum(aqq), skq = hsum(akq);
#pragma unroll
                for (int m = 1; m < 16; m <<= 1) {
                    skk += __shfl_xor_sync(0xffffffffu, skk, m);
                    sqq += __shfl_xor_sync(0xffffffffu, sqq, m);
                    skq += __shfl_xor_sync(0xffffffffu, skq, m);
                }
                kq = skq;
                if (p.is_qk_norm) {
                    const float inv_k = rsqrtf(skk + 1e-6f), inv_q = rsqrtf(sqq + 1e-6f);
                    const f2 ik2 = pk(inv_k, inv_k), iq2 = pk(inv_q, inv_q);
#pragma unroll
                    for (int c = 0; c < NQ; ++c) {
                        k2[c] = mul2(k2[c], ik2);
                        q2[c] = mul2(q2[c], iq2);
                    }
                    kq = skq * inv_k * inv_q;
                }
                        };
        // ---- multi-token unit: prepare the tokens once for all tiles (see RecPrepBuf)
        bool use_prep = false;
        if constexpr (kPrep) {
            use_prep = T.ntok > 1 && T.ntok <= kRecPrepTok && tpu * kRecTileRows <= kRecPrepRows;
            if (use_prep) {
                __syncthreads();  // the previous unit's tiles have read the buffer
                for (int t = warp; t < T.ntok; t += kRecThreads / 32) {
                    const long long tok = T.tok0 + t;
                    const __nv_bfloat16* kp = p.k + T.bidx * p.k_sb + tok * p.k_st + T.khead * p.k_sh;
                    const __nv_bfloat16* qp = p.q + T.bidx * p.q_sb + tok * p.q_st + T.khead * p.q_sh;
                    uint2 kk[NQ / 2], qq[NQ / 2];
#pragma unroll
                    for (int pc = 0; pc < NQ / 2; ++pc) {
                        kk[pc] = __ldg(reinterpret_cast<const uint2*>(kp + pc * 64 + l16 * 4));
                        qq[pc] = __ldg(reinterpret_cast<const uint2*>(qp + pc * 64 + l16 * 4));
                    }
                    float bt, gt;
                    load_scalars(T, t, bt, gt);
                    if (p.fused_gating) apply_gating(T.head, bt, gt);
                    prep_kq(kk, qq);
                    if (half == 0) {
#pragma unroll
                        for (int pc = 0; pc < NQ / 2; ++pc) {
                            float a0, a1, a2, a3;
                            unpk(k2[2 * pc], a0, a1);
                            unpk(k2[2 * pc + 1], a2, a3);
                            *reinterpret_cast<float4*>(&prep.k[t][pc * 64 + l16 * 4]) = make_float4(a0, a1, a2, a3);
                            unpk(q2[2 * pc], a0, a1);
                            unpk(q2[2 * pc + 1], a2, a3);
                            *reinterpret_cast<float4*>(&prep.q[t][pc * 64 + l16 * 4]) = make_float4(a0, a1, a2, a3);
                        }
                    }
                    if (lane == 0) *reinterpret_cast<float4*>(prep.sc[t]) = make_float4(bt, gt, kq, 0.f);
                    const __nv_bfloat16* vp = p.v + T.bidx * p.v_sb + tok * p.v_st + T.head * p.v_sh + T.rb0 * kRecTileRows;
                    for (int i = lane; i < tpu * kRecTileRows; i += 32) prep.v[t][i] = vp[i];
                }
                __syncthreads();
            }
        }

        for (int r = 0; r < tpu; ++r, ++it) {
            const int rb = T.rb0 + r;
            const int stage = it % kStages;
            const uint32_t parity = static_cast<uint32_t>((it / kStages) & 1);
            if (tid == 0) produce_one();  // refills the stage consumed in the previous iteration

            // ---- staged data -> registers
            f2 S[4][NQ];
            float vr[4];
            // `ok` turns false when a wait gives up: the tile's data is then garbage and nothing of it is stored
            bool ok = mbar_wait(&full[stage], parity, &abort_flag);
            const uint8_t* st = smem + stage * Stage::kBytes;
            if (has_in) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int row = warp * 8 + 2 * j + half;
#pragma unroll
                    for (int pc = 0; pc < NQ / 2; ++pc) {
                        if (kF32) {
                            const float4 w = *reinterpret_cast<const float4*>(st + (row * DK + pc * 64 + l16 * 4) * 4);
                            S[j][2 * pc] = pk(w.x, w.y);
                            S[j][2 * pc + 1] = pk(w.z, w.w);
                        } else {
                            const uint2 w = *reinterpret_cast<const uint2*>(st + (row * DK + pc * 64 + l16 * 4) * 2);
                            S[j][2 * pc] = bf2_to_f2(w.x);
                            S[j][2 * pc + 1] = bf2_to_f2(w.y);
                        }
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
#pragma unroll
                    for (int c = 0; c < NQ; ++c) S[j][c] = 0ull;
            }
            const bool fresh_qk = (r == 0) || (!kLean && T.ntok > 1);
            uint2 kw[NQ / 2], qw[NQ / 2];
            if (T.ntok > 0) {
                if (fresh_qk) {
#pragma unroll
                    for (int pc = 0; pc < NQ / 2; ++pc) {
                        kw[pc] = *reinterpret_cast<const uint2*>(st + Stage::kOffK + (pc * 64 + l16 * 4) * 2);
                        qw[pc] = *reinterpret_cast<const uint2*>(st + Stage::kOffQ + (pc * 64 + l16 * 4) * 2);
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    vr[j] = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(st + Stage::kOffV)[warp * 8 + 2 * j + half]);
            }
            __syncthreads();  // every thread has read this stage: it may be refilled

            // ---- token loop (inputs of token t+1 are fetched from global while token t is computed)
            auto load_token = [&](int t, uint2* kk, uint2* qq, float* vv, float& bt, float& gt) {
                const long long tok = T.tok0 + t;
                const __nv_bfloat16* kp = p.k + T.bidx * p.k_sb + tok * p.k_st + T.khead * p.k_sh;
                const __nv_bfloat16* qp = p.q + T.bidx * p.q_sb + tok * p.q_st + T.khead * p.q_sh;
#pragma unroll
                for (int pc = 0; pc < NQ / 2; ++pc) {
                    kk[pc] = __ldg(reinterpret_cast<const uint2*>(kp + pc * 64 + l16 * 4));
                    qq[pc] = __ldg(reinterpret_cast<const uint2*>(qp + pc * 64 + l16 * 4));
                }
                const __nv_bfloat16* vp = p.v + T.bidx * p.v_sb + tok * p.v_st + T.head * p.v_sh + rb * kRecTileRows;
#pragma unroll
                for (int j = 0; j < 4; ++j) vv[j] = __bfloat162float(vp[warp * 8 + 2 * j + half]);
                load_scalars(T, t, bt, gt);
            };

            auto token_step = [&](int t, const float* vr_, float beta_t, float g_t) {
                // ---- S.k and S.q for the thread's 4 rows
                f2 ak[4], aq[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    ak[j] = mul2(S[j][0], k2[0]);
                    aq[j] = mul2(S[j][0], q2[0]);
                }
#pragma unroll
                for (int c = 1; c < NQ; ++c) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        ak[j] = fma2(S[j][c], k2[c], ak[j]);
                        aq[j] = fma2(S[j][c], q2[c], aq[j]);
                    }
                }
                // transposing butterfly over the 16 lanes of a row: 8 values -> lane l16 holds
                // the full sum of value (l16 >> 1): S.k of row j on lanes 2j, 2j+1; S.q on 8+2j, 8+2j+1
                float v8[8];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    v8[j] = hsum(ak[j]);
                    v8[4 + j] = hsum(aq[j]);
                }
                float v4[4], v2[2], v1;
                {
                    const bool up = (l16 & 8) != 0;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float send = up ? v8[i] : v8[4 + i];
                        const float keep = up ? v8[4 + i] : v8[i];
                        v4[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
                    }
                }
                {
                    const bool up = (l16 & 4) != 0;
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const float send = up ? v4[i] : v4[2 + i];
                        const float keep = up ? v4[2 + i] : v4[i];
                        v2[i] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
                    }
                }
                {
                    const bool up = (l16 & 2) != 0;
                    const float send = up ? v2[0] : v2[1];
                    const float keep = up ? v2[1] : v2[0];
                    v1 = keep + __shfl_xor_sync(0xffffffffu, send, 2);
                }
                v1 += __shfl_xor_sync(0xffffffffu, v1, 1);

                const float eg = __expf(g_t);
                const f2 eg2 = pk(eg, eg);
                const int base = lane & 16;
                float o_mine = 0.f;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float dkj = __shfl_sync(0xffffffffu, v1, base + 2 * j);
                    const float r = vr_[j] - eg * dkj;
                    const float br = beta_t * r;
                    if (l16 == 8 + 2 * j) o_mine = p.scale * fmaf(eg, v1, br * kq);
                    const f2 br2 = pk(br, br);
#pragma unroll
                    for (int c = 0; c < NQ; ++c) S[j][c] = fma2(eg2, S[j][c], mul2(br2, k2[c]));
                }
                if (ok && l16 >= 8 && (l16 & 1) == 0) {
                    __nv_bfloat16* op = out_unit + t * p.o_st + rb * kRecTileRows;
                    op[warp * 8 + (l16 - 8) + half] = __float2bfloat16(o_mine);
                }
                if (store_step && ok) {
                    const long long sidx = p.cu_seqlens ? (T.tok0 + t) : (static_cast<long long>(T.seq) * p.seq_len + t);
                    ST* sp = sout_unit + sidx * p.so_ss + rb * (kRecTileRows * DK);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int row = warp * 8 + 2 * j + half;
#pragma unroll
                        for (int pc = 0; pc < NQ / 2; ++pc) {
                            float a0, a1, a2, a3;
                            unpk(S[j][2 * pc], a0, a1);
                            unpk(S[j][2 * pc + 1], a2, a3);
                            if (kF32) {
                                *reinterpret_cast<float4*>(sp + row * DK + pc * 64 + l16 * 4) = make_float4(a0, a1, a2, a3);
                            } else {
                                uint2 w;
                                w.x = pack_bf16(a0, a1);
                                w.y = pack_bf16(a2, a3);
                                *reinterpret_cast<uint2*>(sp + row * DK + pc * 64 + l16 * 4) = w;
                            }
                        }
                    }
                }
            };
            if constexpr (kRing) {
                static_assert(Stage::kOffQ - Stage::kOffK == TokSlot::kOffQ && Stage::kOffV - Stage::kOffK == TokSlot::kOffV,
                              "the stage's token block must be laid out like a ring slot");
                // (every sequence of the launch goes through the ring, the short ones with their first block's
                // latency exposed: the host picks this instance when the sequences average more than kRecTokRingMin tokens)
// k, q, v of 8 tokens per block.  Block 0 came with the tile's stage; blocks 1.. go through
                // the two slots of the token ring, block b + 2 being requested when block b is done.
                constexpr int TB = kRecTokBlock;
                const int nblk = (T.ntok + TB - 1) / TB;
                auto issue_block = [&](int blk) {  // one thread; blk >= 1
                    const int slot = (tb_it + blk - 1) & 1;
                    uint8_t* dst = tokbase + slot * TokSlot::kBytes;
                    const int nt = min(TB, T.ntok - blk * TB);
                    mbar_arrive_expect_tx(&tokfull[slot], static_cast<uint32_t>(nt) * (4 * DK + kRecTileRows * 2));
                    for (int i = 0; i < nt; ++i) {
                        const long long tok = T.tok0 + blk * TB + i;
                        bulk_load(dst + TokSlot::kOffK + i * DK * 2, p.k + T.bidx * p.k_sb + tok * p.k_st + T.khead * p.k_sh,
                                  DK * 2, &tokfull[slot]);
                        bulk_load(dst + TokSlot::kOffQ + i * DK * 2, p.q + T.bidx * p.q_sb + tok * p.q_st + T.khead * p.q_sh,
                                  DK * 2, &tokfull[slot]);
                        bulk_load(dst + TokSlot::kOffV + i * kRecTileRows * 2,
                                  p.v + T.bidx * p.v_sb + tok * p.v_st + T.head * p.v_sh + rb * kRecTileRows,
                                  kRecTileRows * 2, &tokfull[slot]);
                    }
                };
                if (tid == 0) {
                    if (nblk > 1) issue_block(1);
                    if (nblk > 2) issue_block(2);
                }
                // beta and gate: lane l holds those of token 32 * group + l (group 0 was fetched during
                // the previous unit), the next group is fetched one group ahead
                float bsc = beta_first, gsc = g_first, bsn = 0.f, gsn = 0.f;
                for (int blk = 0; blk < nblk; ++blk) {
                    if ((blk & 3) == 0) {
                        if (blk > 0) {
                            bsc = bsn;
                            gsc = gsn;
                            if (p.fused_gating) apply_gating(T.head, bsc, gsc);  // one lane per token
                        }
                        const int tn = (blk + 4) * TB + lane;
                        bsn = 0.f;
                        gsn = 0.f;
                        if (tn < T.ntok) load_scalars(T, tn, bsn, gsn);
                    }
                    const uint8_t* ts;
                    if (blk == 0) {
                        ts = st + Stage::kTileBytes;  // same layout as a ring slot
                    } else {
                        const int slot = (tb_it + blk - 1) & 1;
                        ok = mbar_wait(&tokfull[slot], static_cast<uint32_t>(((tb_it + blk - 1) >> 1) & 1), &abort_flag) && ok;
                        ts = tokbase + slot * TokSlot::kBytes;
                    }
                    const int nt = min(TB, T.ntok - blk * TB);
                    for (int i = 0; i < nt; ++i) {
                        const int t = blk * TB + i;
                        uint2 kt[NQ / 2], qt[NQ / 2];
                        float vt[4];
#pragma unroll
                        for (int pc = 0; pc < NQ / 2; ++pc) {
                            kt[pc] = *reinterpret_cast<const uint2*>(ts + TokSlot::kOffK + i * DK * 2 + (pc * 64 + l16 * 4) * 2);
                            qt[pc] = *reinterpret_cast<const uint2*>(ts + TokSlot::kOffQ + i * DK * 2 + (pc * 64 + l16 * 4) * 2);
                        }
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            vt[j] = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(
                                ts + TokSlot::kOffV + i * kRecTileRows * 2)[warp * 8 + 2 * j + half]);
                        const float beta_t = __shfl_sync(0xffffffffu, bsc, t & 31);
                        const float g_t = __shfl_sync(0xffffffffu, gsc, t & 31);
                        prep_kq(kt, qt);
                        token_step(t, vt, beta_t, g_t);
                    }
                    __syncthreads();  // the block (stage or slot) has been read by every thread
                    if (tid == 0 && blk >= 1 && blk + 2 < nblk) issue_block(blk + 2);
                }
                if (nblk > 1) tb_it += nblk - 1;
            } else {
            float beta_t = beta_first, g_t = g_first;
            if (kLean || T.ntok == 1) {
                // plain decode: no token loop, nothing fetched ahead (an accepted-token cap of 0 copies the state)
                if (T.ntok == 1) {
                    if (fresh_qk) prep_kq(kw, qw);
                    token_step(0, vr, beta_t, g_t);
                }
            } else if (kPrep && use_prep) {
                if constexpr (kPrep) {
                    for (int t = 0; t < T.ntok; ++t) {
#pragma unroll
                        for (int pc = 0; pc < NQ / 2; ++pc) {
                            const float4 a = *reinterpret_cast<const float4*>(&prep.k[t][pc * 64 + l16 * 4]);
                            const float4 b = *reinterpret_cast<const float4*>(&prep.q[t][pc * 64 + l16 * 4]);
                            k2[2 * pc] = pk(a.x, a.y);
                            k2[2 * pc + 1] = pk(a.z, a.w);
                            q2[2 * pc] = pk(b.x, b.y);
                            q2[2 * pc + 1] = pk(b.z, b.w);
                        }
                        const float4 sc = *reinterpret_cast<const float4*>(prep.sc[t]);
                        kq = sc.z;
                        float vt[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) vt[j] = __bfloat162float(prep.v[t][r * kRecTileRows + warp * 8 + 2 * j + half]);
                        token_step(t, vt, sc.x, sc.y);
                    }
                }
            } else
            for (int t = 0; t < T.ntok; ++t) {
                uint2 kn[NQ / 2], qn[NQ / 2];
                float vn[4], beta_n = 0.f, g_n = 0.f;
                if (t + 1 < T.ntok) load_token(t + 1, kn, qn, vn, beta_n, g_n);
                if (t > 0 || fresh_qk) prep_kq(kw, qw);
                token_step(t, vr, beta_t, g_t);
#pragma unroll
                for (int pc = 0; pc < NQ / 2; ++pc) {
                    kw[pc] = kn[pc];
                    qw[pc] = qn[pc];
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) vr[j] = vn[j];
                beta_t = beta_n;
                g_t = g_n;
                if (p.fused_gating && t + 1 < T.ntok) apply_gating(T.head, beta_t, g_t);
            }

            }
            if (!store_step && ok && T.slot >= 0) {
                ST* sp = sout_unit + rb * (kRecTileRows * DK);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int row = warp * 8 + 2 * j + half;
#pragma unroll
                    for (int pc = 0; pc < NQ / 2; ++pc) {
                        float a0, a1, a2, a3;
                        unpk(S[j][2 * pc], a0, a1);
                        unpk(S[j][2 * pc + 1], a2, a3);
                        if (kF32) {
                            *reinterpret_cast<float4*>(sp + row * DK + pc * 64 + l16 * 4) = make_float4(a0, a1, a2, a3);
                        } else {
                            uint2 w;
                            w.x = pack_bf16(a0, a1);
                            w.y = pack_bf16(a2, a3);
                            *reinterpret_cast<uint2*>(sp + row * DK + pc * 64 + l16 * 4) = w;
                        }
                    }
                }
            }
        }
        beta_first = beta_next;
        g_first = g_next;
    }
    if (tid == 0 && abort_flag && p.status) atomicExch(p.status, 1);
}

// (fp32 states at DK = 128: the 16-byte accesses need a few more registers than four CTAs per SM leave)
template <int DK, bool kRing = false, bool kF32 = false>
constexpr int recurrent_ctas_per_sm() {
    return kRing ? (DK <= 64 ? 4 : 3) : (DK <= 128 ? ((kF32 && DK > 64) ? 3 : 4) : 2);
}

template <int DK, bool kRing = false, bool kLean = false, bool kF32 = false>
__global__ void __launch_bounds__(kRecThreads, recurrent_ctas_per_sm<DK, kRing, kF32>()) gdn_recurrent_kernel(const RecurrentParams p) {
    gdn_recurrent_body<DK, kRing, kLean, kF32>(p);
}

}  // namespace gdn
