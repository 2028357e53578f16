// Chunk-parallel stage of the whole-layer chunked prefill (gdn_chunked_forward).
//
// Per (64-token chunk, v-head), with g the chunk-local cumulative gate, g_L its last value and
//     A = tril(diag(beta) K K^T .* exp(g_i - g_j), -1),   X = (I + A)^-1,   T = X diag(beta)
//     P = scale * tril(Q K^T .* exp(g_i - g_j))
// the kernel writes the two matrices the sequential state kernel (prefill_fused.cuh) consumes:
//     Z  = T^T diag(exp(g_L - g)) K      (64 x dk, bf16)
//     PT = P T                           (64 x 64, bf16)
// They fold the WY/UT transform into the chunk-to-chunk recurrence: with R = V - exp(g) .* (K S^T)
//     U_new = T R,   S <- exp(g_L) S + R^T Z,   O = scale * exp(g) .* (Q S^T) + PT R
// so U = T V and W = T (K .* exp(g)) (what the reference's sm90_bf16_compute_u_w writes,
// gdn_cuda/include/gdn_cuda/kernels/sm90_bf16_gdn_compute_u_w.cuh:153-667) never exist, V is not
// read here at all, and the scratch per unit is 24 KB instead of 40 KB.
//
// Work unit = (chunk, k-head): the K and Q tiles are loaded once and K K^T, Q K^T are computed once
// (one M=128 tcgen05 MMA group whose A operand is K stacked on Q) for all the v-heads of the
// k-head group; only beta and the gate differ between them.  A CTA of 256 threads is two teams of
// four warps, each team taking one v-head of the group at a time: A / P pass from tensor memory,
// in-place inverse (fp32 forward substitution on 16x16 blocks, two levels of recursive doubling on
// TF32 warp MMAs), T and (diag(d) T)^T as bf16 tiles, then three M=64 MMAs (the two 64-column
// halves of Z, and PT) and the bf16 epilogue into a staging area that leaves by two bulk copies.
// Persistent CTAs, two per SM (85 KB of shared memory, 256 tensor-memory columns each).
#pragma once
#include <cuda.h>

#include <type_traits>

#include "prefill_common.cuh"
#include "prefill_uw.cuh"  // uw:: helpers (TF32 block products, packed fp32 pairs)

namespace gdn {

struct ZPParams {
    ChunkMap map;
    ScalarView beta;
    ScalarView gate;  // raw per-token log-decay (the chunk-local cumsum is taken here); ptr == NULL: no decay
    uint8_t* blocks;  // kZPBlockBytes per (global chunk, v-head)
    float p_scale;    // output scale, folded into P
    float* norms;     // kNorm: 128 floats per (global chunk, k-head): rsqrt(sum k^2 + eps)[64], the same for q [64]
    int kh, vh;
    int num_chunks;
    int* status;
};

struct ZPSmem {
    static constexpr int kLd = 68;  // fp32 row stride of A, conflict-free for the MMA fragment loads
    // K and Q tiles interleaved atom by atom: [K cols 0-63 | Q cols 0-63 | K cols 64-127 | Q cols 64-127],
    // 8 KB each, so that rows 0-127 of one atom pair are K stacked on Q (the M=128 A operand)
    static constexpr int kOffKQ = 0;
    static constexpr int kTeam = 32768;                  // per-team area starts here, two of them
    static constexpr int kOffA = 0;                      // A / X fp32 (17 KB), later T | (dT)^T, later the staged Z
    static constexpr int kOffP = 64 * kLd * 4;           // 17408: P tile (8 KB), later the staged PT
    static constexpr int kOffVec = kOffP + 8192;         // beta[64], g log2e[64], d[64], scan partials[64], column factors[32]
    static constexpr int kTeamBytes = kOffVec + 2048;    // 27648 (multiple of 1024)
    static constexpr int kOffNorm = kTeam + 2 * kTeamBytes;  // kNorm: inverse row norms of K [64] and Q [64], their log2 [128]
    static constexpr int kOffBar = kOffNorm + 1024;
    static constexpr int kBytes = kOffBar + 128 + 1024;
    static_assert(kOffP % 1024 == 0 && kTeamBytes % 1024 == 0, "swizzled tiles need 1024-byte alignment");
};

namespace zp {
constexpr int kThreads = 256;
constexpr uint32_t kTmKQ = 0;    // fp32 K K^T (lanes 0-63) and Q K^T (lanes 64-127), 64 columns
constexpr uint32_t kTmPT = 64;   // PT of team 0 (lanes +0) and team 1 (lanes +16), 64 columns
constexpr uint32_t kTmZ = 128;   // + 64 * team: Z columns 0-63 (lanes +0) and 64-127 (lanes +16)
__device__ __forceinline__ void team_sync(int team) {
    if (team)
        asm volatile("bar.sync 2, 128;" ::: "memory");
    else
        asm volatile("bar.sync 1, 128;" ::: "memory");
}
}  // namespace zp

// kNorm: q and k are L2-normalised per head (x * rsqrt(sum x^2 + 1e-6)) without touching the tiles:
// (k_i.k_j) r_i r_j and (q_i.k_j) rq_i r_j enter through the row factor of the A / P pass and through
// the column's gate (g_j - log2 r_j in the exponent), Z = (dT)^T diag(r) K through d_i r_i.  The
// factors are also written to `norms` for the state kernel.
template <bool kNorm>
__global__ void __launch_bounds__(zp::kThreads, 2) gdn_zp_kernel(const __grid_constant__ CUtensorMap tmK,
                                                                 const __grid_constant__ CUtensorMap tmQ,
                                                                 const ZPParams p) {
    using namespace ptx;
    using namespace uw;
    using namespace zp;
    using L = ZPSmem;
    constexpr int LD = L::kLd;
    extern __shared__ uint8_t smem_raw[];
    // aligned by an offset from the array itself, so that the compiler still knows the pointer is shared memory
    uint8_t* smem = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int team = warp >> 2, tw = warp & 3, tt = tid & 127;
    uint8_t* sKQ = smem + L::kOffKQ;
    uint8_t* tbase = smem + L::kTeam + team * L::kTeamBytes;
    float* sA = reinterpret_cast<float*>(tbase + L::kOffA);
    uint8_t* sT = tbase + L::kOffA;           // T   = X diag(beta), rows i (128 B), columns j
    uint8_t* sTd = tbase + L::kOffA + 8192;   // dT  = diag(d) T, same layout; read MN-major as (dT)^T
    uint8_t* sP = tbase + L::kOffP;
    float* sBeta = reinterpret_cast<float*>(tbase + L::kOffVec);
    float* sG = sBeta + 64;
    float* sD = sG + 64;
    float* sPart = sD + 64;   // 64 floats: partial sums of the gate scan (each half of the chunk on its own)
    float* sC = sPart + 64;    // 32 floats: e^{g_32 - g_j} for the columns j < 32 of the block below the diagonal
    float* sRn = reinterpret_cast<float*>(smem + L::kOffNorm);  // [128] inverse norms (K rows, then Q rows)
    float* sLr = sRn + 128;                                      // [128] their log2
    uint64_t* bar_load = reinterpret_cast<uint64_t*>(smem + L::kOffBar);
    uint64_t* bar_kq = bar_load + 1;
    uint64_t* bar_mma = bar_load + 2;  // [2], one per team
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_load + 4);
    int* abort_flag = reinterpret_cast<int*>(tmem_slot + 1);
    int* teams_done = abort_flag + 1;  // teams that have finished reading the current unit's K tile

    if (tid == 0) {
        *abort_flag = 0;
        *teams_done = 0;
        mbar_init(bar_load, 1);
        mbar_init(bar_kq, 1);
        mbar_init(&bar_mma[0], 1);
        mbar_init(&bar_mma[1], 1);
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(tmem_slot, 256);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    // This kernel is launched as a programmatic dependent of whatever precedes it in the stream: it is placed
    // and set up while that work drains and waits here, before its first read of global memory.
    grid_dep_wait();
    // The state kernel that follows may be placed on SMs as this grid drains (it takes a whole SM, so
    // never beside a CTA of this kernel) and do its set-up there; it reads this kernel's results only
    // after its own grid_dep_wait.  The release comes AFTER the wait above: the state kernel loads its initial
    // state (which the work before this kernel may have produced: a state handed over from the previous call)
    // without waiting, so it must not be able to start before that work has completed.
    if (tid == 0) grid_dep_launch();

    const int rep = p.vh / p.kh;               // v-heads per k-head
    const int rounds = (rep + 1) >> 1;         // head pairs per unit
    const int total_units = p.num_chunks * p.kh;
    // Order of the work units.  Padded mode: the chunks of all sequences from the LAST chunk position to the
    // first (sequences and k-heads inside), so that what this kernel writes last - the blocks of the first
    // chunks - is what the state kernel, which starts right after it, reads first: still in L2.
    // Packed mode: chunk_indices order.
    const int per_pos = p.map.cu_seqlens ? 0 : (p.num_chunks / p.map.chunks_per_seq) * p.kh;  // units per chunk position
    auto unit_chunk = [&](int unit, int& chunk, int& khead) {
        if (per_pos) {
            const int pos = unit / per_pos, rem = unit - pos * per_pos;
            const int seq = rem / p.kh;
            khead = rem - seq * p.kh;
            chunk = seq * p.map.chunks_per_seq + (p.map.chunks_per_seq - 1 - pos);
        } else {
            chunk = unit / p.kh;
            khead = unit - chunk * p.kh;
        }
    };
    // A unit's coordinates are worked out once (a handful of integer divisions) and carried along.
    struct UnitPos {
        int chunk, khead;
        ChunkPos cp;
        bool valid;
    };
    auto decode_unit = [&](int unit) {
        UnitPos u{};
        u.valid = unit < total_units;
        if (u.valid) {
            unit_chunk(unit, u.chunk, u.khead);
            u.cp = locate_chunk(p.map, u.chunk);
        }
        return u;
    };
    auto issue_loads = [&](const UnitPos& u) {  // one thread
        mbar_arrive_expect_tx(bar_load, 4 * 8192);
        for (int a = 0; a < 2; ++a) {
            tma_load_4d(sKQ + a * 16384, &tmK, bar_load, a * 64, u.khead, static_cast<int>(u.cp.tok0), u.cp.batch);
            tma_load_4d(sKQ + a * 16384 + 8192, &tmQ, bar_load, a * 64, u.khead, static_cast<int>(u.cp.tok0), u.cp.batch);
        }
    };
    UnitPos cur = decode_unit(blockIdx.x), nxt{};
    if (tid == 0 && cur.valid) issue_loads(cur);

    // beta and the raw gate of this thread's token for (unit, round): fetched one round ahead, so that
    // their DRAM latency is not in front of every unit
    auto fetch_scalars = [&](const UnitPos& u, int rd, float& b, float& g) {
        b = 0.f;
        g = 0.f;
        const int hloc = 2 * rd + team;
        if (!u.valid || hloc >= rep) return;
        if (tt < u.cp.n) {
            const int head = u.khead * rep + hloc;
            b = p.beta.load(u.cp.batch, u.cp.tok0 + tt, head);
            if (p.gate.ptr) g = p.gate.load(u.cp.batch, u.cp.tok0 + tt, head);
        }
    };
    float b_next, g_next;
    fetch_scalars(cur, 0, b_next, g_next);

    uint32_t it = 0;      // units done by this CTA (parity of bar_load and bar_kq)
    uint32_t mma_it = 0;  // MMA groups this team has waited for (parity of bar_mma[team])
    bool stores_pending = false;
    for (int unit = blockIdx.x; unit < total_units; unit += gridDim.x, ++it, cur = nxt) {
        const int chunk = cur.chunk, khead = cur.khead;
        const ChunkPos cp = cur.cp;
        const int n = cp.n;
        for (int rd = 0; rd < rounds; ++rd) {
            const int hloc = 2 * rd + team;
            const bool active = hloc < rep;  // team-uniform
            const int head = khead * rep + hloc;
            // ---- beta, chunk-local cumulative gate, decay to the chunk's last token
            if (!active) {  // (odd number of v-heads per k-head: team 1 sits the last round out)
                nxt = decode_unit(unit + gridDim.x);
                fetch_scalars(nxt, 0, b_next, g_next);
            } else {
                const float b_mine = b_next, g_mine = g_next;
                if (tt < 64) {
                    float g = g_mine;
#pragma unroll
                    for (int m = 1; m < 32; m <<= 1) {
                        const float y = __shfl_up_sync(0xffffffffu, g, m);
                        if (lane >= m) g += y;
                    }
                    sPart[tt] = g;  // cumulative sum within each half of the chunk
                }
                team_sync(team);
                if (tt < 64) {
                    // tokens past the end had a raw gate of 0: they carry the last valid value
                    const float g = sPart[tt] + (tt >= 32 ? sPart[31] : 0.f);
                    const float gl = sPart[n - 1] + (n - 1 >= 32 ? sPart[31] : 0.f);
                    sBeta[tt] = b_mine;
                    sG[tt] = g * 1.4426950408889634f;  // times log2(e): decay factors are ex2 of differences
                    sD[tt] = __expf(gl - g);
                    if (tt < 32) sC[tt] = __expf(sPart[32] + sPart[31] - g);  // g_32 is the first entry of the second scan plus the first half's total
                }
                team_sync(team);
            }
            // ---- K K^T (lanes 0-63) and Q K^T (lanes 64-127): once per unit, shared by its v-heads
            if (rd == 0) {
                mbar_wait(bar_load, it & 1u, abort_flag);
                if (kNorm) {
                    // inverse L2 norm of every row of the stacked K | Q tile: two threads per row, 64 columns each
                    const int r = tid >> 1, hf = tid & 1;
                    const uint8_t* rowp = sKQ + hf * 16384 + (r >> 6) * 8192 + (r & 63) * 128;
                    float ss = 0.f;
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        const uint4 w = *reinterpret_cast<const uint4*>(rowp + 16 * c);
                        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float lo = bf16_lo(ww[e]), hi = bf16_hi(ww[e]);
                            ss = fmaf(lo, lo, ss);
                            ss = fmaf(hi, hi, ss);
                        }
                    }
                    ss += __shfl_xor_sync(0xffffffffu, ss, 1);
                    const float rinv = rsqrtf(ss + 1e-6f);
                    if (hf == 0) {
                        sRn[r] = rinv;
                        sLr[r] = log2f(rinv);
                        if (*abort_flag == 0) p.norms[(static_cast<size_t>(chunk) * p.kh + khead) * 128 + r] = rinv;
                    }
                    __syncthreads();
                }
                if (warp == 0) {
                    tc_fence_after_sync();
                    constexpr uint32_t idesc = make_idesc_bf16(128, 64, false, false);
                    const uint64_t dkq = make_smem_desc_sw128(smem_u32(sKQ), 0, 1024);  // A: 128 rows, B: its first 64
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks) {
                        const uint32_t off = kmajor_step(ks, 16384);
                        if (ks == 0)
                            mma_ss_w<false>(tmem + kTmKQ, desc_advance(dkq, off), desc_advance(dkq, off), idesc);
                        else
                            mma_ss_w<true>(tmem + kTmKQ, desc_advance(dkq, off), desc_advance(dkq, off), idesc);
                    }
                    mma_commit_w(bar_kq);
                }
                __syncwarp();
                mbar_wait(bar_kq, it & 1u, abort_flag);
                tc_fence_after_sync();
            }
            if (active) {
                if (stores_pending) {
                    // the previous round's staged Z and PT must have been read out before A and P are rewritten;
                    // by now that has long happened and the wait costs nothing
                    if (tt == 0) bulk_wait_read<0>();
                    stores_pending = false;
                    team_sync(team);
                }
                // ---- A = tril(beta_i (k_i.k_j) e^{g_i-g_j}, -1) in fp32 (warps 0, 1 of the team) and
                //      P = scale tril((q_i.k_j) e^{g_i-g_j}) as a bf16 tile (warps 2, 3); thread = row
                {
                    const bool is_p = tw >= 2;
                    const int rb = tw & 1;
                    const int i = 32 * rb + lane;
                    const float gi = sG[i];
                    float f = is_p ? p.p_scale : sBeta[i];
                    if (kNorm) f *= sRn[is_p ? 64 + i : i];
                    const f2 fv = pk(f, f);
                    const int lim = (i < n) ? (is_p ? i : i - 1) : -1;  // columns kept: col <= lim
                    for (int cb = 0; cb <= rb; ++cb) {
                        uint32_t r[32];
                        tmem_ld32(tmem + kTmKQ + (static_cast<uint32_t>(32 * tw) << 16) + 32 * cb, r);
                        tmem_wait_ld();
                        // kMode 0: the block meets the diagonal (or the chunk is ragged): every element masked.
                        // kMode 1: a block entirely below the diagonal of a full chunk: every element kept.
                        // kMode 2: the same, with the decay of the block factored: for rows i >= 32 and columns j < 32
                        //          e^{g_i-g_j} = e^{g_i-g_32} e^{g_32-g_j}, both factors <= 1 (the cumulative gate only
                        //          falls), so the column factors come from a table and no ex2 is left per element.
                        auto block = [&](auto mode_tag) {
                            constexpr int kMode = decltype(mode_tag)::value;
                            constexpr bool kMask = kMode == 0;
                            f2 fvr = fv;
                            if (kMode == 2) {
                                const float ri = ex2(gi - sG[32]);
                                fvr = mul2(fv, pk(ri, ri));
                            }
#pragma unroll
                            for (int j = 0; j < 32; j += 8) {
                                float o[8];
#pragma unroll
                                for (int e4 = 0; e4 < 2; ++e4) {
                                    const float4 gc = *reinterpret_cast<const float4*>((kMode == 2 ? sC : sG) + 32 * cb + j + 4 * e4);
                                    float gcv[4] = {gc.x, gc.y, gc.z, gc.w};
                                    if (kNorm) {  // the column's key norm enters through the exponent
                                        const float4 lr = *reinterpret_cast<const float4*>(sLr + 32 * cb + j + 4 * e4);
                                        gcv[0] -= lr.x; gcv[1] -= lr.y; gcv[2] -= lr.z; gcv[3] -= lr.w;
                                    }
#pragma unroll
                                    for (int e = 0; e < 4; e += 2) {
                                        const int col = 32 * cb + j + 4 * e4 + e, k = j + 4 * e4 + e;
                                        float d0, d1;
                                        if (kMode == 2) {
                                            d0 = gcv[e];
                                            d1 = gcv[e + 1];
                                        } else {
                                            d0 = (!kMask || col <= lim) ? ex2(gi - gcv[e]) : 0.f;
                                            d1 = (!kMask || col + 1 <= lim) ? ex2(gi - gcv[e + 1]) : 0.f;
                                        }
                                        unpk(mul2(mul2(pk(__uint_as_float(r[k]), __uint_as_float(r[k + 1])), fvr), pk(d0, d1)),
                                             o[4 * e4 + e], o[4 * e4 + e + 1]);
                                    }
                                }
                                if (!is_p) {
                                    *reinterpret_cast<float4*>(&sA[i * LD + 32 * cb + j]) = make_float4(o[0], o[1], o[2], o[3]);
                                    *reinterpret_cast<float4*>(&sA[i * LD + 32 * cb + j + 4]) = make_float4(o[4], o[5], o[6], o[7]);
                                } else {
                                    *reinterpret_cast<uint4*>(sP + tile_off(i, (32 * cb + j) >> 3)) =
                                        make_uint4(pack_bf16(o[0], o[1]), pack_bf16(o[2], o[3]), pack_bf16(o[4], o[5]),
                                                   pack_bf16(o[6], o[7]));
                                }
                            }
                        };
                        if (cb < rb && n == kChunk) {
                            if (kNorm)
                                block(std::integral_constant<int, 1>{});
                            else
                                block(std::integral_constant<int, 2>{});
                        } else {
                            block(std::integral_constant<int, 0>{});
                        }
                    }
                    if (is_p && rb == 0) {  // rows 0-31 of P: columns 32-63 lie above the diagonal
#pragma unroll
                        for (int c16 = 4; c16 < 8; ++c16)
                            *reinterpret_cast<uint4*>(sP + tile_off(i, c16)) = make_uint4(0u, 0u, 0u, 0u);
                    }
                }
                if (rd + 1 < rounds) {
                    fetch_scalars(cur, rd + 1, b_next, g_next);
                } else {
                    nxt = decode_unit(unit + gridDim.x);
                    fetch_scalars(nxt, 0, b_next, g_next);
                }
                tc_fence_before_sync();
                team_sync(team);
                // ---- X = (I + A)^-1 in place.  Every warp owns one 16x16 diagonal block: its two 8x8 diagonal
                //      blocks by forward substitution in fp32 (one column per lane, 16 lanes), then
                //      X_10 = -X_11 A_10 X_00 with two TF32 warp MMAs (the intermediate stays in registers).
                {
                    const int b = tw, hb = (lane >> 3) & 1, j = lane & 7;
                    const int o = 16 * b + 8 * hb;  // first row / column of this lane's 8x8 block
                    float x[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) x[i] = (i == j) ? 1.f : 0.f;
                    // x_j = 1, x_i = -sum_{m<i} A_im x_m
#pragma unroll
                    for (int i = 1; i < 8; ++i) {
                        float a[8];
#pragma unroll
                        for (int q = 0; q < (i + 3) / 4; ++q) {
                            const float4 t = *reinterpret_cast<const float4*>(&sA[(o + i) * LD + o + 4 * q]);
                            a[4 * q] = t.x; a[4 * q + 1] = t.y; a[4 * q + 2] = t.z; a[4 * q + 3] = t.w;
                        }
                        float acc = 0.f;
#pragma unroll
                        for (int m = 0; m + 1 < i; ++m) acc = fmaf(a[m], x[m], acc);
                        if (i > j) x[i] = -fmaf(a[i - 1], x[i - 1], acc);
                    }
                    __syncwarp();  // the block is private to this warp: every lane has read it
                    if (lane < 16) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) sA[(o + i) * LD + o + j] = x[i];
                    }
                    __syncwarp();
                    // level 0 (8 -> 16)
                    const int i0 = 16 * b + 8, j0 = 16 * b;
                    float d[4] = {0.f, 0.f, 0.f, 0.f};
                    mma_block8(d, sA, LD, i0, j0, sA, LD, j0, j0, lane);  // t = A_10 X_00; lane (g, t) holds t[g][2t], t[g][2t+1]
                    // t as the B operand of the next product: lane (g, t) needs t[t][g] and t[t + 4][g]
                    const int g = lane >> 2, tq = lane & 3;
                    const float v00 = __shfl_sync(0xffffffffu, d[0], 4 * tq + (g >> 1));
                    const float v01 = __shfl_sync(0xffffffffu, d[1], 4 * tq + (g >> 1));
                    const float v10 = __shfl_sync(0xffffffffu, d[0], 4 * (tq + 4) + (g >> 1));
                    const float v11 = __shfl_sync(0xffffffffu, d[1], 4 * (tq + 4) + (g >> 1));
                    uint32_t bfrag[2] = {to_tf32((g & 1) ? v01 : v00), to_tf32((g & 1) ? v11 : v10)};
                    uint32_t afrag[4] = {to_tf32(sA[(i0 + g) * LD + i0 + tq]), 0u, to_tf32(sA[(i0 + g) * LD + i0 + tq + 4]), 0u};
                    float e[4] = {0.f, 0.f, 0.f, 0.f};
                    mma_tf32(e, afrag, bfrag);  // X_11 t
                    *reinterpret_cast<float2*>(&sA[(i0 + g) * LD + j0 + 2 * tq]) = make_float2(-e[0], -e[1]);
                }
                team_sync(team);
                // level 1 (16 -> 32): X_10 = -X_11 A_10 X_00, X_32 = -X_33 A_32 X_22; warp = (pair, 8-column half);
                // the intermediate A_10 X_00 is parked in the unused block above the diagonal
                {
                    const int pr = tw >> 1, n0 = 8 * (tw & 1);
                    const int i0 = 16 * (2 * pr + 1), j0 = 16 * (2 * pr);
                    float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int ks = 0; ks < 2; ++ks) mma_block(d, sA, LD, i0, j0 + 8 * ks, sA, LD, j0 + 8 * ks, j0 + n0, lane);
                    store_block(d, 1.f, sA, LD, j0, i0 + n0, lane);
                    team_sync(team);
                    float e[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int ks = 0; ks < 2; ++ks) mma_block(e, sA, LD, i0, i0 + 8 * ks, sA, LD, j0 + 8 * ks, i0 + n0, lane);
                    store_block(e, -1.f, sA, LD, i0, j0 + n0, lane);
                }
                team_sync(team);
                // level 2 (32 -> 64): X_[2:4,0:2] = -X_[2:4,2:4] A_[2:4,0:2] X_[0:2,0:2]; warp = 16x16 block of the
                // result; the intermediate goes to the unused upper-right quadrant
                {
                    const int rb = tw >> 1, cb = tw & 1;
                    float d[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        if (ks >= 2 * cb) {
                            uint32_t af[4], bf[2];
                            load_afrag(af, sA, LD, 32 + 16 * rb, 8 * ks, lane);  // shared by the two column tiles
#pragma unroll
                            for (int nt = 0; nt < 2; ++nt) {
                                load_bfrag(bf, sA, LD, 8 * ks, 16 * cb + 8 * nt, lane);
                                mma_tf32(d[nt], af, bf);
                            }
                        }
                    }
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt) store_block(d[nt], 1.f, sA, LD, 16 * rb, 32 + 16 * cb + 8 * nt, lane);
                    team_sync(team);
                    float e[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        if (ks < 2 * (rb + 1)) {
                            uint32_t af[4], bf[2];
                            load_afrag(af, sA, LD, 32 + 16 * rb, 32 + 8 * ks, lane);
#pragma unroll
                            for (int nt = 0; nt < 2; ++nt) {
                                load_bfrag(bf, sA, LD, 8 * ks, 32 + 16 * cb + 8 * nt, lane);
                                mma_tf32(e[nt], af, bf);
                            }
                        }
                    }
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt) store_block(e[nt], -1.f, sA, LD, 32 + 16 * rb, 16 * cb + 8 * nt, lane);
                }
                team_sync(team);
                // ---- T = X diag(beta) and dT = diag(d) T as bf16 swizzled tiles (row = token i, 64 columns j) over X;
                //      every thread first pulls its 32 values of X into registers
                {
                    const int i = tt >> 1, c0 = (tt & 1) * 32;
                    float xs[32];
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        const float4 t = *reinterpret_cast<const float4*>(&sA[i * LD + c0 + 4 * q]);
                        const bool valid = ((c0 + 4 * q) >> 4) <= (i >> 4);  // blocks above the diagonal hold scratch
                        xs[4 * q] = valid ? t.x : 0.f; xs[4 * q + 1] = valid ? t.y : 0.f;
                        xs[4 * q + 2] = valid ? t.z : 0.f; xs[4 * q + 3] = valid ? t.w : 0.f;
                    }
                    const float di = kNorm ? sD[i] * sRn[i] : sD[i];
                    const f2 di2 = pk(di, di);
                    team_sync(team);
#pragma unroll
                    for (int ch = 0; ch < 4; ++ch) {
                        const float4 b0 = *reinterpret_cast<const float4*>(&sBeta[c0 + 8 * ch]);
                        const float4 b1 = *reinterpret_cast<const float4*>(&sBeta[c0 + 8 * ch + 4]);
                        const float* x = xs + 8 * ch;
                        const f2 t0 = mul2(pk(x[0], x[1]), pk(b0.x, b0.y)), t1 = mul2(pk(x[2], x[3]), pk(b0.z, b0.w));
                        const f2 t2 = mul2(pk(x[4], x[5]), pk(b1.x, b1.y)), t3 = mul2(pk(x[6], x[7]), pk(b1.z, b1.w));
                        float v[8], w[8];
                        unpk(t0, v[0], v[1]); unpk(t1, v[2], v[3]); unpk(t2, v[4], v[5]); unpk(t3, v[6], v[7]);
                        unpk(mul2(t0, di2), w[0], w[1]); unpk(mul2(t1, di2), w[2], w[3]);
                        unpk(mul2(t2, di2), w[4], w[5]); unpk(mul2(t3, di2), w[6], w[7]);
                        const uint32_t off = sw128_offset(i, c0 + 8 * ch);
                        *reinterpret_cast<uint4*>(sT + off) = make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]),
                                                                         pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
                        *reinterpret_cast<uint4*>(sTd + off) = make_uint4(pack_bf16(w[0], w[1]), pack_bf16(w[2], w[3]),
                                                                          pack_bf16(w[4], w[5]), pack_bf16(w[6], w[7]));
                    }
                }
                fence_proxy_async_smem();
                team_sync(team);
                // ---- Z = (dT)^T K as two 64-column halves (lanes +0 / +16 of the team's columns), PT = P T
                if (tw == 0) {
                    tc_fence_after_sync();
                    constexpr uint32_t idesc = make_idesc_bf16(64, 64, false, true);   // PT: A K-major, B MN-major
                    constexpr uint32_t idescz = make_idesc_bf16(64, 64, true, true);   // Z: A = (dT)^T read MN-major too
                    const uint64_t dTd = make_smem_desc_sw128(smem_u32(sTd), 8192, 1024);       // A, read MN-major
                    const uint64_t dPa = make_smem_desc_sw128(smem_u32(sP), 0, 1024);           // A, K-major
                    const uint64_t dTb = make_smem_desc_sw128(smem_u32(sT), 8192, 1024);        // B, read MN-major
                    const uint64_t dK0 = make_smem_desc_sw128(smem_u32(sKQ), 8192, 1024);       // B, K columns 0-63, MN-major
                    const uint64_t dK1 = make_smem_desc_sw128(smem_u32(sKQ + 16384), 8192, 1024);
                    const uint32_t tZ = tmem + kTmZ + 64u * team;
                    const uint32_t tPT = tmem + kTmPT + (team ? (16u << 16) : 0u);
                    mma_ss_w<false>(tZ, dTd, dK0, idescz);
#pragma unroll
                    for (int ks = 1; ks < 4; ++ks) mma_ss_w<true>(tZ, desc_advance(dTd, ks * 2048), desc_advance(dK0, ks * 2048), idescz);
                    mma_ss_w<false>(tZ + (16u << 16), dTd, dK1, idescz);
#pragma unroll
                    for (int ks = 1; ks < 4; ++ks)
                        mma_ss_w<true>(tZ + (16u << 16), desc_advance(dTd, ks * 2048), desc_advance(dK1, ks * 2048), idescz);
                    mma_ss_w<false>(tPT, dPa, dTb, idesc);
#pragma unroll
                    for (int ks = 1; ks < 4; ++ks) mma_ss_w<true>(tPT, desc_advance(dPa, ks * 32), desc_advance(dTb, ks * 2048), idesc);
                    mma_commit_w(&bar_mma[team]);
                }
                __syncwarp();
                mbar_wait(&bar_mma[team], mma_it & 1u, abort_flag);
                ++mma_it;
                tc_fence_after_sync();
            }
            if (rd == rounds - 1 && tt == 0) {
                // This team's MMAs have read the K tile (or it sat the round out).  The team that gets here second
                // knows that both are done with the tiles and requests the next unit's, which land while the
                // epilogues run; the teams do not wait for one another.
                if (atomicAdd(teams_done, 1) == 1) {
                    *teams_done = 0;
                    if (nxt.valid) issue_loads(nxt);
                }
            }
            if (active) {
                // ---- accumulators -> bf16 -> staged tiles (Z over T / dT, PT over P) -> two bulk copies
                uint8_t* stZ = tbase + L::kOffA;
                const int row = 16 * tw + (lane & 15), hi = lane >> 4;
                const uint32_t tl = static_cast<uint32_t>(32 * tw) << 16;
#pragma unroll
                for (int cb = 0; cb < 2; ++cb) {
                    uint32_t r[32];
                    tmem_ld32(tmem + kTmZ + 64u * team + tl + 32 * cb, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        *reinterpret_cast<uint4*>(stZ + tile_off(row, 8 * hi + 4 * cb + q)) = make_uint4(
                            pack_bf16(__uint_as_float(r[8 * q + 0]), __uint_as_float(r[8 * q + 1])),
                            pack_bf16(__uint_as_float(r[8 * q + 2]), __uint_as_float(r[8 * q + 3])),
                            pack_bf16(__uint_as_float(r[8 * q + 4]), __uint_as_float(r[8 * q + 5])),
                            pack_bf16(__uint_as_float(r[8 * q + 6]), __uint_as_float(r[8 * q + 7])));
                }
#pragma unroll
                for (int cb = 0; cb < 2; ++cb) {
                    uint32_t r[32];
                    tmem_ld32(tmem + kTmPT + tl + 32 * cb, r);  // lanes +0: team 0's PT, lanes +16: team 1's
                    tmem_wait_ld();
                    if (hi == team) {
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            *reinterpret_cast<uint4*>(sP + tile_off(row, 4 * cb + q)) = make_uint4(
                                pack_bf16(__uint_as_float(r[8 * q + 0]), __uint_as_float(r[8 * q + 1])),
                                pack_bf16(__uint_as_float(r[8 * q + 2]), __uint_as_float(r[8 * q + 3])),
                                pack_bf16(__uint_as_float(r[8 * q + 4]), __uint_as_float(r[8 * q + 5])),
                                pack_bf16(__uint_as_float(r[8 * q + 6]), __uint_as_float(r[8 * q + 7])));
                    }
                }
                fence_proxy_async_smem();
                tc_fence_before_sync();
                team_sync(team);
                if (tt == 0 && *abort_flag == 0) {  // nothing is written once a wait has given up
                    uint8_t* dst = p.blocks + (static_cast<size_t>(chunk) * p.vh + head) * kZPBlockBytes;
                    // the state kernel reads these blocks back soon: ask L2 to hold on to them
                    const uint64_t keep = l2_policy_evict_last();
                    bulk_store_hint(dst, stZ, 16384, keep);
                    bulk_store_hint(dst + 16384, sP, 8192, keep);
                    bulk_commit();
                }
                stores_pending = true;
            }
        }  // head pairs
    }      // units
    if (stores_pending && tt == 0) bulk_wait_read<0>();
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 256);
    if (tid == 0 && *abort_flag && p.status) atomicExch(p.status, 2);
}

}  // namespace gdn
