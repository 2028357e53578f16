// WY / UT transform of chunked Gated DeltaNet prefill: per (64-token chunk, v-head)
//     A = tril(diag(beta) K K^T .* exp(g_i - g_j), -1),  X = (I + A)^-1
//     U = X diag(beta) V,   W = X diag(beta exp(g)) K
// with g the chunk-local cumulative gate.  Stands in for the reference's
// sm90_bf16_compute_u_w (gdn_cuda/include/gdn_cuda/kernels/sm90_bf16_gdn_compute_u_w.cuh:153-667),
// using the canonical W (gate folded in before the solve).
//
// This is the stage kernel behind the low-level wrapper gdn_compute_u_w; the whole-layer path
// (gdn_chunked_forward) folds the transform into the recurrence instead (prefill_zp.cuh).
// Persistent CTAs of 128 threads (four per SM) walk the (chunk, v-head) units.  tcgen05 tensor
// cores do the big contractions with the TMA-loaded tiles used as they are:
//   K K^T      : M=64 N=32 K=D MMAs, one accumulator per issuing warp (columns 0-31 and 32-63 of
//                the product), interleaved in the same tensor-memory columns (lanes +0 and +16 of
//                every 32-lane quarter), so one 32-lane load hands every thread of a warp half a row;
//   U = T V    : M=64 N=D K=64, A = T (bf16, written by the CTA), B = the V tile read MN-major;
//   W = T' K   : M=64 N=D K=64, A = T' = X diag(beta e^g), B = the K tile read MN-major;
//                U and W are interleaved the same way (U in lanes +0, W in lanes +16).
// One pass over the first accumulators forms A (fp32, shared memory) with one ex2 per element.
// The unit-lower-triangular
// inverse: the 16x16 diagonal blocks in fp32 by forward substitution (one column per thread),
// then two levels of recursive doubling (16 -> 32 -> 64) whose block products use warp-level
// tensor-core MMAs on TF32 operands with fp32 accumulation, all in place.
// Tensor memory: D columns.  Shared memory (52 KB): the K tile (later the U staging tile), the V
// tile (later the W staging tile) and A (later T, T').  U and W go to the caller's token-major
// tensors through tiled TMA stores (row-predicated stores for a ragged packed tail).
#pragma once
#include <cuda.h>

#include "prefill_common.cuh"

namespace gdn {

struct UWParams {
    ChunkMap map;
    ScalarView beta;
    ScalarView gate;      // ptr == NULL: no decay
    int gate_is_raw;      // 1: per-token log-decay (cumsum taken here); 0: already chunk-local cumsum
    TokenView u, w;
    int kh, vh;
    int num_chunks;
    int* status;
};

template <int D>
struct UWSmem {
    static constexpr int kTile = kChunk * D * 2;  // K or V tile; later the U / W staging tile
    static constexpr int kLd = 68;                // fp32 row stride, conflict-free for MMA fragment loads
    static constexpr int kOffK = 0;
    static constexpr int kOffV = kOffK + kTile;
    static constexpr int kOffA = kOffV + kTile;           // A, overwritten block by block with X = (I+A)^-1;
                                                          // blocks above the diagonal are scratch; later T and T'
    static constexpr int kOffVec = kOffA + 64 * kLd * 4;  // beta[64], g log2(e) [64], beta e^g [64]
    static constexpr int kOffBar = kOffVec + 3 * 64 * 4;  // 2 mbarriers, tmem slot, abort flag
    static constexpr int kBytes = kOffBar + 64 + 1024;    // + alignment slack
    static_assert(64 * kLd * 4 >= 2 * 8192, "T and T' must fit over A");
    static_assert(kOffA % 1024 == 0, "swizzled tiles need 1024-byte alignment");
};

namespace uw {
__device__ __forceinline__ uint32_t to_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return r;
}
using f2 = unsigned long long;  // two fp32 values in a 64-bit register pair
__device__ __forceinline__ f2 pk(float lo, float hi) {
    f2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpk(f2 v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f2 mul2(f2 a, f2 b) {
    f2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void mma_tf32(float* d, const uint32_t* a, const uint32_t* b) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
// d(16x8) += A(16x8 at [r0][k0] of `am`) * B(8x8 at [k0b][n0] of `bm`), TF32 operands, fp32 accumulation.
// The operands are entries of A and of (I+A)^-1 blocks; their TF32 rounding (2^-11) perturbs the
// inverse by well under the bf16 rounding (2^-9) its result receives anyway.
__device__ __forceinline__ void mma_block(float* d, const float* am, int lda, int r0, int k0, const float* bm,
                                          int ldb, int k0b, int n0, int lane) {
    const int g = lane >> 2, t = lane & 3;
    uint32_t a[4], b[2];
    a[0] = to_tf32(am[(r0 + g) * lda + k0 + t]);
    a[1] = to_tf32(am[(r0 + g + 8) * lda + k0 + t]);
    a[2] = to_tf32(am[(r0 + g) * lda + k0 + t + 4]);
    a[3] = to_tf32(am[(r0 + g + 8) * lda + k0 + t + 4]);
    b[0] = to_tf32(bm[(k0b + t) * ldb + n0 + g]);
    b[1] = to_tf32(bm[(k0b + t + 4) * ldb + n0 + g]);
    mma_tf32(d, a, b);
}
// The two operand fragments of mma_block on their own, for products that share one of them.
__device__ __forceinline__ void load_afrag(uint32_t* a, const float* am, int lda, int r0, int k0, int lane) {
    const int g = lane >> 2, t = lane & 3;
    a[0] = to_tf32(am[(r0 + g) * lda + k0 + t]);
    a[1] = to_tf32(am[(r0 + g + 8) * lda + k0 + t]);
    a[2] = to_tf32(am[(r0 + g) * lda + k0 + t + 4]);
    a[3] = to_tf32(am[(r0 + g + 8) * lda + k0 + t + 4]);
}
__device__ __forceinline__ void load_bfrag(uint32_t* b, const float* bm, int ldb, int k0b, int n0, int lane) {
    const int g = lane >> 2, t = lane & 3;
    b[0] = to_tf32(bm[(k0b + t) * ldb + n0 + g]);
    b[1] = to_tf32(bm[(k0b + t + 4) * ldb + n0 + g]);
}
// d(rows 0-7 of the 16x8 tile) += A(8x8 at [r0][k0] of `am`) * B(8x8 at [k0b][n0] of `bm`): the upper half of
// the warp MMA; lane (g, t) ends up with d[0], d[1] = rows g, columns 2t, 2t+1 of the product.
__device__ __forceinline__ void mma_block8(float* d, const float* am, int lda, int r0, int k0, const float* bm,
                                           int ldb, int k0b, int n0, int lane) {
    const int g = lane >> 2, t = lane & 3;
    uint32_t a[4], b[2];
    a[0] = to_tf32(am[(r0 + g) * lda + k0 + t]);
    a[1] = 0u;
    a[2] = to_tf32(am[(r0 + g) * lda + k0 + t + 4]);
    a[3] = 0u;
    b[0] = to_tf32(bm[(k0b + t) * ldb + n0 + g]);
    b[1] = to_tf32(bm[(k0b + t + 4) * ldb + n0 + g]);
    mma_tf32(d, a, b);
}
// store sign * d (16x8) at [r0][n0]
__device__ __forceinline__ void store_block(const float* d, float sign, float* m, int ld, int r0, int n0, int lane) {
    const int g = lane >> 2, t = lane & 3;
    *reinterpret_cast<float2*>(&m[(r0 + g) * ld + n0 + 2 * t]) = make_float2(sign * d[0], sign * d[1]);
    *reinterpret_cast<float2*>(&m[(r0 + g + 8) * ld + n0 + 2 * t]) = make_float2(sign * d[2], sign * d[3]);
}
}  // namespace uw

template <int D>
__global__ void __launch_bounds__(128, 4) gdn_uw_kernel(const __grid_constant__ CUtensorMap tmK,
                                                        const __grid_constant__ CUtensorMap tmV,
                                                        const __grid_constant__ CUtensorMap tmUo,
                                                        const __grid_constant__ CUtensorMap tmWo,
                                                        const UWParams p) {
    using namespace ptx;
    using namespace uw;
    using L = UWSmem<D>;
    constexpr int NA = D / 64;  // 64-column swizzle atoms per tile
    constexpr int LD = L::kLd;
    extern __shared__ uint8_t smem_raw[];
    // aligned by an offset from the array itself, so that the compiler still knows the pointer is shared memory
    uint8_t* smem = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* sK = smem + L::kOffK;
    uint8_t* sV = smem + L::kOffV;
    uint8_t* sT = smem + L::kOffA;
    uint8_t* sT2 = sT + 8192;
    float* sA = reinterpret_cast<float*>(smem + L::kOffA);  // A, then X in place
    float* sBeta = reinterpret_cast<float*>(smem + L::kOffVec);
    float* sG = sBeta + 64;
    float* sEg = sG + 64;  // beta e^g per token
    uint64_t* bar_load = reinterpret_cast<uint64_t*>(smem + L::kOffBar);
    uint64_t* bar_mma = bar_load + 1;   // first MMA groups: one commit per issuing warp
    uint64_t* bar_mma2 = bar_load + 2;  // U and W MMAs: two issuing warps
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_load + 3);
    int* abort_flag = reinterpret_cast<int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        *abort_flag = 0;
        mbar_init(bar_load, 1);
        mbar_init(bar_mma, 2);
        mbar_init(bar_mma2, 2);
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(tmem_slot, D);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tLo = tmem, tHi = tmem + (16u << 16);  // the two interleaved M=64 accumulators

    // Persistent CTA: units (chunk, v-head) are walked with the grid as stride, heads fastest, so
    // that the CTAs running at one time share K and Q tiles of a k-head group in L2.  Barriers,
    // tensor memory and the tensor-map fetches are set up once per CTA instead of once per unit
    // (a CTA per unit spent a quarter of its life being launched and retired).
    const int total_units = p.num_chunks * p.vh;
    uint32_t it = 0;
    for (int unit = blockIdx.x; unit < total_units; unit += gridDim.x, ++it) {
    const int chunk = unit / p.vh, head = unit - chunk * p.vh;
    const int khead = head / (p.vh / p.kh);
    const ChunkPos cp = locate_chunk(p.map, chunk);
    const int n = cp.n;
    // beta and gate of this thread's token: requested first, used after the set-up below
    float b_mine = 0.f, g_mine = 0.f;
    if (tid < n) {
        b_mine = p.beta.load(cp.batch, cp.tok0 + tid, head);
        if (p.gate.ptr) g_mine = p.gate.load(cp.batch, cp.tok0 + tid, head);
    }
    // one load phase and two MMA phases per unit
    const uint32_t load_par0 = it & 1u;

    if (tid == 0) {
        mbar_arrive_expect_tx(bar_load, 2 * L::kTile);
        for (int a = 0; a < NA; ++a) {
            tma_load_4d(sK + a * 8192, &tmK, bar_load, a * 64, khead, static_cast<int>(cp.tok0), cp.batch);
            tma_load_4d(sV + a * 8192, &tmV, bar_load, a * 64, head, static_cast<int>(cp.tok0), cp.batch);
        }
    }
    // beta and the chunk-local cumulative gate (rows past the end: beta = 0, g = g of the last row)
    if (tid < 64) {
        float g = g_mine;
        sBeta[tid] = b_mine;
        if (p.gate_is_raw) {
#pragma unroll
            for (int m = 1; m < 32; m <<= 1) {
                const float y = __shfl_up_sync(0xffffffffu, g, m);
                if (lane >= m) g += y;
            }
        }
        sG[tid] = g;
    }
    __syncthreads();
    if (tid < 64) {
        float g = sG[tid];
        if (p.gate_is_raw) {
            if (tid >= 32) g += sG[31];
        } else if (tid >= n) {
            g = sG[n - 1];
        }
        sEg[tid] = g;  // final g, parked here until every thread has read the partial sums
    }
    __syncthreads();
    if (tid < 64) {
        const float g = sEg[tid];
        sG[tid] = g * 1.4426950408889634f;  // from here on the gate times log2(e): decay factors are ex2 of differences
        sEg[tid] = b_mine * __expf(g);  // beta e^g: the column factor of T' = X diag(beta e^g)
    }
    __syncthreads();

    // ---- A_raw = K K^T, columns 0-31 into lanes +0 and columns 32-63 into lanes +16
    mbar_wait(bar_load, load_par0, abort_flag);
    // Every accumulator has its own issuing warp (warp-uniform issue, one elected lane): the issue
    // rate of one warp, not the tensor pipe, is what bounds these small MMAs.
    //   warp 0: K K^T columns 0-31 (lanes +0)    warp 1: K K^T columns 32-63 (lanes +16)
    if (warp < 2) {
        tc_fence_after_sync();
        constexpr uint32_t idesc = make_idesc_bf16(64, 32, false, false);
        const uint64_t dk0 = make_smem_desc_sw128(smem_u32(sK), 0, 1024);
        const uint64_t da = dk0;                                                // A: the K tile
        const uint64_t db = (warp & 1) ? desc_advance(dk0, 32 * 128) : dk0;     // B: rows 32-63 or 0-31 of K
        const uint32_t tacc = (warp & 1) ? tHi : tLo;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            const uint32_t off = kmajor_step(ks, 8192);
            if (ks == 0)
                mma_ss_w<false>(tacc, desc_advance(da, off), desc_advance(db, off), idesc);
            else
                mma_ss_w<true>(tacc, desc_advance(da, off), desc_advance(db, off), idesc);
        }
        mma_commit_w(bar_mma);
    }
    __syncwarp();
    mbar_wait(bar_mma, it & 1u, abort_flag);
    tc_fence_after_sync();
    {
        // row 16*warp + (lane & 15); lanes 0-15 hold columns 0-31, lanes 16-31 columns 32-63.
        const int i = 16 * warp + (lane & 15);
        const int cbase = (lane >> 4) * 32;
        const float bi = sBeta[i], gi = sG[i];
        const f2 bi2 = pk(bi, bi);
        uint32_t r[32];
        tmem_ld32(tmem + (static_cast<uint32_t>(warp * 32) << 16), r);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
            float a[8];
#pragma unroll
            for (int e4 = 0; e4 < 2; ++e4) {
                const float4 gc = *reinterpret_cast<const float4*>(sG + cbase + j + 4 * e4);
                const float gcv[4] = {gc.x, gc.y, gc.z, gc.w};
#pragma unroll
                for (int e = 0; e < 4; e += 2) {
                    // two columns at a time with the two-wide fp32 multiplies; the diagonal entry of
                    // A (which the mask col <= i lets through) is zeroed after the loop
                    const int col = cbase + j + 4 * e4 + e, k = j + 4 * e4 + e;
                    const float d0 = (col <= i && i < n) ? ex2(gi - gcv[e]) : 0.f;
                    const float d1 = (col + 1 <= i && i < n) ? ex2(gi - gcv[e + 1]) : 0.f;
                    const f2 dec2 = pk(d0, d1);
                    unpk(mul2(mul2(pk(__uint_as_float(r[k]), __uint_as_float(r[k + 1])), bi2), dec2), a[4 * e4 + e],
                         a[4 * e4 + e + 1]);
                }
            }
            *reinterpret_cast<float4*>(&sA[i * LD + cbase + j]) = make_float4(a[0], a[1], a[2], a[3]);
            *reinterpret_cast<float4*>(&sA[i * LD + cbase + j + 4]) = make_float4(a[4], a[5], a[6], a[7]);
        }
        if (i >= cbase && i < cbase + 32) sA[i * LD + i] = 0.f;  // A is strictly lower triangular
    }
    tc_fence_before_sync();
    __syncthreads();

    // ---- X = (I + A)^-1, in place.  Diagonal 16x16 blocks: one column per thread.
    {
        const int b = warp, j = lane & 15;
        float x[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) x[i] = (i == j) ? 1.f : 0.f;
        // x_j = 1, x_i = -sum_{m<i} A_im x_m.  Rows are read with 16-byte loads (one address for all
        // lanes: a broadcast); the terms that have been ready for a while are summed in one chain,
        // so that only the newest term waits on x_{i-1}.
#pragma unroll
        for (int i = 1; i < 16; ++i) {
            float a[16];
#pragma unroll
            for (int q = 0; q < (i + 3) / 4; ++q) {
                const float4 t = *reinterpret_cast<const float4*>(&sA[(16 * b + i) * LD + 16 * b + 4 * q]);
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
            for (int i = 0; i < 16; ++i) sA[(16 * b + i) * LD + 16 * b + j] = x[i];
        }
    }
    __syncthreads();
    // level 1 (16 -> 32): X_10 = -X_11 A_10 X_00 and X_32 = -X_33 A_32 X_22; warp = (pair, 8-column half).
    // The intermediate A_10 X_00 is parked in the unused block above the diagonal.
    {
        const int pr = warp >> 1, n0 = 8 * (warp & 1);
        const int i0 = 16 * (2 * pr + 1), j0 = 16 * (2 * pr);
        float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) mma_block(d, sA, LD, i0, j0 + 8 * ks, sA, LD, j0 + 8 * ks, j0 + n0, lane);
        store_block(d, 1.f, sA, LD, j0, i0 + n0, lane);
        __syncthreads();
        float e[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) mma_block(e, sA, LD, i0, i0 + 8 * ks, sA, LD, j0 + 8 * ks, i0 + n0, lane);
        store_block(e, -1.f, sA, LD, i0, j0 + n0, lane);
    }
    __syncthreads();
    // level 2 (32 -> 64): X_[2:4,0:2] = -X_[2:4,2:4] A_[2:4,0:2] X_[0:2,0:2]; warp = 16x16 block of the result.
    // The intermediate goes to the unused upper-right quadrant; K-steps that would only meet the
    // (zero, here scratch) blocks above the diagonal are skipped.
    {
        const int rb = warp >> 1, cb = warp & 1;
        float d[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            if (ks >= 2 * cb) {
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
                    mma_block(d[nt], sA, LD, 32 + 16 * rb, 8 * ks, sA, LD, 8 * ks, 16 * cb + 8 * nt, lane);
            }
        }
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) store_block(d[nt], 1.f, sA, LD, 16 * rb, 32 + 16 * cb + 8 * nt, lane);
        __syncthreads();
        float e[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            if (ks < 2 * (rb + 1)) {
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
                    mma_block(e[nt], sA, LD, 32 + 16 * rb, 32 + 8 * ks, sA, LD, 8 * ks, 32 + 16 * cb + 8 * nt, lane);
            }
        }
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) store_block(e[nt], -1.f, sA, LD, 32 + 16 * rb, 16 * cb + 8 * nt, lane);
    }
    __syncthreads();

    // ---- T = X diag(beta), T' = X diag(beta e^g) as bf16 K-major swizzled tiles written over X:
    //      every thread first pulls its 32 values of X into registers
    {
        const int i = tid >> 1, c0 = (tid & 1) * 32;
        float xs[32], bt[32], eg[32];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const float4 t = *reinterpret_cast<const float4*>(&sA[i * LD + c0 + 4 * q]);
            const bool valid = ((c0 + 4 * q) >> 4) <= (i >> 4);  // blocks above the diagonal hold scratch
            xs[4 * q] = valid ? t.x : 0.f; xs[4 * q + 1] = valid ? t.y : 0.f;
            xs[4 * q + 2] = valid ? t.z : 0.f; xs[4 * q + 3] = valid ? t.w : 0.f;
            const float4 tb = *reinterpret_cast<const float4*>(&sBeta[c0 + 4 * q]);
            bt[4 * q] = tb.x; bt[4 * q + 1] = tb.y; bt[4 * q + 2] = tb.z; bt[4 * q + 3] = tb.w;
            const float4 te = *reinterpret_cast<const float4*>(&sEg[c0 + 4 * q]);
            eg[4 * q] = te.x; eg[4 * q + 1] = te.y; eg[4 * q + 2] = te.z; eg[4 * q + 3] = te.w;
        }
        __syncthreads();
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
            uint32_t t1[4], t2[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = ch * 8 + e * 2;
                const float v0 = xs[j] * bt[j], v1 = xs[j + 1] * bt[j + 1];
                t1[e] = pack_bf16(v0, v1);
                t2[e] = pack_bf16(xs[j] * eg[j], xs[j + 1] * eg[j + 1]);
            }
            const uint32_t off = sw128_offset(i, c0 + ch * 8);
            *reinterpret_cast<uint4*>(sT + off) = make_uint4(t1[0], t1[1], t1[2], t1[3]);
            *reinterpret_cast<uint4*>(sT2 + off) = make_uint4(t2[0], t2[1], t2[2], t2[3]);
        }
    }
    fence_proxy_async_smem();
    __syncthreads();

    // ---- U = T V (lanes +0), W = T' K (lanes +16)
    if (warp < 2) {  // warp 0 issues U, warp 1 issues W
        tc_fence_after_sync();
        constexpr uint32_t idesc = make_idesc_bf16(64, D, false, true);
        const uint64_t dt = make_smem_desc_sw128(smem_u32(warp ? sT2 : sT), 0, 1024);
        const uint64_t db = make_smem_desc_sw128(smem_u32(warp ? sK : sV), 8192, 1024);  // read MN-major
        const uint32_t tacc = warp ? tHi : tLo;
        mma_ss_w<false>(tacc, dt, db, idesc);
#pragma unroll
        for (int ks = 1; ks < 4; ++ks) mma_ss_w<true>(tacc, desc_advance(dt, ks * 32), desc_advance(db, ks * 2048), idesc);
        mma_commit_w(bar_mma2);
    }
    __syncwarp();
    mbar_wait(bar_mma2, it & 1u, abort_flag);
    tc_fence_after_sync();

    // ---- accumulators -> bf16 -> staged tiles (over the K and V tiles) -> coalesced stores
    uint8_t* stU = sK;
    uint8_t* stW = sV;
    {
        const int i = 16 * warp + (lane & 15);
        uint8_t* stg = (lane < 16) ? stU : stW;
#pragma unroll
        for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t r[32];
            tmem_ld32(tmem + (static_cast<uint32_t>(warp * 32) << 16) + c0, r);
            tmem_wait_ld();
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint4 v;
                v.x = pack_bf16(__uint_as_float(r[8 * q + 0]), __uint_as_float(r[8 * q + 1]));
                v.y = pack_bf16(__uint_as_float(r[8 * q + 2]), __uint_as_float(r[8 * q + 3]));
                v.z = pack_bf16(__uint_as_float(r[8 * q + 4]), __uint_as_float(r[8 * q + 5]));
                v.w = pack_bf16(__uint_as_float(r[8 * q + 6]), __uint_as_float(r[8 * q + 7]));
                *reinterpret_cast<uint4*>(stg + tile_off(i, c0 / 8 + q)) = v;
            }
        }
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag != 0) {
        // a wait has given up: nothing is written
    } else if (p.map.cu_seqlens != nullptr && n < kChunk) {
        // a full-box store would spill into the next packed sequence: row-predicated stores
        store_tile_rows<128>(stU, p.u, cp.batch, cp.tok0, head, n, tid);
        store_tile_rows<128>(stW, p.w, cp.batch, cp.tok0, head, n, tid);
    } else if (tid == 0) {
        for (int a = 0; a < NA; ++a) {
            tma_store_4d(&tmUo, stU + a * 8192, a * 64, head, static_cast<int>(cp.tok0), cp.batch);
            tma_store_4d(&tmWo, stW + a * 8192, a * 64, head, static_cast<int>(cp.tok0), cp.batch);
        }
        bulk_commit();
        bulk_wait_read<0>();
    }
    __syncthreads();  // staging tiles and vectors are free for the next unit
    }                 // unit loop
    if (warp == 0) tmem_dealloc(tmem, D);
    if (tid == 0 && *abort_flag && p.status) atomicExch(p.status, 2);
}

}  // namespace gdn
