// WY / UT transform of chunked Gated DeltaNet prefill: per (64-token chunk, v-head)
//     A = tril(diag(beta) K K^T .* exp(g_i - g_j), -1),  X = (I + A)^-1
//     U = X diag(beta) V,   W = X diag(beta exp(g)) K
// with g the chunk-local cumulative gate.  Stands in for the reference's
// sm90_bf16_compute_u_w (gdn_cuda/include/gdn_cuda/kernels/sm90_bf16_gdn_compute_u_w.cuh:153-667),
// using the canonical W (gate folded in before the solve).
//
// One CTA of 128 threads per unit; tcgen05 tensor cores do the three contractions:
//   K K^T      : M=64 N=64 K=D, both operands the same K-major shared-memory tile (TMA, 128B swizzle)
//   U = T V    : M=64 N=D  K=64, A = T (bf16, written by the CTA), B = the V tile read MN-major
//   W = T' K   : M=64 N=D  K=64, A = T' = X diag(beta e^g), B = the K tile read MN-major
// so neither K nor V is ever rescaled or copied.  The unit-lower-triangular inverse is done
// in fp32 on CUDA cores: 16x16 diagonal blocks by forward substitution (one column per
// thread), then three levels of 16x16 block products.
// Accumulators live in tensor memory (2*D columns); the raw K K^T block shares columns with U.
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
    int* status;
};

template <int D>
struct UWSmem {
    static constexpr int kTile = kChunk * D * 2;          // K or V tile
    static constexpr int kOffK = 0;
    static constexpr int kOffV = kOffK + kTile;
    static constexpr int kOffT = kOffV + kTile;           // T  (64x64 bf16, K-major SW128)
    static constexpr int kOffT2 = kOffT + 8192;           // T' (same layout)
    static constexpr int kOffA = kOffT2 + 8192;           // A, fp32 [64][65]; later U staging
    static constexpr int kOffX = kOffA + 64 * 65 * 4 + 64; // X, fp32 [64][65]; later W staging
    static constexpr int kOffTmp = kOffX + 64 * 65 * 4 + 64;
    static constexpr int kOffVec = kOffTmp + 3 * 256 * 4;  // beta[64], g[64], e^g[64]
    static constexpr int kBytes = kOffVec + 3 * 64 * 4 + 1024;  // + alignment slack
    static_assert(64 * 65 * 4 + 64 >= kTile || D > 128, "staging must fit");
};

template <int D>
__global__ void __launch_bounds__(128) gdn_uw_kernel(const __grid_constant__ CUtensorMap tmK,
                                                     const __grid_constant__ CUtensorMap tmV,
                                                     const UWParams p) {
    using namespace ptx;
    using L = UWSmem<D>;
    constexpr int NA = D / 64;  // 64-column swizzle atoms per tile
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sK = smem + L::kOffK;
    uint8_t* sV = smem + L::kOffV;
    uint8_t* sT = smem + L::kOffT;
    uint8_t* sT2 = smem + L::kOffT2;
    float(*sA)[65] = reinterpret_cast<float(*)[65]>(smem + L::kOffA);
    float(*sX)[65] = reinterpret_cast<float(*)[65]>(smem + L::kOffX);
    float* sTmp = reinterpret_cast<float*>(smem + L::kOffTmp);
    float* sBeta = reinterpret_cast<float*>(smem + L::kOffVec);
    float* sG = sBeta + 64;
    float* sEg = sG + 64;
    __shared__ uint64_t bar_load, bar_mma;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int head = blockIdx.y;
    const int khead = head / (p.vh / p.kh);
    const ChunkPos cp = locate_chunk(p.map, blockIdx.x);
    const int n = cp.n;

    if (tid == 0) {
        abort_flag = 0;
        mbar_init(&bar_load, 1);
        mbar_init(&bar_mma, 1);
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(&tmem_slot, 2 * D);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = tmem_slot;
    const uint32_t tU = tmem, tW = tmem + D;

    if (tid == 0) {
        mbar_arrive_expect_tx(&bar_load, 2 * L::kTile);
        for (int a = 0; a < NA; ++a) {
            tma_load_4d(sK + a * 8192, &tmK, &bar_load, a * 64, khead, static_cast<int>(cp.tok0), cp.batch);
            tma_load_4d(sV + a * 8192, &tmV, &bar_load, a * 64, head, static_cast<int>(cp.tok0), cp.batch);
        }
    }
    // beta and gate of the chunk's tokens (rows past the end: beta = 0, g = g of the last row)
    if (tid < 64) {
        float b = 0.f, g = 0.f;
        if (tid < n) {
            b = p.beta.load(cp.batch, cp.tok0 + tid, head);
            if (p.gate.ptr) g = p.gate.load(cp.batch, cp.tok0 + tid, head);
        }
        sBeta[tid] = b;
        sEg[tid] = g;  // raw values; replaced by exp(g) below
    }
    __syncthreads();
    if (tid < 64) {
        float g = 0.f;
        if (p.gate.ptr) {
            const int last = tid < n ? tid : n - 1;
            if (p.gate_is_raw) {
                for (int m = 0; m <= last; ++m) g += sEg[m];
            } else {
                g = sEg[last];
            }
        }
        sG[tid] = g;
    }
    __syncthreads();
    if (tid < 64) sEg[tid] = __expf(sG[tid]);
    __syncthreads();

    // ---- A_raw = K K^T
    mbar_wait(&bar_load, 0, &abort_flag);
    if (tid == 0) {
        tc_fence_after_sync();
        constexpr uint32_t idesc = make_idesc_bf16(64, 64, false, false);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            const uint64_t d = make_smem_desc_sw128(smem_u32(sK) + (ks / 4) * 8192 + (ks % 4) * 32, 0, 1024);
            mma_ss(tU, d, d, idesc, ks > 0);
        }
        mma_commit(&bar_mma);
    }
    __syncwarp();
    mbar_wait(&bar_mma, 0, &abort_flag);
    tc_fence_after_sync();
    {
        // M=64 accumulator: row 16*warp + l sits in lane 32*warp + l for l < 16
        const int i = 16 * warp + (lane & 15);
        const float bi = sBeta[i], gi = sG[i];
#pragma unroll
        for (int c0 = 0; c0 < 64; c0 += 16) {
            uint32_t r[16];
            tmem_ld16(tU + (static_cast<uint32_t>(warp * 32) << 16) + c0, r);
            tmem_wait_ld();
            if (lane < 16) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int col = c0 + j;
                    float a = 0.f;
                    if (col < i && i < n) a = bi * __uint_as_float(r[j]) * __expf(gi - sG[col]);
                    sA[i][col] = a;
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();

    // ---- X = (I + A)^-1 : diagonal 16x16 blocks, one column per thread
    if (tid < 64) {
        const int b = tid >> 4, j = tid & 15;
        float x[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) x[i] = (i == j) ? 1.f : 0.f;
#pragma unroll
        for (int i = 1; i < 16; ++i) {
            float acc = 0.f;
#pragma unroll
            for (int m = 0; m < i; ++m) acc = fmaf(sA[16 * b + i][16 * b + m], x[m], acc);
            if (i > j) x[i] = -acc;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) sX[16 * b + i][16 * b + j] = x[i];
    }
    __syncthreads();
    // off-diagonal blocks, level by level: X_ij = -X_ii * sum_{m=j}^{i-1} A_im X_mj
#pragma unroll 1
    for (int lvl = 1; lvl <= 3; ++lvl) {
        const int nblk = 4 - lvl;
        for (int idx = tid; idx < nblk * 256; idx += 128) {
            const int bi = idx >> 8, rr = (idx >> 4) & 15, cc = idx & 15;
            const int i = bi + lvl, j = bi;
            const float* arow = &sA[16 * i + rr][0];
            float acc = 0.f;
            for (int kk = 16 * j; kk < 16 * i; ++kk) acc = fmaf(arow[kk], sX[kk][16 * j + cc], acc);
            sTmp[idx] = acc;
        }
        __syncthreads();
        for (int idx = tid; idx < nblk * 256; idx += 128) {
            const int bi = idx >> 8, rr = (idx >> 4) & 15, cc = idx & 15;
            const int i = bi + lvl, j = bi;
            float acc = 0.f;
            for (int m = 0; m <= rr; ++m) acc = fmaf(sX[16 * i + rr][16 * i + m], sTmp[(bi << 8) + (m << 4) + cc], acc);
            sX[16 * i + rr][16 * j + cc] = -acc;
        }
        __syncthreads();
    }

    // ---- T = X diag(beta), T' = X diag(beta e^g) as bf16 K-major swizzled tiles
    {
        const int i = tid >> 1, c0 = (tid & 1) * 32;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
            uint32_t t1[4], t2[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float v0[2], v1[2];
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    const int j = c0 + ch * 8 + e * 2 + q;
                    const float x = ((j >> 4) <= (i >> 4)) ? sX[i][j] : 0.f;  // blocks above the diagonal are zero
                    v0[q] = x * sBeta[j];
                    v1[q] = v0[q] * sEg[j];
                }
                t1[e] = pack_bf16(v0[0], v0[1]);
                t2[e] = pack_bf16(v1[0], v1[1]);
            }
            const uint32_t off = sw128_offset(i, c0 + ch * 8);
            *reinterpret_cast<uint4*>(sT + off) = make_uint4(t1[0], t1[1], t1[2], t1[3]);
            *reinterpret_cast<uint4*>(sT2 + off) = make_uint4(t2[0], t2[1], t2[2], t2[3]);
        }
    }
    fence_proxy_async_smem();
    __syncthreads();

    // ---- U = T V, W = T' K
    if (tid == 0) {
        tc_fence_after_sync();
        constexpr uint32_t idesc = make_idesc_bf16(64, D, false, true);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            const uint64_t a1 = make_smem_desc_sw128(smem_u32(sT) + ks * 32, 0, 1024);
            const uint64_t b1 = make_smem_desc_sw128(smem_u32(sV) + ks * 2048, 8192, 1024);
            mma_ss(tU, a1, b1, idesc, ks > 0);
        }
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            const uint64_t a2 = make_smem_desc_sw128(smem_u32(sT2) + ks * 32, 0, 1024);
            const uint64_t b2 = make_smem_desc_sw128(smem_u32(sK) + ks * 2048, 8192, 1024);
            mma_ss(tW, a2, b2, idesc, ks > 0);
        }
        mma_commit(&bar_mma);
    }
    __syncwarp();
    mbar_wait(&bar_mma, 1, &abort_flag);
    tc_fence_after_sync();

    // ---- accumulators -> bf16 -> staged tiles -> coalesced stores
    uint8_t* stU = smem + L::kOffA;
    uint8_t* stW = smem + L::kOffX;
    {
        const int i = 16 * warp + (lane & 15);
#pragma unroll
        for (int which = 0; which < 2; ++which) {
            const uint32_t tacc = which ? tW : tU;
            uint8_t* stg = which ? stW : stU;
#pragma unroll
            for (int c0 = 0; c0 < D; c0 += 16) {
                uint32_t r[16];
                tmem_ld16(tacc + (static_cast<uint32_t>(warp * 32) << 16) + c0, r);
                tmem_wait_ld();
                if (lane < 16) {
                    uint4 lo, hi;
                    lo.x = pack_bf16(__uint_as_float(r[0]), __uint_as_float(r[1]));
                    lo.y = pack_bf16(__uint_as_float(r[2]), __uint_as_float(r[3]));
                    lo.z = pack_bf16(__uint_as_float(r[4]), __uint_as_float(r[5]));
                    lo.w = pack_bf16(__uint_as_float(r[6]), __uint_as_float(r[7]));
                    hi.x = pack_bf16(__uint_as_float(r[8]), __uint_as_float(r[9]));
                    hi.y = pack_bf16(__uint_as_float(r[10]), __uint_as_float(r[11]));
                    hi.z = pack_bf16(__uint_as_float(r[12]), __uint_as_float(r[13]));
                    hi.w = pack_bf16(__uint_as_float(r[14]), __uint_as_float(r[15]));
                    *reinterpret_cast<uint4*>(stg + stage_off<D>(i, c0 / 8)) = lo;
                    *reinterpret_cast<uint4*>(stg + stage_off<D>(i, c0 / 8 + 1)) = hi;
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    store_staged_tile<D, 128>(stU, p.u, cp.batch, cp.tok0, head, n, tid);
    store_staged_tile<D, 128>(stW, p.w, cp.batch, cp.tok0, head, n, tid);
    if (warp == 0) tmem_dealloc(tmem, 2 * D);
    if (tid == 0 && abort_flag && p.status) atomicExch(p.status, 2);
}

}  // namespace gdn
