// Stand-alone output stage of chunked Gated DeltaNet prefill, one CTA of 128 threads per
// (64-token chunk, v-head):
//     O = scale * ( e^{g} .* (Q h^T) + tril(Q K^T .* e^{g_i - g_j}) U_new )
// with h the (dv x dk) state entering the chunk.  Stands in for the reference's
// sm90_bf16_gdn_chunked_compute_O (kernels/sm90_bf16_gdn_chunked_compute_O.cuh:23-530) behind the
// low-level bf16_gdn_chunked_compute_O wrapper; gdn_chunked_forward does not use it (there the
// output is fused into the state kernel and h is never written).
//
// tcgen05: Q K^T as two interleaved M=64 N=32 accumulators (see prefill_uw.cuh), then, transposed
// so that dv is the M dimension,  O1^T = h Q^T (A = the h tile, K-major) and O2^T = U_new^T P^T
// (A = the U_new tile read MN-major, B = P written by the CTA as a bf16 swizzled tile).
#pragma once
#include <cuda.h>

#include "prefill_common.cuh"

namespace gdn {

struct OParams {
    ChunkMap map;
    ScalarView gate;  // chunk-local cumulative gate; ptr == NULL: no decay
    TokenView out;
    int kh, vh;
    float scale;
    int* status;
};

struct OSmem {
    static constexpr int kTile = kChunk * 128 * 2;  // 16 KB
    static constexpr int kOffQ = 0;                 // later the output staging tile
    static constexpr int kOffK = kTile;
    static constexpr int kOffU = 2 * kTile;
    static constexpr int kOffH = 3 * kTile;  // 128 x 128 bf16, two atoms of 128 rows
    static constexpr int kOffP = 3 * kTile + 32768;
    static constexpr int kOffVec = kOffP + 8192;  // g[64], scale * e^g[64]
    static constexpr int kOffBar = kOffVec + 2 * 64 * 4;
    static constexpr int kBytes = kOffBar + 64 + 1024;
};

__global__ void __launch_bounds__(128, 2) gdn_o_kernel(const __grid_constant__ CUtensorMap tmQ,
                                                       const __grid_constant__ CUtensorMap tmK,
                                                       const __grid_constant__ CUtensorMap tmU,
                                                       const __grid_constant__ CUtensorMap tmH,
                                                       const __grid_constant__ CUtensorMap tmO, const OParams p) {
    using namespace ptx;
    using L = OSmem;
    extern __shared__ uint8_t smem_raw[];
    // aligned by an offset from the array itself, so that the compiler still knows the pointer is shared memory
    uint8_t* smem = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* sQ = smem + L::kOffQ;
    uint8_t* sK = smem + L::kOffK;
    uint8_t* sU = smem + L::kOffU;
    uint8_t* sH = smem + L::kOffH;
    uint8_t* sP = smem + L::kOffP;
    float* sG = reinterpret_cast<float*>(smem + L::kOffVec);
    float* sEs = sG + 64;
    uint64_t* bar_load = reinterpret_cast<uint64_t*>(smem + L::kOffBar);
    uint64_t* bar_mma = bar_load + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_load + 2);
    int* abort_flag = reinterpret_cast<int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int head = blockIdx.y;
    const int khead = head / (p.vh / p.kh);
    const ChunkPos cp = locate_chunk(p.map, blockIdx.x);
    const int n = cp.n;
    float g_mine = 0.f;
    if (tid < n && p.gate.ptr) g_mine = p.gate.load(cp.batch, cp.tok0 + tid, head);

    if (tid == 0) {
        *abort_flag = 0;
        mbar_init(bar_load, 1);
        mbar_init(bar_mma, 1);
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(tmem_slot, 256);
    if (tid < 64) sG[tid] = g_mine;
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    if (tid == 0) {
        mbar_arrive_expect_tx(bar_load, 3 * L::kTile + 32768);
        const int tok = static_cast<int>(cp.tok0);
        for (int a = 0; a < 2; ++a) {
            tma_load_4d(sQ + a * 8192, &tmQ, bar_load, a * 64, khead, tok, cp.batch);
            tma_load_4d(sK + a * 8192, &tmK, bar_load, a * 64, khead, tok, cp.batch);
            tma_load_4d(sU + a * 8192, &tmU, bar_load, a * 64, head, tok, cp.batch);
            tma_load_2d(sH + a * 16384, &tmH, bar_load, a * 64, (blockIdx.x * p.vh + head) * 128);
        }
    }
    if (tid < 64) {
        // rows past the end of the sequence carry the last valid gate value
        const float g = p.gate.ptr ? sG[tid < n ? tid : n - 1] : 0.f;
        sEs[tid] = g;  // parked: sG is still being read by other threads
    }
    __syncthreads();
    if (tid < 64) {
        const float g = sEs[tid];
        sG[tid] = g;
        sEs[tid] = p.scale * __expf(g);
    }
    __syncthreads();

    mbar_wait(bar_load, 0, abort_flag);
    const uint32_t tLo = tmem, tHi = tmem + (16u << 16);
    if (warp == 0) {
        tc_fence_after_sync();
        constexpr uint32_t id_qk = make_idesc_bf16(64, 32, false, false);
        constexpr uint32_t id_hq = make_idesc_bf16(128, 64, false, false);
        const uint64_t dq = make_smem_desc_sw128(smem_u32(sQ), 0, 1024);
        const uint64_t dk0 = make_smem_desc_sw128(smem_u32(sK), 0, 1024);
        const uint64_t dk1 = desc_advance(dk0, 32 * 128);
        const uint64_t dh = make_smem_desc_sw128(smem_u32(sH), 0, 1024);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            const uint32_t off = kmajor_step(ks, 8192);
            if (ks == 0) {
                mma_ss_w<false>(tLo, dq, dk0, id_qk);
                mma_ss_w<false>(tHi, dq, dk1, id_qk);
            } else {
                mma_ss_w<true>(tLo, desc_advance(dq, off), desc_advance(dk0, off), id_qk);
                mma_ss_w<true>(tHi, desc_advance(dq, off), desc_advance(dk1, off), id_qk);
            }
        }
        mma_commit_w(bar_mma);
        // O1^T = h Q^T  (tensor-memory columns 64..127), does not need P
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            if (ks == 0)
                mma_ss_w<false>(tmem + 64, dh, dq, id_hq);
            else
                mma_ss_w<true>(tmem + 64, desc_advance(dh, kmajor_step(ks, 16384)), desc_advance(dq, kmajor_step(ks, 8192)), id_hq);
        }
    }
    __syncwarp();
    mbar_wait(bar_mma, 0, abort_flag);
    tc_fence_after_sync();
    {
        // P rows: row 16*warp + (lane & 15); lanes 0-15 hold columns 0-31, lanes 16-31 columns 32-63
        const int i = 16 * warp + (lane & 15);
        const int cbase = (lane >> 4) * 32;
        const float gi = sG[i];
        uint32_t r[32];
        tmem_ld32(tmem + (static_cast<uint32_t>(warp * 32) << 16), r);
        float gc[32];
#pragma unroll
        for (int e4 = 0; e4 < 8; ++e4) {
            const float4 t = *reinterpret_cast<const float4*>(sG + cbase + 4 * e4);
            gc[4 * e4] = t.x; gc[4 * e4 + 1] = t.y; gc[4 * e4 + 2] = t.z; gc[4 * e4 + 3] = t.w;
        }
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float v[2];
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    const int col = cbase + j + 2 * e + q;
                    v[q] = (col <= i && i < n) ? p.scale * __uint_as_float(r[j + 2 * e + q]) * __expf(gi - gc[j + 2 * e + q]) : 0.f;
                }
                w[e] = pack_bf16(v[0], v[1]);
            }
            *reinterpret_cast<uint4*>(sP + tile_off(i, (cbase + j) >> 3)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after_sync();
        // O2^T = U_new^T P^T  (tensor-memory columns 128..191)
        constexpr uint32_t id_up = make_idesc_bf16(128, 64, true, false);
        const uint64_t du = make_smem_desc_sw128(smem_u32(sU), 8192, 1024);
        const uint64_t dp = make_smem_desc_sw128(smem_u32(sP), 0, 1024);
        mma_ss_w<false>(tmem + 128, du, dp, id_up);
#pragma unroll
        for (int ks = 1; ks < 4; ++ks) mma_ss_w<true>(tmem + 128, desc_advance(du, ks * 2048), desc_advance(dp, ks * 32), id_up);
        mma_commit_w(bar_mma);
    }
    __syncwarp();
    mbar_wait(bar_mma, 1, abort_flag);
    tc_fence_after_sync();
    {
        // thread = dv row; O^T columns are tokens; staged into the (dead) Q tile in TMA layout
        const int row = tid;
        const uint32_t tm_lane = static_cast<uint32_t>(warp * 32) << 16;
        uint32_t off8[8];
#pragma unroll
        for (int k = 0; k < 8; ++k)
            off8[k] = static_cast<uint32_t>((row >> 6) * 8192 + ((((row & 63) >> 3) ^ k) << 4) + (row & 7) * 2);
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            uint32_t r1[16], r2[16];
            tmem_ld16(tmem + 64 + tm_lane + 16 * b, r1);
            tmem_ld16(tmem + 128 + tm_lane + 16 * b, r2);
            float gv[16];
#pragma unroll
            for (int e4 = 0; e4 < 4; ++e4) {
                const float4 t = *reinterpret_cast<const float4*>(sEs + 16 * b + 4 * e4);
                gv[4 * e4] = t.x; gv[4 * e4 + 1] = t.y; gv[4 * e4 + 2] = t.z; gv[4 * e4 + 3] = t.w;
            }
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 16; ++e) {
                const int i = 16 * b + e;
                const float o = fmaf(gv[e], __uint_as_float(r1[e]), __uint_as_float(r2[e]));
                *reinterpret_cast<__nv_bfloat16*>(sQ + i * 128 + off8[i & 7]) = __float2bfloat16(o);
            }
        }
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    if (p.map.cu_seqlens != nullptr && n < kChunk) {
        store_tile_rows<128>(sQ, p.out, cp.batch, cp.tok0, head, n, tid);
    } else if (tid == 0) {
        tma_store_4d(&tmO, sQ, 0, head, static_cast<int>(cp.tok0), cp.batch);
        tma_store_4d(&tmO, sQ + 8192, 64, head, static_cast<int>(cp.tok0), cp.batch);
        bulk_commit();
        bulk_wait_read<0>();
    }
    if (warp == 0) tmem_dealloc(tmem, 256);
    if (tid == 0 && *abort_flag && p.status) atomicExch(p.status, 5);
}

}  // namespace gdn
