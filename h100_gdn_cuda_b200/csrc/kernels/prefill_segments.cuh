// Start states of the segments of a segmented prefill run (see FusedParams in prefill_fused.cuh):
//     S_start[0] = initial state,   S_start[p + 1] = S_start[p] M_p + N_p
// with M_p, N_p the composite transition of segment p (fp32, dv x dk and dk x dk with dv = dk = 128)
// produced by the mode-1 launch of gdn_fused_seq_kernel.  Segment p of a sequence sits in launch
// slot first_slot + p (locate_segment in prefill_common.cuh); in packed mode the sequences have
// different numbers of segments.  The work is tiny (one 128 x 128 x 128
// product per chain and segment) and strictly sequential in p; it stays in fp32 on CUDA cores.
// One CTA of 128 threads per (chain, block of 8 state rows); thread = column of the state.
// M_p (64 KB) comes into shared memory by one bulk copy, the copy of M_{p+1} running while M_p is
// being used (element-wise global loads of M made this kernel latency-bound: 235 us instead of
// about 40 at 8 chains x 16 segments).
#pragma once
#include <cuda_bf16.h>

#include "prefill_common.cuh"
#include "sm100_ptx.cuh"

namespace gdn {

struct SegCombineParams {
    const float* seg_mn;   // [slot][head][2][128][128]: N then M
    float* seg_start;      // [slot][head][128][128]
    ChunkMap map;
    int seg_chunks;
    const __nv_bfloat16* state_in;  // or NULL; d x d per (sequence, head), zero outside when d < 128
    long long si_ss, si_sh;
    int d;
    int vh, num_segments;
    int* status;
};

struct SegCombineSmem {
    static constexpr int D = 128, R = 8;
    static constexpr int kOffM = 0;                      // two buffers of D x D fp32
    static constexpr int kOffS = 2 * D * D * 4;          // R x D fp32
    static constexpr int kOffBar = kOffS + R * D * 4;    // 2 mbarriers, abort flag
    static constexpr int kBytes = kOffBar + 32 + 128;
};

__global__ void __launch_bounds__(128) gdn_seg_combine_kernel(const SegCombineParams p) {
    using namespace ptx;
    using L = SegCombineSmem;
    constexpr int D = L::D, R = L::R;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((128u - (ptx::smem_u32(smem_raw) & 127u)) & 127u);
    float* sM = reinterpret_cast<float*>(smem + L::kOffM);
    float(*sS)[D] = reinterpret_cast<float(*)[D]>(smem + L::kOffS);
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem + L::kOffBar);
    int* abort_flag = reinterpret_cast<int*>(bar + 2);

    ptx::grid_dep_wait();  // launched as a programmatic dependent of the composite-transition launch
    const long long chain = blockIdx.x;
    const int r0 = blockIdx.y * R, col = threadIdx.x;
    const int seq = static_cast<int>(chain / p.vh), head = static_cast<int>(chain % p.vh);
    const SegPos sp = sequence_segments(p.map, seq, p.seg_chunks, p.num_segments);
    const int nseg = sp.nseg;
    auto idx = [&](int s) { return static_cast<long long>(sp.first_slot + s) * p.vh + head; };
    auto m_of = [&](int s) { return p.seg_mn + (idx(s) * 2 + 1) * (D * D); };
    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(&bar[0], 1);
        mbar_init(&bar[1], 1);
        mbar_fence_init();
        if (nseg > 1) {
            mbar_arrive_expect_tx(&bar[0], D * D * 4);
            bulk_load(sM, m_of(0), D * D * 4, &bar[0]);
        }
    }
    float acc[R], nxt[R];  // nxt: the N rows of the coming segment, fetched one iteration ahead
#pragma unroll
    for (int r = 0; r < R; ++r)
        acc[r] = (p.state_in && r0 + r < p.d && col < p.d)
                     ? __bfloat162float(p.state_in[seq * p.si_ss + head * p.si_sh + static_cast<long long>(r0 + r) * p.d + col])
                     : 0.f;
    auto load_n = [&](int s) {
        const float* N = p.seg_mn + idx(s) * 2 * (D * D);
#pragma unroll
        for (int r = 0; r < R; ++r) nxt[r] = (s + 1 < nseg) ? N[(r0 + r) * D + col] : 0.f;
    };
    load_n(0);
    __syncthreads();
    for (int s = 0; s < nseg; ++s) {
        float* dst = p.seg_start + idx(s) * (D * D);
#pragma unroll
        for (int r = 0; r < R; ++r) dst[(r0 + r) * D + col] = acc[r];
        if (s + 1 == nseg) break;
        const int b = s & 1;
        // the other buffer was last read in iteration s - 1, which every thread has left (barrier below)
        if (threadIdx.x == 0 && s + 2 < nseg) {
            mbar_arrive_expect_tx(&bar[b ^ 1], D * D * 4);
            bulk_load(sM + (b ^ 1) * D * D, m_of(s + 1), D * D * 4, &bar[b ^ 1]);
        }
#pragma unroll
        for (int r = 0; r < R; ++r) sS[r][col] = acc[r];
#pragma unroll
        for (int r = 0; r < R; ++r) acc[r] = nxt[r];
        load_n(s + 1);
        __syncthreads();  // sS complete
        mbar_wait(&bar[b], static_cast<uint32_t>((s >> 1) & 1), abort_flag);
        const float* M = sM + b * D * D;
#pragma unroll 2
        for (int k = 0; k < D; k += 4) {
            const float m0 = M[k * D + col], m1 = M[(k + 1) * D + col], m2 = M[(k + 2) * D + col], m3 = M[(k + 3) * D + col];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const float4 s4 = *reinterpret_cast<const float4*>(&sS[r][k]);  // one address for all lanes: a broadcast
                acc[r] = fmaf(s4.w, m3, fmaf(s4.z, m2, fmaf(s4.y, m1, fmaf(s4.x, m0, acc[r]))));
            }
        }
        __syncthreads();  // sS and this M buffer are free again
    }
    if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, 6);
}

}  // namespace gdn
