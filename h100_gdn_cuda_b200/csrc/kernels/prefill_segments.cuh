// Start states of the segments of a segmented prefill run (see FusedParams in prefill_fused.cuh):
//     S_start[0] = initial state,   S_start[p + 1] = S_start[p] M_p + N_p
// with M_p, N_p the composite transition of segment p (fp32, dv x dk and dk x dk with dv = dk = 128)
// produced by the mode-1 launch of gdn_fused_seq_kernel.  The work is tiny (one 128 x 128 x 128
// product per chain and segment) and strictly sequential in p; it stays in fp32 on CUDA cores.
// One CTA of 128 threads per (chain, block of 16 state rows); thread = column of the state.
#pragma once
#include <cuda_bf16.h>

namespace gdn {

struct SegCombineParams {
    const float* seg_mn;   // [chain][segment][2][128][128]: N then M
    float* seg_start;      // [chain][segment][128][128]
    const __nv_bfloat16* state_in;  // or NULL
    long long si_ss, si_sh;
    int vh, num_segments;
};

__global__ void __launch_bounds__(128) gdn_seg_combine_kernel(const SegCombineParams p) {
    constexpr int D = 128, R = 16;
    __shared__ float sS[R][D];
    const long long chain = blockIdx.x;
    const int r0 = blockIdx.y * R, col = threadIdx.x;
    const int seq = static_cast<int>(chain / p.vh), head = static_cast<int>(chain % p.vh);
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r)
        acc[r] = p.state_in ? __bfloat162float(p.state_in[seq * p.si_ss + head * p.si_sh + static_cast<long long>(r0 + r) * D + col]) : 0.f;
    for (int s = 0; s < p.num_segments; ++s) {
        float* dst = p.seg_start + (chain * p.num_segments + s) * (D * D);
#pragma unroll
        for (int r = 0; r < R; ++r) dst[(r0 + r) * D + col] = acc[r];
        if (s + 1 == p.num_segments) break;
        __syncthreads();  // previous iteration's readers of sS are done
#pragma unroll
        for (int r = 0; r < R; ++r) sS[r][col] = acc[r];
        __syncthreads();
        const float* N = p.seg_mn + (chain * p.num_segments + s) * 2 * (D * D);
        const float* M = N + D * D;
#pragma unroll
        for (int r = 0; r < R; ++r) acc[r] = N[(r0 + r) * D + col];
#pragma unroll 4
        for (int k = 0; k < D; ++k) {
            const float m = M[k * D + col];
#pragma unroll
            for (int r = 0; r < R; ++r) acc[r] = fmaf(sS[r][k], m, acc[r]);
        }
    }
}

}  // namespace gdn
