// Launch-shape choices for B200 (148 SMs, 227 KB shared memory and 512 tensor-memory columns per
// SM, 64 K registers).  Stands in for the reference's get_*_config functions
// (csrc/jit_kernels/heuristics/common.hpp:8-398, sm90_arch.hpp:8-15), which pick tiles, stages
// and grids for H100.  Tile shapes are fixed by the kernels here (64-token chunks, 32-row state
// tiles); what remains to choose is how many CTAs share an SM and how large a persistent grid is.
#pragma once
#include <algorithm>

namespace gdn {

struct RecurrentConfig {
    int stages;        // ring stages of 32 x DK state tiles
    int ctas_per_sm;   // limited by registers (128 threads x <=128 registers at DK <= 128)
    int smem_bytes;
    long long grid;    // persistent CTAs
};

inline RecurrentConfig recurrent_config(int dk, long long num_tiles, int sms) {
    RecurrentConfig c;
    c.stages = 4;
    c.ctas_per_sm = dk <= 128 ? 4 : 2;
    const int stage = (32 * dk * 2 + 4 * dk + 64 + 127) / 128 * 128;
    c.smem_bytes = c.stages * stage + 128;
    c.grid = std::min<long long>(num_tiles, static_cast<long long>(sms) * c.ctas_per_sm);
    return c;
}

struct PrefillConfig {
    int uw_ctas_per_sm;     // WY/UT kernel: 4 (52 KB shared memory, 128 tensor-memory columns, 128 registers)
    int fused_threads;      // state/output kernel: 16 warps, one CTA per SM (all 512 tensor-memory columns)
};

inline PrefillConfig prefill_config() { return PrefillConfig{4, 512}; }

// Segmented state propagation for few long padded sequences.  The state kernel is a serial chain
// per (sequence, v-head); with fewer chains than SMs most of the GPU idles.  The chain obeys
// S' = S M_c + N_c per chunk, so the sequence is cut into P segments: one launch finds every
// segment's composite (M, N) (two CTAs per chain and segment), a small kernel chains them into the
// segments' start states, and a second launch of the state kernel produces the output of all
// segments at once.  Three passes instead of one, P segments wide: worth it from P = 3 on.
// The plan must not depend on the device (the scratch size is computed without one), so it is
// made for the 148 SMs of a B200.
struct SegmentPlan {
    int num_segments;  // 1: not segmented
    int seg_chunks;    // chunks per segment
};
inline SegmentPlan prefill_segments(long long chains, int chunks_per_seq, bool packed) {
    SegmentPlan plan{1, chunks_per_seq};
    if (packed || chains <= 0) return plan;
    constexpr long long kSms = 148;
    // cost model in units of "one chunk of the state kernel": a CTA wave of the first pass costs
    // 0.8 per chunk (no output), of the second 1.0; waves = CTAs / SMs rounded up
    auto waves = [&](long long ctas) { return static_cast<double>((ctas + kSms - 1) / kSms); };
    const double n = chunks_per_seq;
    double best = waves(chains) * n * 0.75;  // segment only for a gain of a quarter or more
    for (int P = 2; P <= 16 && chunks_per_seq / P >= 32; ++P) {
        const double len = static_cast<double>((chunks_per_seq + P - 1) / P);
        const double cost = waves(2 * chains * P) * len * 0.8 + waves(chains * P) * len;
        if (cost < best) {
            best = cost;
            plan.num_segments = P;
            plan.seg_chunks = (chunks_per_seq + P - 1) / P;
        }
    }
    return plan;
}

// Grid of the persistent WY/UT kernel: every CTA slot of the GPU, or one CTA per unit if fewer.
inline int uw_grid(long long units, int sms) {
    return static_cast<int>(std::min<long long>(units, static_cast<long long>(sms) * prefill_config().uw_ctas_per_sm));
}

}  // namespace gdn
