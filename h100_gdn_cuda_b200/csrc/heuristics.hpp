// Launch-shape choices for B200 (148 SMs, 227 KB shared memory and 512 tensor-memory columns per
// SM, 64 K registers).  Stands in for the reference's get_*_config functions
// (csrc/jit_kernels/heuristics/common.hpp:8-398, sm90_arch.hpp:8-15), which pick tiles, stages
// and grids for H100.  Tile shapes are fixed by the kernels here (64-token chunks, 32-row state
// tiles); what remains to choose is how many CTAs share an SM and how large a persistent grid is.
#pragma once
#include <algorithm>
#include <cstdlib>

namespace gdn {

struct RecurrentConfig {
    int stages;        // ring stages of 32 x DK state tiles
    int ctas_per_sm;   // limited by registers (128 threads x <=128 registers at DK <= 128)
    int smem_bytes;
    long long grid;    // persistent CTAs
};

// `ring`: the multi-token instance (two tile stages, the token ring, every tile a work unit);
// otherwise the decode instance (four tile stages).
inline RecurrentConfig recurrent_config(int dk, long long num_tiles, int sms, bool ring = false) {
    RecurrentConfig c;
    c.stages = ring ? 2 : 4;
    c.ctas_per_sm = ring ? (dk <= 64 ? 4 : (dk <= 256 ? 3 : 1)) : (dk <= 128 ? 4 : 2);
    const int tok_slot = 8 * (4 * dk + 64);  // k, q, v slice of 8 tokens (two ring slots; one more in every stage)
    const int stage = (32 * dk * 2 + (ring ? tok_slot : 4 * dk + 64) + 127) / 128 * 128;
    c.smem_bytes = c.stages * stage + 128 + (ring ? 2 * tok_slot : 0);
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
// S' = S M_c + N_c per chunk, so the sequence is cut into P (at most 32) segments: one launch finds every
// segment's composite (M, N) (two CTAs per chain and segment), a small kernel chains them into the
// segments' start states, and a second launch of the state kernel produces the output of all
// segments at once.  Three passes instead of one, P segments wide.
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
    // Cost model fitted to measurements (B=1..2, T=4096..131072, 4..32 v-heads), in units of "one
    // chunk of the state kernel": a CTA costs its chunks plus about 3 for start-up and pipeline
    // fill; a launch costs that times its CTA waves.  Plans whose second launch needs more than
    // one wave, or whose first needs more than two, measured worse than the model and are not made.
    auto waves = [&](long long ctas) { return (ctas + kSms - 1) / kSms; };
    constexpr int kFixed = 3, kMinSegment = 32;
    double best = 0.8 * static_cast<double>(waves(chains) * (chunks_per_seq + kFixed));
    for (int P = 2; P <= 32 && chunks_per_seq / P >= kMinSegment; ++P) {
        const long long w1 = waves(2 * chains * P), w3 = waves(chains * P);
        if (w3 > 1 || w1 > 2) break;
        const int len = (chunks_per_seq + P - 1) / P;
        const double cost = static_cast<double>((w1 + w3) * (len + kFixed));
        if (cost < best) {
            best = cost;
            plan.num_segments = P;
            plan.seg_chunks = len;
        }
    }
    return plan;
}

// Grid of the persistent WY/UT kernel: every CTA slot of the GPU, or one CTA per unit if fewer.
inline int uw_grid(long long units, int sms) {
    return static_cast<int>(std::min<long long>(units, static_cast<long long>(sms) * prefill_config().uw_ctas_per_sm));
}

// Grid of the persistent chunk-parallel kernel of the whole-layer path (units = chunks x k-heads,
// two CTAs of 256 threads per SM).
inline int zp_grid(long long units, int sms) {
    return static_cast<int>(std::min<long long>(units, static_cast<long long>(sms) * 2));
}

}  // namespace gdn
