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

// Segmented state propagation for few long sequences.  The state kernel is a serial chain
// per (sequence, v-head); with fewer chains than SMs most of the GPU idles.  The chain obeys
// S' = S M_c + N_c per chunk, so a sequence is cut into segments: one launch finds every
// segment's composite (M, N) (two CTAs per chain and segment), a small kernel chains them into the
// segments' start states, and a second launch of the state kernel produces the output of all
// segments at once.  Three passes instead of one, many segments wide.
// The plan must not depend on the device (the scratch size is computed without one), so it is
// made for the 148 SMs of a B200.
struct SegmentPlan {
    int num_segments;  // padded mode: segments per sequence; 1: not segmented
    int seg_chunks;    // chunks per segment
    int slots;         // (sequence, segment) pairs the launches cover: batch x num_segments in padded mode,
                       // an upper bound in packed mode (the lengths are only known on the device)
};
namespace plan_detail {
constexpr long long kSms = 148;
// Cost model fitted to measurements (B=1..2, T=4096..131072, 4..32 v-heads), in units of "one
// chunk of the state kernel": a CTA costs its chunks plus about 3 for start-up and pipeline
// fill; a launch costs that times its CTA waves.  Plans whose second launch needs more than
// one wave, or whose first needs more than two, measured worse than the model and are not made.
constexpr int kFixed = 3, kMinSegment = 32;
inline long long waves(long long ctas) { return (ctas + kSms - 1) / kSms; }
}  // namespace plan_detail

inline SegmentPlan prefill_segments(long long chains, int chunks_per_seq, bool packed) {
    using namespace plan_detail;
    SegmentPlan plan{1, chunks_per_seq, 0};
    if (packed || chains <= 0) return plan;
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

// Packed mode: the host sees the number of sequences and the total number of chunks, not the
// lengths.  Segments have one length L for all sequences; sequence s gets max(1, ceil(chunks_s / L))
// of them, at most total / L + num_seqs altogether: that many slots are launched and the surplus
// CTAs leave at once.  The unsegmented run is costed as if all sequences were equally long (its
// best case), so unequal lengths only make the segmented plan better than assumed.
constexpr int kMaxSegmentedSeqs = 64;
inline SegmentPlan prefill_segments_packed(int num_seqs, int num_v_heads, long long total_chunks) {
    using namespace plan_detail;
    SegmentPlan plan{1, static_cast<int>(std::min<long long>(total_chunks, 1 << 30)), 0};
    if (num_seqs <= 0 || num_seqs > kMaxSegmentedSeqs || num_v_heads <= 0 || total_chunks <= 0 || total_chunks > (1 << 30)) return plan;
    const long long chains = static_cast<long long>(num_seqs) * num_v_heads;
    const long long even = (total_chunks + num_seqs - 1) / num_seqs;
    double best = 0.8 * static_cast<double>(waves(chains) * (even + kFixed));
    for (int P = 2; P <= 128 && total_chunks / P >= kMinSegment; ++P) {
        const int len = static_cast<int>((total_chunks + P - 1) / P);
        const long long slots = total_chunks / len + num_seqs;  // launched (and given scratch): the upper bound
        // CTAs of surplus slots leave at once and free their SM, so the waves are counted for the slots that
        // hold work when the sequences are about equally long: every sequence end but the last may add one
        // short segment
        const long long work = (total_chunks + len - 1) / len + num_seqs - 1;
        const long long w1 = waves(2 * work * num_v_heads), w3 = waves(work * num_v_heads);
        if (w3 > 1 || w1 > 2) break;
        const double cost = static_cast<double>((w1 + w3) * (len + kFixed));
        if (cost < best) {
            best = cost;
            plan.num_segments = P;
            plan.seg_chunks = len;
            plan.slots = static_cast<int>(slots);
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
