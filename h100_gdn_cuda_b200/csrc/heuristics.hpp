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

// Grid of the persistent WY/UT kernel: every CTA slot of the GPU, or one CTA per unit if fewer.
inline int uw_grid(long long units, int sms) {
    return static_cast<int>(std::min<long long>(units, static_cast<long long>(sms) * prefill_config().uw_ctas_per_sm));
}

}  // namespace gdn
