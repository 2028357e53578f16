// Pieces shared by the chunked-prefill kernels: chunk lookup, gate/beta loading with the
// chunk-local cumulative sum, and the coalesced row-predicated store of a staged tile.
#pragma once
#include "sm100_ptx.cuh"

namespace gdn {

constexpr int kChunk = 64;

// Scratch of the whole-layer path since the WY/UT transform was folded into the recurrence (see
// prefill_zp.cuh): per (global chunk, v-head) unit Z (64 x 128 bf16 as two 64 x 64 swizzled atoms, the
// shared-memory image of an MN-major B operand) and then PT (64 x 64, one atom).
constexpr int kZPBlockBytes = kChunk * 128 * 2 + kChunk * kChunk * 2;

// per-token scalar tensor (beta or gate) as the kernels see it
struct ScalarView {
    const void* ptr;
    int is_f32;
    long long sb, st, sh;
    __device__ __forceinline__ float load(long long b, long long t, int h) const {
        const long long o = b * sb + t * st + static_cast<long long>(h) * sh;
        return is_f32 ? __ldg(reinterpret_cast<const float*>(ptr) + o)
                      : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(ptr)[o]);
    }
};

struct TokenView {
    __nv_bfloat16* ptr;
    long long sb, st, sh;
};

// Where the chunks of the problem are.
struct ChunkMap {
    const int* cu_seqlens;     // packed mode or NULL
    const int* chunk_indices;  // packed mode: [seq, chunk] pairs
    const int* cu_chunks;      // packed mode: first global chunk of each sequence
    int seq_len;               // padded mode
    int chunks_per_seq;        // padded mode
};

struct ChunkPos {
    int seq;          // sequence index
    int batch;        // batch coordinate for addressing (0 in packed mode)
    long long tok0;   // first token of the chunk (index along the token axis of `batch`)
    int n;            // valid tokens in the chunk (1..64)
};

// chunk `c` (in chunk_indices order / batch-major order) -> position
__device__ __forceinline__ ChunkPos locate_chunk(const ChunkMap& m, int c) {
    ChunkPos r;
    if (m.cu_seqlens) {
        r.seq = m.chunk_indices[2 * c];
        const int ci = m.chunk_indices[2 * c + 1];
        const int bos = m.cu_seqlens[r.seq], eos = m.cu_seqlens[r.seq + 1];
        r.batch = 0;
        r.tok0 = static_cast<long long>(bos) + static_cast<long long>(ci) * kChunk;
        const long long rem = eos - r.tok0;
        r.n = rem < kChunk ? static_cast<int>(rem) : kChunk;
    } else {
        r.seq = c / m.chunks_per_seq;
        const int ci = c % m.chunks_per_seq;
        r.batch = r.seq;
        r.tok0 = static_cast<long long>(ci) * kChunk;
        const int rem = m.seq_len - ci * kChunk;
        r.n = rem < kChunk ? rem : kChunk;
    }
    return r;
}

// Segmented runs of the state kernel (few long sequences): which (sequence, segment) a launch slot is.
// Padded mode: every sequence has `num_segments` segments, slot = seq * num_segments + segment.
// Packed mode: segments of `seg_chunks` chunks, sequence s has max(1, ceil(chunks_s / seg_chunks)) of
// them (an empty sequence keeps one, so that its final state is still written); slots follow the
// sequences in order and the launch covers an upper bound of them (seq = -1 for the surplus).
struct SegPos {
    int seq, segment, nseg, first_slot;  // nseg, first_slot: segments of the sequence and the slot of its first one
};
__device__ __forceinline__ int packed_seq_segments(const int* cu_seqlens, int s, int seg_chunks) {
    const int chunks = (cu_seqlens[s + 1] - cu_seqlens[s] + kChunk - 1) / kChunk;
    const int n = (chunks + seg_chunks - 1) / seg_chunks;
    return n > 0 ? n : 1;
}
__device__ __forceinline__ SegPos locate_segment(const ChunkMap& m, int slot, int seg_chunks, int num_segments, int num_seqs) {
    if (!m.cu_seqlens) return SegPos{slot / num_segments, slot % num_segments, num_segments, slot - slot % num_segments};
    int first = 0;
    for (int s = 0; s < num_seqs; ++s) {
        const int n = packed_seq_segments(m.cu_seqlens, s, seg_chunks);
        if (slot < first + n) return SegPos{s, slot - first, n, first};
        first += n;
    }
    return SegPos{-1, 0, 0, 0};
}
// the segments of sequence `seq` (the `segment` field is not meaningful)
__device__ __forceinline__ SegPos sequence_segments(const ChunkMap& m, int seq, int seg_chunks, int num_segments) {
    if (!m.cu_seqlens) return SegPos{seq, 0, num_segments, seq * num_segments};
    int first = 0;
    for (int s = 0; s < seq; ++s) first += packed_seq_segments(m.cu_seqlens, s, seg_chunks);
    return SegPos{seq, 0, packed_seq_segments(m.cu_seqlens, seq, seg_chunks), first};
}

// Offset of 16-byte chunk `chunk` of row `row` in a staging tile of D bf16 per row whose
// chunks are XOR-swizzled by the row so that 16 rows written at once hit distinct banks.
template <int D>
__device__ __forceinline__ uint32_t stage_off(int row, int chunk) {
    constexpr int CPR = D / 8;
    return static_cast<uint32_t>(row) * (D * 2) + static_cast<uint32_t>((chunk ^ (row & (CPR - 1))) * 16);
}

// Copy rows [0, n) of a staged 64 x D bf16 tile to global memory, 16 bytes per thread,
// consecutive threads on consecutive 16-byte pieces of a row.
template <int D, int THREADS>
__device__ __forceinline__ void store_staged_tile(const uint8_t* stage, const TokenView& dst, int batch,
                                                  long long tok0, int head, int n, int tid) {
    constexpr int CPR = D / 8;
    __nv_bfloat16* base = dst.ptr + batch * dst.sb + tok0 * dst.st + static_cast<long long>(head) * dst.sh;
    for (int idx = tid; idx < kChunk * CPR; idx += THREADS) {
        const int row = idx / CPR, chunk = idx % CPR;
        if (row < n) {
            const uint4 v = *reinterpret_cast<const uint4*>(stage + stage_off<D>(row, chunk));
            *reinterpret_cast<uint4*>(base + row * dst.st + chunk * 8) = v;
        }
    }
}

// Byte offset of 16-byte piece `c16` (0..15) of row `row` in a 64 x 128 bf16 tile kept as two
// 64 x 64 atoms in the layout TMA uses with the 128-byte swizzle (what a tiled TMA store or
// load with box 64 x 64 expects in shared memory).
__device__ __forceinline__ uint32_t tile_off(int row, int c16) {
    return static_cast<uint32_t>((c16 >> 3) * 8192 + row * 128 + (((c16 & 7) ^ (row & 7)) << 4));
}

// Row-predicated copy of rows [0, n) of such a tile to global memory (used where a TMA store
// would write past the end of a packed sequence).
// `pieces`: 16-byte pieces of a row that exist in the destination (head dim / 8).
template <int THREADS>
__device__ __forceinline__ void store_tile_rows(const uint8_t* tile, const TokenView& dst, int batch, long long tok0,
                                                int head, int n, int tid, int pieces = 16) {
    __nv_bfloat16* base = dst.ptr + batch * dst.sb + tok0 * dst.st + static_cast<long long>(head) * dst.sh;
    for (int idx = tid; idx < kChunk * 16; idx += THREADS) {
        const int row = idx >> 4, c16 = idx & 15;
        if (row < n && c16 < pieces) {
            const uint4 v = *reinterpret_cast<const uint4*>(tile + tile_off(row, c16));
            *reinterpret_cast<uint4*>(base + row * dst.st + c16 * 8) = v;
        }
    }
}

}  // namespace gdn
