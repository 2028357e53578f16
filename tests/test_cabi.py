"""CPU checks of the C-ABI library: it loads without a GPU and exports every declared symbol."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from h100_gdn_cuda_b200 import build, _cabi
    build.build()
    return _cabi.load()


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "gdn_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gdn_[a-z_0-9]+)\s*\(", text)))


def test_header_symbols_exported(lib):
    names = _declared_symbols()
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), "symbol %s declared in include/gdn_b200.h is not exported" % n


def test_binding_table_covers_header():
    from h100_gdn_cuda_b200 import _cabi
    assert set(_declared_symbols()) == set(_cabi.SYMBOLS)


def test_version_and_error_text(lib):
    assert lib.gdn_version() >= 100
    assert lib.gdn_init(b"/tmp", b"/usr/local/cuda") == 0
    # argument validation happens before any CUDA call, so it is testable without a GPU
    rc = lib.gdn_recurrent_forward(None, None)
    assert rc == -1 and b"NULL" in lib.gdn_last_error()
    rc = lib.gdn_transpose_mn_major(None, None, 2, 1, 1, 1, 1, None)
    assert rc == -1


def test_struct_sizes_match_c(lib):
    # sizes computed by the C compiler for the structs in the header
    import subprocess, tempfile, textwrap
    from h100_gdn_cuda_b200 import _cabi
    src = textwrap.dedent('''
        #include <stdio.h>
        #include "gdn_b200.h"
        int main(void) {
            printf("%zu %zu %zu %zu %zu %zu %zu %zu %zu %zu\\n", sizeof(GdnTokenTensor), sizeof(GdnTokenScalar),
                   sizeof(GdnState), sizeof(GdnShape), sizeof(GdnRecurrentArgs), sizeof(GdnComputeUWArgs),
                   sizeof(GdnSeqStateArgs), sizeof(GdnComputeOArgs), sizeof(GdnChunkedArgs), sizeof(GdnConvArgs));
            return 0;
        }''')
    with tempfile.TemporaryDirectory() as d:
        c = os.path.join(d, "s.c")
        open(c, "w").write(src)
        exe = os.path.join(d, "s")
        subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), c, "-o", exe])
        sizes = [int(x) for x in subprocess.check_output([exe]).split()]
    py = [ctypes.sizeof(t) for t in (_cabi.TokenTensor, _cabi.TokenScalar, _cabi.State, _cabi.Shape,
                                     _cabi.RecurrentArgs, _cabi.ComputeUWArgs, _cabi.SeqStateArgs,
                                     _cabi.ComputeOArgs, _cabi.ChunkedArgs, _cabi.ConvArgs)]
    assert sizes == py


def test_workspace_bytes(lib):
    """Scratch of chunked_forward: 24 KB per (64-token chunk, v-head); for few long sequences
    three fp32 states per v-head and segment slot on top (the segmented state propagation)."""
    from h100_gdn_cuda_b200 import api
    unit = 64 * 128 * 2 + 64 * 64 * 2
    norm = 512  # q/k norm factors per (chunk, k-head); the size queries below are made with one k-head
    assert api.chunked_forward_workspace_bytes(4, 4096, 32, num_k_heads=1) == 4 * 64 * (32 * unit + norm) + 256
    assert api.chunked_forward_workspace_bytes(1, 65, 2, num_k_heads=1) == 2 * (2 * unit + norm) + 256   # ragged tail: whole chunks
    # packed mode counts chunks, not tokens; 256 bytes more hold the sequences ordered by length
    assert api.chunked_forward_workspace_bytes(3, 0, 4, total_tokens=200, total_chunks=6, packed=True, num_k_heads=1) == 6 * (4 * unit + norm) + 256 + 256
    assert api.chunked_forward_workspace_bytes(1, 0, 4, total_tokens=200, total_chunks=4, packed=True, num_k_heads=1) == 4 * (4 * unit + norm) + 256
    # B=2, T=131072, 4 v-heads: 8 chains -> 18 segments
    long_ctx = api.chunked_forward_workspace_bytes(2, 131072, 4, num_k_heads=1)
    assert long_ctx == 2 * 2048 * (4 * unit + norm) + 256 + 8 * 18 * 3 * 128 * 128 * 4 + 256
    # the same two sequences packed: segments of 114 chunks, at most 4096 // 114 + 2 = 37 slots
    packed_long = api.chunked_forward_workspace_bytes(2, 0, 4, total_tokens=2 * 131072, total_chunks=4096, packed=True, num_k_heads=1)
    assert packed_long == 4096 * (4 * unit + norm) + 256 + 37 * 4 * 3 * 128 * 128 * 4 + 256
    # 128 chains: never segmented
    assert api.chunked_forward_workspace_bytes(4, 131072, 32, num_k_heads=1) == 4 * 2048 * (32 * unit + norm) + 256


def test_segment_plan_heuristic():
    """Host-side choice of the number of segments for the state propagation (heuristics.hpp)."""
    import subprocess, tempfile, textwrap
    src = textwrap.dedent('''
        #include <cstdio>
        #include "heuristics.hpp"
        int main() {
            const long long chains[] = {8, 16, 32, 64, 128, 2, 8, 8};
            const int chunks[] = {2048, 2048, 2048, 2048, 64, 97, 2048, 40};
            const bool packed[] = {false, false, false, false, false, false, true, false};
            for (int i = 0; i < 8; ++i) {
                const gdn::SegmentPlan p = gdn::prefill_segments(chains[i], chunks[i], packed[i]);
                std::printf("%d %d\\n", p.num_segments, p.seg_chunks);
            }
            // packed mode: sequences, v-heads, total chunks
            const int seqs[] = {2, 1, 16, 65, 2, 4}, vh[] = {4, 32, 32, 2, 1, 2};
            const long long total[] = {4096, 2048, 520, 6000, 259, 267};
            for (int i = 0; i < 6; ++i) {
                const gdn::SegmentPlan p = gdn::prefill_segments_packed(seqs[i], vh[i], total[i]);
                std::printf("%d %d %d\\n", p.num_segments, p.seg_chunks, p.slots);
            }
            return 0;
        }''')
    with tempfile.TemporaryDirectory() as d:
        c = os.path.join(d, "h.cpp")
        open(c, "w").write(src)
        exe = os.path.join(d, "h")
        subprocess.check_call(["g++", "-std=c++17", "-I", os.path.join(ROOT, "h100_gdn_cuda_b200", "csrc"), c, "-o", exe])
        rows = [tuple(int(x) for x in l.split()) for l in subprocess.check_output([exe]).decode().splitlines()]
    assert rows[0] == (18, 114)          # 8 chains: two CTA waves of short segments beat one of long ones
    assert rows[1][0] == 9               # 16 chains: 9 segments fill 144 SMs in the second pass
    assert rows[2][0] >= 2               # 32 chains: still worth it
    assert rows[3] == (1, 2048)          # 64 chains: three passes cost more than they save
    assert rows[4] == (1, 64)            # the benchmark shape is never segmented
    assert rows[5][0] == 3 and rows[5][0] * rows[5][1] >= 97
    assert rows[6][:2] == (1, 2048)      # the padded plan is not made for packed inputs
    assert rows[7] == (1, 40)            # too short for 32-chunk segments
    assert rows[8] == (36, 114, 37)      # two long packed sequences of 4 heads: like the padded plan, one CTA wave
    assert rows[8][2] * 4 <= 148
    assert rows[9] == (4, 512, 5)        # 32 heads of one sequence: as the padded plan; the slack slot holds no work
    assert rows[10][0] == 1              # the packed benchmark batch (512 chains) is never segmented
    assert rows[11][0] == 1              # more sequences than the lookup scans
    assert rows[12] == (8, 33, 9)        # total // 33 + 2 slots cover any split of 259 chunks over 2 sequences
    assert rows[13][0] == 1              # four equal sequences would already run side by side


def test_state_alignment_is_checked_on_the_host(lib):
    """States are accessed 16 bytes at a time: a misaligned pointer or a stride that is not a multiple of
    8 elements is refused with GDN_ERR_INVALID before anything touches a device."""
    from h100_gdn_cuda_b200 import _cabi as cabi, api
    tok = cabi.TokenTensor(0x10000, 64 * 4 * 128, 4 * 128, 128)
    sc = cabi.TokenScalar(0x20000, cabi.GDN_BF16, 64 * 4, 4, 1)
    for state in (cabi.State(0x30002, 4 * 128 * 128, 128 * 128), cabi.State(0x30000, 4 * 128 * 128 + 4, 128 * 128)):
        a = cabi.ChunkedArgs()
        a.shape = api._shape(1, 64, 64, 4, 4, 128, 128)
        a.q = a.k = a.v = a.out = tok
        a.beta = sc
        a.initial_state = state
        assert lib.gdn_chunked_forward(ctypes.byref(a), None) == -1
        assert b"initial_state" in lib.gdn_last_error()
        s = cabi.SeqStateArgs()
        s.shape = a.shape
        s.k = s.u = s.w = tok
        s.final_state = state
        s.chunk_states = 0x40000
        assert lib.gdn_seq_state_update(ctypes.byref(s), None) == -1
        assert b"final_state" in lib.gdn_last_error()
