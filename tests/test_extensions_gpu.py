"""GPU parity of the paths added on top of the reference's surface, against the CPU oracle and the
golden fixtures: gating fused into the recurrent kernel, q/k L2 normalisation inside
chunked_forward, the qk-norm / step-state fixtures, the in-place state on a strided cache, and the
bounded-wait self-test.  Tolerances as in test_recurrent_gpu.py: relative Frobenius <= 1e-2 and
max-abs <= 5e-2 * max|ref| (bf16 outputs against the fp32 oracle on the same bf16-rounded inputs).
"""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from oracle import gdn_oracle as O
from h100_gdn_cuda_b200 import synthetic

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
REL_FRO, MAX_ABS = 1e-2, 5e-2


def close(x, ref, what):
    x = x.float().cpu()
    rf, ma = O.rel_fro(x, ref), O.max_abs_over_max(x, ref)
    assert rf <= REL_FRO and ma <= MAX_ABS, "%s: rel_fro %.3e max_abs/max %.3e" % (what, rf, ma)


@pytest.fixture(scope="module")
def gdn():
    import h100_gdn_cuda_b200 as g
    from h100_gdn_cuda_b200 import build
    build.build()
    return g


def dev(d):
    return {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in d.items()}


def check_status(gdn):
    from h100_gdn_cuda_b200 import _cabi
    st = C.c_int(-1)
    assert _cabi.load().gdn_device_status(0, C.byref(st)) == 0
    return st.value


@pytest.mark.parametrize("B,T,kh,vh,d,dtype", [
    (8, 1, 16, 32, 128, torch.bfloat16),   # decode at the benchmark's head configuration
    (5, 1, 2, 6, 64, torch.float32),
    (3, 20, 2, 4, 128, torch.bfloat16),    # more than 16 tokens: the multi-token instance
])
def test_recurrent_fused_gating(gdn, B, T, kh, vh, d, dtype):
    """beta and the gate computed inside the kernel from A_log, dt_bias, a, b."""
    p = synthetic.decode_inputs(B, T, kh, vh, d, seed=31 + B, dtype=torch.bfloat16)
    A, dt, a, b = (p[k].to(dtype) for k in ("A_log", "dt_bias", "a", "b"))
    pd = dev(p)
    o, s = gdn.recurrent_forward(pd["q"], pd["k"], pd["v"], pd["state"], None, None, is_qk_norm=True,
                                 inference_mode=gdn.Decode, gating=(A.cuda(), dt.cuda(), a.cuda(), b.cuda()))
    beta_ref, g_ref = O.gating_ref(A.float(), dt.float(), a.float(), b.float())  # fp32, nothing rounded
    o_ref, s_ref = O.recurrent_ref(p["q"].float(), p["k"].float(), p["v"].float(), beta_ref, g_ref, p["state"].float(),
                                   is_qk_norm=True)
    close(o, o_ref, "o")
    close(s, s_ref, "state")
    with pytest.raises(RuntimeError):
        gdn.recurrent_forward(pd["q"], pd["k"], pd["v"], pd["state"], pd["b"], None,
                              gating=(A.cuda(), dt.cuda(), a.cuda(), b.cuda()))
    assert check_status(gdn) == 0


def test_spec_verify_fused_gating(gdn):
    """Speculative verify of the benchmark configuration (T=4, per-token states, accepted-token cap) with
    the gating fused."""
    B, T, kh, vh, d = 6, 4, 4, 8, 128
    p = synthetic.decode_inputs(B, T, kh, vh, d, seed=77)
    acc = torch.tensor([1, 4, 2, 3, 4, 1], dtype=torch.int32)
    pd = dev(p)
    gating = (pd["A_log"], pd["dt_bias"], pd["a"], pd["b"])
    o, steps = gdn.recurrent_forward(pd["q"], pd["k"], pd["v"], pd["state"], None, None, None, acc.cuda(),
                                     inference_mode=gdn.SpecVerify, is_qk_norm=True, gating=gating)
    beta_ref, g_ref = O.gating_ref(p["A_log"].float(), p["dt_bias"].float(), p["a"].float(), p["b"].float())
    o_ref, st_ref = O.recurrent_ref(p["q"].float(), p["k"].float(), p["v"].float(), beta_ref, g_ref, p["state"].float(),
                                    is_qk_norm=True, num_accepted_tokens=acc.tolist(), store_step_state=True)
    for bi, n in enumerate(acc.tolist()):
        close(o[bi, :n], o_ref[bi, :n], "o of sequence %d" % bi)
        close(steps[bi, :n], st_ref[bi, :n], "step states of sequence %d" % bi)
    # mode 1 (one state per sequence): the state after the accepted prefix
    o1, s1 = gdn.recurrent_forward(pd["q"], pd["k"], pd["v"], pd["state"], None, None, None, acc.cuda(),
                                   inference_mode=gdn.Decode, is_qk_norm=True, gating=gating)
    for bi, n in enumerate(acc.tolist()):
        close(s1[bi], st_ref[bi, n - 1], "final state of sequence %d" % bi)


@pytest.mark.parametrize("B,T,kh,vh,d,mild", [
    (2, 200, 2, 4, 128, False),
    (1, 1000, 2, 4, 128, True),
    (2, 130, 2, 2, 64, True),       # kh == vh, head dim padded to 128
    (1, 8256, 1, 2, 128, True),     # few long sequences: segmented state propagation
])
def test_chunked_forward_qk_norm(gdn, B, T, kh, vh, d, mild):
    """q/k L2 normalisation inside chunked_forward: raw (un-normalised) q and k in, the oracle normalises."""
    p = synthetic.prefill_inputs(B, T, kh, vh, d, seed=T, mild_gate=mild, normalize=False)
    pd = dev(p)
    o, s = gdn.chunked_forward(pd["q"], pd["k"], pd["v"], pd["beta"], pd["g"], None, pd["state"], is_qk_norm=True)
    o_ref, s_ref = O.recurrent_ref(p["q"].float(), p["k"].float(), p["v"].float(), p["beta"].float(), p["g"],
                                   p["state"].float(), is_qk_norm=True)
    close(o, o_ref, "o")
    close(s, s_ref, "final state")
    assert check_status(gdn) == 0


def test_chunked_forward_qk_norm_varlen(gdn):
    lens = [1, 63, 64, 65, 200, 7]
    p = synthetic.varlen_inputs(lens, 2, 4, 128, seed=9, normalize=False)
    pd = dev(p)
    o, s = gdn.chunked_forward(pd["q"], pd["k"], pd["v"], pd["beta"], pd["g"], None, pd["state"], pd["cu_seqlens"],
                               pd["chunk_indices"], pd["cu_chunks"], p["total_chunks"], is_qk_norm=True)
    o_ref, s_ref = O.recurrent_ref(p["q"].float(), p["k"].float(), p["v"].float(), p["beta"].float(), p["g"],
                                   p["state"].float(), is_qk_norm=True, cu_seqlens=p["cu_seqlens"].tolist())
    close(o, o_ref, "o")
    close(s, s_ref, "final state")


def _load(name):
    z = np.load(os.path.join(GOLDEN, name))
    return {k: torch.from_numpy(z[k]) for k in z.files if k != "fla_version"}


def test_golden_qk_norm_both_paths(gdn):
    """The qk-norm fixture (third-party recurrence on q, k normalised by the generating script; the
    fixture holds the raw q, k) through the recurrent kernel and through chunked_forward."""
    t = _load("branch_qknorm_B2_T40_kh2_vh4_d64.npz")
    bf = lambda x: x.bfloat16().cuda()
    o, s = gdn.recurrent_forward(bf(t["q"]), bf(t["k"]), bf(t["v"]), bf(t["state"]), bf(t["beta"]), t["g"].cuda(),
                                 is_qk_norm=True)
    close(o, t["o"], "recurrent o vs golden")
    close(s, t["final_state"], "recurrent state vs golden")
    o2, s2 = gdn.chunked_forward(bf(t["q"]), bf(t["k"]), bf(t["v"]), bf(t["beta"]), t["g"].cuda(), None, bf(t["state"]),
                                 is_qk_norm=True)
    close(o2, t["o"], "chunked o vs golden")
    close(s2, t["final_state"], "chunked state vs golden")


def test_golden_step_states(gdn):
    t = _load("branch_steps_B3_T6_h2_d64.npz")
    bf = lambda x: x.bfloat16().cuda()
    o, steps = gdn.recurrent_forward(bf(t["q"]), bf(t["k"]), bf(t["v"]), bf(t["state"]), bf(t["beta"]), t["g"].cuda(),
                                     inference_mode=gdn.SpecVerify)
    close(o, t["o"], "o vs golden")
    close(steps, t["step_states"], "step states vs golden")


def test_inplace_state_on_strided_cache(gdn):
    """A state cache whose sequences are every other slot: the (dv, dk) blocks are contiguous, the
    sequence stride is not the packed one; in-place decode must update the caller's tensor."""
    B, kh, vh, d = 4, 2, 4, 128
    p = synthetic.decode_inputs(B, 1, kh, vh, d, seed=3)
    beta, g = O.gating_ref(p["A_log"], p["dt_bias"], p["a"], p["b"])
    cache = torch.zeros(2 * B, vh, d, d, dtype=torch.bfloat16, device="cuda")
    view = cache[::2]
    view.copy_(p["state"].cuda())
    pd = dev(p)
    o, s = gdn.recurrent_forward(pd["q"], pd["k"], pd["v"], view, beta.bfloat16().cuda(), g.cuda(), inference_mode=gdn.Decode,
                                 inplace_state=True)
    o_ref, s_ref = O.recurrent_ref(p["q"].float(), p["k"].float(), p["v"].float(), beta.bfloat16().float(), g, p["state"].float())
    assert s.data_ptr() == view.data_ptr()
    close(cache[::2], s_ref, "cache slots in use")
    assert float(cache[1::2].abs().max()) == 0.0
    close(o, o_ref, "o")
    # blocks that are not contiguous cannot be updated in place: refuse instead of working on a copy
    bad = torch.zeros(B, vh, d, 2 * d, dtype=torch.bfloat16, device="cuda")[..., :d]
    with pytest.raises(RuntimeError):
        gdn.recurrent_forward(pd["q"], pd["k"], pd["v"], bad, beta.bfloat16().cuda(), g.cuda(), inplace_state=True)


def test_bounded_wait_gives_up_and_context_survives(gdn):
    """A wait that nothing will ever satisfy runs into its (here: short) cycle limit, the kernel reports
    status 7 and returns; the next kernels run normally and report nothing."""
    from h100_gdn_cuda_b200 import _cabi
    lib = _cabi.load()
    assert check_status(gdn) == 0
    assert lib.gdn_selftest_bounded_wait(200000, None) == 0
    assert check_status(gdn) == 7
    assert check_status(gdn) == 0          # reading clears the word
    assert lib.gdn_selftest_bounded_wait(0, None) == -1   # limit out of range: refused on the host
    p = synthetic.decode_inputs(2, 1, 2, 4, 128, seed=1)
    beta, g = O.gating_ref(p["A_log"], p["dt_bias"], p["a"], p["b"])
    pd = dev(p)
    o, s = gdn.recurrent_forward(pd["q"], pd["k"], pd["v"], pd["state"], beta.bfloat16().cuda(), g.cuda())
    o_ref, _ = O.recurrent_ref(p["q"].float(), p["k"].float(), p["v"].float(), beta.bfloat16().float(), g, p["state"].float())
    close(o, o_ref, "o after the self-test")
    assert check_status(gdn) == 0


@pytest.mark.parametrize("T", [1, 3])
def test_indexed_state_pool(gdn, T):
    """A pool of states addressed through state_indices (what a serving engine keeps): the sequences of the
    batch read and update their own slots, a negative slot skips the sequence, the other slots stay as they were."""
    B, kh, vh, d, P = 6, 2, 4, 128, 10
    p = synthetic.decode_inputs(B, T, kh, vh, d, seed=21 + T)
    beta, g = O.gating_ref(p["A_log"], p["dt_bias"], p["a"], p["b"])
    gen = torch.Generator().manual_seed(5)
    pool0 = (torch.randn(P, vh, d, d, generator=gen) * 0.02).bfloat16()
    idx = torch.tensor([7, 2, -1, 9, 0, 4], dtype=torch.int32)
    pool = pool0.clone().cuda()
    pd = dev(p)
    o, ret = gdn.recurrent_forward(pd["q"], pd["k"], pd["v"], pool, beta.bfloat16().cuda(), g.cuda(), inference_mode=gdn.Decode,
                                   is_qk_norm=True, state_indices=idx.cuda())
    assert ret.data_ptr() == pool.data_ptr()
    live = [i for i in range(B) if idx[i] >= 0]
    s0 = pool0[idx[live].long()].float()
    o_ref, s_ref = O.recurrent_ref(p["q"][live].float(), p["k"][live].float(), p["v"][live].float(), beta.bfloat16()[live].float(),
                                   g[live], s0, is_qk_norm=True)
    close(o[live], o_ref, "o of the live sequences")
    close(pool[idx[live].long()], s_ref, "updated slots")
    untouched = [s for s in range(P) if s not in idx.tolist()]
    assert torch.equal(pool[untouched].cpu(), pool0[untouched])
    assert check_status(gdn) == 0


@pytest.mark.parametrize("B,T,kh,vh,d", [(6, 1, 2, 4, 128), (3, 4, 2, 4, 64), (2, 40, 1, 2, 128)])
def test_fp32_state(gdn, B, T, kh, vh, d):
    """A state kept in fp32: read, updated and returned as fp32 (decode, a few tokens, and a run long enough for
    the multi-token instance).  The state is compared with a tighter gate than bf16 states allow."""
    p = synthetic.decode_inputs(B, T, kh, vh, d, seed=51 + T)
    beta, g = O.gating_ref(p["A_log"], p["dt_bias"], p["a"], p["b"])
    s0 = p["state"].float() + 1e-4 * torch.randn(p["state"].shape, generator=torch.Generator().manual_seed(1))  # not bf16-exact
    pd = dev(p)
    o, s = gdn.recurrent_forward(pd["q"], pd["k"], pd["v"], s0.cuda(), beta.bfloat16().cuda(), g.cuda(), inference_mode=gdn.Decode,
                                 is_qk_norm=True)
    assert s.dtype == torch.float32
    o_ref, s_ref = O.recurrent_ref(p["q"].float(), p["k"].float(), p["v"].float(), beta.bfloat16().float(), g, s0, is_qk_norm=True)
    close(o, o_ref, "o")
    assert O.rel_fro(s.cpu(), s_ref) < 1e-5, O.rel_fro(s.cpu(), s_ref)
    # two decode steps on an fp32 state equal one two-token call bit for bit in the state's precision class
    if T == 1:
        o2, s2 = gdn.recurrent_forward(pd["q"], pd["k"], pd["v"], s, beta.bfloat16().cuda(), g.cuda(), inference_mode=gdn.Decode, is_qk_norm=True)
        _, s2_ref = O.recurrent_ref(p["q"].float(), p["k"].float(), p["v"].float(), beta.bfloat16().float(), g, s_ref, is_qk_norm=True)
        assert O.rel_fro(s2.cpu(), s2_ref) < 1e-5
    assert check_status(gdn) == 0


@pytest.mark.parametrize("B,T,C_,W,bias,state", [(2, 70, 64, 4, True, True), (1, 5, 24, 3, False, False), (3, 1, 128, 4, True, True),
                                                (2, 33, 8, 2, True, True)])
def test_causal_conv1d_padded(gdn, B, T, C_, W, bias, state):
    """Causal depthwise convolution + SiLU against the fp32 definition; bf16 in and out (gate: relative
    Frobenius <= 1e-2, as for the other bf16 outputs); the final state is a copy of inputs and must be exact."""
    gen = torch.Generator().manual_seed(B * 100 + T)
    x = torch.randn(B, T, C_, generator=gen).bfloat16()
    w = (torch.randn(C_, W, generator=gen) * 0.5).bfloat16()
    b = torch.randn(C_, generator=gen).bfloat16() if bias else None
    s0 = torch.randn(B, W - 1, C_, generator=gen).bfloat16() if state else None
    y, fin = gdn.api.causal_conv1d(x.cuda(), w.cuda(), None if b is None else b.cuda(), None if s0 is None else s0.cuda(),
                                   return_final_state=True)
    y_ref, fin_ref = O.causal_conv1d_ref(x, w, b, s0)
    close(y, y_ref, "y")
    assert torch.equal(fin.float().cpu(), fin_ref)
    if T <= 32 and state:   # decode-sized call: the state may be updated in place
        s_io = s0.clone().cuda()
        y2, fin2 = gdn.api.causal_conv1d(x.cuda(), w.cuda(), None if b is None else b.cuda(), s_io, final_state=s_io)
        assert torch.equal(y2, y) and torch.equal(s_io.float().cpu(), fin_ref)
    # continuation: the two halves with the state handed over equal the whole
    if T >= 8:
        h = T // 2
        ya, sa = gdn.api.causal_conv1d(x[:, :h].cuda(), w.cuda(), None if b is None else b.cuda(), None if s0 is None else s0.cuda(),
                                       return_final_state=True)
        yb, sb = gdn.api.causal_conv1d(x[:, h:].cuda(), w.cuda(), None if b is None else b.cuda(), sa, return_final_state=True)
        assert torch.equal(torch.cat([ya, yb], dim=1), y) and torch.equal(sb, fin)


def test_causal_conv1d_packed(gdn):
    lens = [1, 40, 0, 3, 64, 2]
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    C_, W = 40, 4
    gen = torch.Generator().manual_seed(3)
    x = torch.randn(sum(lens), C_, generator=gen).bfloat16()
    w = (torch.randn(C_, W, generator=gen) * 0.5).bfloat16()
    b = torch.randn(C_, generator=gen).bfloat16()
    s0 = torch.randn(len(lens), W - 1, C_, generator=gen).bfloat16()
    y, fin = gdn.api.causal_conv1d(x.cuda(), w.cuda(), b.cuda(), s0.cuda(), cu_seqlens=cu.cuda(), return_final_state=True)
    y_ref, fin_ref = O.causal_conv1d_ref(x, w, b, s0, cu_seqlens=cu.tolist())
    close(y, y_ref, "y")
    assert torch.equal(fin.float().cpu(), fin_ref)   # the empty sequence keeps its state
    with pytest.raises(RuntimeError):                # a sequence spanning several blocks cannot be updated in place
        s_io = s0.clone().cuda()
        gdn.api.causal_conv1d(x.cuda(), w.cuda(), b.cuda(), s_io, cu_seqlens=cu.cuda(), final_state=s_io)


@pytest.mark.parametrize("shape", [(2, 50, 4, 128), (3, 7, 64), (5, 1024), (4, 3, 2, 200)])
def test_gated_rmsnorm(gdn, shape):
    gen = torch.Generator().manual_seed(len(shape))
    x = torch.randn(*shape, generator=gen).bfloat16()
    z = torch.randn(*shape, generator=gen).bfloat16()
    w = (1 + 0.1 * torch.randn(shape[-1], generator=gen)).bfloat16()
    y = gdn.api.gated_rmsnorm(x.cuda(), z.cuda(), w.cuda(), 1e-6)
    close(y, O.gated_rmsnorm_ref(x, z, w, 1e-6), "y")


def test_cuda_graph_replay_of_decode_and_prefill(gdn):
    """Launch-bound loops are meant to be captured: a decode step (gating inside, state updated in place) and a
    prefill call are recorded into CUDA graphs after one eager warm-up call each and replayed; the replays must
    give the bits of the eager calls (nothing is allocated, synchronised or compiled inside the entry points)."""
    d = dev(synthetic.decode_inputs(8, 1, 2, 4, 128, seed=31))
    gating = (d["A_log"], d["dt_bias"], d["a"], d["b"])
    steps = 3
    qs = [torch.nn.functional.normalize(torch.randn_like(d["q"].float()), dim=-1).bfloat16() for _ in range(steps)]
    # eager reference: three in-place steps
    s_eager = d["state"].clone()
    o_eager = []
    for q in qs:
        o, _ = gdn.recurrent_forward(q, d["k"], d["v"], s_eager, None, None, inference_mode=1, is_qk_norm=True,
                                     gating=gating, inplace_state=True)
        o_eager.append(o.clone())
    # captured: static input and state buffers, one graph, replayed per step
    q_buf, s_graph = qs[0].clone(), d["state"].clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):   # warm-up on the capture stream, on a scratch state
        gdn.recurrent_forward(q_buf, d["k"], d["v"], d["state"].clone(), None, None, inference_mode=1, is_qk_norm=True,
                              gating=gating, inplace_state=True)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        o_buf, _ = gdn.recurrent_forward(q_buf, d["k"], d["v"], s_graph, None, None, inference_mode=1, is_qk_norm=True,
                                         gating=gating, inplace_state=True)
    for i, q in enumerate(qs):
        q_buf.copy_(q)
        graph.replay()
        assert torch.equal(o_buf, o_eager[i]), "decode step %d" % i
    assert torch.equal(s_graph, s_eager)
    # prefill (two kernels, the second launched with programmatic stream serialization)
    p = dev(synthetic.prefill_inputs(2, 300, 2, 4, 128, seed=32, mild_gate=True))
    o_ref, s_ref = gdn.chunked_forward(p["q"], p["k"], p["v"], p["beta"], p["g"], None, p["state"])
    graph2 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph2):
        o_g, s_g = gdn.chunked_forward(p["q"], p["k"], p["v"], p["beta"], p["g"], None, p["state"])
    o_g.zero_()
    graph2.replay()
    graph2.replay()
    assert torch.equal(o_g, o_ref) and torch.equal(s_g, s_ref)
    check_status(gdn)
