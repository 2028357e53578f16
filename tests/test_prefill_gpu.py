"""GPU parity of the chunked-prefill path (tcgen05 kernels) against the CPU oracle.

Tolerances (bf16 tensors out, fp32 oracle on the same bf16-rounded inputs): relative
Frobenius error <= 1e-2 and max-abs error <= 5e-2 * max|ref| for O, final state, U, W,
U_new and per-chunk states.  The end-to-end checks compare with the *token recurrence*
(the layer semantics), not with a chunked re-statement.
"""
import pytest
import torch

from oracle import gdn_oracle as O
from h100_gdn_cuda_b200 import synthetic

pytestmark = pytest.mark.gpu

REL_FRO, MAX_ABS = 1e-2, 5e-2


def close(x, ref, what, rel=REL_FRO, mx=MAX_ABS):
    x = x.float().cpu()
    assert torch.isfinite(x).all(), "%s has non-finite values" % what
    rf, ma = O.rel_fro(x, ref), O.max_abs_over_max(x, ref)
    assert rf <= rel and ma <= mx, "%s: rel_fro %.3e max_abs/max %.3e" % (what, rf, ma)
    return rf, ma


@pytest.fixture(scope="module")
def gdn():
    import h100_gdn_cuda_b200 as g
    from h100_gdn_cuda_b200 import build
    build.build()
    return g


def dev(d):
    return {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in d.items()}


def f32(p, *names):
    return [None if p[n] is None else p[n].float() for n in names]


def check_status(gdn):
    import ctypes
    from h100_gdn_cuda_b200 import _cabi
    st = ctypes.c_int(0)
    assert _cabi.load().gdn_device_status(torch.cuda.current_device(), ctypes.byref(st)) == 0
    assert st.value == 0, "a kernel reported a bounded wait that ran out (status %d)" % st.value


# ---------------------------------------------------------------- per-stage
@pytest.mark.parametrize("B,T,kh,vh,mild", [(1, 64, 1, 1, False), (2, 130, 2, 4, True), (1, 255, 1, 2, False)])
def test_compute_u_w_padded(gdn, B, T, kh, vh, mild):
    p = synthetic.prefill_inputs(B, T, kh, vh, 128, seed=T, with_state=False, mild_gate=mild)
    gc = O.chunk_local_cumsum_ref(p["g"])
    u_ref, w_ref = O.compute_u_w_ref(*f32(p, "k", "v", "beta"), gc)
    pd = dev(p)
    u = torch.full_like(pd["v"], float("nan"))
    w = torch.full_like(pd["v"], float("nan"))
    # MN-major beta / gate as the reference's wrappers require
    beta_mn = gdn.transpose_to_mn_major(pd["beta"])
    gate_mn = gdn.transpose_to_mn_major(gc.cuda())
    gdn.bf16_gdn_compute_u_w(pd["k"], pd["v"], u, w, beta_mn, gate_mn)
    check_status(gdn)
    close(u, u_ref, "U")
    close(w, w_ref, "W")
    # token-major scalars give the same bits
    u2, w2 = torch.empty_like(u), torch.empty_like(w)
    gdn.bf16_gdn_compute_u_w(pd["k"], pd["v"], u2, w2, pd["beta"], gc.cuda())
    assert torch.equal(u2, u) and torch.equal(w2, w)


def test_compute_u_w_varlen_ragged(gdn):
    lens = [1, 63, 64, 65, 130, 2]
    p = synthetic.varlen_inputs(lens, 2, 4, 128, seed=5, with_state=False, mild_gate=True)
    gc = O.chunk_local_cumsum_ref(p["g"], p["cu_seqlens"])
    u_ref, w_ref = O.compute_u_w_ref(*f32(p, "k", "v", "beta"), gc, p["cu_seqlens"])
    pd = dev(p)
    u = torch.full_like(pd["v"], float("nan"))
    w = torch.full_like(pd["v"], float("nan"))
    gdn.bf16_gdn_compute_u_w(pd["k"], pd["v"], u, w, pd["beta"], gc.cuda(), cu_seqlens=pd["cu_seqlens"],
                             chunk_indices=pd["chunk_indices"])
    check_status(gdn)
    close(u, u_ref, "U")
    close(w, w_ref, "W")


@pytest.mark.parametrize("varlen", [False, True])
def test_seq_state_update(gdn, varlen):
    if varlen:
        lens = [65, 1, 200, 64]
        p = synthetic.varlen_inputs(lens, 2, 4, 128, seed=8, mild_gate=True)
        cu = p["cu_seqlens"]
    else:
        p = synthetic.prefill_inputs(2, 200, 2, 4, 128, seed=8, mild_gate=True)
        cu = None
    gc = O.chunk_local_cumsum_ref(p["g"], cu)
    u_ref, w_ref = O.compute_u_w_ref(*f32(p, "k", "v", "beta"), gc, cu)
    u_bf, w_bf = u_ref.bfloat16(), w_ref.bfloat16()
    h_ref, un_ref, s_ref = O.seq_state_update_ref(p["k"].float(), u_bf.float(), w_bf.float(), gc, p["state"].float(), cu)
    pd = dev(p)
    u, w = u_bf.cuda(), w_bf.cuda()
    state = torch.full(h_ref.shape, float("nan"), dtype=torch.bfloat16, device="cuda")
    final = torch.empty_like(pd["state"])
    kw = dict(cu_seqlens=pd["cu_seqlens"], cu_chunks=pd["cu_chunks"], total_chunks=p["total_chunks"]) if varlen else {}
    gdn.bf16_chunked_seq_state_update(pd["k"], u, w, pd["state"], state, final, gc.cuda(), **kw)
    check_status(gdn)
    close(state, h_ref, "chunk states")
    close(u, un_ref, "U_new")
    close(final, s_ref, "final state")


# ---------------------------------------------------------------- end to end
PADDED = [
    # (B, T, kh, vh, d)   shapes from the reference's test lists plus BASELINE-like ones
    (1, 63, 1, 1, 64), (2, 500, 3, 3, 60), (2, 1000, 3, 3, 64), (3, 1024, 4, 4, 100), (4, 1024, 4, 4, 128),
    (2, 1500, 4, 4, 128), (1, 130, 2, 4, 128), (1, 97, 1, 2, 128), (2, 65, 2, 2, 128), (1, 255, 2, 8, 128),
    (1, 256, 4, 4, 64), (2, 512, 16, 32, 128),
]


@pytest.mark.parametrize("B,T,kh,vh,d", PADDED)
@pytest.mark.parametrize("mild", [False, True])
def test_chunked_forward_padded(gdn, B, T, kh, vh, d, mild):
    p = synthetic.prefill_inputs(B, T, kh, vh, d, seed=T + d, mild_gate=mild)
    o_ref, s_ref = O.recurrent_ref(*f32(p, "q", "k", "v", "beta"), p["g"], p["state"].float())
    pd = dev(p)
    o, s = gdn.chunked_forward(pd["q"], pd["k"], pd["v"], pd["beta"], pd["g"], None, pd["state"])
    check_status(gdn)
    assert o.shape == p["v"].shape and s.shape == p["state"].shape
    close(o, o_ref, "O")
    close(s, s_ref, "final state")


@pytest.mark.parametrize("B,T,kh,vh,with_state", [(1, 6161, 1, 2, True), (3, 6144, 4, 8, True), (1, 9000, 2, 2, False),
                                                 (2, 16384 + 70, 1, 1, True)])
def test_chunked_forward_segmented(gdn, B, T, kh, vh, with_state):
    """Few long padded sequences take the segmented path (composite transitions per segment, start
    states chained in fp32, all segments at once); the result must still be the token recurrence."""
    p = synthetic.prefill_inputs(B, T, kh, vh, 128, seed=T, with_state=with_state)
    o_ref, s_ref = O.recurrent_ref(*f32(p, "q", "k", "v", "beta"), p["g"],
                                   p["state"].float() if with_state else None)
    pd = dev(p)
    o, s = gdn.chunked_forward(pd["q"], pd["k"], pd["v"], pd["beta"], pd["g"], None, pd["state"])
    check_status(gdn)
    close(o, o_ref, "O")
    close(s, s_ref, "final state")


@pytest.mark.parametrize("lens,kh,vh,qk_norm", [([6161], 1, 2, False), ([16384 + 70, 70], 1, 1, False),
                                                ([20000, 0, 5600], 2, 2, False), ([9000, 9100], 1, 2, True)])
def test_chunked_forward_segmented_packed(gdn, lens, kh, vh, qk_norm):
    """Few long PACKED sequences take the segmented path as well: segments of one length for all sequences,
    a sequence shorter than a segment (or empty) keeps one segment, surplus launch slots leave at once."""
    from h100_gdn_cuda_b200 import api
    p = synthetic.varlen_inputs(lens, kh, vh, 128, seed=sum(lens), mild_gate=True, normalize=not qk_norm)
    plain = (64 * 128 * 2 + 64 * 64 * 2) * vh * p["total_chunks"] + 512 * kh * p["total_chunks"]
    need = api.chunked_forward_workspace_bytes(len(lens), 0, vh, total_tokens=sum(lens), total_chunks=p["total_chunks"],
                                               packed=True, num_k_heads=kh)
    assert need > plain + 3 * 128 * 128 * 4, "this shape is meant to be segmented"
    o_ref, s_ref = O.recurrent_ref(*f32(p, "q", "k", "v", "beta"), p["g"], p["state"].float(),
                                   cu_seqlens=p["cu_seqlens"], is_qk_norm=qk_norm)
    pd = dev(p)
    o, s = gdn.chunked_forward(pd["q"], pd["k"], pd["v"], pd["beta"], pd["g"], None, pd["state"],
                               pd["cu_seqlens"], pd["chunk_indices"], pd["cu_chunks"], p["total_chunks"],
                               is_qk_norm=qk_norm)
    check_status(gdn)
    close(o, o_ref, "O")
    close(s, s_ref, "final states")
    for i, n in enumerate(lens):
        if n == 0:
            assert torch.equal(s[i], pd["state"][i])


def test_chunked_forward_no_state_custom_scale(gdn):
    p = synthetic.prefill_inputs(2, 300, 2, 4, 128, seed=77, with_state=False, mild_gate=True)
    o_ref, s_ref = O.recurrent_ref(*f32(p, "q", "k", "v", "beta"), p["g"], None, scale=0.5)
    pd = dev(p)
    o, s = gdn.chunked_forward(pd["q"], pd["k"], pd["v"], pd["beta"], pd["g"], 0.5)
    close(o, o_ref, "O")
    close(s, s_ref, "final state")


RAGGED = [
    [64, 64], [128, 64, 192], [1], [2, 1, 63, 65], [130, 97, 65, 255], [1, 64, 1, 65, 1],
    [63, 63, 63], [300, 5, 1000, 64, 17], [700, 1, 1, 129],
]


@pytest.mark.parametrize("lens", RAGGED)
def test_chunked_forward_varlen(gdn, lens):
    p = synthetic.varlen_inputs(lens, 2, 4, 128, seed=sum(lens), mild_gate=(len(lens) % 2 == 0))
    o_ref, s_ref = O.recurrent_ref(*f32(p, "q", "k", "v", "beta"), p["g"], p["state"].float(),
                                   cu_seqlens=p["cu_seqlens"])
    pd = dev(p)
    o, s = gdn.chunked_forward(pd["q"], pd["k"], pd["v"], pd["beta"], pd["g"], None, pd["state"],
                               pd["cu_seqlens"], pd["chunk_indices"], pd["cu_chunks"], p["total_chunks"])
    check_status(gdn)
    close(o, o_ref, "O")
    close(s, s_ref, "final state")


@pytest.mark.parametrize("d,lens,kh,vh", [(64, [130, 97, 65, 255], 2, 4), (96, [300, 5, 1000, 64, 17], 1, 2),
                                          (8, [70, 1], 1, 1), (64, [9000, 9100], 1, 2)])
def test_chunked_forward_small_head_dims_unpadded(gdn, d, lens, kh, vh):
    """Head dims below 128 that are multiples of 8 go to the kernels as they are (zero columns come from the
    tensor maps, states are d x d): packed inputs with ragged chunk tails, and one segmented case."""
    p = synthetic.varlen_inputs(lens, kh, vh, d, seed=d + sum(lens), mild_gate=True)
    o_ref, s_ref = O.recurrent_ref(*f32(p, "q", "k", "v", "beta"), p["g"], p["state"].float(),
                                   cu_seqlens=p["cu_seqlens"])
    pd = dev(p)
    o, s = gdn.chunked_forward(pd["q"], pd["k"], pd["v"], pd["beta"], pd["g"], None, pd["state"],
                               pd["cu_seqlens"], pd["chunk_indices"], pd["cu_chunks"], p["total_chunks"])
    check_status(gdn)
    assert o.shape == p["v"].shape and s.shape == p["state"].shape and o.is_contiguous()
    close(o, o_ref, "O")
    close(s, s_ref, "final states")
    # a strided view of a wider buffer (the layout of a fused projection): neighbours must stay untouched
    wide = torch.randn(sum(lens), kh, 3 * d, device="cuda").bfloat16()
    wide[..., :d], wide[..., d:2 * d] = pd["q"], pd["k"]
    o2, s2 = gdn.chunked_forward(wide[..., :d], wide[..., d:2 * d], pd["v"], pd["beta"], pd["g"], None, pd["state"],
                                 pd["cu_seqlens"], pd["chunk_indices"], pd["cu_chunks"], p["total_chunks"])
    assert torch.equal(o2, o) and torch.equal(s2, s)
    # a view TMA cannot address (head stride not a multiple of 8 elements) is compacted by the front end, not refused
    odd = torch.zeros(sum(lens), kh, d + 4, device="cuda", dtype=torch.bfloat16)
    odd[..., :d] = pd["q"]
    o3, s3 = gdn.chunked_forward(odd[..., :d], pd["k"], pd["v"], pd["beta"], pd["g"], None, pd["state"],
                                 pd["cu_seqlens"], pd["chunk_indices"], pd["cu_chunks"], p["total_chunks"])
    assert torch.equal(o3, o) and torch.equal(s3, s)


def test_varlen_equals_padded_per_sequence(gdn):
    lens = [200, 77]
    p = synthetic.varlen_inputs(lens, 2, 4, 128, seed=4, mild_gate=True)
    pd = dev(p)
    o, s = gdn.chunked_forward(pd["q"], pd["k"], pd["v"], pd["beta"], pd["g"], None, pd["state"],
                               pd["cu_seqlens"], pd["chunk_indices"], pd["cu_chunks"], p["total_chunks"])
    off = 0
    for i, n in enumerate(lens):
        sl = slice(off, off + n)
        oi, si = gdn.chunked_forward(pd["q"][None, sl], pd["k"][None, sl], pd["v"][None, sl], pd["beta"][None, sl],
                                     pd["g"][None, sl], None, pd["state"][i:i + 1])
        assert torch.equal(oi[0], o[sl]) and torch.equal(si[0], s[i])
        off += n


def test_chunked_forward_varlen_with_empty_sequences(gdn):
    # sequences without tokens own no chunk; their final state is their initial state
    lens = [70, 0, 5, 0]
    p = synthetic.varlen_inputs(lens, 2, 4, 128, seed=3, mild_gate=True)
    assert p["total_chunks"] == 3
    o_ref, s_ref = O.recurrent_ref(*f32(p, "q", "k", "v", "beta"), p["g"], p["state"].float(),
                                   cu_seqlens=p["cu_seqlens"])
    pd = dev(p)
    o, s = gdn.chunked_forward(pd["q"], pd["k"], pd["v"], pd["beta"], pd["g"], None, pd["state"],
                               pd["cu_seqlens"], pd["chunk_indices"], pd["cu_chunks"], p["total_chunks"])
    check_status(gdn)
    close(o, o_ref, "O")
    close(s, s_ref, "final states")
    assert torch.equal(s[1], pd["state"][1]) and torch.equal(s[3], pd["state"][3])


def test_varlen_more_chains_than_sms(gdn):
    # 40 sequences x 4 v-heads = 160 chains: the state kernel takes the sequences longest first
    # (ties, single-token and empty sequences included); every sequence must still land in its own slot
    lens = [1 + (37 * i) % 150 for i in range(35)] + [0, 64, 64, 150, 1]
    p = synthetic.varlen_inputs(lens, 2, 4, 128, seed=40, mild_gate=True)
    o_ref, s_ref = O.recurrent_ref(*f32(p, "q", "k", "v", "beta"), p["g"], p["state"].float(),
                                   cu_seqlens=p["cu_seqlens"])
    pd = dev(p)
    o, s = gdn.chunked_forward(pd["q"], pd["k"], pd["v"], pd["beta"], pd["g"], None, pd["state"],
                               pd["cu_seqlens"], pd["chunk_indices"], pd["cu_chunks"], p["total_chunks"])
    check_status(gdn)
    close(o, o_ref, "O")
    close(s, s_ref, "final states")
    off = 0
    for i, n in enumerate(lens):
        if i % 7 == 0 and n > 0:
            sl = slice(off, off + n)
            oi, si = gdn.chunked_forward(pd["q"][None, sl], pd["k"][None, sl], pd["v"][None, sl], pd["beta"][None, sl],
                                         pd["g"][None, sl], None, pd["state"][i:i + 1])
            assert torch.equal(oi[0], o[sl]) and torch.equal(si[0], s[i])
        off += n


def test_prefill_state_handoff(gdn):
    # prefill(T1) -> state -> prefill(T2) == prefill(T1+T2); then hand the state to decode
    p = synthetic.prefill_inputs(1, 384, 2, 4, 128, seed=12, mild_gate=True)
    pd = dev(p)
    a = [pd[k] for k in ("q", "k", "v", "beta", "g")]
    o, s = gdn.chunked_forward(*a, None, pd["state"])
    o1, s1 = gdn.chunked_forward(*(x[:, :128] for x in a), None, pd["state"])
    o2, s2 = gdn.chunked_forward(*(x[:, 128:] for x in a), None, s1)
    o_ref, s_ref = O.recurrent_ref(*f32(p, "q", "k", "v", "beta"), p["g"], p["state"].float())
    close(torch.cat([o1, o2], 1), o_ref, "O (two-part)")
    close(s2, s_ref, "state (two-part)")
    # decode continues from the prefill state
    d = synthetic.decode_inputs(1, 1, 2, 4, 128, seed=3)
    beta, g = O.gating_ref(d["A_log"], d["dt_bias"], d["a"], d["b"])
    od, sd = gdn.recurrent_forward(d["q"].cuda(), d["k"].cuda(), d["v"].cuda(), s, beta.bfloat16().cuda(), g.cuda(),
                                   is_qk_norm=True, inference_mode=1)
    od_ref, sd_ref = O.recurrent_ref(d["q"].float(), d["k"].float(), d["v"].float(), beta.bfloat16().float(), g,
                                     s.float().cpu(), is_qk_norm=True)
    close(od, od_ref, "decode O after prefill")
    close(sd, sd_ref, "decode state after prefill")


def test_chunked_head_sliced_views(gdn):
    # value-head sharding: non-contiguous head slices must give the same bits as the full call
    p = synthetic.prefill_inputs(1, 200, 4, 8, 128, seed=31, mild_gate=True)
    pd = dev(p)
    o, s = gdn.chunked_forward(pd["q"], pd["k"], pd["v"], pd["beta"], pd["g"], None, pd["state"])
    oh, sh = gdn.chunked_forward(pd["q"][:, :, 2:4], pd["k"][:, :, 2:4], pd["v"][:, :, 4:8], pd["beta"][:, :, 4:8],
                                 pd["g"][:, :, 4:8], None, pd["state"][:, 4:8])
    assert torch.equal(oh, o[:, :, 4:8]) and torch.equal(sh, s[:, 4:8])


def test_chunked_errors(gdn):
    p = dev(synthetic.prefill_inputs(1, 64, 1, 1, 128, seed=1))
    with pytest.raises(RuntimeError):
        gdn.chunked_forward(p["q"].float(), p["k"], p["v"], p["beta"], p["g"])
    big = torch.zeros(1, 64, 1, 320, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        gdn.chunked_forward(big, big, big, p["beta"], p["g"])


@pytest.mark.parametrize("B,T,kh,vh,d", [(2, 200, 2, 4, 192), (1, 130, 1, 2, 256), (2, 77, 2, 2, 200)])
def test_chunked_forward_wide_heads(gdn, B, T, kh, vh, d):
    # head dims in (128, 256] (the reference's chunked kernels go up to 256): same call, same semantics
    p = synthetic.prefill_inputs(B, T, kh, vh, d, seed=T + d, mild_gate=True)
    o_ref, s_ref = O.recurrent_ref(*f32(p, "q", "k", "v", "beta"), p["g"], p["state"].float())
    pd = dev(p)
    o, s = gdn.chunked_forward(pd["q"], pd["k"], pd["v"], pd["beta"], pd["g"], None, pd["state"])
    check_status(gdn)
    assert o.shape == p["v"].shape and s.shape == p["state"].shape
    close(o, o_ref, "O")
    close(s, s_ref, "final state")


def test_chunked_forward_wide_heads_varlen(gdn):
    lens = [65, 1, 130, 0, 64]
    p = synthetic.varlen_inputs(lens, 2, 4, 256, seed=9, mild_gate=True)
    o_ref, s_ref = O.recurrent_ref(*f32(p, "q", "k", "v", "beta"), p["g"], p["state"].float(),
                                   cu_seqlens=p["cu_seqlens"])
    pd = dev(p)
    o, s = gdn.chunked_forward(pd["q"], pd["k"], pd["v"], pd["beta"], pd["g"], None, pd["state"],
                               pd["cu_seqlens"], pd["chunk_indices"], pd["cu_chunks"], p["total_chunks"])
    check_status(gdn)
    close(o, o_ref, "O")
    close(s, s_ref, "final states")


@pytest.mark.parametrize("varlen", [False, True])
def test_compute_o_stage(gdn, varlen):
    """Low-level output stage from oracle-made per-chunk states and U_new; then the three
    low-level stages chained equal the token recurrence."""
    if varlen:
        lens = [65, 1, 200, 64]
        p = synthetic.varlen_inputs(lens, 2, 4, 128, seed=18, mild_gate=True)
        cu = p["cu_seqlens"]
    else:
        p = synthetic.prefill_inputs(2, 200, 2, 4, 128, seed=18, mild_gate=True)
        cu = None
    gc = O.chunk_local_cumsum_ref(p["g"], cu)
    u_ref, w_ref = O.compute_u_w_ref(*f32(p, "k", "v", "beta"), gc, cu)
    h_ref, un_ref, s_ref = O.seq_state_update_ref(p["k"].float(), u_ref, w_ref, gc, p["state"].float(), cu)
    h_bf, un_bf = h_ref.bfloat16(), un_ref.bfloat16()
    o_ref = O.compute_o_ref(p["q"].float(), p["k"].float(), un_bf.float(), h_bf.float(), gc, None, cu)
    pd = dev(p)
    kw = dict(cu_seqlens=pd["cu_seqlens"], chunk_indices=pd["chunk_indices"], cu_chunks=pd["cu_chunks"]) if varlen else {}
    o = torch.full_like(pd["v"], float("nan"))
    gdn.bf16_gdn_chunked_compute_O(pd["q"], h_bf.cuda(), pd["k"], un_bf.cuda(), o, gc.cuda(), **kw)
    check_status(gdn)
    close(o, o_ref, "O (stage)")
    # chain of the three low-level wrappers == recurrence
    u, w = torch.empty_like(pd["v"]), torch.empty_like(pd["v"])
    kw_uw = dict(cu_seqlens=pd["cu_seqlens"], chunk_indices=pd["chunk_indices"]) if varlen else {}
    gdn.bf16_gdn_compute_u_w(pd["k"], pd["v"], u, w, pd["beta"], gc.cuda(), **kw_uw)
    state = torch.empty(h_ref.shape, dtype=torch.bfloat16, device="cuda")
    final = torch.empty_like(pd["state"])
    kw_st = dict(cu_seqlens=pd["cu_seqlens"], cu_chunks=pd["cu_chunks"], total_chunks=p["total_chunks"]) if varlen else {}
    gdn.bf16_chunked_seq_state_update(pd["k"], u, w, pd["state"], state, final, gc.cuda(), **kw_st)
    o2 = torch.empty_like(pd["v"])
    gdn.bf16_gdn_chunked_compute_O(pd["q"], state, pd["k"], u, o2, gc.cuda(), **kw)
    check_status(gdn)
    o_rec, s_rec = O.recurrent_ref(*f32(p, "q", "k", "v", "beta"), p["g"], p["state"].float(), cu_seqlens=cu)
    close(o2, o_rec, "O (three stages)")
    close(final, s_rec, "final state (three stages)")


def test_back_to_back_calls_hand_the_state_over(gdn):
    """The kernels are launched as programmatic dependents of the work before them (they are placed and set up while it
    drains).  A state produced by one call and consumed by the next, with nothing in between, must still be the
    finished state: chains of prefill and decode calls issued without any synchronisation give the bits of the same
    chains run with a device synchronisation after every call.  Small problems, so that a following kernel could start
    while most of the GPU is still free."""
    for (B, T, kh, vh) in ((1, 130, 2, 4), (2, 64, 1, 2), (1, 700, 2, 4)):
        p = dev(synthetic.prefill_inputs(B, T, kh, vh, 128, seed=T, mild_gate=True))
        dq, dk, dv = (p[n][:, :1].contiguous() for n in ("q", "k", "v"))
        db, dg = p["beta"][:, :1].contiguous(), p["g"][:, :1].contiguous()

        def chain(sync):
            s = p["state"]
            outs = []
            for it in range(12):
                o, s = gdn.chunked_forward(p["q"], p["k"], p["v"], p["beta"], p["g"], None, s)
                if sync:
                    torch.cuda.synchronize()
                o2, s = gdn.recurrent_forward(dq, dk, dv, s, db, dg)
                if sync:
                    torch.cuda.synchronize()
                outs.append((o[:, -1].clone(), o2.clone()))
            torch.cuda.synchronize()
            return s, outs
        s_sync, outs_sync = chain(True)
        for _ in range(3):
            s_async, outs_async = chain(False)
            assert torch.equal(s_async, s_sync)
            assert all(torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]) for a, b in zip(outs_async, outs_sync))
    check_status(gdn)
