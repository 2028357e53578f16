"""The C++/pybind11 `gdn_cuda` extension (same module surface as the reference's
csrc/python_api.cpp) gives the same bits as the ctypes mirror, and raises RuntimeError."""
import pytest
import torch

from h100_gdn_cuda_b200 import synthetic

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mods():
    import h100_gdn_cuda_b200 as py
    from h100_gdn_cuda_b200 import build
    build.build()
    build.build_ext()
    from h100_gdn_cuda_b200 import gdn_cuda as ext
    return py, ext


def dev(d):
    return {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in d.items()}


def test_surface(mods):
    _, ext = mods
    for name in ("init", "chunked_forward", "recurrent_forward", "fused_gdn_gating", "bf16_gdn_compute_u_w",
                 "bf16_chunked_seq_state_update", "bf16_gdn_chunked_compute_O", "bf16_gdn_recurrent", "chunk_local_cumsum_bf16",
                 "transpose_to_mn_major", "InferenceMode"):
        assert hasattr(ext, name)
    assert int(ext.Prefill) == 0 and int(ext.Decode) == 1 and int(ext.SpecVerify) == 2


def test_chunked_forward_same_bits(mods):
    py, ext = mods
    p = dev(synthetic.prefill_inputs(2, 200, 2, 4, 128, seed=3, mild_gate=True))
    o1, s1 = py.chunked_forward(p["q"], p["k"], p["v"], p["beta"], p["g"], None, p["state"])
    o2, s2 = ext.chunked_forward(p["q"], p["k"], p["v"], p["beta"], p["g"], None, p["state"])
    assert torch.equal(o1, o2) and torch.equal(s1, s2)
    v = dev(synthetic.varlen_inputs([65, 1, 200], 2, 4, 100, seed=4))
    a = (v["q"], v["k"], v["v"], v["beta"], v["g"], None, v["state"], v["cu_seqlens"], v["chunk_indices"],
         v["cu_chunks"], v["total_chunks"])
    o1, s1 = py.chunked_forward(*a)
    o2, s2 = ext.chunked_forward(*a)
    assert o2.shape == v["v"].shape and torch.equal(o1, o2) and torch.equal(s1, s2)
    # head dim above 128: both layers hand the call to the token-recurrent kernel
    w = dev(synthetic.prefill_inputs(1, 100, 1, 2, 200, seed=6, mild_gate=True))
    o1, s1 = py.chunked_forward(w["q"], w["k"], w["v"], w["beta"], w["g"], None, w["state"])
    o2, s2 = ext.chunked_forward(w["q"], w["k"], w["v"], w["beta"], w["g"], None, w["state"])
    assert o2.shape == w["v"].shape and s2.shape == w["state"].shape
    assert torch.equal(o1, o2) and torch.equal(s1, s2)


def test_recurrent_and_helpers_same_bits(mods):
    py, ext = mods
    d = dev(synthetic.decode_inputs(8, 4, 2, 4, 128, seed=5, spec=True))
    b1, g1 = py.fused_gdn_gating(d["A_log"], d["dt_bias"], d["a"], d["b"])
    b2, g2 = ext.fused_gdn_gating(d["A_log"], d["dt_bias"], d["a"], d["b"], False)
    assert torch.equal(b1, b2) and torch.equal(g1, g2)
    for mode in (1, 2):
        o1, s1 = py.recurrent_forward(d["q"], d["k"], d["v"], d["state"], b1, g1, None, d["num_accepted_tokens"],
                                      mode, True)
        o2, s2 = ext.recurrent_forward(d["q"], d["k"], d["v"], d["state"], b2, g2, None, d["num_accepted_tokens"],
                                       mode, True)
        mask = torch.arange(4, device="cuda")[None, :] < d["num_accepted_tokens"][:, None]
        assert torch.equal(o1[mask], o2[mask]) and s1.shape == s2.shape
        if mode == 1:
            assert torch.equal(s1, s2)
    x = torch.randn(3, 70, 5, device="cuda")
    assert torch.equal(py.transpose_to_mn_major(x), ext.transpose_to_mn_major(x))
    out1 = torch.empty(3, 70, 5, device="cuda")
    out2 = torch.empty(3, 70, 5, device="cuda")
    py.chunk_local_cumsum_bf16(x, out1, 3, 70, 5, True)
    ext.chunk_local_cumsum_bf16(x, out2, 3, 70, 5, True)
    assert torch.equal(out1, out2)


def test_low_level_chain_same_bits(mods):
    py, ext = mods
    p = dev(synthetic.prefill_inputs(1, 130, 2, 4, 128, seed=6, mild_gate=True))
    gc = torch.empty_like(p["g"])
    ext.chunk_local_cumsum_bf16(p["g"], gc, 1, 130, 4, True)
    res = []
    for m in (py, ext):
        u, w = torch.empty_like(p["v"]), torch.empty_like(p["v"])
        m.bf16_gdn_compute_u_w(p["k"], p["v"], u, w, m.transpose_to_mn_major(p["beta"]), m.transpose_to_mn_major(gc))
        state = torch.empty(1, 3, 4, 128, 128, dtype=torch.bfloat16, device="cuda")
        final = torch.empty_like(p["state"])
        m.bf16_chunked_seq_state_update(p["k"], u, w, p["state"], state, final, gc)
        o = torch.empty_like(p["v"])
        m.bf16_gdn_chunked_compute_O(p["q"], state, p["k"], u, o, gc)
        res.append((u, w, state, final, o))
    for a, b in zip(*res):
        assert torch.equal(a, b)


def test_errors_raise(mods):
    _, ext = mods
    p = dev(synthetic.prefill_inputs(1, 64, 1, 1, 128, seed=1))
    with pytest.raises(RuntimeError):
        ext.chunked_forward(p["q"].float(), p["k"], p["v"], p["beta"], p["g"])
    big = torch.zeros(1, 64, 1, 320, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        ext.chunked_forward(big, big, big, p["beta"], p["g"])


@pytest.mark.parametrize("d,varlen", [(64, False), (100, False), (64, True)])
def test_low_level_chain_small_head_dims_vs_oracle(mods, d, varlen):
    """The reference's per-stage chain (compute_u_w -> seq_state_update -> compute_O) at head dims below
    128, through the pybind module, against the fp32 token recurrence.  Tolerance of the prefill tests:
    relative Frobenius <= 1e-2, max-abs <= 5e-2 * max|ref|."""
    from oracle import gdn_oracle as O
    _, ext = mods
    if varlen:
        lens = [65, 1, 130]
        p = synthetic.varlen_inputs(lens, 2, 4, d, seed=40 + d, mild_gate=True)
        cu = p["cu_seqlens"]
        nck = p["total_chunks"]
    else:
        p = synthetic.prefill_inputs(2, 130, 2, 4, d, seed=40 + d, mild_gate=True)
        cu, nck = None, 3
    gc = O.chunk_local_cumsum_ref(p["g"], cu)
    pd = dev(p)
    g = gc.cuda()
    kw_uw = dict(cu_seqlens=pd["cu_seqlens"], chunk_indices=pd["chunk_indices"]) if varlen else {}
    kw_st = dict(cu_seqlens=pd["cu_seqlens"], cu_chunks=pd["cu_chunks"], total_chunks=nck) if varlen else {}
    kw_o = dict(cu_seqlens=pd["cu_seqlens"], chunk_indices=pd["chunk_indices"], cu_chunks=pd["cu_chunks"]) if varlen else {}
    u, w = torch.empty_like(pd["v"]), torch.empty_like(pd["v"])
    ext.bf16_gdn_compute_u_w(pd["k"], pd["v"], u, w, pd["beta"], g, **kw_uw)
    state = torch.empty((nck, 4, d, d) if varlen else (2, nck, 4, d, d), dtype=torch.bfloat16, device="cuda")
    final = torch.empty_like(pd["state"])
    ext.bf16_chunked_seq_state_update(pd["k"], u, w, pd["state"], state, final, g, **kw_st)
    o = torch.empty_like(pd["v"])
    ext.bf16_gdn_chunked_compute_O(pd["q"], state, pd["k"], u, o, g, **kw_o)
    o_ref, s_ref = O.recurrent_ref(p["q"].float(), p["k"].float(), p["v"].float(), p["beta"].float(), p["g"],
                                   p["state"].float(), cu_seqlens=None if cu is None else cu.tolist())
    for x, ref, what in ((o, o_ref, "o"), (final, s_ref, "final state")):
        x = x.float().cpu()
        assert O.rel_fro(x, ref) <= 1e-2 and O.max_abs_over_max(x, ref) <= 5e-2, what


def test_bf16_gdn_recurrent_on_caller_tensors(mods):
    """gdn_cuda::bf16_gdn_recurrent: same bits as recurrent_forward, written into the caller's tensors."""
    py, ext = mods
    d = dev(synthetic.decode_inputs(4, 3, 2, 4, 128, seed=8))
    beta, gate = py.fused_gdn_gating(d["A_log"], d["dt_bias"], d["a"], d["b"])
    o1, s1 = py.recurrent_forward(d["q"], d["k"], d["v"], d["state"], beta, gate, None, None, 1, True, 0.25)
    out, fin = torch.empty_like(d["v"]), torch.empty_like(d["state"])
    ext.bf16_gdn_recurrent(d["q"], d["k"], d["v"], d["state"], fin, out, gate, beta, "t", None, None, False, True, 0.25)
    assert torch.equal(o1, out) and torch.equal(s1, fin)
    steps = torch.empty(4, 3, 4, 128, 128, dtype=torch.bfloat16, device="cuda")
    ext.bf16_gdn_recurrent(d["q"], d["k"], d["v"], d["state"], steps, out, gate, beta, store_step_state=True, is_qk_norm=True,
                           scale=0.25)
    assert torch.equal(steps[:, -1], fin)
    with pytest.raises(RuntimeError):
        ext.bf16_gdn_recurrent(d["q"][..., :100], d["k"][..., :100], d["v"], d["state"], fin, out, gate, beta)


def test_extensions_same_bits(mods):
    py, ext = mods
    d = dev(synthetic.decode_inputs(4, 1, 2, 4, 128, seed=9))
    gating = (d["A_log"], d["dt_bias"], d["a"], d["b"])
    o1, s1 = py.recurrent_forward(d["q"], d["k"], d["v"], d["state"], None, None, inference_mode=1, is_qk_norm=True, gating=gating)
    o2, s2 = ext.recurrent_forward(d["q"], d["k"], d["v"], d["state"], None, None, inference_mode=1, is_qk_norm=True, gating=gating)
    assert torch.equal(o1, o2) and torch.equal(s1, s2)
    p = dev(synthetic.prefill_inputs(1, 200, 2, 4, 128, seed=3, mild_gate=True, normalize=False))
    o1, s1 = py.chunked_forward(p["q"], p["k"], p["v"], p["beta"], p["g"], None, p["state"], is_qk_norm=True)
    o2, s2 = ext.chunked_forward(p["q"], p["k"], p["v"], p["beta"], p["g"], None, p["state"], is_qk_norm=True)
    assert torch.equal(o1, o2) and torch.equal(s1, s2)


def test_state_pool_fp32_state_and_layer_adjacent_same_bits(mods):
    """The pybind front end carries the same keyword-only extensions as the ctypes one: an indexed state pool,
    an in-place state, fp32 states, and the two layer-adjacent kernels."""
    py, ext = mods
    d = dev(synthetic.decode_inputs(5, 1, 2, 4, 128, seed=21))
    gating = (d["A_log"], d["dt_bias"], d["a"], d["b"])
    # indexed pool: 8 slots, sequence 2 is padding (negative slot)
    idx = torch.tensor([6, 0, -1, 3, 5], dtype=torch.int32, device="cuda")
    pool = (torch.randn(8, 4, 128, 128, device="cuda") * 0.05).bfloat16()
    pool1, pool2 = pool.clone(), pool.clone()
    o1, r1 = py.recurrent_forward(d["q"], d["k"], d["v"], pool1, None, None, inference_mode=1, is_qk_norm=True, gating=gating,
                                  state_indices=idx)
    o2, r2 = ext.recurrent_forward(d["q"], d["k"], d["v"], pool2, None, None, inference_mode=1, is_qk_norm=True, gating=gating,
                                   state_indices=idx)
    assert r1.data_ptr() == pool1.data_ptr() and r2.data_ptr() == pool2.data_ptr()
    keep = [i for i in range(5) if i != 2]
    assert torch.equal(o1[keep], o2[keep]) and torch.equal(pool1, pool2)
    assert torch.equal(pool2[[1, 2, 4, 7]], pool[[1, 2, 4, 7]]) and not torch.equal(pool2[6], pool[6])
    # in-place state
    s1, s2 = d["state"].clone(), d["state"].clone()
    py.recurrent_forward(d["q"], d["k"], d["v"], s1, None, None, inference_mode=1, gating=gating, inplace_state=True)
    _, r2 = ext.recurrent_forward(d["q"], d["k"], d["v"], s2, None, None, inference_mode=1, gating=gating, inplace_state=True)
    assert r2.data_ptr() == s2.data_ptr() and torch.equal(s1, s2) and not torch.equal(s2, d["state"])
    with pytest.raises(RuntimeError):
        ext.recurrent_forward(d["q"], d["k"], d["v"], d["state"].transpose(-1, -2), None, None, inference_mode=1, gating=gating,
                              inplace_state=True)
    # fp32 state stays fp32
    f1, f2 = d["state"].float(), d["state"].float()
    o1, r1 = py.recurrent_forward(d["q"], d["k"], d["v"], f1, None, None, inference_mode=1, gating=gating)
    o2, r2 = ext.recurrent_forward(d["q"], d["k"], d["v"], f2, None, None, inference_mode=1, gating=gating)
    assert r2.dtype == torch.float32 and torch.equal(o1, o2) and torch.equal(r1, r2)
    # causal conv1d (+ SiLU) with a carried state, and the gated RMS norm
    x = torch.randn(2, 100, 256, device="cuda").bfloat16()
    w = (torch.randn(256, 4, device="cuda") * 0.5).bfloat16()
    b = torch.randn(256, device="cuda").bfloat16()
    s0 = torch.randn(2, 3, 256, device="cuda").bfloat16()
    y1, t1 = py.causal_conv1d(x, w, b, s0, return_final_state=True)
    y2, t2 = ext.causal_conv1d(x, w, b, s0, return_final_state=True)
    assert torch.equal(y1, y2) and torch.equal(t1, t2)
    assert torch.equal(ext.causal_conv1d(x, w, activation=False), py.causal_conv1d(x, w, activation=False))
    cu = torch.tensor([0, 37, 200], dtype=torch.int32, device="cuda")
    xp = x.reshape(200, 256)
    assert torch.equal(ext.causal_conv1d(xp, w, b, cu_seqlens=cu), py.causal_conv1d(xp, w, b, cu_seqlens=cu))
    z = torch.randn(3, 50, 4, 128, device="cuda").bfloat16()
    xo = torch.randn(3, 50, 4, 128, device="cuda").bfloat16()
    g = torch.randn(128, device="cuda").bfloat16()
    assert torch.equal(ext.gated_rmsnorm(xo, z, g, 1e-5), py.gated_rmsnorm(xo, z, g, 1e-5))
