"""GPU parity of the recurrent path and the helper kernels against the CPU oracle.

Tolerances (bf16 outputs, fp32 oracle on the same bf16-rounded inputs):
relative Frobenius error <= 1e-2 and max-abs error <= 5e-2 * max|ref| for outputs and states.
Typical values are 2-3e-3 (the floor from rounding the oracle's result to bf16 is 1.7e-3).
"""
import numpy as np
import os
import glob
import pytest
import torch

from oracle import gdn_oracle as O
from h100_gdn_cuda_b200 import synthetic

pytestmark = pytest.mark.gpu

REL_FRO, MAX_ABS = 1e-2, 5e-2


def close(x, ref, what):
    x = x.float().cpu()
    rf, ma = O.rel_fro(x, ref), O.max_abs_over_max(x, ref)
    assert rf <= REL_FRO and ma <= MAX_ABS, "%s: rel_fro %.3e max_abs/max %.3e" % (what, rf, ma)
    return rf, ma


@pytest.fixture(scope="module")
def gdn():
    import h100_gdn_cuda_b200 as g
    from h100_gdn_cuda_b200 import build
    build.build()
    return g


def dev(d):
    return {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in d.items()}


GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("path", sorted(f for f in glob.glob(os.path.join(GOLDEN, "*.npz"))
                                        if not os.path.basename(f).startswith("branch_")))
def test_recurrent_matches_golden(gdn, path):
    z = np.load(path)
    t = {k: torch.from_numpy(z[k]) for k in z.files if k != "fla_version"}
    bf = lambda x: x.bfloat16().cuda()
    s0 = bf(t["state"]) if "state" in t else None
    o, s = gdn.recurrent_forward(bf(t["q"]), bf(t["k"]), bf(t["v"]), s0, bf(t["beta"]), t["g"].cuda())
    # golden inputs of the fp32 case are not bf16-exact: compare against the oracle on rounded inputs too
    r = lambda x: x.bfloat16().float()
    o_ref, s_ref = O.recurrent_ref(r(t["q"]), r(t["k"]), r(t["v"]), r(t["beta"]), t["g"],
                                   r(t["state"]) if "state" in t else None)
    close(o, o_ref, "o vs oracle")
    close(s, s_ref, "state vs oracle")
    rf = O.rel_fro(o.float().cpu(), t["o"])
    assert rf < 2e-2, "o vs golden rel_fro %.3e" % rf


@pytest.mark.parametrize("B,T,kh,vh,d,norm,gate_dtype", [
    (8, 1, 16, 32, 128, True, torch.bfloat16),     # decode, BASELINE shape at small batch
    (3, 1, 2, 4, 64, False, torch.float32),
    (2, 5, 2, 2, 256, True, torch.float32),
    (2, 3, 1, 2, 192, False, torch.bfloat16),
    (1, 256, 4, 4, 64, False, torch.float32),      # recurrent_forward as short prefill
    (2, 7, 2, 4, 100, True, torch.float32),        # head dim padded to 128
])
def test_recurrent_padded(gdn, B, T, kh, vh, d, norm, gate_dtype):
    p = synthetic.decode_inputs(B, T, kh, vh, d, seed=B * 100 + T)
    beta_ref, g_ref = O.gating_ref(p["A_log"], p["dt_bias"], p["a"], p["b"])
    beta = beta_ref.bfloat16()
    g = g_ref.to(gate_dtype)
    pd = dev(p)
    o, s = gdn.recurrent_forward(pd["q"], pd["k"], pd["v"], pd["state"], beta.cuda(), g.cuda(),
                                 is_qk_norm=norm, inference_mode=gdn.Decode)
    o_ref, s_ref = O.recurrent_ref(p["q"].float(), p["k"].float(), p["v"].float(), beta.float(), g.float(),
                                   p["state"].float(), is_qk_norm=norm)
    assert o.shape == p["v"].shape and s.shape == p["state"].shape
    close(o, o_ref, "o")
    close(s, s_ref, "state")


def test_recurrent_no_state_no_gate(gdn):
    p = synthetic.decode_inputs(2, 4, 2, 4, 128, seed=9)
    beta = torch.sigmoid(p["b"].float()).bfloat16()
    pd = dev(p)
    o, s = gdn.recurrent_forward(pd["q"], pd["k"], pd["v"], None, beta.cuda(), None, is_qk_norm=True)
    o_ref, s_ref = O.recurrent_ref(p["q"].float(), p["k"].float(), p["v"].float(), beta.float(),
                                   torch.zeros(2, 4, 4), None, is_qk_norm=True)
    close(o, o_ref, "o")
    close(s, s_ref, "state")


def test_spec_verify_step_states_and_accepted(gdn):
    B, T = 16, 4
    p = synthetic.decode_inputs(B, T, 16, 32, 128, seed=21, spec=True)
    beta_ref, g_ref = O.gating_ref(p["A_log"], p["dt_bias"], p["a"], p["b"])
    beta, g = beta_ref.bfloat16(), g_ref.bfloat16()
    pd = dev(p)
    nat = pd["num_accepted_tokens"]
    common = (p["q"].float(), p["k"].float(), p["v"].float(), beta.float(), g.float(), p["state"].float())
    # mode Decode with an accepted-token cap: final state after the accepted prefix
    o, s = gdn.recurrent_forward(pd["q"], pd["k"], pd["v"], pd["state"], beta.cuda(), g.cuda(),
                                 num_accepted_tokens=nat, inference_mode=1, is_qk_norm=True)
    o_ref, s_ref = O.recurrent_ref(*common, is_qk_norm=True, num_accepted_tokens=p["num_accepted_tokens"])
    mask = (torch.arange(T)[None, :] < p["num_accepted_tokens"][:, None])
    close(o.float().cpu()[mask], o_ref[mask], "o (accepted tokens)")
    close(s, s_ref, "state after accepted prefix")
    # mode SpecVerify: one state per token
    o2, steps = gdn.recurrent_forward(pd["q"], pd["k"], pd["v"], pd["state"], beta.cuda(), g.cuda(),
                                      inference_mode=gdn.SpecVerify, is_qk_norm=True)
    o2_ref, steps_ref = O.recurrent_ref(*common, is_qk_norm=True, store_step_state=True)
    assert steps.shape == (B, T, 32, 128, 128)
    close(o2, o2_ref, "o (spec)")
    close(steps, steps_ref, "step states")
    # step states equal successive single-token decodes
    s_run = pd["state"]
    for t in range(T):
        _, s_run = gdn.recurrent_forward(pd["q"][:, t:t + 1], pd["k"][:, t:t + 1], pd["v"][:, t:t + 1], s_run,
                                         beta.cuda()[:, t:t + 1], g.cuda()[:, t:t + 1], is_qk_norm=True)
        # the chained decode re-rounds the state to bf16 every step; allow for that
        assert O.rel_fro(s_run.float().cpu(), steps_ref[:, t]) < 1e-2


@pytest.mark.parametrize("d", [64, 128, 256])
def test_long_runs_step_states_and_accepted(gdn, d):
    # more than 16 tokens per sequence: the instance that streams k, q, v through its token ring;
    # 41 tokens = five full blocks of 8 and a ragged one, caps that end inside and between blocks
    B, T, kh, vh = 3, 41, 2, 4
    p = synthetic.decode_inputs(B, T, kh, vh, d, seed=31 + d)
    beta_ref, g_ref = O.gating_ref(p["A_log"], p["dt_bias"], p["a"], p["b"])
    beta, g = beta_ref.bfloat16(), g_ref.float()
    pd = dev(p)
    common = (p["q"].float(), p["k"].float(), p["v"].float(), beta.float(), g, p["state"].float())
    o, steps = gdn.recurrent_forward(pd["q"], pd["k"], pd["v"], pd["state"], beta.cuda(), g.cuda(),
                                     inference_mode=gdn.SpecVerify, is_qk_norm=True)
    o_ref, steps_ref = O.recurrent_ref(*common, is_qk_norm=True, store_step_state=True)
    assert steps.shape == (B, T, vh, d, d)
    close(o, o_ref, "o")
    close(steps, steps_ref, "step states")
    nat = torch.tensor([41, 24, 17], dtype=torch.int32)
    o, s = gdn.recurrent_forward(pd["q"], pd["k"], pd["v"], pd["state"], beta.cuda(), g.cuda(),
                                 num_accepted_tokens=nat.cuda(), inference_mode=1, is_qk_norm=True)
    o_ref, s_ref = O.recurrent_ref(*common, is_qk_norm=True, num_accepted_tokens=nat)
    mask = torch.arange(T)[None, :] < nat[:, None]
    close(o.float().cpu()[mask], o_ref[mask], "o (accepted tokens)")
    close(s, s_ref, "state after the accepted prefix")


def test_recurrent_varlen_short_and_long_sequences(gdn):
    # one launch with sequences on both sides of the 16-token threshold (and an empty one)
    lens = [40, 3, 0, 17, 100, 1, 16, 33]
    p = synthetic.varlen_inputs(lens, 2, 4, 128, seed=14, mild_gate=True)
    pd = dev(p)
    o, s = gdn.recurrent_forward(pd["q"], pd["k"], pd["v"], pd["state"], pd["beta"], pd["g"],
                                 cu_seqlens=pd["cu_seqlens"])
    o_ref, s_ref = O.recurrent_ref(p["q"].float(), p["k"].float(), p["v"].float(), p["beta"].float(), p["g"],
                                   p["state"].float(), cu_seqlens=p["cu_seqlens"])
    close(o, o_ref, "o")
    close(s, s_ref, "state")


def test_recurrent_varlen_and_inplace(gdn):
    lens = [1, 5, 2, 9]
    p = synthetic.varlen_inputs(lens, 2, 4, 128, seed=2)
    pd = dev(p)
    o, s = gdn.recurrent_forward(pd["q"], pd["k"], pd["v"], pd["state"], pd["beta"], pd["g"],
                                 cu_seqlens=pd["cu_seqlens"])
    o_ref, s_ref = O.recurrent_ref(p["q"].float(), p["k"].float(), p["v"].float(), p["beta"].float(), p["g"],
                                   p["state"].float(), cu_seqlens=p["cu_seqlens"])
    close(o, o_ref, "o")
    close(s, s_ref, "state")
    st = pd["state"].clone()
    o3, s3 = gdn.recurrent_forward(pd["q"], pd["k"], pd["v"], st, pd["beta"], pd["g"],
                                   cu_seqlens=pd["cu_seqlens"], inplace_state=True)
    assert s3.data_ptr() == st.data_ptr()
    assert torch.equal(s3, s) and torch.equal(o3, o)


def test_recurrent_varlen_with_empty_sequences(gdn):
    # a sequence without tokens produces no output rows and hands its state through unchanged
    lens = [3, 0, 1, 0]
    p = synthetic.varlen_inputs(lens, 2, 4, 128, seed=12)
    pd = dev(p)
    o, s = gdn.recurrent_forward(pd["q"], pd["k"], pd["v"], pd["state"], pd["beta"], pd["g"],
                                 cu_seqlens=pd["cu_seqlens"])
    o_ref, s_ref = O.recurrent_ref(p["q"].float(), p["k"].float(), p["v"].float(), p["beta"].float(), p["g"],
                                   p["state"].float(), cu_seqlens=p["cu_seqlens"])
    close(o, o_ref, "o")
    close(s, s_ref, "state")
    assert torch.equal(s[1], pd["state"][1]) and torch.equal(s[3], pd["state"][3])


def test_recurrent_head_sliced_views(gdn):
    # value-head sharding passes non-contiguous head slices: results must equal the full call
    p = synthetic.decode_inputs(4, 2, 4, 8, 128, seed=13)
    beta_ref, g_ref = O.gating_ref(p["A_log"], p["dt_bias"], p["a"], p["b"])
    pd = dev(p)
    beta, g = beta_ref.bfloat16().cuda(), g_ref.cuda()
    o, s = gdn.recurrent_forward(pd["q"], pd["k"], pd["v"], pd["state"], beta, g, is_qk_norm=True)
    o_h, s_h = gdn.recurrent_forward(pd["q"][:, :, 2:4], pd["k"][:, :, 2:4], pd["v"][:, :, 4:8],
                                     pd["state"][:, 4:8], beta[:, :, 4:8], g[:, :, 4:8], is_qk_norm=True)
    assert torch.equal(o_h, o[:, :, 4:8]) and torch.equal(s_h, s[:, 4:8])


def test_fused_gating(gdn):
    p = synthetic.decode_inputs(7, 3, 2, 32, 64, seed=1)
    for dt in (torch.bfloat16, torch.float32):
        A, dtb, a, b = (p[k].to(dt).cuda() for k in ("A_log", "dt_bias", "a", "b"))
        beta, g = gdn.fused_gdn_gating(A, dtb, a, b)
        beta_ref, g_ref = O.gating_ref(A.cpu(), dtb.cpu(), a.cpu(), b.cpu())
        assert beta.dtype == dt and g.dtype == dt and g.shape == a.shape
        tol = 1e-2 if dt == torch.bfloat16 else 1e-5
        assert torch.allclose(beta.float().cpu(), beta_ref, rtol=tol, atol=tol)
        assert torch.allclose(g.float().cpu(), g_ref, rtol=tol, atol=tol)
    # reference-style call: A_log shaped like a (first vh entries are the per-head values)
    A_full = p["A_log"].float().cuda().expand(7, 3, 32).contiguous()
    beta2, g2 = gdn.fused_gdn_gating(A_full, p["dt_bias"].float().cuda(), p["a"].float().cuda(), p["b"].float().cuda(), False)
    assert torch.allclose(g2.cpu(), O.gating_ref(p["A_log"].float(), p["dt_bias"].float(), p["a"].float(), p["b"].float())[1], rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_chunk_local_cumsum(gdn, dtype):
    B, T, H = 2, 130, 5
    g = (torch.randn(B, T, H) * 0.3).to(dtype)
    ref = O.chunk_local_cumsum_ref(g.float())
    out = torch.empty(B, T, H, dtype=torch.float32, device="cuda")
    gdn.chunk_local_cumsum_bf16(g.cuda(), out, B, T, H, True)
    assert torch.allclose(out.cpu(), ref, atol=1e-4, rtol=1e-3)
    # time-contiguous layout (B*H, T)
    gt = g.permute(0, 2, 1).contiguous()
    out2 = torch.empty(B, H, T, dtype=torch.float32, device="cuda")
    gdn.chunk_local_cumsum_bf16(gt.cuda(), out2, B, T, H, False)
    assert torch.allclose(out2.cpu().permute(0, 2, 1), ref, atol=1e-4, rtol=1e-3)
    # packed
    lens = [1, 63, 64, 65, 130]
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    N = cu[-1]
    gv = (torch.randn(N, H) * 0.3).to(dtype)
    refv = O.chunk_local_cumsum_ref(gv.float(), cu)
    cu_t = torch.tensor(cu, dtype=torch.int32, device="cuda")
    ci = torch.tensor(O.prepare_chunk_indices(cu), dtype=torch.int32, device="cuda")
    outv = torch.empty(N, H, dtype=torch.float32, device="cuda")
    gdn.chunk_local_cumsum_bf16(gv.cuda(), outv, 1, N, H, True, cu_t, ci)
    assert torch.allclose(outv.cpu(), refv, atol=1e-4, rtol=1e-3)
    outv2 = torch.empty(H, N, dtype=torch.float32, device="cuda")
    gdn.chunk_local_cumsum_bf16(gv.t().contiguous().cuda(), outv2, 1, N, H, False, cu_t, ci)
    assert torch.allclose(outv2.cpu().t(), refv, atol=1e-4, rtol=1e-3)


@pytest.mark.parametrize("dtype,shape", [(torch.float32, (2, 130, 5)), (torch.bfloat16, (3, 2, 67, 33)),
                                          (torch.bfloat16, (64, 32))])
def test_transpose_to_mn_major(gdn, dtype, shape):
    x = torch.randn(*shape).to(dtype)
    t = gdn.transpose_to_mn_major(x.cuda())
    ref = O.transpose_mn_major_ref(x)
    assert t.shape == ref.shape and t.stride(-2) == 1
    assert torch.equal(t.cpu(), ref)


def test_errors_raise(gdn):
    p = dev(synthetic.decode_inputs(2, 1, 2, 4, 128, seed=1))
    beta = torch.sigmoid(p["b"].float()).bfloat16()
    with pytest.raises(RuntimeError):
        gdn.recurrent_forward(p["q"].float(), p["k"], p["v"], p["state"], beta, None)
    with pytest.raises(RuntimeError):
        gdn.recurrent_forward(p["q"][:, :, :, ::2], p["k"], p["v"], p["state"], beta, None)
    with pytest.raises(RuntimeError):
        gdn.transpose_to_mn_major(torch.zeros(4, dtype=torch.float32, device="cuda"))


def test_many_multi_token_units_per_cta(gdn):
    """More (sequence, v-head) units than CTAs, with 0 .. 17 tokens each in no particular order: every CTA walks
    several units, some through the once-per-unit token buffer (2 .. 8 tokens), some through the per-tile path
    (1, or 9 and more), some empty; q/k norm on, fp32 and bf16 gates."""
    lens = [(7 * i + 3) % 18 for i in range(220)]
    p = synthetic.varlen_inputs(lens, 2, 4, 128, seed=77, mild_gate=True, normalize=False)
    pd = dev(p)
    for g in (pd["g"], pd["g"].bfloat16()):
        o, s = gdn.recurrent_forward(pd["q"], pd["k"], pd["v"], pd["state"], pd["beta"], g,
                                     cu_seqlens=pd["cu_seqlens"], is_qk_norm=True)
        o_ref, s_ref = O.recurrent_ref(p["q"].float(), p["k"].float(), p["v"].float(), p["beta"].float(), g.float().cpu(),
                                       p["state"].float(), cu_seqlens=p["cu_seqlens"], is_qk_norm=True)
        close(o, o_ref, "o")
        close(s, s_ref, "state")
    # the same launch twice gives the same bits (no stale token buffer between units)
    o2, s2 = gdn.recurrent_forward(pd["q"], pd["k"], pd["v"], pd["state"], pd["beta"], pd["g"].bfloat16(),
                                   cu_seqlens=pd["cu_seqlens"], is_qk_norm=True)
    assert torch.equal(o2, o) and torch.equal(s2, s)
