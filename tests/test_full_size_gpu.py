"""GPU parity at the full sizes of the benchmark configurations.

configs[1] padded prefill B=4 T=4096 kh=16 vh=32 d=128 (fp32 gate in the time-contiguous
"MN-major" layout), configs[2] packed prefill of 16 log-normal sequences totalling 32768 tokens,
configs[3] decode B=256 and spec-verify B=64 T=4 with fused gating and qk-norm, and one GPU's
share of configs[4] (B=2, T=131072, 4 of the 32 value heads with their 2 q/k heads).

The first three are compared with the fp32 CPU oracle outright (a few seconds of CPU each).  The
long-context case is too long for a token loop on the CPU, so it is checked through properties:
the chunked kernels against the token-recurrent kernel (a different code path) over the whole
length, the oracle on a prefix (outputs of a prefix depend on that prefix only), and
prefill(T) against prefill(T/2) -> state -> prefill(T/2).
"""
import pytest
import torch

from oracle import gdn_oracle as O
from h100_gdn_cuda_b200 import synthetic

pytestmark = pytest.mark.gpu

REL_FRO, MAX_ABS = 1e-2, 5e-2


def close(x, ref, what, rel=REL_FRO, mx=MAX_ABS):
    x, ref = x.float().cpu(), ref.float().cpu()
    assert torch.isfinite(x).all(), "%s has non-finite values" % what
    rf, ma = O.rel_fro(x, ref), O.max_abs_over_max(x, ref)
    assert rf <= rel and ma <= mx, "%s: rel_fro %.3e max_abs/max %.3e" % (what, rf, ma)


@pytest.fixture(scope="module")
def gdn():
    import h100_gdn_cuda_b200 as g
    from h100_gdn_cuda_b200 import build
    build.build()
    return g


def dev(d):
    return {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in d.items()}


def check_status():
    import ctypes
    from h100_gdn_cuda_b200 import _cabi
    st = ctypes.c_int(0)
    assert _cabi.load().gdn_device_status(torch.cuda.current_device(), ctypes.byref(st)) == 0
    assert st.value == 0, "a kernel reported a bounded wait that ran out (status %d)" % st.value


def time_contiguous(x):
    """(B, T, H) tensor whose memory is (B, H, T): the reference's MN-major scalar layout."""
    return x.transpose(1, 2).contiguous().transpose(1, 2)


def test_config1_padded_prefill_full_size(gdn):
    B, T, kh, vh, d = 4, 4096, 16, 32, 128
    p = synthetic.prefill_inputs(B, T, kh, vh, d, seed=0)
    o_ref, s_ref = O.recurrent_ref(p["q"].float(), p["k"].float(), p["v"].float(), p["beta"].float(), p["g"],
                                   p["state"].float())
    pd = dev(p)
    g_mn, beta_mn = time_contiguous(pd["g"]), time_contiguous(pd["beta"])
    assert g_mn.stride() == (vh * T, 1, T)
    o, s = gdn.chunked_forward(pd["q"], pd["k"], pd["v"], beta_mn, g_mn, None, pd["state"])
    check_status()
    assert o.shape == (B, T, vh, d) and s.shape == (B, vh, d, d)
    close(o, o_ref, "O")
    close(s, s_ref, "final state")
    # the scalar layout does not change a bit of the result
    o2, s2 = gdn.chunked_forward(pd["q"], pd["k"], pd["v"], pd["beta"], pd["g"], None, pd["state"])
    assert torch.equal(o, o2) and torch.equal(s, s2)


def test_config2_packed_prefill_full_size(gdn):
    lens = synthetic.lognormal_lengths(16, 32768, 64, 8192, seed=0)
    assert sum(lens) == 32768 and len(lens) == 16
    p = synthetic.varlen_inputs(lens, 16, 32, 128, seed=1)
    o_ref, s_ref = O.recurrent_ref(p["q"].float(), p["k"].float(), p["v"].float(), p["beta"].float(), p["g"],
                                   p["state"].float(), cu_seqlens=p["cu_seqlens"])
    pd = dev(p)
    o, s = gdn.chunked_forward(pd["q"], pd["k"], pd["v"], pd["beta"], pd["g"], None, pd["state"],
                               pd["cu_seqlens"], pd["chunk_indices"], pd["cu_chunks"], p["total_chunks"])
    check_status()
    assert o.shape == (32768, 32, 128) and s.shape == (16, 32, 128, 128)
    close(o, o_ref, "O")
    close(s, s_ref, "final states")


def test_config3_decode_and_spec_verify_full_size(gdn):
    # plain decode, state updated in place
    B = 256
    p = synthetic.decode_inputs(B, 1, 16, 32, 128, seed=3)
    pd = dev(p)
    beta, g = gdn.fused_gdn_gating(pd["A_log"], pd["dt_bias"], pd["a"], pd["b"])
    beta_ref, g_ref = O.gating_ref(p["A_log"], p["dt_bias"], p["a"], p["b"])
    close(beta, beta_ref, "beta")
    close(g, g_ref, "gate")
    o_ref, s_ref = O.recurrent_ref(p["q"].float(), p["k"].float(), p["v"].float(), beta.float().cpu(),
                                   g.float().cpu(), p["state"].float(), is_qk_norm=True)
    state = pd["state"].clone()
    o, s = gdn.recurrent_forward(pd["q"], pd["k"], pd["v"], state, beta, g, inference_mode=1, is_qk_norm=True,
                                 inplace_state=True)
    check_status()
    assert s.data_ptr() == state.data_ptr()
    close(o, o_ref, "decode O")
    close(s, s_ref, "decode state")
    # spec-verify: one state per token, and the accepted-token cap in decode mode
    B, T = 64, 4
    p = synthetic.decode_inputs(B, T, 16, 32, 128, seed=4, spec=True)
    pd = dev(p)
    beta, g = gdn.fused_gdn_gating(pd["A_log"], pd["dt_bias"], pd["a"], pd["b"])
    common = (p["q"].float(), p["k"].float(), p["v"].float(), beta.float().cpu(), g.float().cpu(), p["state"].float())
    o, steps = gdn.recurrent_forward(pd["q"], pd["k"], pd["v"], pd["state"], beta, g,
                                     inference_mode=gdn.SpecVerify, is_qk_norm=True)
    o_ref, steps_ref = O.recurrent_ref(*common, is_qk_norm=True, store_step_state=True)
    check_status()
    assert steps.shape == (B, T, 32, 128, 128)
    close(o, o_ref, "spec O")
    close(steps, steps_ref, "step states")
    nat = p["num_accepted_tokens"]
    o, s = gdn.recurrent_forward(pd["q"], pd["k"], pd["v"], pd["state"], beta, g, num_accepted_tokens=pd["num_accepted_tokens"],
                                 inference_mode=1, is_qk_norm=True)
    o_ref, s_ref = O.recurrent_ref(*common, is_qk_norm=True, num_accepted_tokens=nat)
    mask = torch.arange(T)[None, :] < nat[:, None]
    close(o.float().cpu()[mask], o_ref[mask], "O of accepted tokens")
    close(s, s_ref, "state after the accepted prefix")


def test_config4_long_context_one_gpu_share(gdn):
    B, T, kh, vh, d = 2, 131072, 2, 4, 128   # one GPU's value heads of the 8-way head sharding
    p = synthetic.prefill_inputs(B, T, kh, vh, d, seed=5)
    pd = dev(p)
    a = [pd[k] for k in ("q", "k", "v", "beta", "g")]
    o, s = gdn.chunked_forward(*a, None, pd["state"])
    check_status()
    assert o.shape == (B, T, vh, d)
    # (1) the oracle on a prefix
    n = 2048
    o_ref, _ = O.recurrent_ref(p["q"][:, :n].float(), p["k"][:, :n].float(), p["v"][:, :n].float(),
                               p["beta"][:, :n].float(), p["g"][:, :n], p["state"].float())
    close(o[:, :n], o_ref, "O of the prefix")
    # (2) the token-recurrent kernel over the whole length (a different code path, fp32 state throughout)
    o_rec, s_rec = gdn.recurrent_forward(*a[:3], pd["state"], a[3], a[4], inference_mode=0)
    check_status()
    close(o, o_rec, "O vs the recurrent kernel")
    close(s, s_rec, "final state vs the recurrent kernel")
    # (2b) the oracle over ALL 131072 tokens of one (sequence, v-head) chain: an independent check of every
    # segment of the segmented state propagation (tens of seconds of CPU work)
    b, h = 1, 3
    kk = h // (vh // kh)
    o_1, s_1 = O.recurrent_ref(p["q"][b:b + 1, :, kk:kk + 1].float(), p["k"][b:b + 1, :, kk:kk + 1].float(),
                               p["v"][b:b + 1, :, h:h + 1].float(), p["beta"][b:b + 1, :, h:h + 1].float(),
                               p["g"][b:b + 1, :, h:h + 1], p["state"][b:b + 1, h:h + 1].float())
    close(o[b:b + 1, :, h:h + 1], o_1, "O of one chain over the whole length")
    for lo in range(0, T, T // 16):   # and segment by segment, so that a late deviation cannot hide in the norm
        close(o[b:b + 1, lo:lo + T // 16, h:h + 1], o_1[:, lo:lo + T // 16], "O of tokens %d.." % lo)
    close(s[b:b + 1, h:h + 1], s_1, "final state of one chain")
    # (3) two halves with the state handed over (the hand-over rounds the state to bf16 once)
    h = T // 2
    o1, s1 = gdn.chunked_forward(*(x[:, :h] for x in a), None, pd["state"])
    o2, s2 = gdn.chunked_forward(*(x[:, h:] for x in a), None, s1)
    assert torch.equal(o1, o[:, :h])
    close(o2, o[:, h:], "second half after the hand-over")
    close(s2, s, "final state after the hand-over")
