"""CPU tests of the oracle itself: golden vectors, known answers, internal consistency."""
import glob
import math
import os

import numpy as np
import pytest
import torch

from oracle import gdn_oracle as O
from h100_gdn_cuda_b200 import synthetic

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


PLAIN = sorted(f for f in glob.glob(os.path.join(GOLDEN, "*.npz")) if not os.path.basename(f).startswith("branch_"))


@pytest.mark.parametrize("path", PLAIN)
def test_oracle_matches_golden(path):
    z = np.load(path)
    t = {k: torch.from_numpy(z[k]) for k in z.files if k != "fla_version"}
    o, s = O.recurrent_ref(t["q"], t["k"], t["v"], t["beta"], t["g"], t.get("state"))
    # fp32 vs fp32, different summation order only
    assert (o - t["o"]).abs().max().item() < 2e-6
    assert (s - t["final_state"]).abs().max().item() < 2e-6


def test_golden_present():
    assert len(PLAIN) >= 3


def _load(name):
    z = np.load(os.path.join(GOLDEN, name))
    return {k: torch.from_numpy(z[k]) for k in z.files if k != "fla_version"}


def test_oracle_qk_norm_matches_golden():
    """The fixture holds RAW q, k and the outputs of the third-party recurrence on q, k normalised
    by the generating script: the oracle's own normalisation branch has to reproduce them."""
    t = _load("branch_qknorm_B2_T40_kh2_vh4_d64.npz")
    o, s = O.recurrent_ref(t["q"], t["k"], t["v"], t["beta"], t["g"], t["state"], is_qk_norm=True)
    assert (o - t["o"]).abs().max().item() < 2e-6
    assert (s - t["final_state"]).abs().max().item() < 2e-6
    # and without the flag the answer is a different one (the fixture does exercise the branch)
    o_raw, _ = O.recurrent_ref(t["q"], t["k"], t["v"], t["beta"], t["g"], t["state"])
    assert (o_raw - t["o"]).abs().max().item() > 1e-2


def test_oracle_step_states_and_accept_cap_match_golden():
    """Per-token states (the third-party recurrence called one token at a time) and the accepted-token
    cap: the state after the accepted prefix is the step state of its last token."""
    t = _load("branch_steps_B3_T6_h2_d64.npz")
    o, steps = O.recurrent_ref(t["q"], t["k"], t["v"], t["beta"], t["g"], t["state"], store_step_state=True)
    assert (o - t["o"]).abs().max().item() < 2e-6
    assert (steps - t["step_states"]).abs().max().item() < 2e-6
    acc = [2, 6, 1]
    o_c, s_c = O.recurrent_ref(t["q"], t["k"], t["v"], t["beta"], t["g"], t["state"], num_accepted_tokens=acc)
    for b, a in enumerate(acc):
        assert (s_c[b] - t["step_states"][b, a - 1]).abs().max().item() < 2e-6
        assert (o_c[b, :a] - t["o"][b, :a]).abs().max().item() < 2e-6
        assert o_c[b, a:].abs().max().item() == 0 if a < 6 else True


def test_known_answer_single_step():
    # dk = dv = 2, one head, one token, S0 = 0: S = beta v k^T, o = scale * beta v (k.q)
    q = torch.tensor([[[[1.0, 2.0]]]])
    k = torch.tensor([[[[0.5, -1.0]]]])
    v = torch.tensor([[[[3.0, 4.0]]]])
    beta = torch.tensor([[[0.5]]])
    g = torch.tensor([[[-0.3]]])
    o, s = O.recurrent_ref(q, k, v, beta, g, scale=1.0)
    assert torch.allclose(s[0, 0], 0.5 * torch.outer(v[0, 0, 0], k[0, 0, 0]))
    assert torch.allclose(o[0, 0, 0], 0.5 * v[0, 0, 0] * (0.5 * 1.0 - 1.0 * 2.0))


def test_known_answer_decay_and_delta():
    # second step: S1 = e^g S0 + beta (v - e^g S0 k) k^T, hand-expanded
    S0 = torch.tensor([[[[1.0, 0.0], [0.0, 2.0]]]])
    k = torch.tensor([[[[1.0, 0.0]]]])
    q = torch.tensor([[[[0.0, 1.0]]]])
    v = torch.tensor([[[[1.0, 1.0]]]])
    beta = torch.tensor([[[1.0]]])
    g = torch.tensor([[[math.log(0.5)]]])
    o, s = O.recurrent_ref(q, k, v, beta, g, S0, scale=1.0)
    # e^g S0 = [[.5,0],[0,1]]; S k = [.5, 0]; r = [.5, 1]; S1 = [[.5+.5, 0],[1, 1]]
    assert torch.allclose(s[0, 0], torch.tensor([[1.0, 0.0], [1.0, 1.0]]))
    assert torch.allclose(o[0, 0, 0], torch.tensor([0.0, 1.0]))


def test_default_scale_and_qk_norm():
    p = synthetic.prefill_inputs(1, 5, 2, 2, 64, seed=5, with_state=False, dtype=torch.float32, normalize=False)
    o1, _ = O.recurrent_ref(p["q"], p["k"], p["v"], p["beta"], p["g"], is_qk_norm=True)
    qn, kn = O.l2norm_ref(p["q"]), O.l2norm_ref(p["k"])
    o2, _ = O.recurrent_ref(qn, kn, p["v"], p["beta"], p["g"], scale=1 / 8.0)
    assert torch.allclose(o1, o2, atol=1e-6)


@pytest.mark.parametrize("lens", [[1], [63, 64, 65], [130, 2, 97, 255]])
def test_chunked_stages_equal_recurrence(lens):
    p = synthetic.varlen_inputs(lens, 2, 4, 64, seed=11)
    args = (p["q"], p["k"], p["v"], p["beta"], p["g"], p["state"])
    o, s = O.recurrent_ref(*args, cu_seqlens=p["cu_seqlens"], dtype=torch.float64)
    oc, sc = O.chunked_ref(*args, cu_seqlens=p["cu_seqlens"], dtype=torch.float64)
    assert (o - oc).abs().max().item() < 1e-5
    assert (s - sc).abs().max().item() < 1e-5


def test_chunked_padded_equals_recurrence_partial_tail():
    p = synthetic.prefill_inputs(2, 130, 2, 4, 64, seed=3)
    args = (p["q"], p["k"], p["v"], p["beta"], p["g"], p["state"])
    o, s = O.recurrent_ref(*args, dtype=torch.float64)
    oc, sc = O.chunked_ref(*args, dtype=torch.float64)
    assert (o - oc).abs().max().item() < 1e-5 and (s - sc).abs().max().item() < 1e-5


def test_state_handoff_equals_one_pass():
    p = synthetic.prefill_inputs(1, 100, 2, 2, 64, seed=4)
    a = (p["q"], p["k"], p["v"], p["beta"], p["g"])
    o, s = O.recurrent_ref(*a, p["state"])
    o1, s1 = O.recurrent_ref(*(x[:, :37] for x in a), p["state"])
    o2, s2 = O.recurrent_ref(*(x[:, 37:] for x in a), s1)
    assert torch.allclose(torch.cat([o1, o2], 1), o, atol=1e-6) and torch.allclose(s2, s, atol=1e-6)


def test_num_accepted_and_step_states():
    p = synthetic.decode_inputs(3, 4, 2, 4, 64, seed=7, spec=True, dtype=torch.float32)
    beta, g = O.gating_ref(p["A_log"], p["dt_bias"], p["a"], p["b"])
    nat = p["num_accepted_tokens"]
    o, steps = O.recurrent_ref(p["q"], p["k"], p["v"], beta, g, p["state"], is_qk_norm=True,
                               num_accepted_tokens=nat, store_step_state=True)
    o2, fin = O.recurrent_ref(p["q"], p["k"], p["v"], beta, g, p["state"], is_qk_norm=True,
                              num_accepted_tokens=nat)
    for b in range(3):
        n = int(nat[b])
        assert torch.equal(steps[b, n - 1], fin[b])
        assert (o[b, n:] == 0).all() and (steps[b, n:] == 0).all()
    assert torch.equal(o, o2)


def test_varlen_metadata():
    cu = [0, 1, 64, 129, 129 + 200]
    assert O.prepare_cu_chunks(cu) == [0, 1, 2, 4, 8]
    assert O.prepare_chunk_indices(cu) == [0, 0, 1, 0, 2, 0, 2, 1, 3, 0, 3, 1, 3, 2, 3, 3]
    assert synthetic.prepare_cu_chunks(cu) == O.prepare_cu_chunks(cu)
    assert synthetic.prepare_chunk_indices(cu) == O.prepare_chunk_indices(cu)


def test_gating_ref_values():
    A_log = torch.tensor([0.0, math.log(2.0)])
    dt = torch.tensor([0.0, 0.0])
    a = torch.tensor([[0.0, 30.0]])
    b = torch.tensor([[0.0, 0.0]])
    beta, g = O.gating_ref(A_log, dt, a, b)
    assert torch.allclose(beta, torch.tensor([[0.5, 0.5]]))
    assert torch.allclose(g, torch.tensor([[-math.log(2.0), -60.0]]))


def test_cumsum_and_transpose_ref():
    g = torch.arange(1, 131, dtype=torch.float32).reshape(1, 130, 1)
    c = O.chunk_local_cumsum_ref(g)
    assert c[0, 63, 0] == sum(range(1, 65)) and c[0, 64, 0] == 65 and c[0, 129, 0] == 129 + 130
    x = torch.arange(10, dtype=torch.float32).reshape(1, 5, 2)
    t = O.transpose_mn_major_ref(x, 16)
    assert t.shape == (1, 8, 2) and t.stride(-2) == 1
    assert torch.equal(t[:, :5], x) and (t[:, 5:] == 0).all()


def test_lognormal_lengths_sum():
    lens = synthetic.lognormal_lengths(16, 32768, 64, 8192)
    assert sum(lens) == 32768 and min(lens) >= 64 and max(lens) <= 8192 and len(lens) == 16
