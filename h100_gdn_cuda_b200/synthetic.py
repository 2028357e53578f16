"""Seeded synthetic inputs for the benchmark configurations (CPU tensors).

Self-contained: the gating and normalisation formulas used to draw the inputs
are restated here so that the benchmark's GPU arm does not touch the oracle.

Distributions: q,k ~ N(0,1) L2-normalised per head (or raw N(0,1) when the
kernel normalises); v ~ N(0,1); beta = sigmoid(N(0,1));
g = -exp(A_log) * softplus(a + dt_bias) with A_log = log U(1,16), a ~ N(0,1),
dt_bias ~ N(0,0.1); initial state ~ N(0,0.02).  One torch.Generator per call,
draws in a fixed order, generated in fp32 then cast.
"""
from __future__ import annotations

import math
from typing import Optional

import torch



def l2norm_ref(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + eps)


def gating_ref(A_log, dt_bias, a, b):
    """beta = sigmoid(b), g = -exp(A_log) * softplus(a + dt_bias) in fp32."""
    x = a.float() + dt_bias.float()
    return torch.sigmoid(b.float()), -torch.exp(A_log.float()) * torch.nn.functional.softplus(x)


def prepare_cu_chunks(cu, chunk: int = 64):
    out = [0]
    for s in range(len(cu) - 1):
        out.append(out[-1] + (int(cu[s + 1]) - int(cu[s]) + chunk - 1) // chunk)
    return out


def prepare_chunk_indices(cu, chunk: int = 64):
    out = []
    for s in range(len(cu) - 1):
        for c in range((int(cu[s + 1]) - int(cu[s]) + chunk - 1) // chunk):
            out += [s, c]
    return out


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator()
    g.manual_seed(seed)
    return g


def gate_params(gen, lead_shape, vh):
    A_log = torch.log(torch.rand(vh, generator=gen) * 15.0 + 1.0)
    a = torch.randn(*lead_shape, vh, generator=gen)
    dt_bias = torch.randn(vh, generator=gen) * 0.1
    b = torch.randn(*lead_shape, vh, generator=gen)
    return A_log, dt_bias, a, b


def prefill_inputs(B: int, T: int, kh: int, vh: int, d: int, seed: int = 0,
                   with_state: bool = True, state_std: float = 0.02, dtype=torch.bfloat16,
                   normalize: bool = True, mild_gate: bool = False):
    """Padded prefill inputs: q,k (B,T,kh,d), v (B,T,vh,d), beta (B,T,vh) in
    `dtype`, g (B,T,vh) fp32, state (B,vh,d,d) in `dtype` or None."""
    gen = _gen(seed)
    q = torch.randn(B, T, kh, d, generator=gen)
    k = torch.randn(B, T, kh, d, generator=gen)
    if normalize:
        q, k = l2norm_ref(q), l2norm_ref(k)
    v = torch.randn(B, T, vh, d, generator=gen)
    A_log, dt_bias, a, b = gate_params(gen, (B, T), vh)
    beta, g = gating_ref(A_log, dt_bias, a, b)
    if mild_gate:
        g = g * 0.02
    S0 = (torch.randn(B, vh, d, d, generator=gen) * state_std).to(dtype) if with_state else None
    return dict(q=q.to(dtype), k=k.to(dtype), v=v.to(dtype), beta=beta.to(dtype),
                g=g.float().contiguous(), state=S0)


def lognormal_lengths(num_seqs: int, total: int, lo: int, hi: int, seed: int = 0):
    """`num_seqs` lengths ~ lognormal(7,1) clipped to [lo,hi], rescaled to sum
    to `total` (remainder fixed on the longest, re-clipped)."""
    gen = _gen(seed)
    x = torch.exp(torch.randn(num_seqs, generator=gen) + 7.0).clamp(lo, hi)
    lens = [max(lo, min(hi, int(round(float(v) * total / float(x.sum()))))) for v in x]
    for _ in range(64):
        diff = total - sum(lens)
        if diff == 0:
            break
        order = sorted(range(num_seqs), key=lambda i: -lens[i])
        for i in order:
            step = max(lo - lens[i], min(hi - lens[i], diff))
            lens[i] += step
            diff -= step
            if diff == 0:
                break
    assert sum(lens) == total, (lens, total)
    return lens


def varlen_inputs(lens, kh: int, vh: int, d: int, seed: int = 0, with_state: bool = True,
                  dtype=torch.bfloat16, mild_gate: bool = False, normalize: bool = True):
    N = sum(lens)
    p = prefill_inputs(1, N, kh, vh, d, seed, with_state=False, dtype=dtype, mild_gate=mild_gate, normalize=normalize)
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    gen = _gen(seed + 1)
    S0 = (torch.randn(len(lens), vh, d, d, generator=gen) * 0.02).to(dtype) if with_state else None
    ci = prepare_chunk_indices(cu)
    cc = prepare_cu_chunks(cu)
    return dict(q=p["q"][0], k=p["k"][0], v=p["v"][0], beta=p["beta"][0], g=p["g"][0], state=S0,
                cu_seqlens=torch.tensor(cu, dtype=torch.int32),
                chunk_indices=torch.tensor(ci, dtype=torch.int32),
                cu_chunks=torch.tensor(cc, dtype=torch.int32), total_chunks=cc[-1])


def decode_inputs(B: int, T: int, kh: int, vh: int, d: int, seed: int = 0, dtype=torch.bfloat16,
                  spec: bool = False):
    """Raw (un-normalised) q,k ~ N(0,1); gate parameters for fused_gdn_gating;
    state (B,vh,d,d) ~ N(0,0.02).  With `spec`, num_accepted_tokens ~ U{1..T}."""
    gen = _gen(seed)
    q = torch.randn(B, T, kh, d, generator=gen)
    k = torch.randn(B, T, kh, d, generator=gen)
    v = torch.randn(B, T, vh, d, generator=gen)
    A_log, dt_bias, a, b = gate_params(gen, (B, T), vh)
    S0 = torch.randn(B, vh, d, d, generator=gen) * 0.02
    out = dict(q=q.to(dtype), k=k.to(dtype), v=v.to(dtype), A_log=A_log.to(dtype),
               dt_bias=dt_bias.to(dtype), a=a.to(dtype), b=b.to(dtype), state=S0.to(dtype))
    if spec:
        out["num_accepted_tokens"] = torch.randint(1, T + 1, (B,), generator=gen, dtype=torch.int32)
    return out
