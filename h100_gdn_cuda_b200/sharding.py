"""Sharding of the Gated DeltaNet layer over the GPUs of one box.

The recurrence is independent per sequence and per value head (a v-head only needs the
q/k of its own k-head), so the layer shards with no exchange step inside it:

* by value head: rank r takes a contiguous group of vh/G v-heads and the kh/G k-heads they
  use (G must divide kh so that groups stay aligned);
* by sequence: rank r takes a contiguous block of the batch.

The functions here only compute index ranges and slice views; every rank then calls the
unchanged single-GPU API on its slice (strided head slices are accepted as they are).
Outputs are concatenated on the sharded axis; a collective is needed only by callers that
want the full result on every rank.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch


def head_shard(rank: int, world: int, num_k_heads: int, num_v_heads: int) -> Tuple[slice, slice]:
    """(k-head slice, v-head slice) of `rank` for value-head sharding."""
    if num_k_heads % world != 0:
        raise ValueError("world size %d must divide num_k_heads %d" % (world, num_k_heads))
    if num_v_heads % num_k_heads != 0:
        raise ValueError("num_v_heads must be a multiple of num_k_heads")
    kper = num_k_heads // world
    rep = num_v_heads // num_k_heads
    ks = slice(rank * kper, (rank + 1) * kper)
    vs = slice(rank * kper * rep, (rank + 1) * kper * rep)
    return ks, vs


def seq_shard(rank: int, world: int, batch: int) -> slice:
    """Contiguous block of sequences of `rank` (blocks differ by at most one sequence)."""
    base, extra = divmod(batch, world)
    lo = rank * base + min(rank, extra)
    return slice(lo, lo + base + (1 if rank < extra else 0))


def shard_prefill_by_head(t: Dict[str, torch.Tensor], rank: int, world: int) -> Dict[str, torch.Tensor]:
    """Views of padded prefill inputs (q,k: (B,T,kh,d); v: (B,T,vh,d); beta,g: (B,T,vh);
    state: (B,vh,d,d)) for `rank` under value-head sharding.  No copies."""
    ks, vs = head_shard(rank, world, t["q"].shape[2], t["v"].shape[2])
    out = dict(q=t["q"][:, :, ks], k=t["k"][:, :, ks], v=t["v"][:, :, vs], beta=t["beta"][:, :, vs],
               g=t["g"][:, :, vs])
    out["state"] = None if t.get("state") is None else t["state"][:, vs]
    return out


def shard_by_sequence(t: Dict[str, torch.Tensor], rank: int, world: int) -> Dict[str, torch.Tensor]:
    """Views of padded inputs whose leading axis is the batch, for `rank` under sequence sharding."""
    any_t = next(v for v in t.values() if torch.is_tensor(v))
    sl = seq_shard(rank, world, any_t.shape[0])
    return {k: (v[sl] if torch.is_tensor(v) else v) for k, v in t.items()}
