"""Multi-rank sharding logic on CPU: world_size-2 gloo ranks each take their shard (by value head
and by sequence), compute it with the oracle (there is no GPU here), gather, and the
assembled result must equal the unsharded computation (to fp32 summation-order noise: the
oracle batches its einsums over whatever it is given)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from h100_gdn_cuda_b200 import sharding, synthetic
from oracle import gdn_oracle as O


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        p = synthetic.prefill_inputs(2, 70, 2, 4, 64, seed=0, dtype=torch.float32)
        o_full, s_full = O.recurrent_ref(p["q"], p["k"], p["v"], p["beta"], p["g"], p["state"])
        # --- by value head
        sh = sharding.shard_prefill_by_head(p, rank, world)
        o, s = O.recurrent_ref(sh["q"], sh["k"], sh["v"], sh["beta"], sh["g"], sh["state"])
        outs = [torch.empty_like(o) for _ in range(world)]
        sts = [torch.empty_like(s) for _ in range(world)]
        dist.all_gather(outs, o.contiguous())
        dist.all_gather(sts, s.contiguous())
        ok_head = torch.allclose(torch.cat(outs, dim=2), o_full, atol=1e-6) and torch.allclose(torch.cat(sts, dim=1), s_full, atol=1e-6)
        # --- by sequence
        sq = sharding.shard_by_sequence(p, rank, world)
        o2, s2 = O.recurrent_ref(sq["q"], sq["k"], sq["v"], sq["beta"], sq["g"], sq["state"])
        outs = [torch.empty_like(o2) for _ in range(world)]
        sts = [torch.empty_like(s2) for _ in range(world)]
        dist.all_gather(outs, o2.contiguous())
        dist.all_gather(sts, s2.contiguous())
        ok_seq = torch.allclose(torch.cat(outs, dim=0), o_full, atol=1e-6) and torch.allclose(torch.cat(sts, dim=0), s_full, atol=1e-6)
        # timing reduction used by the benchmark: max over ranks
        t = torch.tensor([float(rank + 1)])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ret[rank] = (ok_head, ok_seq, float(t.item()))
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding_matches_unsharded():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    for r in range(world):
        ok_head, ok_seq, tmax = ret[r]
        assert ok_head and ok_seq and tmax == float(world)


def test_shard_ranges():
    assert sharding.head_shard(3, 8, 16, 32) == (slice(6, 8), slice(12, 16))
    assert [sharding.seq_shard(r, 4, 10) for r in range(4)] == [slice(0, 3), slice(3, 6), slice(6, 8), slice(8, 10)]
    with pytest.raises(ValueError):
        sharding.head_shard(0, 3, 16, 32)
