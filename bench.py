#!/usr/bin/env python
"""Benchmark of the Gated DeltaNet hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one pass of chunked prefill (`chunked_forward`) over one batch of the padded
prefill configuration: B=4, T=4096, kh=16, vh=32, dk=dv=128, bf16 q/k/v/beta, fp32 gate, bf16
initial state (synthetic, seeded).  With N > 1 (launched under torchrun, one rank per GPU)
every rank processes its own batch of that size - sequences are independent, so the path
shards by sequence with no collective - and `value` is the total over ranks (weak scaling).

The printed JSON line carries:
  value      prefill tokens/s with inputs resident in HBM (CUDA events, max over ranks)
  e2e        the same through the public API from pinned HOST buffers: host->device copies of
             q, k, v, beta, gate and the state and the device->host copy of O and the final
             state are inside the timed region
  roofline   for the dominant kernel (the longer of the two prefill launches), timed live with CUDA
             events, against the HBM roof that bounds both of them
  decode     decode tokens/s of `recurrent_forward` (B=256, T=1, qk-norm, fused gating) and its
             HBM roofline fraction
  packed     packed (varlen) prefill of 16 sequences with log-normal lengths, 32768 tokens per GPU
  long_context  the B=2, T=131072 layer with the value heads sharded over the N ranks (strong scaling)
  cpu_baseline  the fp32 CPU token recurrence (the oracle) on a bounded sample, rank 0, N=1

`--impl reference` times only that CPU recurrence (the reference library's own sm_90a kernels
cannot run on a B200 and it has no CPU path).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG = dict(B=4, T=4096, kh=16, vh=32, d=128)
DECODE = dict(B=256, T=1, kh=16, vh=32, d=128)
CHUNK = 64
WORKLOAD = "padded chunked prefill B=4 T=4096 kh=16 vh=32 dk=dv=128 chunk=64 per GPU"


def flops_per_unit(d: int, c: int = CHUNK) -> float:
    """All contractions of one (64-token chunk, v-head): 2C(5Cd + 3dd) + (2/3)C^3."""
    return 2.0 * c * (5 * c * d + 3 * d * d) + (2.0 / 3.0) * c ** 3


def seq_kernel_flops_per_unit(d: int, c: int = CHUNK) -> float:
    """Contractions done by the state/output kernel: P U_new (2CCd) and
    W S^T, Q S^T, U_new^T K (2Cdd each)."""
    return 2.0 * c * (c * d + 3 * d * d)


def uw_kernel_flops_per_unit(d: int, c: int = CHUNK) -> float:
    """K K^T, Q K^T, T V, T' K (2CCd each) and the triangular inverse."""
    return 2.0 * c * (4 * c * d) + (2.0 / 3.0) * c ** 3


# Algorithmic HBM bytes of the two prefill kernels per (64-token chunk, v-head) unit at d = 128:
#   gdn_uw_kernel        : K, Q tiles 16 KB each per k-head (shared by the vh/kh v-heads of a group),
#                          V tile 16 KB in; U, W 16 KB each and P 8 KB out
#   gdn_fused_seq_kernel : U, W, P 40 KB and K, Q (shared as above) in; O 16 KB out
# Both sit well below the ridge of the measured peaks (1636 TFLOP/s / 6546 GB/s = 250 FLOP/B):
# 4.37 MFLOP / 72 KB = 61 FLOP/B and 7.34 MFLOP / 72 KB = 102 FLOP/B at vh/kh = 2, so HBM is the
# roof that bounds them.
def uw_kernel_bytes_per_unit(kh: int, vh: int, d: int, c: int = CHUNK) -> float:
    tile = c * d * 2
    return 2 * tile * kh / vh + tile + 2 * tile + c * c * 2


def seq_kernel_bytes_per_unit(kh: int, vh: int, d: int, c: int = CHUNK) -> float:
    tile = c * d * 2
    return 2 * tile + c * c * 2 + 2 * tile * kh / vh + tile


# DRAM read + write bytes per launch seen by one ncu capture (dram__bytes_read.sum +
# dram__bytes_write.sum), divided by the units that launch processed.  Traffic is proportional
# to the units (every CTA streams its own tiles), so a full launch is units x this figure.
#   gdn_uw_kernel        : B=2 T=4096 vh=32 capture, 135.84 MB read + 116.15 MB written, 4096 units
#   gdn_fused_seq_kernel : same capture, 238.15 MB read + 50.26 MB written, 4096 units
#   gdn_recurrent_kernel : B=128 capture, 136.37 MB read + 87.44 MB written, 128 sequence-tokens
# (written data still in L2 when a launch ends is not counted by the DRAM counters)
NCU_UW_TRAFFIC_PER_UNIT = (135.840512e6 + 116.147456e6) / 4096
NCU_FUSED_TRAFFIC_PER_UNIT = (238.145280e6 + 50.258944e6) / 4096
NCU_DECODE_TRAFFIC_PER_TOKEN = (136.370432e6 + 87.435776e6) / 128


def decode_bytes_per_token(kh, vh, d) -> float:
    return vh * (2 * d * d * 2) + 2 * (2 * kh * d + 2 * vh * d) + vh * 4


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], tflops=p["bf16_tflops"], tflops_sustained=p["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, tflops=1590.0, tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx = float(f[2])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return dict(sm_mhz=sm[len(sm) // 2] if sm else None, sm_max_mhz=mx, reasons=sorted(reasons),
                    samples=len(sm))


def cpu_recurrence_tokens_per_s(sample_tokens: int, repeats: int = 1):
    """fp32 CPU token recurrence (the oracle) on one sequence of `sample_tokens` tokens of the
    prefill configuration; returns (tokens/s, threads, description)."""
    from oracle import gdn_oracle as O
    from h100_gdn_cuda_b200 import synthetic
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    p = synthetic.prefill_inputs(1, sample_tokens, CFG["kh"], CFG["vh"], CFG["d"], seed=0)
    args = [p[k].float() for k in ("q", "k", "v", "beta")] + [p["g"], p["state"].float()]
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        O.recurrent_ref(*args)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return sample_tokens / best, threads, "B=1 x T=%d of the prefill config (kh=16, vh=32, d=128), fp32 torch" % sample_tokens


def run_reference(args):
    """The reference arm: the CPU recurrence, the only implementation of the path that can run
    on this box (rank 0 only)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample = 1024
    from oracle import gdn_oracle as O
    from h100_gdn_cuda_b200 import synthetic
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    p = synthetic.prefill_inputs(1, sample, CFG["kh"], CFG["vh"], CFG["d"], seed=0)
    a = [p[k].float() for k in ("q", "k", "v", "beta")] + [p["g"], p["state"].float()]
    for _ in range(args.warmup):
        O.recurrent_ref(*a)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        O.recurrent_ref(*a)
    dt = (time.perf_counter() - t0) / args.steps
    tps = sample / dt
    line = {
        "impl": "reference", "metric": "prefill_tokens_per_s", "value": tps, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sharding": "rank 0 only", "l2": "not applicable (CPU)"},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port",
                         "sample": "each step = B=1 x T=%d of the prefill config, fp32 torch token recurrence" % sample},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_only(args, gdn, synthetic, dev, peaks):
    """Small single-path runs for profiler captures (few launches, a few hundred MB)."""
    kh, vh, d = CFG["kh"], CFG["vh"], CFG["d"]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if args.only == "prefill":
        B, T = args.batch or 2, CFG["T"]
        p = synthetic.prefill_inputs(B, T, kh, vh, d, seed=0)
        t = {k: p[k].to(dev) for k in ("q", "k", "v", "beta", "g", "state")}
        run = lambda i: gdn.chunked_forward(t["q"], t["k"], t["v"], t["beta"], t["g"], None, t["state"])
        work, unit = B * T, "tokens/s"
    elif args.only == "long":
        # one GPU's share of the long-context configuration: B=2, T=131072, `--heads` v-heads
        B, T, lvh = args.batch or 2, 131072, args.heads or 4
        lkh = max(1, lvh * kh // vh)
        gen = torch.Generator(device=dev).manual_seed(7)
        t = {"q": torch.nn.functional.normalize(torch.randn(B, T, lkh, d, device=dev, generator=gen), dim=-1).bfloat16(),
             "k": torch.nn.functional.normalize(torch.randn(B, T, lkh, d, device=dev, generator=gen), dim=-1).bfloat16(),
             "v": torch.randn(B, T, lvh, d, device=dev, generator=gen).bfloat16(),
             "beta": torch.sigmoid(torch.randn(B, T, lvh, device=dev, generator=gen)).bfloat16(),
             "g": -torch.nn.functional.softplus(torch.randn(B, T, lvh, device=dev, generator=gen)) * 0.1,
             "state": (torch.randn(B, lvh, d, d, device=dev, generator=gen) * 0.02).bfloat16()}
        ws = torch.empty(gdn.api.chunked_forward_workspace_bytes(B, T, lvh), dtype=torch.uint8, device=dev)
        run = lambda i: gdn.chunked_forward(t["q"], t["k"], t["v"], t["beta"], t["g"], None, t["state"], _workspace=ws)
        work, unit = B * T, "tokens/s"
    elif args.only == "packed":
        # 16 sequences of log-normal lengths in one packed batch of 32768 tokens
        lens = synthetic.lognormal_lengths(16, 32768, 64, 8192, seed=0)
        p = synthetic.varlen_inputs(lens, kh, vh, d, seed=200)
        t = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in p.items()}
        run = lambda i: gdn.chunked_forward(t["q"], t["k"], t["v"], t["beta"], t["g"], None, t["state"], t["cu_seqlens"],
                                            t["chunk_indices"], t["cu_chunks"], p["total_chunks"])
        B, work, unit = len(lens), sum(lens), "tokens/s"
    else:
        B = args.batch or 128
        p = synthetic.decode_inputs(B, 1, kh, vh, d, seed=0)
        t = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in p.items()}
        beta, gate = gdn.fused_gdn_gating(t["A_log"], t["dt_bias"], t["a"], t["b"])
        states = [t["state"], t["state"].clone()]
        run = lambda i: gdn.recurrent_forward(t["q"], t["k"], t["v"], states[i & 1], beta, gate, inference_mode=1,
                                              is_qk_norm=True)
        work, unit = B, "tokens/s"
    for i in range(args.warmup):
        run(i)
    torch.cuda.synchronize()
    e0.record()
    for i in range(args.steps):
        run(i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    print(json.dumps({"only": args.only, "batch": B, "ms_per_step": ms, "value": work / (ms * 1e-3), "unit": unit,
                      "steps": args.steps, "warmup": args.warmup}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-long-context", action="store_true", help="skip the B=2 T=131072 head-sharded leg")
    ap.add_argument("--no-packed", action="store_true", help="skip the packed (varlen) prefill leg")
    ap.add_argument("--only", default=None, choices=["prefill", "decode", "long", "packed"],
                    help="profiling aid: run only this path, resident inputs, reduced JSON line")
    ap.add_argument("--batch", type=int, default=None, help="with --only: override the batch size")
    ap.add_argument("--heads", type=int, default=None, help="with --only long: v-heads of this GPU's share (default 4)")
    args = ap.parse_args()
    if args.only is None:
        args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        return run_reference(args)

    import h100_gdn_cuda_b200 as gdn
    from h100_gdn_cuda_b200 import build, synthetic
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
    torch.cuda.set_device(local)
    if world > 1:
        # NCCL prints a version banner on stdout when it initialises; stdout must carry the one JSON
        # line only, so it points at stderr until the first collective has run.
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if rank == 0:
        build.build()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        os.dup2(saved_stdout, 1)
        os.close(saved_stdout)
    gdn.init(ROOT, os.environ.get("CUDA_HOME", "/usr/local/cuda"))
    peaks = load_peaks()
    dev = torch.device("cuda", local)

    B, T, kh, vh, d = (CFG[k] for k in ("B", "T", "kh", "vh", "d"))
    if args.only is not None:
        return run_only(args, gdn, synthetic, dev, peaks)
    p = synthetic.prefill_inputs(B, T, kh, vh, d, seed=rank)
    host = {k: p[k].pin_memory() for k in ("q", "k", "v", "beta", "g", "state")}
    devt = {k: v.to(dev) for k, v in host.items()}
    tokens = B * T
    units = B * ((T + CHUNK - 1) // CHUNK) * vh

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    from h100_gdn_cuda_b200 import api as gdn_api
    ws = torch.empty(gdn_api.chunked_forward_workspace_bytes(B, T, vh), dtype=torch.uint8, device=dev)
    stage_ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    for e in stage_ev:
        e.record()

    def step_resident(events=None):
        return gdn.chunked_forward(devt["q"], devt["k"], devt["v"], devt["beta"], devt["g"], None, devt["state"],
                                   _workspace=ws, _stage_events=events)

    # ---------------- device-resident timing (inputs 0.4 GB per step: larger than the 126 MB L2)
    for _ in range(args.warmup):
        step_resident()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    uw_ms, seq_ms = 0.0, 0.0
    e0.record()
    for _ in range(args.steps):
        step_resident()
    e1.record()
    barrier()
    ms_res = max_over_ranks(e0.elapsed_time(e1) / args.steps)
    # per-kernel durations: same steps again with events between the two kernels
    for _ in range(args.steps):
        step_resident(stage_ev)
        torch.cuda.synchronize()
        uw_ms += stage_ev[0].elapsed_time(stage_ev[1])
        seq_ms += stage_ev[1].elapsed_time(stage_ev[2])
    uw_ms /= args.steps
    seq_ms /= args.steps

    # ---------------- end to end from host buffers
    out_host = torch.empty(B, T, vh, d, dtype=torch.bfloat16).pin_memory()
    st_host = torch.empty(B, vh, d, d, dtype=torch.bfloat16).pin_memory()
    # Three streams (host->device, compute, device->host) and two sets of device staging buffers:
    # every step still copies all of its inputs in and its results out, but the copies of
    # neighbouring steps overlap the kernels and each other (PCIe is full duplex).
    stages = [{k: torch.empty_like(v) for k, v in devt.items()} for _ in range(2)]
    s_in, s_out, s_main = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]   # compute that read staging set i has finished
    ev_out = torch.cuda.Event()
    for e in ev_done:
        e.record(s_main)
    step_no = [0]

    def step_e2e():
        i = step_no[0] & 1
        step_no[0] += 1
        st = stages[i]
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_done[i])
            for k in ("q", "k", "v", "beta", "g", "state"):
                st[k].copy_(host[k], non_blocking=True)
            ev_in[i].record(s_in)
        s_main.wait_event(ev_in[i])
        o, s = gdn.chunked_forward(st["q"], st["k"], st["v"], st["beta"], st["g"], None, st["state"], _workspace=ws)
        ev_done[i].record(s_main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_done[i])
            out_host.copy_(o, non_blocking=True)
            st_host.copy_(s, non_blocking=True)
            o.record_stream(s_out)
            s.record_stream(s_out)
            ev_out.record(s_out)

    for _ in range(3):
        step_e2e()
    s_main.wait_event(ev_out)
    barrier()
    e2e_steps = max(4, min(args.steps, 10))
    e0.record()
    for _ in range(e2e_steps):
        step_e2e()
    s_main.wait_event(ev_out)
    e1.record()
    barrier()
    ms_e2e = max_over_ranks(e0.elapsed_time(e1) / e2e_steps)
    h2d = sum(host[k].numel() * host[k].element_size() for k in host)
    d2h = out_host.numel() * 2 + st_host.numel() * 2

    # ---------------- decode (B=256, T=1): state 268 MB per step, larger than L2
    dB = DECODE["B"]
    dp = synthetic.decode_inputs(dB, 1, kh, vh, d, seed=100 + rank)
    dd = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in dp.items()}
    states = [dd["state"].clone() for _ in range(2)]

    def step_decode(i):
        beta, gate = gdn.fused_gdn_gating(dd["A_log"], dd["dt_bias"], dd["a"], dd["b"])
        return gdn.recurrent_forward(dd["q"], dd["k"], dd["v"], states[i & 1], beta, gate, inference_mode=1,
                                     is_qk_norm=True)

    for i in range(5):
        step_decode(i)
    barrier()
    dsteps = max(args.steps, 20)
    e0.record()
    for i in range(dsteps):
        step_decode(i)
    e1.record()
    barrier()
    ms_dec = max_over_ranks(e0.elapsed_time(e1) / dsteps)
    # the recurrent kernel alone (gating excluded) for its roofline
    beta, gate = gdn.fused_gdn_gating(dd["A_log"], dd["dt_bias"], dd["a"], dd["b"])
    torch.cuda.synchronize()
    e0.record()
    for i in range(dsteps):
        gdn.recurrent_forward(dd["q"], dd["k"], dd["v"], states[i & 1], beta, gate, inference_mode=1, is_qk_norm=True)
    e1.record()
    torch.cuda.synchronize()
    ms_dec_kernel = e0.elapsed_time(e1) / dsteps
    # ---------------- packed prefill: 16 sequences of log-normal lengths, 32768 tokens per rank
    pk = None
    if not args.no_packed:
        lens = synthetic.lognormal_lengths(16, 32768, 64, 8192, seed=rank)
        pp = synthetic.varlen_inputs(lens, kh, vh, d, seed=200 + rank)
        pd = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in pp.items()}
        pws = torch.empty(gdn.api.chunked_forward_workspace_bytes(len(lens), 0, vh, total_tokens=sum(lens),
                                                                  total_chunks=pp["total_chunks"], packed=True),
                          dtype=torch.uint8, device=dev)
        pev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        for e in pev:
            e.record()

        def step_packed(events=None):
            return gdn.chunked_forward(pd["q"], pd["k"], pd["v"], pd["beta"], pd["g"], None, pd["state"], pd["cu_seqlens"],
                                       pd["chunk_indices"], pd["cu_chunks"], pp["total_chunks"], _workspace=pws,
                                       _stage_events=events)
        for _ in range(3):
            step_packed()
        barrier()
        psteps = 10
        e0.record()
        for _ in range(psteps):
            step_packed()
        e1.record()
        barrier()
        ms_pk = max_over_ranks(e0.elapsed_time(e1) / psteps)
        step_packed(pev)
        torch.cuda.synchronize()
        pk = {"metric": "prefill_tokens_per_s", "value": world * sum(lens) / (ms_pk * 1e-3), "unit": "tokens/s",
              "config": "packed: 16 sequences of log-normal lengths (%d ... %d tokens), %d tokens per GPU, kh=16 vh=32 d=128"
                        % (min(lens), max(lens), sum(lens)),
              "ms_per_step": ms_pk, "gdn_uw_kernel_ms": pev[0].elapsed_time(pev[1]),
              "gdn_fused_seq_kernel_ms": pev[1].elapsed_time(pev[2])}
        del pd, pws
    # ---------------- long context: B=2, T=131072, the 32 value heads sharded over the ranks
    # (each rank takes vh / world v-heads with their q/k heads; no collective).  Strong scaling:
    # every rank works on the same two sequences, the layer's time is the slowest rank's.
    lc = None
    if not args.no_long_context and vh % world == 0 and kh % world == 0:
        lB, lT, lvh, lkh = 2, 131072, vh // world, kh // world
        gen = torch.Generator(device=dev).manual_seed(7 + rank)
        lq = torch.nn.functional.normalize(torch.randn(lB, lT, lkh, d, device=dev, generator=gen), dim=-1).bfloat16()
        lk = torch.nn.functional.normalize(torch.randn(lB, lT, lkh, d, device=dev, generator=gen), dim=-1).bfloat16()
        lv = torch.randn(lB, lT, lvh, d, device=dev, generator=gen).bfloat16()
        lbeta = torch.sigmoid(torch.randn(lB, lT, lvh, device=dev, generator=gen)).bfloat16()
        lg = -torch.nn.functional.softplus(torch.randn(lB, lT, lvh, device=dev, generator=gen)) * 0.1
        ls0 = (torch.randn(lB, lvh, d, d, device=dev, generator=gen) * 0.02).bfloat16()
        lws = torch.empty(gdn.api.chunked_forward_workspace_bytes(lB, lT, lvh), dtype=torch.uint8, device=dev)
        for _ in range(2):
            gdn.chunked_forward(lq, lk, lv, lbeta, lg, None, ls0, _workspace=lws)
        barrier()
        lsteps = 5
        e0.record()
        for _ in range(lsteps):
            gdn.chunked_forward(lq, lk, lv, lbeta, lg, None, ls0, _workspace=lws)
        e1.record()
        barrier()
        ms_lc = max_over_ranks(e0.elapsed_time(e1) / lsteps)
        lc = {"metric": "prefill_tokens_per_s", "value": lB * lT / (ms_lc * 1e-3), "unit": "tokens/s", "scaling": "strong",
              "config": "B=2 T=131072 kh=16 vh=32 d=128, value heads sharded over %d GPU(s): %d v-heads per GPU" % (world, lvh),
              "ms_per_step": ms_lc}
        del lq, lk, lv, lbeta, lg, ls0, lws
    # the sampler ran across every timed region above (prefill resident, end to end, decode, packed, long context)
    clocks = sampler.stop() if rank == 0 else None
    dec_bytes = dB * decode_bytes_per_token(kh, vh, d)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        tps, cores, what = cpu_recurrence_tokens_per_s(4096)
        cpu = {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": what}

    seq_flops = units * seq_kernel_flops_per_unit(d)
    uw_flops = units * uw_kernel_flops_per_unit(d)
    total_flops = units * flops_per_unit(d)
    uw_bytes = units * uw_kernel_bytes_per_unit(kh, vh, d)
    seq_bytes = units * seq_kernel_bytes_per_unit(kh, vh, d)
    # the dominant kernel is the one with the longer launch; both are HBM-bound (see above)
    if uw_ms >= seq_ms:
        dom = ("gdn_uw_kernel (WY/UT transform + intra-chunk attention block)", uw_ms, uw_bytes, uw_flops,
               units * NCU_UW_TRAFFIC_PER_UNIT)
    else:
        dom = ("gdn_fused_seq_kernel (state propagation + output)", seq_ms, seq_bytes, seq_flops,
               units * NCU_FUSED_TRAFFIC_PER_UNIT)
    achieved = dom[2] / (dom[1] * 1e-3) / 1e9
    line = {
        "metric": "prefill_tokens_per_s", "value": world * tokens / (ms_res * 1e-3), "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_res,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD,
                   "sharding": "by sequence, no collective", "l2": "inputs (0.41 GB per step) larger than L2"},
        "e2e": {"value": world * tokens / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e},
        "gpu_launches": 2 * args.steps,
        "roofline": {"kernel": dom[0], "bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "traffic": dom[4],
                     "traffic_source": "ncu capture at B=2 scaled by units", "peak_source": peaks["source"],
                     "ms_per_launch": dom[1], "bytes_per_launch": dom[2], "flops_per_launch": dom[3],
                     "flop_per_byte": dom[3] / dom[2]},
        "kernels": {"gdn_uw_kernel_ms": uw_ms, "gdn_fused_seq_kernel_ms": seq_ms,
                    "uw_gbs": uw_bytes / (uw_ms * 1e-3) / 1e9, "uw_frac_of_hbm_peak": uw_bytes / (uw_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                    "fused_gbs": seq_bytes / (seq_ms * 1e-3) / 1e9,
                    "fused_frac_of_hbm_peak": seq_bytes / (seq_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                    "uw_tflops": uw_flops / (uw_ms * 1e-3) / 1e12, "fused_tflops": seq_flops / (seq_ms * 1e-3) / 1e12,
                    "whole_step_tflops": total_flops / (ms_res * 1e-3) / 1e12,
                    "whole_step_frac_of_tensor_peak": total_flops / (ms_res * 1e-3) / 1e12 / peaks["tflops"],
                    "whole_step_hbm_gbs": (uw_bytes + seq_bytes) / (ms_res * 1e-3) / 1e9,
                    "whole_step_frac_of_hbm_peak": (uw_bytes + seq_bytes) / (ms_res * 1e-3) / 1e9 / peaks["hbm_gbs"]},
        "decode": {"metric": "decode_tokens_per_s", "value": world * dB / (ms_dec * 1e-3), "unit": "tokens/s",
                   "config": "B=256 T=1 kh=16 vh=32 d=128, qk-norm, fused gating, per GPU", "ms_per_step": ms_dec,
                   "roofline": {"kernel": "gdn_recurrent_kernel", "bound": "hbm",
                                "achieved": dec_bytes / (ms_dec_kernel * 1e-3) / 1e9, "peak": peaks["hbm_gbs"],
                                "unit": "GB/s", "frac": dec_bytes / (ms_dec_kernel * 1e-3) / 1e9 / peaks["hbm_gbs"],
                                "frac_of_nominal_8TBs": dec_bytes / (ms_dec_kernel * 1e-3) / 1e9 / 8000.0,
                                "ms_per_launch": ms_dec_kernel, "bytes_per_launch": dec_bytes,
                                "traffic": dB * NCU_DECODE_TRAFFIC_PER_TOKEN}},
        "packed": pk,
        "long_context": lc,
        "clocks": clocks,
    }
    if cpu is not None:
        line["cpu_baseline"] = cpu
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
