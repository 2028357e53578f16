#!/usr/bin/env python
"""Benchmark of the Gated DeltaNet hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one pass of chunked prefill (`chunked_forward`) over one batch of the padded
prefill configuration: B=4, T=4096, kh=16, vh=32, dk=dv=128, bf16 q/k/v/beta, fp32 gate, bf16
initial state (synthetic, seeded).  With N > 1 (launched under torchrun, one rank per GPU)
every rank processes its own batch of that size - sequences are independent, so the path
shards by sequence with no collective - and `value` is the total over ranks (weak scaling).

The printed JSON line carries:
  value      prefill tokens/s with inputs resident in HBM (CUDA events, max over ranks; the K-step
             loop is repeated and the median repeat is reported, min and max beside it)
  e2e        the same through the public API from pinned HOST buffers: host->device copies of
             q, k, v, beta, gate and the state and the device->host copy of O and the final
             state are inside the timed region
  roofline   the whole prefill step against the tensor-core roof: algorithmic FLOPs (11.709 MFLOP per
             64-token chunk and v-head) / step time against the measured bf16 peak, with the byte view
             (24 768 B per token + the states against the measured copy bandwidth) and the two kernels'
             own figures beside it
  decode     decode tokens/s of `recurrent_forward` (B=256, T=1, qk-norm, gating fused in the kernel:
             one launch per step) and its HBM roofline fraction
  spec_verify   speculative verify (B=64, T=4, accepted-token caps ~ U{1..4}, qk-norm, fused gating)
  decode_sharded  a decode batch of B=1024 split by sequence over the N ranks (strong scaling)
  decode_small_batch  B=8 decode steps issued one by one against the same steps replayed as a CUDA graph
  layer_adjacent  the causal conv1d + SiLU in front of the layer and the gated RMS norm behind it (HBM-bound)
  packed     packed (varlen) prefill of 16 sequences with log-normal lengths, 32768 tokens per GPU
  long_context  the B=2, T=131072 layer with the value heads sharded over the N ranks (strong scaling)
  parity     N > 1 only: one shared-seed problem, every rank computes its head shard on its GPU, the
             shards are gathered with NCCL and rank 0 compares them with the CPU oracle (untimed)
  cpu_baseline  the fp32 CPU token recurrence (the oracle) on a bounded sample, rank 0, N=1

`--impl reference` times only that CPU recurrence (the reference library's own sm_90a kernels
cannot run on a B200 and it has no CPU path).
"""
from __future__ import annotations

import argparse
import contextlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG = dict(B=4, T=4096, kh=16, vh=32, d=128)
DECODE = dict(B=256, T=1, kh=16, vh=32, d=128)
SPEC = dict(B=64, T=4)
DECODE_SHARDED_B = 1024
CHUNK = 64
WORKLOAD = "padded chunked prefill B=4 T=4096 kh=16 vh=32 dk=dv=128 chunk=64 per GPU"
REF_SAMPLE_TOKENS = 1024
REPEATS = 5  # the K-step loop is timed this many times; the median is reported


def flops_per_unit(d: int, c: int = CHUNK) -> float:
    """Algorithmic work of one (64-token chunk, v-head), every contraction counted dense and per v-head:
    K K^T, Q K^T, T V, T K, P U_new (2CCd each), W S^T, U_new^T K, Q S^T (2Cdd each), the triangular
    inverse (2/3 C^3):  2C(5Cd + 3dd) + (2/3)C^3 = 11.709 MFLOP at d = 128."""
    return 2.0 * c * (5 * c * d + 3 * d * d) + (2.0 / 3.0) * c ** 3


def zp_kernel_flops_per_unit(kh: int, vh: int, d: int, c: int = CHUNK) -> float:
    """What gdn_zp_kernel executes per (chunk, v-head): K K^T and Q K^T once per k-head (2CCd each, shared
    by vh/kh v-heads), Z = (dT)^T K (2CCd), PT = P T (2CCC), the inverse (2/3 C^3)."""
    return 2.0 * c * c * d * (2.0 * kh / vh + 1.0) + 2.0 * c ** 3 + (2.0 / 3.0) * c ** 3


def seq_kernel_flops_per_unit(d: int, c: int = CHUNK) -> float:
    """What gdn_fused_seq_kernel executes per (chunk, v-head): S K^T, S Q^T, R Z (2Cdd each), R PT^T (2CCd)."""
    return 2.0 * c * (3 * d * d + c * d)


def prefill_min_bytes(tokens: int, seqs: int, kh: int, vh: int, d: int) -> float:
    """HBM bytes no implementation can avoid: q, k, v in and o out (bf16), beta bf16 and gate fp32 per
    token and v-head, plus the bf16 state read and written once per sequence."""
    return tokens * (2.0 * (2 * kh * d + 2 * vh * d) + vh * (2 + 4)) + seqs * 2.0 * vh * d * d * 2


# HBM bytes the two kernels of this design move per (chunk, v-head) unit at d = 128 (algorithmic):
#   gdn_zp_kernel        : K, Q tiles 16 KB each per k-head (shared by the vh/kh v-heads of a group) in;
#                          Z 16 KB and PT 8 KB out
#   gdn_fused_seq_kernel : V 16 KB, Z, PT 24 KB and K, Q (shared as above) in; O 16 KB out
def zp_kernel_bytes_per_unit(kh: int, vh: int, d: int, c: int = CHUNK) -> float:
    tile = c * d * 2
    return 2 * tile * kh / vh + tile + c * c * 2


def seq_kernel_bytes_per_unit(kh: int, vh: int, d: int, c: int = CHUNK) -> float:
    tile = c * d * 2
    return tile + (tile + c * c * 2) + 2 * tile * kh / vh + tile


# DRAM read + write bytes per launch seen by one ncu capture (dram__bytes_read.sum +
# dram__bytes_write.sum), divided by the units that launch processed.  Traffic is proportional
# to the units (every CTA streams its own tiles), so a full launch is units x this figure.
# The captures and their commands are summarised under profiles/.
#   gdn_zp_kernel        : B=2 T=4096 vh=32 capture, 4096 units
#   gdn_fused_seq_kernel : same capture, 4096 units
#   gdn_recurrent_kernel : B=128 capture (gating fused), 128 sequence-tokens
# (written data still in L2 when a launch ends is not counted by the DRAM counters)
NCU_ZP_TRAFFIC_PER_UNIT = (68.743168e6 + 41.161216e6) / 4096
NCU_FUSED_TRAFFIC_PER_UNIT = (238.593280e6 + 39.856384e6) / 4096
NCU_DECODE_TRAFFIC_PER_TOKEN = (136.373248e6 + 84.418816e6) / 128


def decode_bytes_per_token(kh, vh, d) -> float:
    """State read + written (2 * vh * d * d bf16), q, k, v, o, and beta, gate (bf16) per v-head."""
    return vh * (2 * d * d * 2) + 2 * (2 * kh * d + 2 * vh * d) + vh * 4


def spec_bytes_per_seq(T, kh, vh, d) -> float:
    """Speculative verify, one state per sequence out: state read once and written once, T tokens of q, k, v, o."""
    return vh * (2 * d * d * 2) + T * (2 * (2 * kh * d + 2 * vh * d) + vh * 4)


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


def _cpu_sample(sample_tokens: int):
    """Inputs of the CPU recurrence: one sequence of `sample_tokens` tokens of the prefill configuration."""
    from h100_gdn_cuda_b200 import synthetic
    p = synthetic.prefill_inputs(1, sample_tokens, CFG["kh"], CFG["vh"], CFG["d"], seed=0)
    return [p[k].float() for k in ("q", "k", "v", "beta")] + [p["g"], p["state"].float()]


def cpu_recurrence_tokens_per_s(sample_tokens: int, repeats: int = 1):
    """fp32 CPU token recurrence (the oracle) on one sequence of `sample_tokens` tokens of the
    prefill configuration; returns (tokens/s, threads, description)."""
    from oracle import gdn_oracle as O
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    args = _cpu_sample(sample_tokens)
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        O.recurrent_ref(*args)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return sample_tokens / best, threads, "B=1 x T=%d of the prefill config (kh=16, vh=32, d=128), fp32 torch" % sample_tokens


def run_reference(args):
    """The reference arm: the CPU recurrence, the only implementation of the path that can run
    on this box (rank 0 only).  Each step is a bounded sample of the workload, one sequence of
    REF_SAMPLE_TOKENS tokens; the figure is a per-token throughput."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import gdn_oracle as O
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    a = _cpu_sample(REF_SAMPLE_TOKENS)
    for _ in range(args.warmup):
        O.recurrent_ref(*a)
    per_step = []
    for _ in range(args.steps):
        t0 = time.perf_counter()
        O.recurrent_ref(*a)
        per_step.append(time.perf_counter() - t0)
    dt = sum(per_step) / len(per_step)
    tps = REF_SAMPLE_TOKENS / dt
    what = ("each step = ONE sequence of %d tokens (B=1 x T=%d) of the prefill config kh=16 vh=32 dk=dv=128, "
            "fp32 torch token recurrence on %d host threads; 1/16 of the GPU arm's step, so the ratio of the two "
            "arms is a per-token throughput ratio" % (REF_SAMPLE_TOKENS, REF_SAMPLE_TOKENS, threads))
    line = {
        "impl": "reference", "metric": "prefill_tokens_per_s", "value": tps, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "ms_per_step_min": min(per_step) * 1e3, "ms_per_step_max": max(per_step) * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "CPU sample of the padded chunked prefill config: B=1 T=%d kh=16 vh=32 dk=dv=128 per step "
                               "(the GPU arm's step is B=4 T=4096)" % REF_SAMPLE_TOKENS,
                   "sharding": "rank 0 only", "l2": "not applicable (CPU)"},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": what},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


@contextlib.contextmanager
def near_gpu(dev, note):
    """Bind the process to the CPUs NVML reports as local to the GPU while pinned host buffers are
    allocated (the pages are first touched there, so they land on the GPU's NUMA node and the
    copies of several ranks do not all cross the socket link); the previous affinity is restored
    on exit, so nothing else in the run is restricted.  `note` receives what was done."""
    old = os.sched_getaffinity(0)
    try:
        import pynvml
        pynvml.nvmlInit()
        uuid = str(torch.cuda.get_device_properties(dev).uuid)
        h = pynvml.nvmlDeviceGetHandleByUUID(uuid if uuid.startswith("GPU-") else "GPU-" + uuid)
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (max(old) + 64) // 64)
        local = {64 * w + b for w, x in enumerate(words) for b in range(64) if (x >> b) & 1}
        cpus = local & old
        if cpus and cpus != old:
            os.sched_setaffinity(0, cpus)
            note["host_affinity"] = "pinned buffers allocated on %d of %d allowed CPUs (local to the GPU)" % (len(cpus), len(old))
        else:
            note["host_affinity"] = "not bound (%d local CPUs among the %d allowed)" % (len(cpus), len(old))
    except Exception as e:  # no NVML, no affinity call: allocate wherever the pages fall
        note["host_affinity"] = "not bound (%s)" % type(e).__name__
    try:
        yield
    finally:
        os.sched_setaffinity(0, old)


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
        if args.varlen:
            # the same sequences as one packed batch (cu_seqlens): segments are then found on the device
            cu = [i * T for i in range(B + 1)]
            m = [torch.tensor(x, dtype=torch.int32, device=dev) for x in
                 (cu, synthetic.prepare_chunk_indices(cu), synthetic.prepare_cu_chunks(cu))]
            f = {k: t[k].view(B * T, *t[k].shape[2:]) for k in ("q", "k", "v", "beta", "g")}
            nc = B * (T // 64)
            ws = torch.empty(gdn.api.chunked_forward_workspace_bytes(B, 0, lvh, total_tokens=B * T, total_chunks=nc, packed=True),
                             dtype=torch.uint8, device=dev)
            run = lambda i: gdn.chunked_forward(f["q"], f["k"], f["v"], f["beta"], f["g"], None, t["state"], m[0], m[1], m[2], nc,
                                                _workspace=ws)
        work, unit = B * T, "tokens/s"
    elif args.only == "layer":
        # the layer-adjacent kernels: conv1d + SiLU over the q/k/v projections, then the gated RMS norm of the output
        B, T = args.batch or 2, CFG["T"]
        C_ = (2 * kh + vh) * d
        gen = torch.Generator(device=dev).manual_seed(11)
        x = torch.randn(B, T, C_, device=dev, generator=gen).bfloat16()
        w = (torch.randn(C_, 4, device=dev, generator=gen) * 0.5).bfloat16()
        bia = torch.randn(C_, device=dev, generator=gen).bfloat16()
        o = torch.randn(B, T, vh, d, device=dev, generator=gen).bfloat16()
        z = torch.randn(B, T, vh, d, device=dev, generator=gen).bfloat16()
        gw = torch.randn(d, device=dev, generator=gen).bfloat16()

        def run(i):
            gdn.causal_conv1d(x, w, bia)
            gdn.gated_rmsnorm(o, z, gw)
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
        states = [t["state"], t["state"].clone()]
        run = lambda i: gdn.recurrent_forward(t["q"], t["k"], t["v"], states[i & 1], None, None, inference_mode=1,
                                              is_qk_norm=True, gating=(t["A_log"], t["dt_bias"], t["a"], t["b"]))
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
    ap.add_argument("--only", default=None, choices=["prefill", "decode", "long", "packed", "layer"],
                    help="profiling aid: run only this path, resident inputs, reduced JSON line")
    ap.add_argument("--batch", type=int, default=None, help="with --only: override the batch size")
    ap.add_argument("--heads", type=int, default=None, help="with --only long: v-heads of this GPU's share (default 4)")
    ap.add_argument("--varlen", action="store_true", help="with --only long: pass the sequences as one packed batch")
    args = ap.parse_args()
    if args.only is None:
        args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        return run_reference(args)

    import h100_gdn_cuda_b200 as gdn
    from h100_gdn_cuda_b200 import build, sharding, synthetic
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
    affinity_note = {}
    with near_gpu(dev, affinity_note):
        host = {k: p[k].pin_memory() for k in ("q", "k", "v", "beta", "g", "state")}
        out_host = torch.empty(B, T, vh, d, dtype=torch.bfloat16).pin_memory()
        st_host = torch.empty(B, vh, d, d, dtype=torch.bfloat16).pin_memory()
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

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(step, steps, repeats=REPEATS):
        """`repeats` times: barrier, `steps` calls of step(i) between two events, barrier; every figure is the
        maximum over the ranks.  Returns (median ms per step, [ms per step of every repeat])."""
        out = []
        for _ in range(repeats):
            barrier()
            e0.record()
            for i in range(steps):
                step(i)
            e1.record()
            barrier()
            out.append(max_over_ranks(e0.elapsed_time(e1) / steps))
        return statistics.median(out), out

    def spread(xs):
        return {"repeats": len(xs), "ms_min": min(xs), "ms_max": max(xs)}

    from h100_gdn_cuda_b200 import api as gdn_api
    ws = torch.empty(gdn_api.chunked_forward_workspace_bytes(B, T, vh, num_k_heads=kh), dtype=torch.uint8, device=dev)
    stage_ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    for e in stage_ev:
        e.record()

    def step_resident(i=0, events=None):
        return gdn.chunked_forward(devt["q"], devt["k"], devt["v"], devt["beta"], devt["g"], None, devt["state"],
                                   _workspace=ws, _stage_events=events)

    # ---------------- device-resident timing (inputs 0.4 GB per step: larger than the 126 MB L2)
    for _ in range(args.warmup):
        step_resident()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_res, ms_res_all = timed(step_resident, args.steps)
    # per-kernel durations: the same steps again with events between the two kernels
    zp_ms, seq_ms = 0.0, 0.0
    for _ in range(args.steps):
        step_resident(0, stage_ev)
        torch.cuda.synchronize()
        zp_ms += stage_ev[0].elapsed_time(stage_ev[1])
        seq_ms += stage_ev[1].elapsed_time(stage_ev[2])
    zp_ms /= args.steps
    seq_ms /= args.steps

    # ---------------- end to end from host buffers
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
    del stages

    # ---------------- decode (B=256, T=1): state 268 MB per step, larger than L2.  beta and the gate are
    # computed inside the kernel from A_log, dt_bias, a, b: one launch per step.
    dB = DECODE["B"]
    dp = synthetic.decode_inputs(dB, 1, kh, vh, d, seed=100 + rank)
    dd = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in dp.items()}
    states = [dd["state"].clone() for _ in range(2)]
    gating = (dd["A_log"], dd["dt_bias"], dd["a"], dd["b"])

    def step_decode(i):
        return gdn.recurrent_forward(dd["q"], dd["k"], dd["v"], states[i & 1], None, None, inference_mode=1,
                                     is_qk_norm=True, gating=gating)

    for i in range(5):
        step_decode(i)
    # (a step lasts 0.05 - 0.1 ms: 50 of them per timed loop, so that the first call's launch latency after the
    # synchronisation that opens the loop does not show)
    dsteps = max(args.steps, 50)
    ms_dec, ms_dec_all = timed(step_decode, dsteps)
    del states

    # ---------------- small-batch decode (B=8): the step is bound by launch overhead, so a serving loop captures
    # it.  16 consecutive in-place steps, issued one by one from Python and replayed as one CUDA graph.
    gB, gsteps = 8, 16
    gp = synthetic.decode_inputs(gB, 1, kh, vh, d, seed=150 + rank)
    gd = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in gp.items()}
    g_gating = (gd["A_log"], gd["dt_bias"], gd["a"], gd["b"])
    g_state = gd["state"].clone()

    def steps_small(i=0):
        for _ in range(gsteps):
            gdn.recurrent_forward(gd["q"], gd["k"], gd["v"], g_state, None, None, inference_mode=1, is_qk_norm=True,
                                  gating=g_gating, inplace_state=True)
    steps_small()
    ms_small_eager, _ = timed(steps_small, 5, repeats=3)
    ms_small_ext = None
    try:  # the same steps through the pybind front end (built in-tree; optional)
        from h100_gdn_cuda_b200 import gdn_cuda as gdn_ext
        gdn_ext.init(os.path.dirname(os.path.abspath(__file__)), os.environ.get("CUDA_HOME", "/usr/local/cuda"))

        def steps_small_ext(i=0):
            for _ in range(gsteps):
                gdn_ext.recurrent_forward(gd["q"], gd["k"], gd["v"], g_state, None, None, inference_mode=1, is_qk_norm=True,
                                          gating=g_gating, inplace_state=True)
        steps_small_ext()
        ms_small_ext, _ = timed(steps_small_ext, 5, repeats=3)
    except ImportError:
        pass
    cap = torch.cuda.Stream()
    cap.wait_stream(torch.cuda.current_stream())
    small_graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(cap):
        steps_small()
        with torch.cuda.graph(small_graph, stream=cap):
            steps_small()
    torch.cuda.current_stream().wait_stream(cap)
    small_graph.replay()
    ms_small_graph, _ = timed(lambda i=0: small_graph.replay(), 5, repeats=3)
    decode_small = {"config": "B=%d T=1 kh=16 vh=32 d=128, qk-norm, gating inside, state in place; %d steps per measurement" % (gB, gsteps),
                    "eager_us_per_step": 1e3 * ms_small_eager / gsteps,
                    "eager_pybind_us_per_step": None if ms_small_ext is None else 1e3 * ms_small_ext / gsteps,
                    "cuda_graph_us_per_step": 1e3 * ms_small_graph / gsteps,
                    "note": "eager: one Python call per step through the ctypes / the pybind front end; graph: the same launches replayed"}
    del small_graph, g_state

    # ---------------- speculative verify (B=64, T=4, accepted-token caps ~ U{1..4}, one state per sequence out)
    sB, sT = SPEC["B"], SPEC["T"]
    sp = synthetic.decode_inputs(sB, sT, kh, vh, d, seed=300 + rank, spec=True)
    sd = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in sp.items()}
    s_states = [sd["state"].clone() for _ in range(4)]  # 4 x 67 MB, cycled: larger than L2 between reuses
    s_gating = (sd["A_log"], sd["dt_bias"], sd["a"], sd["b"])

    def step_spec(i):
        return gdn.recurrent_forward(sd["q"], sd["k"], sd["v"], s_states[i & 3], None, None, None, sd["num_accepted_tokens"],
                                     inference_mode=1, is_qk_norm=True, gating=s_gating)

    for i in range(5):
        step_spec(i)
    ms_spec, ms_spec_all = timed(step_spec, dsteps)
    accepted = int(sp["num_accepted_tokens"].sum())
    del s_states

    # ---------------- decode batch of 1024 sequences split by sequence over the ranks (strong scaling)
    sl = sharding.seq_shard(rank, world, DECODE_SHARDED_B)
    nB = sl.stop - sl.start
    np_ = synthetic.decode_inputs(nB, 1, kh, vh, d, seed=500 + rank)
    nd = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in np_.items()}
    n_states = [nd["state"], nd["state"].clone()] if nB * vh * d * d * 2 > (160 << 20) else [nd["state"].clone() for _ in range(4)]
    n_gating = (nd["A_log"], nd["dt_bias"], nd["a"], nd["b"])

    def step_decode_sharded(i):
        return gdn.recurrent_forward(nd["q"], nd["k"], nd["v"], n_states[i % len(n_states)], None, None, inference_mode=1,
                                     is_qk_norm=True, gating=n_gating)

    for i in range(5):
        step_decode_sharded(i)
    ms_dsh, ms_dsh_all = timed(step_decode_sharded, dsteps)
    del n_states, nd

    # ---------------- the layer-adjacent steps at the benchmark shape: causal conv1d + SiLU over the q/k/v
    # projections (B=4, T=4096, 2*kh*d + vh*d = 8192 channels, width 4) and the gated RMS norm of the output
    gen_la = torch.Generator(device=dev).manual_seed(900 + rank)
    la_C = 2 * kh * d + vh * d
    la_x = torch.randn(B, T, la_C, device=dev, generator=gen_la).bfloat16()
    la_w = (torch.randn(la_C, 4, device=dev, generator=gen_la) * 0.5).bfloat16()
    la_b = torch.randn(la_C, device=dev, generator=gen_la).bfloat16()
    for _ in range(3):
        gdn.causal_conv1d(la_x, la_w, la_b)
    ms_conv, ms_conv_all = timed(lambda i: gdn.causal_conv1d(la_x, la_w, la_b), 10)
    conv_bytes = 2 * la_x.numel() * 2
    del la_x
    la_o = torch.randn(B, T, vh, d, device=dev, generator=gen_la).bfloat16()
    la_z = torch.randn(B, T, vh, d, device=dev, generator=gen_la).bfloat16()
    la_g = torch.ones(d, device=dev).bfloat16()
    for _ in range(3):
        gdn.gated_rmsnorm(la_o, la_z, la_g)
    ms_norm, ms_norm_all = timed(lambda i: gdn.gated_rmsnorm(la_o, la_z, la_g), 10)
    norm_bytes = 3 * la_o.numel() * 2
    del la_o, la_z

    # ---------------- packed prefill: 16 sequences of log-normal lengths, 32768 tokens per rank
    pk = None
    if not args.no_packed:
        lens = synthetic.lognormal_lengths(16, 32768, 64, 8192, seed=rank)
        pp = synthetic.varlen_inputs(lens, kh, vh, d, seed=200 + rank)
        pd = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in pp.items()}
        pws = torch.empty(gdn_api.chunked_forward_workspace_bytes(len(lens), 0, vh, total_tokens=sum(lens),
                                                                  total_chunks=pp["total_chunks"], packed=True, num_k_heads=kh),
                          dtype=torch.uint8, device=dev)
        pev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        for e in pev:
            e.record()

        def step_packed(i=0, events=None):
            return gdn.chunked_forward(pd["q"], pd["k"], pd["v"], pd["beta"], pd["g"], None, pd["state"], pd["cu_seqlens"],
                                       pd["chunk_indices"], pd["cu_chunks"], pp["total_chunks"], _workspace=pws,
                                       _stage_events=events)
        for _ in range(3):
            step_packed()
        ms_pk, ms_pk_all = timed(step_packed, 10)
        step_packed(0, pev)
        torch.cuda.synchronize()
        pk = {"metric": "prefill_tokens_per_s", "value": world * sum(lens) / (ms_pk * 1e-3), "unit": "tokens/s",
              "config": "packed: 16 sequences of log-normal lengths (%d ... %d tokens), %d tokens per GPU, kh=16 vh=32 d=128"
                        % (min(lens), max(lens), sum(lens)),
              "ms_per_step": ms_pk, "spread": spread(ms_pk_all), "gdn_zp_kernel_ms": pev[0].elapsed_time(pev[1]),
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
        lws = torch.empty(gdn_api.chunked_forward_workspace_bytes(lB, lT, lvh, num_k_heads=lkh), dtype=torch.uint8, device=dev)

        def step_long(i=0):
            return gdn.chunked_forward(lq, lk, lv, lbeta, lg, None, ls0, _workspace=lws)
        for _ in range(2):
            step_long()
        ms_lc, ms_lc_all = timed(step_long, 5, repeats=3)
        lc = {"metric": "prefill_tokens_per_s", "value": lB * lT / (ms_lc * 1e-3), "unit": "tokens/s", "scaling": "strong",
              "config": "B=2 T=131072 kh=16 vh=32 d=128, value heads sharded over %d GPU(s): %d v-heads per GPU" % (world, lvh),
              "ms_per_step": ms_lc, "spread": spread(ms_lc_all)}
        # the same two sequences as one packed (varlen) batch: what a serving engine passes
        cu_host = [0, lT, 2 * lT]
        lnc = 2 * (lT // 64)
        lcu, lci, lcc = (torch.tensor(x, dtype=torch.int32, device=dev) for x in
                         (cu_host, synthetic.prepare_chunk_indices(cu_host), synthetic.prepare_cu_chunks(cu_host)))
        lpws = torch.empty(gdn_api.chunked_forward_workspace_bytes(lB, 0, lvh, total_tokens=lB * lT, total_chunks=lnc, packed=True,
                                                                   num_k_heads=lkh), dtype=torch.uint8, device=dev)
        pq, pk_, pv, pb, pg = (t.view(lB * lT, *t.shape[2:]) for t in (lq, lk, lv, lbeta, lg))

        def step_long_packed(i=0):
            return gdn.chunked_forward(pq, pk_, pv, pb, pg, None, ls0, lcu, lci, lcc, lnc, _workspace=lpws)
        for _ in range(2):
            step_long_packed()
        ms_lcp, ms_lcp_all = timed(step_long_packed, 5, repeats=3)
        lc["packed_ms_per_step"] = ms_lcp
        lc["packed_spread"] = spread(ms_lcp_all)
        del lq, lk, lv, lbeta, lg, ls0, lws, lpws, pq, pk_, pv, pb, pg
    # the sampler ran across every timed region above
    clocks = sampler.stop() if rank == 0 else None

    # ---------------- N > 1: sharded result against the oracle (untimed).  One problem from a shared seed;
    # every rank computes its value-head shard on its own GPU; O and the final state are gathered with
    # NCCL; rank 0 compares the assembled result with the fp32 CPU recurrence.
    parity = None
    if world > 1 and 8 % world == 0:
        pB, pT, pkh, pvh = 2, 520, 8, 16
        pp = synthetic.prefill_inputs(pB, pT, pkh, pvh, d, seed=4242)
        full = {k: pp[k].to(dev) for k in ("q", "k", "v", "beta", "g", "state")}
        mine = sharding.shard_prefill_by_head(full, rank, world)
        o_sh, s_sh = gdn.chunked_forward(mine["q"], mine["k"], mine["v"], mine["beta"], mine["g"], None, mine["state"])
        o_sh, s_sh = o_sh.contiguous(), s_sh.contiguous()
        o_all = [torch.empty_like(o_sh) for _ in range(world)]
        s_all = [torch.empty_like(s_sh) for _ in range(world)]
        dist.all_gather(o_all, o_sh)
        dist.all_gather(s_all, s_sh)
        torch.cuda.synchronize()
        if rank == 0:
            from oracle import gdn_oracle as O
            o_ref, s_ref = O.recurrent_ref(pp["q"].float(), pp["k"].float(), pp["v"].float(), pp["beta"].float(), pp["g"],
                                           pp["state"].float())
            o_cat, s_cat = torch.cat(o_all, dim=2).float().cpu(), torch.cat(s_all, dim=1).float().cpu()
            parity = {"config": "B=2 T=520 kh=8 vh=16 d=128, value heads sharded over %d GPUs, NCCL all_gather of O and final state" % world,
                      "o_rel_fro": O.rel_fro(o_cat, o_ref), "o_max_abs_over_max": O.max_abs_over_max(o_cat, o_ref),
                      "state_rel_fro": O.rel_fro(s_cat, s_ref), "state_max_abs_over_max": O.max_abs_over_max(s_cat, s_ref),
                      "gate": "rel_fro <= 1e-2 and max_abs <= 5e-2 * max|ref|"}
            parity["rel_fro"] = max(parity["o_rel_fro"], parity["state_rel_fro"])
            parity["ok"] = bool(parity["rel_fro"] <= 1e-2 and max(parity["o_max_abs_over_max"], parity["state_max_abs_over_max"]) <= 5e-2)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        tps, cores, what = cpu_recurrence_tokens_per_s(4096)
        cpu = {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": what}

    total_flops = units * flops_per_unit(d)
    zp_flops = units * zp_kernel_flops_per_unit(kh, vh, d)
    seq_flops = units * seq_kernel_flops_per_unit(d)
    zp_bytes = units * zp_kernel_bytes_per_unit(kh, vh, d)
    seq_bytes = units * seq_kernel_bytes_per_unit(kh, vh, d)
    min_bytes = prefill_min_bytes(tokens, B, kh, vh, d)
    step_tflops = total_flops / (ms_res * 1e-3) / 1e12
    traffic = None
    if NCU_ZP_TRAFFIC_PER_UNIT is not None and NCU_FUSED_TRAFFIC_PER_UNIT is not None:
        traffic = units * (NCU_ZP_TRAFFIC_PER_UNIT + NCU_FUSED_TRAFFIC_PER_UNIT)
    dec_bytes = dB * decode_bytes_per_token(kh, vh, d)
    spec_bytes = sB * spec_bytes_per_seq(sT, kh, vh, d)
    dsh_bytes = nB * decode_bytes_per_token(kh, vh, d)

    def hbm_roof(nbytes, ms, kernel, traffic=None):
        gbs = nbytes / (ms * 1e-3) / 1e9
        return {"kernel": kernel, "bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": gbs / peaks["hbm_gbs"], "frac_of_nominal_8TBs": gbs / 8000.0, "ms_per_launch": ms,
                "bytes_per_launch": nbytes, "traffic": traffic, "peak_source": peaks["source"]}

    line = {
        "metric": "prefill_tokens_per_s", "value": world * tokens / (ms_res * 1e-3), "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_res,
        "spread": spread(ms_res_all),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD,
                   "sharding": "by sequence, no collective", "l2": "inputs (0.41 GB per step) larger than L2"},
        "e2e": {"value": world * tokens / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e, "host_affinity": affinity_note.get("host_affinity"),
                "note": "bound by the pinned-host <-> device copies (%.0f MB per rank and step, %.1f GB/s in + %.1f GB/s out per rank); "
                        "at N > 1 the ranks share the host's memory and PCIe path" % (
                            (h2d + d2h) / 1e6, h2d / (ms_e2e * 1e-3) / 1e9, d2h / (ms_e2e * 1e-3) / 1e9)},
        "gpu_launches": 2 * args.steps * REPEATS,
        "gpu_launches_per_step": 2,
        # the whole step (two launches) against the tensor-core roof: the path is a dense contraction
        "roofline": {"kernel": "gdn_zp_kernel + gdn_fused_seq_kernel (one prefill step)", "bound": "tensor",
                     "achieved": step_tflops, "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": step_tflops / peaks["tflops"],
                     "peak_kind": "burst cuBLAS bf16 figure (the timed region lasts milliseconds)",
                     "frac_of_sustained_peak": step_tflops / peaks["tflops_sustained"],
                     "flops_per_step": total_flops, "flops_per_unit": flops_per_unit(d), "units_per_step": units,
                     "traffic": traffic, "traffic_source": "ncu captures at B=2 scaled by units, both kernels",
                     "peak_source": peaks["source"],
                     "bytes": {"min_bytes_per_step": min_bytes, "achieved_gbs": min_bytes / (ms_res * 1e-3) / 1e9,
                               "peak_gbs": peaks["hbm_gbs"], "frac": min_bytes / (ms_res * 1e-3) / 1e9 / peaks["hbm_gbs"],
                               "what": "24 768 B per token (q, k, v, o, beta, gate) + the states, against the measured copy bandwidth"}},
        "kernels": {
            "gdn_zp_kernel": {"ms": zp_ms, "executed_tflops": zp_flops / (zp_ms * 1e-3) / 1e12,
                              "frac_of_tensor_peak": zp_flops / (zp_ms * 1e-3) / 1e12 / peaks["tflops"],
                              "algorithmic_gbs": zp_bytes / (zp_ms * 1e-3) / 1e9,
                              "frac_of_hbm_peak": zp_bytes / (zp_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                              "traffic": None if NCU_ZP_TRAFFIC_PER_UNIT is None else units * NCU_ZP_TRAFFIC_PER_UNIT},
            "gdn_fused_seq_kernel": {"ms": seq_ms, "executed_tflops": seq_flops / (seq_ms * 1e-3) / 1e12,
                                     "frac_of_tensor_peak": seq_flops / (seq_ms * 1e-3) / 1e12 / peaks["tflops"],
                                     "algorithmic_gbs": seq_bytes / (seq_ms * 1e-3) / 1e9,
                                     "frac_of_hbm_peak": seq_bytes / (seq_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                                     "traffic": None if NCU_FUSED_TRAFFIC_PER_UNIT is None else units * NCU_FUSED_TRAFFIC_PER_UNIT}},
        "decode": {"metric": "decode_tokens_per_s", "value": world * dB / (ms_dec * 1e-3), "unit": "tokens/s",
                   "config": "B=256 T=1 kh=16 vh=32 d=128, qk-norm, gating fused in the kernel (one launch per step), per GPU",
                   "ms_per_step": ms_dec, "spread": spread(ms_dec_all), "gpu_launches_per_step": 1,
                   "roofline": hbm_roof(dec_bytes, ms_dec, "gdn_recurrent_kernel", dB * NCU_DECODE_TRAFFIC_PER_TOKEN)},
        "spec_verify": {"metric": "verified_tokens_per_s", "value": world * sB * sT / (ms_spec * 1e-3), "unit": "tokens/s",
                        "accepted_tokens_per_s": world * accepted / (ms_spec * 1e-3),
                        "config": "B=64 T=4 inference_mode=1, num_accepted_tokens ~ U{1..4} (%d of %d accepted), qk-norm, "
                                  "gating fused in the kernel, per GPU" % (accepted, sB * sT),
                        "ms_per_step": ms_spec, "spread": spread(ms_spec_all), "gpu_launches_per_step": 1,
                        "roofline": hbm_roof(spec_bytes, ms_spec, "gdn_recurrent_kernel")},
        "decode_sharded": {"metric": "decode_tokens_per_s", "value": DECODE_SHARDED_B / (ms_dsh * 1e-3), "unit": "tokens/s",
                           "scaling": "strong",
                           "config": "B=1024 T=1 kh=16 vh=32 d=128 split by sequence over %d GPU(s): %d sequences on rank 0, "
                                     "qk-norm, fused gating" % (world, nB),
                           "ms_per_step": ms_dsh, "spread": spread(ms_dsh_all),
                           "roofline": hbm_roof(dsh_bytes, ms_dsh, "gdn_recurrent_kernel (rank 0's share)")},
        "decode_small_batch": decode_small,
        "layer_adjacent": {
            "causal_conv1d_silu": {"config": "B=4 T=4096 channels=8192 (q, k, v projections) width=4, bias, SiLU, per GPU",
                                   "value": world * tokens / (ms_conv * 1e-3), "unit": "tokens/s", "ms_per_step": ms_conv,
                                   "spread": spread(ms_conv_all), "roofline": hbm_roof(conv_bytes, ms_conv, "gdn_causal_conv1d_kernel<4>")},
            "gated_rmsnorm": {"config": "B=4 T=4096 vh=32 d=128: 524288 rows of 128, per GPU",
                              "value": world * tokens / (ms_norm * 1e-3), "unit": "tokens/s", "ms_per_step": ms_norm,
                              "spread": spread(ms_norm_all), "roofline": hbm_roof(norm_bytes, ms_norm, "gdn_gated_rmsnorm_kernel")}},
        "packed": pk,
        "long_context": lc,
        "parity": parity,
        "clocks": clocks,
    }
    if cpu is not None:
        line["cpu_baseline"] = cpu
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
