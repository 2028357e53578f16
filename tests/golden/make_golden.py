"""Generate the golden vectors in this directory.

Run once, in a container where the reference's third-party arithmetic is
importable:  python tests/golden/make_golden.py

The reference library stores no golden vectors; at its own test boundary the
expected values come from the `flash-linear-attention` package
(test/test_py/fla_comparison.py:8-28, test_fla_recurrent_comparison.py:8-11;
pinned 0.4.1 in uv.lock).  This script calls that package's pure-PyTorch naive
token recurrence (fla.ops.gated_delta_rule.naive, runs on CPU) on seeded
inputs and stores inputs and outputs, so the oracle in oracle/gdn_oracle.py is
pinned against an implementation that is not ours.  The state is stored in the
reference layout (vh, dv, dk), i.e. the transpose of the package's (H, K, V).
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

from h100_gdn_cuda_b200 import synthetic  # noqa: E402


def main():
    import fla
    from fla.ops.gated_delta_rule.naive import naive_recurrent_gated_delta_rule as naive

    cases = {
        # BASELINE configs[0]: fp32, no initial state
        "cfg0_T256_h4_d64": dict(B=1, T=256, kh=4, vh=4, d=64, seed=0, state=False, dtype=torch.float32),
        # GQA, initial state, partial last chunk, bf16-rounded inputs
        "gqa_T130_kh2_vh4_d128": dict(B=1, T=130, kh=2, vh=4, d=128, seed=1, state=True, dtype=torch.bfloat16),
        # short sequence (single partial chunk)
        "short_T7_h2_d64": dict(B=1, T=7, kh=2, vh=2, d=64, seed=2, state=True, dtype=torch.bfloat16),
    }
    for name, c in cases.items():
        p = synthetic.prefill_inputs(c["B"], c["T"], c["kh"], c["vh"], c["d"], seed=c["seed"],
                                     with_state=c["state"], dtype=c["dtype"])
        rep = c["vh"] // c["kh"]
        q = p["q"].float().repeat_interleave(rep, dim=2)
        k = p["k"].float().repeat_interleave(rep, dim=2)
        s0 = None if p["state"] is None else p["state"].float().transpose(-1, -2).contiguous()
        o, s = naive(q, k, p["v"].float(), p["beta"].float(), p["g"], initial_state=s0,
                     output_final_state=True)
        out = dict(q=p["q"].float().numpy(), k=p["k"].float().numpy(), v=p["v"].float().numpy(),
                   beta=p["beta"].float().numpy(), g=p["g"].numpy(),
                   o=o.numpy(), final_state=s.transpose(-1, -2).contiguous().numpy(),
                   fla_version=np.array(fla.__version__))
        if p["state"] is not None:
            out["state"] = p["state"].float().numpy()
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
        print(name, "o", tuple(o.shape), "absmax", float(o.abs().max()))


def branch_cases():
    """Fixtures for the branches of the oracle that the plain recurrence above does not reach:
    q/k L2 normalisation, per-token (step) states and the accepted-token cap.  The package's
    normalisation kernel needs a GPU, so q and k are normalised here in float64 with the formula
    the reference kernel uses (x * rsqrt(sum x^2 + 1e-6), sm90_bf16_gdn_recurrent.cuh:299,350)
    and the package's naive recurrence runs on the normalised tensors; the fixture stores the RAW
    q and k, so the oracle has to do the normalisation itself.  Step states come from calling the
    naive recurrence one token at a time, each call starting from the state the previous returned."""
    import fla
    from fla.ops.gated_delta_rule.naive import naive_recurrent_gated_delta_rule as naive

    def norm64(x):
        x = x.double()
        return (x * torch.rsqrt((x * x).sum(-1, keepdim=True) + 1e-6)).float()

    # --- qk-norm, GQA, initial state, raw (un-normalised) bf16-rounded q and k
    p = synthetic.prefill_inputs(2, 40, 2, 4, 64, seed=11, with_state=True, dtype=torch.bfloat16, normalize=False)
    q, k = norm64(p["q"].float()).repeat_interleave(2, dim=2), norm64(p["k"].float()).repeat_interleave(2, dim=2)
    s0 = p["state"].float().transpose(-1, -2).contiguous()
    o, s = naive(q, k, p["v"].float(), p["beta"].float(), p["g"], initial_state=s0, output_final_state=True)
    np.savez_compressed(os.path.join(HERE, "branch_qknorm_B2_T40_kh2_vh4_d64.npz"),
                        q=p["q"].float().numpy(), k=p["k"].float().numpy(), v=p["v"].float().numpy(),
                        beta=p["beta"].float().numpy(), g=p["g"].numpy(), state=p["state"].float().numpy(),
                        o=o.numpy(), final_state=s.transpose(-1, -2).contiguous().numpy(),
                        fla_version=np.array(fla.__version__))
    print("branch_qknorm", tuple(o.shape), float(o.abs().max()))

    # --- step states (speculative verify): B=3, T=6, token by token
    p = synthetic.prefill_inputs(3, 6, 2, 2, 64, seed=12, with_state=True, dtype=torch.bfloat16)
    st = p["state"].float().transpose(-1, -2).contiguous()
    outs, steps = [], []
    for t in range(6):
        sl = slice(t, t + 1)
        o, st = naive(p["q"].float()[:, sl], p["k"].float()[:, sl], p["v"].float()[:, sl], p["beta"].float()[:, sl],
                      p["g"][:, sl], initial_state=st, output_final_state=True)
        outs.append(o)
        steps.append(st.transpose(-1, -2).contiguous())
    np.savez_compressed(os.path.join(HERE, "branch_steps_B3_T6_h2_d64.npz"),
                        q=p["q"].float().numpy(), k=p["k"].float().numpy(), v=p["v"].float().numpy(),
                        beta=p["beta"].float().numpy(), g=p["g"].numpy(), state=p["state"].float().numpy(),
                        o=torch.cat(outs, dim=1).numpy(), step_states=torch.stack(steps, dim=1).numpy(),
                        fla_version=np.array(fla.__version__))
    print("branch_steps", tuple(torch.stack(steps, dim=1).shape))


if __name__ == "__main__":
    main()
    branch_cases()
