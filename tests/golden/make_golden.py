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


if __name__ == "__main__":
    main()
