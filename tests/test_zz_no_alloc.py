"""The workspace-free prefill entry point (gdn_chunked_forward_static_scratch).

Some callers of the library cannot hand it a workspace because they may not allocate device
memory when the call happens (all HBM already given to their own pool, or cudaMalloc ruled
out on their path because it synchronises the device).  For them the library keeps the U/W
scratch of chunked prefill in a fixed array inside its own image.  This test drives that
entry point through the C ABI, twice in a row on different problems (the array is shared
and keeps the previous call's contents), and requires the same bits as the regular entry
point given a caller-provided workspace.  It also checks that a problem beyond the array's
stated limit is refused.  The file name makes pytest collect it last.
"""
import ctypes as C

import pytest
import torch

from h100_gdn_cuda_b200 import synthetic

pytestmark = pytest.mark.gpu


def _args(api, cabi, p, out, final, ws, ws_bytes):
    q, k, v = p["q"], p["k"], p["v"]
    B, T, kh, d = q.shape
    vh = v.shape[2]
    shape = api._shape(B, T, B * T, kh, vh, d, d)
    return cabi.ChunkedArgs(shape, api._token_tensor(q, False), api._token_tensor(k, False),
                            api._token_tensor(v, False), api._token_tensor(out, False),
                            api._token_scalar(p["beta"], False), api._token_scalar(p["g"], False),
                            api._state_desc(p["state"]), api._state_desc(final), float(d) ** -0.5,
                            ws, ws_bytes, None)


def test_static_scratch_matches_workspace_path_twice():
    from h100_gdn_cuda_b200 import _cabi as cabi, api, build
    build.build()
    lib = cabi.load()
    stream = torch.cuda.current_stream().cuda_stream
    # two calls in a row, the second smaller than the first so stale scratch lies beyond it
    for (B, T, kh, vh, seed) in ((2, 300, 2, 4, 5), (1, 130, 2, 4, 6)):
        p = {k: (v.cuda() if torch.is_tensor(v) else v)
             for k, v in synthetic.prefill_inputs(B, T, kh, vh, 128, seed=seed, mild_gate=True).items()}
        outs = []
        for static in (False, True):
            out = torch.full_like(p["v"], float("nan"))
            final = torch.full_like(p["state"], float("nan"))
            if static:
                a = _args(api, cabi, p, out, final, None, 0)
                rc = lib.gdn_chunked_forward_static_scratch(C.byref(a), stream)
            else:
                n = lib.gdn_chunked_forward_workspace_bytes(C.byref(api._shape(B, T, B * T, kh, vh, 128, 128)))
                ws = torch.empty(n, dtype=torch.uint8, device="cuda")
                a = _args(api, cabi, p, out, final, ws.data_ptr(), n)
                rc = lib.gdn_chunked_forward(C.byref(a), stream)
            assert rc == 0, lib.gdn_last_error()
            torch.cuda.synchronize()
            outs.append((out, final))
        (o_ws, s_ws), (o_st, s_st) = outs
        assert torch.isfinite(o_st.float()).all() and torch.isfinite(s_st.float()).all()
        # same kernels, same inputs: the tolerance of the prefill tests (1e-2 relative
        # Frobenius) is met with zero difference
        assert torch.equal(o_st, o_ws) and torch.equal(s_st, s_ws)


def test_static_scratch_refuses_oversize():
    from h100_gdn_cuda_b200 import _cabi as cabi, api, build
    build.build()
    lib = cabi.load()
    # 4097 tokens x 32 heads is one token over the limit; validation precedes any device work
    shape = api._shape(1, 4097, 4097, 16, 32, 128, 128)
    a = cabi.ChunkedArgs()
    a.shape = shape
    rc = lib.gdn_chunked_forward_static_scratch(C.byref(a), None)
    assert rc == -4 and b"built-in" in lib.gdn_last_error()
