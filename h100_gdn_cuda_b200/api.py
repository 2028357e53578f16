"""Python mirror of the reference's `gdn_cuda` module (csrc/python_api.cpp:17-393).

Same function names, argument order, keywords and defaults; every function runs on the
current CUDA stream by calling the C ABI of libgdn_b200.so (include/gdn_b200.h).  Errors
raise RuntimeError (the reference's docstrings promise that; its code exits the process).
"""
from __future__ import annotations

import ctypes as C
import enum
import math
from typing import Optional, Tuple

import torch

from . import _cabi as cabi

CHUNK = 64


class InferenceMode(enum.IntEnum):
    """gdn_cuda/include/gdn_cuda/types.h:5 (SpecDecode is declared there but unused)."""
    Prefill = 0
    Decode = 1
    SpecVerify = 2


Prefill, Decode, SpecVerify = InferenceMode.Prefill, InferenceMode.Decode, InferenceMode.SpecVerify

_state = {"library_root": None, "cuda_home": None}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return cabi.GDN_BF16
    if t.dtype == torch.float32:
        return cabi.GDN_F32
    raise RuntimeError("unsupported dtype %s (bf16 or fp32 expected)" % t.dtype)


def _require(cond: bool, msg: str):
    if not cond:
        raise RuntimeError(msg)


def _cuda_bf16(t: torch.Tensor, name: str):
    _require(t.is_cuda, "%s must be a CUDA tensor" % name)
    _require(t.dtype == torch.bfloat16, "%s must be bf16 (got %s)" % (name, t.dtype))


def _token_tensor(t: torch.Tensor, varlen: bool) -> cabi.TokenTensor:
    """(B,T,H,D) or (N,H,D) view with contiguous last dim -> strides in elements."""
    _require(t.stride(-1) == 1, "head dimension must be contiguous")
    if varlen:
        _require(t.dim() == 3, "packed tensors are rank 3 (tokens, heads, dim)")
        return cabi.TokenTensor(t.data_ptr(), 0, t.stride(0), t.stride(1))
    _require(t.dim() == 4, "padded tensors are rank 4 (batch, tokens, heads, dim)")
    return cabi.TokenTensor(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))


def _token_scalar(t: Optional[torch.Tensor], varlen: bool) -> cabi.TokenScalar:
    if t is None:
        return cabi.TokenScalar(None, 0, 0, 0, 0)
    if varlen:
        _require(t.dim() == 2, "packed beta/gate are rank 2 (tokens, heads)")
        return cabi.TokenScalar(t.data_ptr(), _dt(t), 0, t.stride(0), t.stride(1))
    _require(t.dim() == 3, "padded beta/gate are rank 3 (batch, tokens, heads)")
    return cabi.TokenScalar(t.data_ptr(), _dt(t), t.stride(0), t.stride(1), t.stride(2))


def _state_desc(t: Optional[torch.Tensor]) -> cabi.State:
    if t is None:
        return cabi.State(None, 0, 0)
    _require(t.stride(-1) == 1 and t.stride(-2) == t.shape[-1], "state (dv, dk) block must be contiguous")
    return cabi.State(t.data_ptr(), t.stride(0), t.stride(1))


def _i32(t: Optional[torch.Tensor], name: str):
    if t is None:
        return None
    _require(t.is_cuda and t.dtype == torch.int32 and t.is_contiguous(), "%s must be a contiguous int32 CUDA tensor" % name)
    return t.data_ptr()


def _shape(batch, seq_len, total_tokens, kh, vh, dk, dv, cu_seqlens=None, chunk_indices=None,
           cu_chunks=None, total_chunks=0) -> cabi.Shape:
    return cabi.Shape(batch, seq_len, total_tokens, kh, vh, dk, dv, _i32(cu_seqlens, "cu_seqlens"),
                      _i32(chunk_indices, "chunk_indices"), _i32(cu_chunks, "cu_chunks"), int(total_chunks))


def _tma_ready(t: torch.Tensor) -> torch.Tensor:
    """The prefill kernels read token tensors through TMA: 16-byte aligned base, contiguous head dim, every other
    stride a multiple of 8 elements.  A view that does not qualify is compacted (a copy), anything else passes."""
    ok = t.stride(-1) == 1 and t.data_ptr() % 16 == 0 and all(st % 8 == 0 for st in t.stride()[:-1])
    return t if ok else t.contiguous()


def _pad_last(t: torch.Tensor, to: int) -> torch.Tensor:
    return t if t.shape[-1] == to else torch.nn.functional.pad(t, (0, to - t.shape[-1]))


def _pad_state(t: Optional[torch.Tensor], to: int) -> Optional[torch.Tensor]:
    if t is None or (t.shape[-1] == to and t.shape[-2] == to):
        return t
    return torch.nn.functional.pad(t, (0, to - t.shape[-1], 0, to - t.shape[-2]))


def _aligned_dim(d: int) -> int:
    return (d + 63) // 64 * 64


# --------------------------------------------------------------------------
def init(library_root: str, cuda_home: str) -> None:
    """Record the repository root (holding the kernel headers) and the CUDA toolkit root
    for the run-time kernel compiler.  Mirrors gdn_cuda.init (python_api.cpp:20)."""
    _state["library_root"], _state["cuda_home"] = library_root, cuda_home
    cabi.check(cabi.load().gdn_init(library_root.encode(), cuda_home.encode()), "init")


def fused_gdn_gating(A_log, dt_bias, a, b, is_var_len: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """(beta, gate) = (sigmoid(b), -exp(A_log) * softplus(a + dt_bias)); python_api.cpp:161-168.

    `A_log` may be the per-head vector (vh,) or, as in the reference, a tensor shaped like
    `a` whose first vh entries are the per-head values.  Output dtype = input dtype."""
    _require(a.is_cuda and b.is_cuda and A_log.is_cuda and dt_bias.is_cuda, "inputs must be CUDA tensors")
    _require(a.dtype == b.dtype == A_log.dtype == dt_bias.dtype, "A_log, dt_bias, a, b must share a dtype")
    vh = a.shape[-1]
    _require(dt_bias.numel() >= vh and A_log.numel() >= vh, "A_log and dt_bias need one entry per head")
    a_c, b_c = a.contiguous(), b.contiguous()
    A_c, dt_c = A_log.contiguous(), dt_bias.contiguous()
    beta = torch.empty_like(b_c)
    gate = torch.empty_like(a_c)
    n = a_c.numel() // vh
    cabi.check(cabi.load().gdn_fused_gating(A_c.data_ptr(), dt_c.data_ptr(), a_c.data_ptr(), b_c.data_ptr(),
                                             beta.data_ptr(), gate.data_ptr(), n, vh, _dt(a_c), _dt(gate),
                                             _stream()), "fused_gdn_gating")
    return beta, gate


def chunk_local_cumsum_bf16(input, output, batch_size: int, seq_len: int, num_heads: int,
                            head_first: bool = False, cu_seqlens=None, chunk_indices=None) -> None:
    """Chunk-local inclusive cumsum, bf16 (or fp32) in, fp32 out; python_api.cpp:328-339.

    As in the reference, `head_first=True` means the token-major layout (B,T,H)/(N,H) and
    `False` the time-contiguous one (B*H,T)/(H,N)."""
    _require(input.is_cuda and output.is_cuda, "tensors must be CUDA tensors")
    _require(output.dtype == torch.float32, "output must be fp32")
    _require(input.is_contiguous() and output.is_contiguous(), "input and output must be contiguous")
    tc = 0 if chunk_indices is None else chunk_indices.numel() // 2
    cabi.check(cabi.load().gdn_chunk_local_cumsum(
        input.data_ptr(), output.data_ptr(), _dt(input), batch_size, seq_len, num_heads, 1 if head_first else 0,
        _i32(cu_seqlens, "cu_seqlens"), _i32(chunk_indices, "chunk_indices"), tc, _stream()),
        "chunk_local_cumsum")


def _chunk_local_cumsum_f32(gate: torch.Tensor, batch, seq_len, vh, cu_seqlens, chunk_indices) -> torch.Tensor:
    out = torch.empty(gate.shape, dtype=torch.float32, device=gate.device)
    chunk_local_cumsum_bf16(gate.contiguous(), out, batch, seq_len, vh, True, cu_seqlens, chunk_indices)
    return out


def transpose_to_mn_major(input: torch.Tensor, alignment: int = 16) -> torch.Tensor:
    """(..., mn, k) -> same logical shape with mn padded to `alignment` bytes and
    stride(-2) == 1; python_api.cpp:362-368 / csrc/apis/layout.hpp:13-57.  Pad rows are zero."""
    _require(input.is_cuda and input.dim() >= 2, "input must be a CUDA tensor of rank >= 2")
    _require(input.dtype in (torch.float32, torch.bfloat16), "only fp32 and bf16 are supported")
    es = input.element_size()
    _require(alignment % es == 0, "alignment must be a multiple of the element size")
    x = input.contiguous()
    mn, k = x.shape[-2], x.shape[-1]
    per = alignment // es
    mn_al = (mn + per - 1) // per * per
    groups = x.numel() // max(mn * k, 1)
    store = torch.empty(*x.shape[:-2], k, mn_al, dtype=x.dtype, device=x.device)
    cabi.check(cabi.load().gdn_transpose_mn_major(x.data_ptr(), store.data_ptr(), es, groups, mn, k, mn_al,
                                                   _stream()), "transpose_to_mn_major")
    return store.transpose(-1, -2)


def recurrent_forward(query, key, value, initial_state=None, beta=None, gate=None, cu_seqlens=None,
                      num_accepted_tokens=None, inference_mode: int = 0, is_qk_norm: bool = False,
                      scale: Optional[float] = None, *, inplace_state: bool = False, gating=None,
                      state_indices=None, _max_head_dim: int = 256):
    """Token recurrence for decode / speculative verify / short prefill; python_api.cpp:107-122
    and csrc/apis/gdn_forward.cpp:134-206.

    Returns (output, new_state).  new_state is (B, vh, dv, dk), or one state per token
    ((B,T,vh,dv,dk) / (N,vh,dv,dk)) when inference_mode == SpecVerify.  `gate` may be bf16
    or fp32 (or None for no decay).  An fp32 `initial_state` (extension; head dims 64 and 128) keeps the
    state in fp32: it is read, updated and returned as fp32.  Extensions (keyword-only): with `inplace_state=True` the new
    state overwrites `initial_state`, which is returned (its (dv, dk) blocks must be contiguous);
    with `gating=(A_log, dt_bias, a, b)` the kernel computes beta = sigmoid(b) and
    gate = -exp(A_log) * softplus(a + dt_bias) itself from the layer's raw projections (what
    fused_gdn_gating would produce, without the extra launch or the bf16 rounding of its
    outputs) and `beta` / `gate` must be None; with `state_indices` (int32, one entry per sequence)
    `initial_state` is a pool of states (P, vh, dv, dk): sequence s uses slot state_indices[s], the new
    state is written back to the same slot (the pool is returned), and a negative slot marks a padding
    sequence that is skipped altogether."""
    if gating is not None:
        _require(beta is None and gate is None, "pass either gating=(A_log, dt_bias, a, b) or beta/gate, not both")
        g_A, g_dt, g_a, g_b = gating
        _require(g_a.dtype == g_b.dtype == g_A.dtype == g_dt.dtype, "A_log, dt_bias, a, b must share a dtype")
        _require(g_a.shape == g_b.shape and g_A.numel() >= g_a.shape[-1] and g_dt.numel() >= g_a.shape[-1],
                 "gating: a and b are (B,T,vh) / (N,vh); A_log and dt_bias hold one entry per v-head")
        g_A, g_dt = g_A.contiguous(), g_dt.contiguous()
    else:
        _require(beta is not None, "beta is required")
    for t, n in ((query, "query"), (key, "key"), (value, "value")):
        _cuda_bf16(t, n)
    varlen = cu_seqlens is not None
    mode = int(inference_mode)
    store_steps = mode == int(InferenceMode.SpecVerify)
    d = query.shape[-1]
    _require(key.shape[-1] == d, "query and key head dims differ")
    dv_in = value.shape[-1]
    d_al, dv_al = _aligned_dim(d), _aligned_dim(dv_in)
    _require(d_al <= _max_head_dim and dv_al <= _max_head_dim, "head dims above %d are not supported" % _max_head_dim)
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    q, k, v = _pad_last(query, d_al), _pad_last(key, d_al), _pad_last(value, dv_al)
    s_in = initial_state
    state_dtype = torch.bfloat16
    if s_in is not None:
        # an fp32 initial state selects the fp32-state kernels: the state stays fp32 (extension)
        _require(s_in.is_cuda and s_in.dtype in (torch.bfloat16, torch.float32), "initial_state must be a bf16 or fp32 CUDA tensor")
        state_dtype = s_in.dtype
        if s_in.shape[-1] != d_al or s_in.shape[-2] != dv_al:
            _require(not inplace_state, "in-place state needs head dims that are multiples of 64")
            s_in = torch.nn.functional.pad(s_in, (0, d_al - s_in.shape[-1], 0, dv_al - s_in.shape[-2]))
        if not (s_in.stride(-1) == 1 and s_in.stride(-2) == d_al):
            # a copy would silently break the in-place promise: the caller's tensor would never change
            _require(not inplace_state, "inplace_state needs contiguous (dv, dk) blocks in initial_state")
            s_in = s_in.contiguous()
    kh, vh = q.shape[-2], v.shape[-2]
    if varlen:
        batch, seq_len, total = cu_seqlens.numel() - 1, 0, q.shape[0]
    else:
        batch, seq_len, total = q.shape[0], q.shape[1], q.shape[0] * q.shape[1]
    out = torch.empty_like(v)
    if store_steps:
        lead = (total,) if varlen else (batch, seq_len)
        s_out = torch.empty(*lead, vh, dv_al, d_al, dtype=state_dtype, device=q.device)
        so_desc = cabi.State(s_out.data_ptr(), vh * dv_al * d_al, dv_al * d_al)
    elif inplace_state or state_indices is not None:
        _require(s_in is not None, "inplace_state / state_indices need an initial_state")
        _require(s_in is initial_state or s_in.data_ptr() == initial_state.data_ptr(),
                 "the state pool must have head dims that are multiples of 64 and contiguous (dv, dk) blocks")
        s_out = s_in
        so_desc = _state_desc(s_out)
    else:
        s_out = torch.empty(batch, vh, dv_al, d_al, dtype=state_dtype, device=q.device)
        so_desc = _state_desc(s_out)
    args = cabi.RecurrentArgs(
        _shape(batch, seq_len, total, kh, vh, d_al, dv_al, cu_seqlens),
        _token_tensor(q, varlen), _token_tensor(k, varlen), _token_tensor(v, varlen), _token_tensor(out, varlen),
        _token_scalar(beta, varlen), _token_scalar(gate, varlen), _state_desc(s_in), so_desc,
        _i32(num_accepted_tokens, "num_accepted_tokens"), float(scale), int(bool(is_qk_norm)), int(store_steps))
    args.state_dtype = cabi.GDN_F32 if state_dtype == torch.float32 else cabi.GDN_BF16
    if state_indices is not None:
        _require(not store_steps, "state_indices cannot be combined with per-token states")
        _require(state_indices.numel() == batch, "state_indices needs one entry per sequence")
        args.state_indices = _i32(state_indices, "state_indices")
    if gating is not None:
        args.gating_a, args.gating_b = _token_scalar(g_a, varlen), _token_scalar(g_b, varlen)
        args.A_log, args.dt_bias = g_A.data_ptr(), g_dt.data_ptr()
    cabi.check(cabi.load().gdn_recurrent_forward(C.byref(args), _stream()), "recurrent_forward")
    if dv_al != dv_in:
        out = out[..., :dv_in]
    if d_al != d or dv_al != dv_in:
        s_out = s_out[..., :dv_in, :d]
    return out, s_out


# --------------------------------------------------------------------------
# chunked prefill
# --------------------------------------------------------------------------
_PREFILL_D = 128  # head dimension the tensor-core kernels are built for


def _prefill_dims(query, value, cu_seqlens):
    varlen = cu_seqlens is not None
    if varlen:
        batch, seq_len, total = cu_seqlens.numel() - 1, 0, query.shape[0]
    else:
        batch, seq_len, total = query.shape[0], query.shape[1], query.shape[0] * query.shape[1]
    return varlen, batch, seq_len, total


def _check_head_dim(d: int):
    _require(0 < d <= _PREFILL_D, "chunked kernels support head dims up to %d (got %d)" % (_PREFILL_D, d))


_PREFILL_D_MAX = 256  # chunked_forward takes head dims up to here (above 128: the token-recurrent kernel)


def chunked_forward_workspace_bytes(batch: int, seq_len: int, num_v_heads: int, total_tokens: int = 0,
                                    total_chunks: int = 0, packed: bool = False,
                                    num_k_heads: Optional[int] = None) -> int:
    """Bytes of scratch `chunked_forward` needs for a problem of this size (head dim 128).  Without
    `num_k_heads` the figure is the upper bound num_k_heads = num_v_heads."""
    kh = num_v_heads if num_k_heads is None else num_k_heads
    shape = cabi.Shape(batch, seq_len, total_tokens if packed else batch * seq_len, kh, num_v_heads, _PREFILL_D,
                       _PREFILL_D, 1 if packed else None, None, None, total_chunks)
    return int(cabi.load().gdn_chunked_forward_workspace_bytes(C.byref(shape)))


def chunked_forward(query, key, value, beta, gate, scale: Optional[float] = None, initial_state=None,
                    cu_seqlens=None, chunk_indices=None, cu_chunks=None, total_chunks: Optional[int] = None,
                    *, is_qk_norm: bool = False, _stage_events=None, _workspace=None):
    """Chunked (64-token) Gated DeltaNet prefill; python_api.cpp:47-60, csrc/apis/gdn_forward.cpp:18-132.

    query/key (B,T,kh,d) or (N,kh,d); value (B,T,vh,d) or (N,vh,d); beta bf16 and gate fp32
    (raw per-token log-decay, before any cumsum) shaped (B,T,vh) / (N,vh); initial_state
    (B|S, vh, d, d) bf16 or None.  Packed mode needs int32 cu_seqlens, chunk_indices and
    cu_chunks.  Returns (output shaped like value, final_state (B|S, vh, d, d)), both bf16.
    The default scale is d ** -0.5 with d the caller's (unpadded) head dimension.
    `is_qk_norm=True` (keyword-only extension; the reference lists it as future work) L2-normalises
    q and k per head inside the kernels, as recurrent_forward does."""
    for t, n in ((query, "query"), (key, "key"), (value, "value")):
        _cuda_bf16(t, n)
    _require(gate is None or gate.dtype in (torch.float32, torch.bfloat16), "gate must be fp32 (or bf16)")
    varlen, batch, seq_len, total = _prefill_dims(query, value, cu_seqlens)
    d = query.shape[-1]
    _require(key.shape[-1] == d and value.shape[-1] == d, "chunked kernels need dk == dv")
    _require(0 < d <= _PREFILL_D_MAX, "chunked_forward supports head dims up to %d (got %d)" % (_PREFILL_D_MAX, d))
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    # up to 128: the tensor-core kernels, which compute on 128 columns.  A head dim that is a multiple of 8
    # goes in as it is (the library's tensor maps supply the zero columns, nothing is copied); any other is
    # zero-padded to 128 here.  129..256: the library runs the token recurrence on 192 or 256 columns instead.
    D = (d if d % 8 == 0 else _PREFILL_D) if d <= _PREFILL_D else _aligned_dim(d)
    q, k, v = (_tma_ready(_pad_last(t, D)) for t in (query, key, value))
    s_in = _pad_state(initial_state, D)
    if s_in is not None:
        _cuda_bf16(s_in, "initial_state")
        s_in = s_in if s_in.stride(-1) == 1 and s_in.stride(-2) == D else s_in.contiguous()
    kh, vh = q.shape[-2], v.shape[-2]
    if varlen:
        _require(chunk_indices is not None and cu_chunks is not None,
                 "packed mode needs cu_seqlens, chunk_indices and cu_chunks")
        tc = chunk_indices.numel() // 2 if total_chunks is None else int(total_chunks)
    else:
        tc = 0
    out = torch.empty_like(v)
    final = torch.empty(batch, vh, D, D, dtype=torch.bfloat16, device=q.device)
    shape = _shape(batch, seq_len, total, kh, vh, D, D, cu_seqlens, chunk_indices, cu_chunks, tc)
    lib = cabi.load()
    ws_bytes = lib.gdn_chunked_forward_workspace_bytes(C.byref(shape))
    ws = _workspace if _workspace is not None and _workspace.numel() >= ws_bytes else \
        torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
    ev = None
    if _stage_events is not None:  # three torch.cuda.Event(enable_timing=True), already recorded once
        ev = (C.c_void_p * 3)(*[e.cuda_event for e in _stage_events])
    args = cabi.ChunkedArgs(shape, _token_tensor(q, varlen), _token_tensor(k, varlen), _token_tensor(v, varlen),
                            _token_tensor(out, varlen), _token_scalar(beta, varlen), _token_scalar(gate, varlen),
                            _state_desc(s_in), _state_desc(final), float(scale), ws.data_ptr(), ws_bytes,
                            ev, int(bool(is_qk_norm)))
    cabi.check(lib.gdn_chunked_forward(C.byref(args), _stream()), "chunked_forward")
    if d != D:
        out, final = out[..., :d], final[..., :d, :d]
    return out, final


def bf16_gdn_compute_u_w(k, v, u, w, beta, gate=None, compiled_dims: str = "t", cu_seqlens=None,
                         chunk_indices=None) -> None:
    """Low-level WY/UT transform; python_api.cpp:199-210.  Writes u and w in place.

    beta and gate (chunk-local cumsum, fp32) may be MN-major views (stride(-2) == 1, as
    transpose_to_mn_major returns) or plain token-major tensors; `compiled_dims` is accepted
    and ignored (no dimension is baked into the kernels)."""
    for t, n in ((k, "k"), (v, "v"), (u, "u"), (w, "w")):
        _cuda_bf16(t, n)
    varlen, batch, seq_len, total = _prefill_dims(k, v, cu_seqlens)
    d = k.shape[-1]
    _require(0 < d <= _PREFILL_D and v.shape[-1] == d, "low-level chunked kernels need dk = dv <= %d" % _PREFILL_D)
    if d != _PREFILL_D:
        # the kernels are built for head dim 128: run on zero-padded copies (exact) and copy the results back
        up, wp = torch.empty(*u.shape[:-1], _PREFILL_D, dtype=u.dtype, device=u.device), \
            torch.empty(*w.shape[:-1], _PREFILL_D, dtype=w.dtype, device=w.device)
        bf16_gdn_compute_u_w(_pad_last(k, _PREFILL_D), _pad_last(v, _PREFILL_D), up, wp, beta, gate, compiled_dims,
                             cu_seqlens, chunk_indices)
        u.copy_(up[..., :d])
        w.copy_(wp[..., :d])
        return
    beta, gate = _crop_tokens(beta, total if varlen else seq_len), _crop_tokens(gate, total if varlen else seq_len)
    tc = 0 if chunk_indices is None else chunk_indices.numel() // 2
    shape = _shape(batch, seq_len, total, k.shape[-2], v.shape[-2], d, d, cu_seqlens, chunk_indices, None, tc)
    args = cabi.ComputeUWArgs(shape, _token_tensor(k, varlen), _token_tensor(v, varlen), _token_tensor(u, varlen),
                              _token_tensor(w, varlen), _token_scalar(beta, varlen), _token_scalar(gate, varlen))
    cabi.check(cabi.load().gdn_compute_u_w(C.byref(args), _stream()), "bf16_gdn_compute_u_w")


def _crop_tokens(t: Optional[torch.Tensor], tokens: int) -> Optional[torch.Tensor]:
    """MN-major tensors carry a padded token axis; cut the view back to the real length."""
    if t is None:
        return None
    return t[..., :tokens, :] if t.shape[-2] != tokens else t


def bf16_chunked_seq_state_update(k, u, w, initial_state, state, final_state, gate=None,
                                  compiled_dims: str = "t", cu_seqlens=None, cu_chunks=None,
                                  total_chunks: Optional[int] = None, chunk_size: int = 64) -> None:
    """Low-level chunk-to-chunk state pass; python_api.cpp:243-258.  Writes `state` (the state
    entering every chunk, (B,nc,vh,d,d) / (total_chunks,vh,d,d)), `final_state`, and
    overwrites `u` with U_new."""
    _require(chunk_size == CHUNK, "only chunk_size 64 is supported")
    for t, n in ((k, "k"), (u, "u"), (w, "w"), (state, "state")):
        _cuda_bf16(t, n)
    varlen, batch, seq_len, total = _prefill_dims(k, u, cu_seqlens)
    d = k.shape[-1]
    _require(0 < d <= _PREFILL_D and u.shape[-1] == d, "low-level chunked kernels need dk = dv <= %d" % _PREFILL_D)
    _require(state.is_contiguous(), "state must be contiguous")
    if d != _PREFILL_D:
        # as the reference's wrapper does (csrc/apis/gdn_forward.cpp:252-302): zero-padded copies, results copied back
        D = _PREFILL_D
        up = _pad_last(u, D)
        sp = torch.empty(*state.shape[:-2], D, D, dtype=state.dtype, device=state.device)
        fp = None if final_state is None else torch.empty(*final_state.shape[:-2], D, D, dtype=state.dtype, device=state.device)
        bf16_chunked_seq_state_update(_pad_last(k, D), up, _pad_last(w, D), _pad_state(initial_state, D), sp, fp, gate,
                                      compiled_dims, cu_seqlens, cu_chunks, total_chunks, chunk_size)
        u.copy_(up[..., :d])
        state.copy_(sp[..., :d, :d])
        if final_state is not None:
            final_state.copy_(fp[..., :d, :d])
        return
    gate = _crop_tokens(gate, total if varlen else seq_len)
    if varlen:
        _require(cu_chunks is not None, "packed mode needs cu_chunks")
        tc = state.shape[0] if total_chunks is None else int(total_chunks)
    else:
        tc = 0
    shape = _shape(batch, seq_len, total, k.shape[-2], u.shape[-2], d, d, cu_seqlens, None, cu_chunks, tc)
    args = cabi.SeqStateArgs(shape, _token_tensor(k, varlen), _token_tensor(u, varlen), _token_tensor(w, varlen),
                             _token_scalar(gate, varlen), _state_desc(initial_state), _state_desc(final_state),
                             state.data_ptr())
    cabi.check(cabi.load().gdn_seq_state_update(C.byref(args), _stream()), "bf16_chunked_seq_state_update")


def bf16_gdn_chunked_compute_O(q, state, k, u, o, gate=None, scale: Optional[float] = None,
                               compiled_dims: str = "t", cu_seqlens=None, chunk_indices=None, cu_chunks=None,
                               chunk_size: int = 64) -> None:
    """Low-level output stage; python_api.cpp:287-302.  Writes `o`."""
    _require(chunk_size == CHUNK, "only chunk_size 64 is supported")
    for t, n in ((q, "q"), (k, "k"), (u, "u"), (o, "o"), (state, "state")):
        _cuda_bf16(t, n)
    varlen, batch, seq_len, total = _prefill_dims(q, u, cu_seqlens)
    d = q.shape[-1]
    _require(0 < d <= _PREFILL_D and u.shape[-1] == d, "low-level chunked kernels need dk = dv <= %d" % _PREFILL_D)
    _require(state.is_contiguous(), "state must be contiguous")
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    if d != _PREFILL_D:
        D = _PREFILL_D
        op = torch.empty(*o.shape[:-1], D, dtype=o.dtype, device=o.device)
        bf16_gdn_chunked_compute_O(_pad_last(q, D), _pad_state(state, D).contiguous(), _pad_last(k, D), _pad_last(u, D), op,
                                   gate, scale, compiled_dims, cu_seqlens, chunk_indices, cu_chunks, chunk_size)
        o.copy_(op[..., :d])
        return
    gate = _crop_tokens(gate, total if varlen else seq_len)
    tc = 0
    if varlen:
        _require(chunk_indices is not None, "packed mode needs chunk_indices")
        tc = chunk_indices.numel() // 2
    shape = _shape(batch, seq_len, total, q.shape[-2], u.shape[-2], d, d, cu_seqlens, chunk_indices, cu_chunks, tc)
    args = cabi.ComputeOArgs(shape, _token_tensor(q, varlen), _token_tensor(k, varlen), _token_tensor(u, varlen),
                             _token_tensor(o, varlen), _token_scalar(gate, varlen), state.data_ptr(), float(scale))
    cabi.check(cabi.load().gdn_compute_o(C.byref(args), _stream()), "bf16_gdn_chunked_compute_O")


# --------------------------------------------------------------------------
# layer-adjacent steps (not in the reference: its callers run them)
# --------------------------------------------------------------------------
def causal_conv1d(x, weight, bias=None, initial_state=None, cu_seqlens=None, activation: bool = True,
                  final_state=None, return_final_state: bool = False):
    """Depthwise causal convolution along the token axis (+ SiLU), as applied to the q/k/v projections in
    front of Gated DeltaNet.  x: (B, T, C) or packed (N, C) bf16 with contiguous channels; weight: (C, W)
    bf16, W = 2 .. 4; bias: (C) or None; initial_state: (sequences, W-1, C) holding the W-1 inputs before
    each sequence (None: zeros).  Returns y, or (y, final_state) with the last W-1 inputs of every sequence
    when `return_final_state` (or when a `final_state` buffer is given; it may be `initial_state` itself for
    decode-sized calls)."""
    _cuda_bf16(x, "x")
    _cuda_bf16(weight, "weight")
    _require(x.stride(-1) == 1, "channels must be contiguous")
    varlen = cu_seqlens is not None
    C_, W = weight.shape
    _require(x.shape[-1] == C_, "weight must be (channels, width)")
    if varlen:
        _require(x.dim() == 2, "packed input is (tokens, channels)")
        batch, seq_len, total, xsb, xst = cu_seqlens.numel() - 1, 0, x.shape[0], 0, x.stride(0)
    else:
        _require(x.dim() == 3, "padded input is (batch, tokens, channels)")
        batch, seq_len, total, xsb, xst = x.shape[0], x.shape[1], x.shape[0] * x.shape[1], x.stride(0), x.stride(1)
    y = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    w = weight.contiguous()
    b = None if bias is None else bias.contiguous()
    s_in = None if initial_state is None else initial_state.contiguous()
    if s_in is not None:
        _require(tuple(s_in.shape) == (batch, W - 1, C_) and s_in.dtype == torch.bfloat16, "initial_state must be (sequences, W-1, C) bf16")
    s_out = final_state
    if s_out is None and return_final_state:
        s_out = torch.empty(batch, W - 1, C_, dtype=x.dtype, device=x.device)
    if s_out is not None:
        _require(s_out.is_contiguous() and tuple(s_out.shape) == (batch, W - 1, C_), "final_state must be contiguous (sequences, W-1, C)")
    args = cabi.ConvArgs(x.data_ptr(), y.data_ptr(), w.data_ptr(), None if b is None else b.data_ptr(),
                         None if s_in is None else s_in.data_ptr(), None if s_out is None else s_out.data_ptr(),
                         xsb, xst, 0 if varlen else y.stride(0), y.stride(0) if varlen else y.stride(1),
                         batch, seq_len, total, _i32(cu_seqlens, "cu_seqlens"), C_, W, int(bool(activation)))
    cabi.check(cabi.load().gdn_causal_conv1d(C.byref(args), _stream()), "causal_conv1d")
    return (y, s_out) if s_out is not None else y


def gated_rmsnorm(x, z, weight, eps: float = 1e-6):
    """y = x * rsqrt(mean(x^2) + eps) * weight * silu(z) over the last axis: the output norm that follows Gated
    DeltaNet (x: the layer's output, z: the gate projection, both (..., D) bf16; weight (D))."""
    _cuda_bf16(x, "x")
    _cuda_bf16(z, "z")
    _cuda_bf16(weight, "weight")
    _require(x.shape == z.shape and x.shape[-1] == weight.numel(), "x and z must have the same shape, weight one entry per column")
    D = x.shape[-1]
    x2 = x.reshape(-1, D) if x.is_contiguous() else x.contiguous().view(-1, D)
    z2 = z.reshape(-1, D) if z.is_contiguous() else z.contiguous().view(-1, D)
    y = torch.empty(x2.shape, dtype=x.dtype, device=x.device)
    cabi.check(cabi.load().gdn_gated_rmsnorm(x2.data_ptr(), z2.data_ptr(), y.data_ptr(), weight.contiguous().data_ptr(), x2.shape[0], D,
                                             x2.stride(0), z2.stride(0), y.stride(0), float(eps), _stream()), "gated_rmsnorm")
    return y.view(x.shape)
