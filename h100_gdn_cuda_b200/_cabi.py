"""ctypes binding of libgdn_b200.so (declared in include/gdn_b200.h).

Loading fails loudly when the shared library has not been built; there is no
CPU or PyTorch fallback for any operation.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libgdn_b200.so")

GDN_BF16, GDN_F32 = 0, 1


class TokenTensor(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("stride_batch", C.c_int64), ("stride_token", C.c_int64),
                ("stride_head", C.c_int64)]


class TokenScalar(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("dtype", C.c_int32), ("stride_batch", C.c_int64),
                ("stride_token", C.c_int64), ("stride_head", C.c_int64)]


class State(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("stride_seq", C.c_int64), ("stride_head", C.c_int64)]


class Shape(C.Structure):
    _fields_ = [("batch", C.c_int32), ("seq_len", C.c_int32), ("total_tokens", C.c_int64),
                ("num_k_heads", C.c_int32), ("num_v_heads", C.c_int32), ("head_dim_k", C.c_int32),
                ("head_dim_v", C.c_int32), ("cu_seqlens", C.c_void_p), ("chunk_indices", C.c_void_p),
                ("cu_chunks", C.c_void_p), ("total_chunks", C.c_int32)]


class RecurrentArgs(C.Structure):
    _fields_ = [("shape", Shape), ("q", TokenTensor), ("k", TokenTensor), ("v", TokenTensor),
                ("out", TokenTensor), ("beta", TokenScalar), ("gate", TokenScalar),
                ("state_in", State), ("state_out", State), ("num_accepted_tokens", C.c_void_p),
                ("scale", C.c_float), ("is_qk_norm", C.c_int32), ("store_step_state", C.c_int32),
                ("gating_a", TokenScalar), ("gating_b", TokenScalar), ("A_log", C.c_void_p), ("dt_bias", C.c_void_p),
                ("state_indices", C.c_void_p), ("state_dtype", C.c_int32)]


class ComputeUWArgs(C.Structure):
    _fields_ = [("shape", Shape), ("k", TokenTensor), ("v", TokenTensor), ("u", TokenTensor),
                ("w", TokenTensor), ("beta", TokenScalar), ("gate_cumsum", TokenScalar)]


class SeqStateArgs(C.Structure):
    _fields_ = [("shape", Shape), ("k", TokenTensor), ("u", TokenTensor), ("w", TokenTensor),
                ("gate_cumsum", TokenScalar), ("initial_state", State), ("final_state", State),
                ("chunk_states", C.c_void_p)]


class ComputeOArgs(C.Structure):
    _fields_ = [("shape", Shape), ("q", TokenTensor), ("k", TokenTensor), ("u_new", TokenTensor),
                ("out", TokenTensor), ("gate_cumsum", TokenScalar), ("chunk_states", C.c_void_p),
                ("scale", C.c_float)]


class ChunkedArgs(C.Structure):
    _fields_ = [("shape", Shape), ("q", TokenTensor), ("k", TokenTensor), ("v", TokenTensor),
                ("out", TokenTensor), ("beta", TokenScalar), ("gate", TokenScalar),
                ("initial_state", State), ("final_state", State), ("scale", C.c_float),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
                ("stage_events", C.POINTER(C.c_void_p)), ("is_qk_norm", C.c_int32)]


class ConvArgs(C.Structure):
    _fields_ = [("x", C.c_void_p), ("y", C.c_void_p), ("weight", C.c_void_p), ("bias", C.c_void_p),
                ("state_in", C.c_void_p), ("state_out", C.c_void_p), ("x_stride_batch", C.c_int64),
                ("x_stride_token", C.c_int64), ("y_stride_batch", C.c_int64), ("y_stride_token", C.c_int64),
                ("batch", C.c_int32), ("seq_len", C.c_int32), ("total_tokens", C.c_int64), ("cu_seqlens", C.c_void_p),
                ("channels", C.c_int32), ("width", C.c_int32), ("silu", C.c_int32)]


# name -> (restype, argtypes); every symbol include/gdn_b200.h declares
SYMBOLS = {
    "gdn_init": (C.c_int, [C.c_char_p, C.c_char_p]),
    "gdn_last_error": (C.c_char_p, []),
    "gdn_version": (C.c_int, []),
    "gdn_device_status": (C.c_int, [C.c_int, C.POINTER(C.c_int)]),
    "gdn_selftest_bounded_wait": (C.c_int, [C.c_int64, C.c_void_p]),
    "gdn_jit_compile": (C.c_int, [C.c_char_p, C.c_char_p, C.c_char_p, C.c_size_t, C.POINTER(C.c_int)]),
    "gdn_fused_gating": (C.c_int, [C.c_void_p] * 6 + [C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "gdn_chunk_local_cumsum": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int64, C.c_int32,
                                         C.c_int32, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p]),
    "gdn_transpose_mn_major": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int64, C.c_int64,
                                         C.c_int64, C.c_void_p]),
    "gdn_recurrent_forward": (C.c_int, [C.POINTER(RecurrentArgs), C.c_void_p]),
    "gdn_compute_u_w": (C.c_int, [C.POINTER(ComputeUWArgs), C.c_void_p]),
    "gdn_seq_state_update": (C.c_int, [C.POINTER(SeqStateArgs), C.c_void_p]),
    "gdn_compute_o": (C.c_int, [C.POINTER(ComputeOArgs), C.c_void_p]),
    "gdn_chunked_forward_workspace_bytes": (C.c_size_t, [C.POINTER(Shape)]),
    "gdn_chunked_forward": (C.c_int, [C.POINTER(ChunkedArgs), C.c_void_p]),
    "gdn_chunked_forward_static_scratch": (C.c_int, [C.POINTER(ChunkedArgs), C.c_void_p]),
    "gdn_causal_conv1d": (C.c_int, [C.POINTER(ConvArgs), C.c_void_p]),
    "gdn_gated_rmsnorm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int64,
                                    C.c_int64, C.c_int64, C.c_float, C.c_void_p]),
}

_lib = None


def load():
    """Load the shared library once and attach prototypes."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                "libgdn_b200.so is not built (expected at %s); run `python -m h100_gdn_cuda_b200.build`. "
                "There is no fallback path." % LIB_PATH)
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(rc: int, what: str):
    if rc != 0:
        msg = load().gdn_last_error().decode("utf-8", "replace")
        raise RuntimeError("%s failed (%d): %s" % (what, rc, msg))
