"""B200-native Gated DeltaNet kernels behind the `gdn_cuda` API of kingsleykimm/h100_gdn_cuda.

    import h100_gdn_cuda_b200 as gdn_cuda
    gdn_cuda.init(repo_root, "/usr/local/cuda")
    o, s = gdn_cuda.chunked_forward(q, k, v, beta, gate, None, s0)

All compute happens in libgdn_b200.so (hand-written sm_100a CUDA behind a C ABI, declared
in include/gdn_b200.h).  Importing this package does not need a GPU; calling an operation
without the built library or on a non-sm_100 device raises RuntimeError.
"""
from . import api  # noqa: F401
from .api import (  # noqa: F401
    Decode,
    InferenceMode,
    Prefill,
    SpecVerify,
    bf16_chunked_seq_state_update,
    bf16_gdn_chunked_compute_O,
    bf16_gdn_compute_u_w,
    causal_conv1d,
    chunk_local_cumsum_bf16,
    chunked_forward,
    fused_gdn_gating,
    gated_rmsnorm,
    init,
    recurrent_forward,
    transpose_to_mn_major,
)

__version__ = "0.1.0"
