/* gdn_b200.h - C ABI of libgdn_b200.so, a Gated DeltaNet kernel library for NVIDIA B200
 * (sm_100a).
 *
 * Every entry point replaces one function of the `gdn_cuda` C++ API of
 * kingsleykimm/h100_gdn_cuda (csrc/apis/gdn_forward.hpp:15-73); the citation beside each
 * declaration names the reference function it stands in for.  The functions take plain
 * device pointers, sizes and element strides, enqueue their work on the given stream,
 * never synchronise, never allocate unless stated, never exit the process and never throw:
 * they return GDN_OK or a negative error code, and gdn_last_error() returns a message for
 * the calling thread's last failure.
 *
 * Conventions
 *   - "token tensors" (q, k, v, u, w, o) are bf16 with the head dimension contiguous; they are
 *     addressed as  base + batch*stride_batch + token*stride_token + head*stride_head  (in
 *     elements).  In packed variable-length mode (`cu_seqlens != NULL`) there is no batch
 *     axis and `token` is the global token index.
 *   - "per-token scalars" (beta, gate) are addressed the same way with a head stride, so
 *     both the token-major (B,T,H) layout and the time-contiguous "MN-major" (B,H,T_pad)
 *     layout of the reference are expressed by strides.
 *   - states are bf16, laid out (sequence, v_head, dv, dk) with dk contiguous and dv rows
 *     packed (the reference's layout, csrc/apis/gdn_forward.cpp:102-112).
 *   - the chunk size is 64 tokens.
 *   - q and k have `num_k_heads` heads, v/u/w/o/beta/gate/state have `num_v_heads`;
 *     v-head h uses k-head h / (num_v_heads / num_k_heads).
 */
#ifndef GDN_B200_H
#define GDN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* gdn_stream_t; /* a cudaStream_t */

enum {
    GDN_OK = 0,
    GDN_ERR_INVALID = -1,     /* bad shape, stride, alignment, dtype or NULL pointer          */
    GDN_ERR_UNSUPPORTED = -2, /* valid request this build has no kernel for (or non-sm_100 GPU) */
    GDN_ERR_CUDA = -3,        /* a CUDA runtime / driver call failed                          */
    GDN_ERR_WORKSPACE = -4,   /* workspace missing, misaligned or too small                   */
    GDN_ERR_DEVICE = -5       /* a kernel reported a bounded wait that ran out                */
};

enum { GDN_BF16 = 0, GDN_F32 = 1 };
enum { GDN_MODE_PREFILL = 0, GDN_MODE_DECODE = 1, GDN_MODE_SPEC_VERIFY = 2 };

/* bf16 tensor with a contiguous last (head-dim) axis. */
typedef struct {
    void* ptr;
    int64_t stride_batch;
    int64_t stride_token;
    int64_t stride_head;
} GdnTokenTensor;

/* one scalar per (token, v-head); dtype GDN_BF16 or GDN_F32; ptr == NULL means absent. */
typedef struct {
    void* ptr;
    int32_t dtype;
    int64_t stride_batch;
    int64_t stride_token;
    int64_t stride_head;
} GdnTokenScalar;

/* (sequence, v_head, dv, dk) bf16 state; the inner (dv, dk) block is contiguous. */
typedef struct {
    void* ptr;
    int64_t stride_seq;
    int64_t stride_head;
} GdnState;

/* Shape of a call.  Padded mode: `batch` sequences of `seq_len` tokens.  Packed mode
 * (`cu_seqlens` given): `batch` sequences, `total_tokens` tokens, `seq_len` ignored. */
typedef struct {
    int32_t batch;
    int32_t seq_len;
    int64_t total_tokens;
    int32_t num_k_heads;
    int32_t num_v_heads;
    int32_t head_dim_k; /* dk */
    int32_t head_dim_v; /* dv */
    const int32_t* cu_seqlens;    /* device, batch+1 entries, or NULL                    */
    const int32_t* chunk_indices; /* device, 2*total_chunks entries [seq, chunk], or NULL */
    const int32_t* cu_chunks;     /* device, batch+1 entries, or NULL                    */
    int32_t total_chunks;         /* packed mode: number of 64-token chunks              */
} GdnShape;

/* ---------------------------------------------------------------- runtime
 * Replaces gdn_cuda::init (csrc/apis/gdn_forward.cpp:14-16 -> Compiler::init_static_vars,
 * csrc/jit/compiler.hpp:34-40): records where the kernel headers and the CUDA toolkit are
 * for the run-time kernel compiler.  Either argument may be NULL (built-in kernels only). */
int gdn_init(const char* library_root, const char* cuda_home);

/* Message for the calling thread's most recent failure ("" if none). */
const char* gdn_last_error(void);

/* Library version as major*10000 + minor*100 + patch. */
int gdn_version(void);

/* Reads and clears the device-side status word of `device` (synchronises that device's
 * work first).  0 = no kernel reported a problem.  Debug / test aid; has no counterpart in
 * the reference, whose device asserts trap (kernels/common/common.hpp:485-493). */
int gdn_device_status(int device, int* status_out);

/* Self-test of the bounded waits every kernel of this library uses (no counterpart in the
 * reference, whose waits spin without a limit, kernels/common/sm90_utils.cuh): launches one warp
 * that waits on a barrier nothing will ever complete, with a limit of `limit_cycles` SM clock
 * cycles (1 .. 1e9).  The wait gives up, the kernel sets the device status word to 7 and returns;
 * gdn_device_status() then reads 7 and the context stays usable.  Status codes of the product
 * kernels: 1 recurrent, 2 WY/UT and chunk-parallel stage, 4 state/output stage, 6 other prefill
 * stages.  A kernel whose wait gave up writes none of its outputs where that is cheap to arrange
 * (recurrent, whole-layer prefill); the entry point has long returned GDN_OK by then, so the
 * status word, not a return code, is how GDN_ERR_DEVICE conditions are observed. */
int gdn_selftest_bounded_wait(int64_t limit_cycles, gdn_stream_t stream);

/* Replaces Compiler::build (csrc/jit/compiler.hpp:82-103): compiles `source`, a complete CUDA
 * translation unit that may include the library's kernel headers ("kernels/...") and defines
 * an extern "C" kernel, to an sm_100a cubin, or finds it in the on-disk cache
 * ($JIT_CACHE_DIR or ~/.gdn_b200/cache, directory kernel.<name>.<hash>).  NVRTC is used when it
 * can be loaded and JIT_USE_NVRTC is not 0, otherwise <cuda_home>/bin/nvcc.  Needs gdn_init()
 * first and no GPU.  Writes the cubin path and whether it was a cache hit.  The library uses this
 * itself for kernels it has no prebuilt instance of (recurrent head dims above 256). */
int gdn_jit_compile(const char* name, const char* source, char* cubin_path_out, size_t cubin_path_cap,
                    int* cache_hit_out);

/* ---------------------------------------------------------------- helpers
 * Replaces kernels::gdn_gating (src/gdn_ops.cu:13-33; kernel gdn_helpers.cuh:41-122):
 *   beta = sigmoid(b),  gate = -exp(A_log[h]) * softplus(a + dt_bias[h])   (softplus(x) = x for x > 20)
 * a, b, beta, gate are contiguous (num_tokens, num_v_heads); A_log, dt_bias have num_v_heads
 * entries.  `dtype` is the type of all four inputs and of beta; `gate_dtype` that of gate. */
int gdn_fused_gating(const void* A_log, const void* dt_bias, const void* a, const void* b,
                     void* beta, void* gate, int64_t num_tokens, int32_t num_v_heads,
                     int32_t dtype, int32_t gate_dtype, gdn_stream_t stream);

/* Replaces kernels::chunk_local_cumsum (src/gdn_ops.cu:38-57; kernels gdn_helpers.cuh:142-256):
 * inclusive prefix sum of `input` restarted at every 64-token chunk of every sequence;
 * fp32 output in the same layout.  `token_major` != 0: (batch, seq_len, heads) / (tokens, heads)
 * (the reference's head_first=true); 0: time-contiguous (batch*heads, seq_len) / (heads, tokens).
 * Packed mode needs cu_seqlens and chunk_indices (total_chunks pairs). */
int gdn_chunk_local_cumsum(const void* input, float* output, int32_t in_dtype, int32_t batch,
                           int64_t seq_len, int32_t num_heads, int32_t token_major,
                           const int32_t* cu_seqlens, const int32_t* chunk_indices,
                           int32_t total_chunks, gdn_stream_t stream);

/* Replaces api::transpose_to_mn_major (csrc/apis/layout.hpp:13-57; kernels sm90_layout.cuh:10-87):
 * `groups` row-major (mn, k) matrices -> (k, mn_aligned) each, pad columns written as zero.
 * elem_size is 2 or 4 bytes. */
int gdn_transpose_mn_major(const void* input, void* output, int32_t elem_size, int64_t groups,
                           int64_t mn, int64_t k, int64_t mn_aligned, gdn_stream_t stream);

/* ---------------------------------------------------------------- recurrent decode / spec-verify
 * Replaces gdn_cuda::bf16_gdn_recurrent / recurrent_forward (csrc/apis/gdn_forward.cpp:134-206,
 * 240-250; kernel sm90_bf16_gdn_recurrent.cuh:20-440).  Per token t of sequence s, v-head h:
 *     S <- exp(g) S ;  S <- S + beta (v - S k) k^T ;  o = scale * S q
 * with optional L2 normalisation of q and k (x * rsqrt(sum x^2 + 1e-6)).
 *   state_in.ptr == NULL  : start from zero.
 *   num_accepted_tokens   : optional device int32[batch]; caps the tokens processed per sequence
 *                           (outputs past the cap are left untouched).
 *   store_step_state != 0 : state_out holds one state per token, addressed
 *                           token_index*stride_seq + head*stride_head (token_index =
 *                           b*seq_len + t, or the packed token index); otherwise one per
 *                           sequence.  state_out may alias state_in when not storing steps.
 *   gating_a.ptr != NULL  : the gating of the layer is computed inside the kernel from its raw
 *                           projections (what gdn_fused_gating does, csrc/apis/gdn_forward.cpp:208-229,
 *                           without the extra launch and without rounding beta and the gate to bf16):
 *                               beta = sigmoid(gating_b),  g = -exp(A_log[h]) * softplus(gating_a + dt_bias[h])
 *                           gating_a / gating_b are per-token scalars like beta / gate (same dtype for
 *                           both, bf16 or f32); A_log and dt_bias are contiguous vectors of num_v_heads
 *                           entries of that dtype.  `beta` and `gate` are then ignored.
 *   state_indices != NULL : indexed state pool, as serving engines keep one (no counterpart in the reference):
 *                           device int32[batch]; sequence s reads its state from slot state_indices[s] of
 *                           state_in and writes the new one to the same slot of state_out (addressed
 *                           slot*stride_seq; the two may be the same pool).  A negative slot marks a padding
 *                           sequence: nothing is read, computed or written for it.  Not combined with
 *                           store_step_state. */
typedef struct {
    GdnShape shape;
    GdnTokenTensor q, k, v, out;
    GdnTokenScalar beta, gate; /* gate.ptr may be NULL (no decay) */
    GdnState state_in, state_out;
    const int32_t* num_accepted_tokens;
    float scale;
    int32_t is_qk_norm;
    int32_t store_step_state;
    /* fused gating (all four given, or gating_a.ptr == NULL) */
    GdnTokenScalar gating_a, gating_b;
    const void* A_log;
    const void* dt_bias;
    const int32_t* state_indices;
    /* GDN_BF16 (0, the reference's only state type) or GDN_F32: element type of state_in and state_out, whose
     * strides then count fp32 elements.  A state kept in fp32 is not rounded between decode steps.  No
     * counterpart in the reference; built for dk = 64 and 128. */
    int32_t state_dtype;
} GdnRecurrentArgs;
int gdn_recurrent_forward(const GdnRecurrentArgs* args, gdn_stream_t stream);

/* ---------------------------------------------------------------- chunked prefill, stage by stage
 * Replaces api::bf16_gdn_compute_u_w (csrc/apis/gdn.hpp:14-24; kernel
 * sm90_bf16_gdn_compute_u_w.cuh:153-667).  Per 64-token chunk and v-head, with g the
 * chunk-local cumulative gate (fp32; absent = no decay):
 *     A = tril(diag(beta) K K^T .* exp(g_i - g_j), -1),  T = (I + A)^-1 diag(beta)
 *     U = T V,   W = T (K .* exp(g))
 * (W is the canonical form; the reference scales rows after the solve instead.) */
typedef struct {
    GdnShape shape;
    GdnTokenTensor k, v, u, w;
    GdnTokenScalar beta, gate_cumsum;
} GdnComputeUWArgs;
int gdn_compute_u_w(const GdnComputeUWArgs* args, gdn_stream_t stream);

/* Replaces api::bf16_chunked_seq_state_update (csrc/apis/gdn.hpp:26-39; kernel
 * sm90_bf16_chunked_seq_state_update2.cuh).  Sequential over the chunks of a sequence:
 *     h[c] = S ;  U_new = U - W S^T ;  S <- exp(g_last) S + U_new^T (K .* exp(g_last - g))
 * `u` is overwritten with U_new.  chunk_states is (batch, num_chunks, vh, dv, dk) in padded
 * mode and (total_chunks, vh, dv, dk) in packed mode, contiguous.  initial_state.ptr and
 * final_state.ptr may be NULL. */
typedef struct {
    GdnShape shape;
    GdnTokenTensor k, u, w;
    GdnTokenScalar gate_cumsum;
    GdnState initial_state, final_state;
    void* chunk_states;
} GdnSeqStateArgs;
int gdn_seq_state_update(const GdnSeqStateArgs* args, gdn_stream_t stream);

/* Replaces api::bf16_gdn_chunked_compute_O (csrc/apis/gdn.hpp:41-55; kernel
 * sm90_bf16_gdn_chunked_compute_O.cuh:23-530):
 *     O = scale * ( exp(g) .* (Q h[c]^T) + tril(Q K^T .* exp(g_i - g_j)) U_new ) */
typedef struct {
    GdnShape shape;
    GdnTokenTensor q, k, u_new, out;
    GdnTokenScalar gate_cumsum;
    const void* chunk_states;
    float scale;
} GdnComputeOArgs;
int gdn_compute_o(const GdnComputeOArgs* args, gdn_stream_t stream);

/* ---------------------------------------------------------------- chunked prefill, whole layer
 * Replaces gdn_cuda::chunked_forward (csrc/apis/gdn_forward.cpp:18-132): raw (pre-cumsum)
 * fp32 or bf16 gate, token-major beta; writes `out` (like v) and final_state.  The per-chunk
 * state tensor of the reference is never materialised.  `workspace` is caller-provided device
 * memory of at least gdn_chunked_forward_workspace_bytes(&shape) bytes, 256-byte aligned; its
 * contents need not be initialised and are garbage afterwards.  It holds one 24 KiB block per
 * 64-token chunk and v-head (the WY/UT transform folded into a 64 x 128 and a 64 x 64 bf16
 * matrix that the state kernel consumes) and, when few long sequences (padded, or packed with
 * at most 64 sequences) are propagated in segments, three fp32 states (192 KiB) per (sequence,
 * v-head) and segment; other packed inputs of 2 to 2048 sequences add 4 bytes per sequence (the
 * sequences ordered by length: the state kernel takes the longest first when there are more
 * (sequence, v-head) pairs than SMs).
 * Head dims: the tensor-core kernels compute on dk = dv = 128; any dk = dv that is a multiple of 8 up to
 * 128 is taken as it is (the tensor maps deliver zero columns past it, states are d x d; no padded copies),
 * callers zero-pad other head dims below 128;
 * dk = dv = 192 or 256 are accepted as well and run on the kernel of gdn_recurrent_forward
 * (no workspace: gdn_chunked_forward_workspace_bytes returns 0; final_state.ptr must be given). */
typedef struct {
    GdnShape shape;
    GdnTokenTensor q, k, v, out;
    GdnTokenScalar beta, gate;
    GdnState initial_state, final_state; /* either ptr may be NULL */
    float scale;
    void* workspace;
    size_t workspace_bytes;
    /* Optional profiling aid: NULL, or three cudaEvent_t recorded on `stream` before the first
     * kernel, between the chunk-parallel kernel and the state/output kernel, and after the last. */
    void* const* stage_events;
    /* != 0: q and k are L2-normalised per head (x * rsqrt(sum x^2 + 1e-6)) inside the kernels, as
     * gdn_recurrent_forward does; the tiles are not touched, the factors enter the gate vectors.
     * (The reference lists this as future work, README.md:113.)  Adds 512 bytes of workspace per
     * (chunk, k-head); gdn_chunked_forward_workspace_bytes() always includes them. */
    int32_t is_qk_norm;
} GdnChunkedArgs;
size_t gdn_chunked_forward_workspace_bytes(const GdnShape* shape);
int gdn_chunked_forward(const GdnChunkedArgs* args, gdn_stream_t stream);

/* ---------------------------------------------------------------- chunked prefill without a workspace
 * No counterpart in the reference (its wrapper always allocates scratch through torch).
 *
 * Some hosts of this library may not allocate device memory at the moment they need a
 * prefill: a serving engine that has handed all HBM to its own pool, a plugin running
 * inside someone else's memory plan, or code on a path where cudaMalloc is forbidden
 * because it synchronises the device.  For them this entry point runs the same two kernels
 * as gdn_chunked_forward but keeps their scratch in a fixed array that is part of the
 * library image (GDN_STATIC_SCRATCH_BYTES of device memory on every GPU that loads the
 * library, held until the process exits).  `workspace` and `workspace_bytes` in `args` are
 * ignored; inputs and outputs are passed as usual.
 *
 *   - Limit: gdn_chunked_forward_workspace_bytes(&args->shape) must not exceed
 *     GDN_STATIC_SCRATCH_BYTES (49 MiB + 8.5 KiB).  The scratch holds 24 KiB per 64-token
 *     chunk and v-head (384 bytes per token and v-head) plus 512 bytes per chunk and k-head,
 *     so with whole chunks that is tokens * num_v_heads <= 131072, for example 4096
 *     tokens of 32 v-heads (less where long sequences of few heads add their segment states).
 *     Larger problems are refused with GDN_ERR_WORKSPACE and a message.
 *   - It calls no cudaMalloc / cudaFree and no allocating library routine.
 *   - The first call on each device looks up the array's device address; make that first
 *     call outside any stream capture.  With CUDA's lazy module loading that first call (or the
 *     first gdn_chunked_forward on the device, which loads the same module) is also the moment
 *     the array's memory is claimed on that device: a host that is about to hand all HBM to its
 *     own pool should make one small warm-up call on each device before it does so, or the
 *     first real call can fail for lack of memory.
 *   - All calls on a device share the one array and it keeps whatever the previous call
 *     left there.  Nothing in it has to start at zero (every element that is read has been
 *     written earlier in the same call), but two calls whose kernels overlap on the GPU -
 *     different streams, or different host threads - race on it: serialise them. */
#define GDN_STATIC_SCRATCH_BYTES ((49u << 20) + 8192u + 512u)
int gdn_chunked_forward_static_scratch(const GdnChunkedArgs* args, gdn_stream_t stream);

/* ---------------------------------------------------------------- layer-adjacent steps
 * No counterpart in the reference, which leaves them to its callers: the two memory-bound steps on either
 * side of Gated DeltaNet in Qwen3-Next-style blocks.
 *
 * gdn_causal_conv1d: depthwise causal convolution along the token axis, optionally followed by SiLU, as
 * applied to the q/k/v projections before the layer:
 *     y[t, c] = act( bias[c] + sum_{i < width} weight[c, i] * x[t - (width-1) + i, c] )
 * x, y are bf16 with the channels contiguous (addressed batch*stride_batch + token*stride_token + c; packed
 * mode: global token index, no batch stride); weight is (channels, width) bf16, bias (channels) bf16 or
 * NULL; width 2 .. 4; channels a multiple of 8.  Inputs before a sequence's first token come from
 * state_in (sequences, width-1, channels; row width-2 is the input right before the sequence) or are zero
 * when it is NULL; state_out (same shape, or NULL) receives the sequence's last width-1 inputs, so that a
 * later call continues it (decode).  state_out may be the same buffer as state_in only when no sequence
 * spans more than one 32-token block: padded mode with seq_len <= 32, packed mode with one token per
 * sequence at most (total_tokens <= batch). */
typedef struct {
    const void* x;
    void* y;
    const void* weight;
    const void* bias;
    const void* state_in;
    void* state_out;
    int64_t x_stride_batch, x_stride_token, y_stride_batch, y_stride_token;
    int32_t batch;
    int32_t seq_len;
    int64_t total_tokens;
    const int32_t* cu_seqlens;
    int32_t channels;
    int32_t width;
    int32_t silu; /* != 0: SiLU after the convolution */
} GdnConvArgs;
int gdn_causal_conv1d(const GdnConvArgs* args, gdn_stream_t stream);

/* gdn_gated_rmsnorm: the output norm of the block, one row per (token, v-head):
 *     y = x * rsqrt(mean(x^2) + eps) * weight * silu(z)
 * x, z, y bf16 (rows, dim) with row strides in elements (multiples of 8) and contiguous rows; weight (dim)
 * bf16; dim a multiple of 8 up to 1024. */
int gdn_gated_rmsnorm(const void* x, const void* z, void* y, const void* weight, int64_t rows, int32_t dim,
                      int64_t x_row_stride, int64_t z_row_stride, int64_t y_row_stride, float eps,
                      gdn_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* GDN_B200_H */
