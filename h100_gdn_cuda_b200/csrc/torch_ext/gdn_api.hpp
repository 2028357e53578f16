// C++ API `namespace gdn_cuda` over the C ABI of libgdn_b200.so, with the signatures of the
// reference's csrc/apis/gdn_forward.hpp:15-73 (at::Tensor arguments, an explicit stream).
// Errors are thrown as std::runtime_error (pybind turns them into RuntimeError).
#pragma once
#include <ATen/ATen.h>
#include <cuda_runtime_api.h>

#include <optional>
#include <string>
#include <tuple>
#include <utility>

namespace gdn_cuda {

enum class InferenceMode : int { Prefill = 0, Decode = 1, SpecVerify = 2, SpecDecode = 3 };

void init(const std::string& library_root, const std::string& cuda_home);

std::pair<at::Tensor, at::Tensor> chunked_forward(at::Tensor& query, at::Tensor& key, at::Tensor& value,
                                                  at::Tensor& beta, at::Tensor& gate, std::optional<float> scale,
                                                  std::optional<at::Tensor>& initial_state,
                                                  std::optional<at::Tensor>& cu_seqlens,
                                                  std::optional<at::Tensor>& chunk_indices,
                                                  std::optional<at::Tensor>& cu_chunks,
                                                  std::optional<int> total_chunks, cudaStream_t stream,
                                                  bool is_qk_norm = false);  // last argument: extension, see gdn_b200.h

std::pair<at::Tensor, at::Tensor> recurrent_forward(at::Tensor& query, at::Tensor& key, at::Tensor& value,
                                                    std::optional<at::Tensor>& initial_state, at::Tensor& beta,
                                                    at::Tensor& gate, std::optional<at::Tensor>& cu_seqlens,
                                                    std::optional<at::Tensor>& num_accepted_tokens,
                                                    InferenceMode inference_mode, cudaStream_t stream,
                                                    bool is_qk_norm, std::optional<float> scale);

// Extension: recurrent_forward with the layer's gating computed inside the kernel from its raw
// projections (beta = sigmoid(b), gate = -exp(A_log) softplus(a + dt_bias)); no separate gating launch.
std::pair<at::Tensor, at::Tensor> recurrent_forward_fused_gating(
    at::Tensor& query, at::Tensor& key, at::Tensor& value, std::optional<at::Tensor>& initial_state, at::Tensor& A_log,
    at::Tensor& dt_bias, at::Tensor& a, at::Tensor& b, std::optional<at::Tensor>& cu_seqlens,
    std::optional<at::Tensor>& num_accepted_tokens, InferenceMode inference_mode, cudaStream_t stream, bool is_qk_norm,
    std::optional<float> scale);

// Extensions of recurrent_forward beyond the reference's signature (all off by default):
//   inplace_state  the new state overwrites `initial_state`, which is returned;
//   state_indices  int32, one entry per sequence: `initial_state` is a pool of states (P, vh, dv, dk), sequence s
//                  uses and updates slot state_indices[s]; a negative slot marks a padding sequence (skipped).
// An fp32 `initial_state` (head dims 64 and 128) keeps the state in fp32: read, updated and returned as fp32.
struct RecurrentExtensions {
    bool inplace_state = false;
    std::optional<at::Tensor> state_indices;
};
// recurrent_forward with either beta / gate or gating = (A_log, dt_bias, a, b), and the extensions above
std::pair<at::Tensor, at::Tensor> recurrent_forward_ext(
    at::Tensor& query, at::Tensor& key, at::Tensor& value, std::optional<at::Tensor>& initial_state,
    std::optional<at::Tensor>& beta, std::optional<at::Tensor>& gate,
    std::optional<std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor>>& gating, std::optional<at::Tensor>& cu_seqlens,
    std::optional<at::Tensor>& num_accepted_tokens, InferenceMode inference_mode, cudaStream_t stream, bool is_qk_norm,
    std::optional<float> scale, const RecurrentExtensions& ext);

// The two memory-bound steps around the layer in Qwen3-Next-style blocks (no counterpart in the reference, whose
// callers run them): depthwise causal convolution (+ SiLU) over (B, T, C) or packed (N, C) with an optional carried
// state (sequences, W-1, C), returning (y, final_state or nothing); and y = rmsnorm(x) * weight * silu(z).
std::pair<at::Tensor, std::optional<at::Tensor>> causal_conv1d(at::Tensor& x, at::Tensor& weight,
                                                               std::optional<at::Tensor>& bias,
                                                               std::optional<at::Tensor>& initial_state,
                                                               std::optional<at::Tensor>& cu_seqlens, bool activation,
                                                               std::optional<at::Tensor>& final_state,
                                                               bool return_final_state, cudaStream_t stream);
at::Tensor gated_rmsnorm(at::Tensor& x, at::Tensor& z, at::Tensor& weight, float eps, cudaStream_t stream);

// csrc/apis/gdn_forward.hpp:43-49: the recurrence on caller-provided output tensors.  `final_state` is
// (B, vh, dv, dk), or one state per token when `store_step_state`; head dims must be multiples of 64
// here (no padding can be done on the caller's tensors); `compiled_dims` is accepted and ignored.
void bf16_gdn_recurrent(at::Tensor& q, at::Tensor& k, at::Tensor& v, std::optional<at::Tensor>& initial_state,
                        at::Tensor& final_state, at::Tensor& out, std::optional<at::Tensor>& gate, at::Tensor& beta,
                        const std::string& compiled_dims, cudaStream_t stream, std::optional<at::Tensor>& cu_seqlens,
                        std::optional<at::Tensor>& num_accepted_tokens, bool store_step_state = false,
                        bool is_qk_norm = false, float scale = 1.0f);

std::pair<at::Tensor, at::Tensor> fused_gdn_gating(at::Tensor& A_log, at::Tensor& dt_bias, at::Tensor& a,
                                                   at::Tensor& b, bool is_var_len, cudaStream_t stream);

void bf16_gdn_compute_u_w(at::Tensor& k, at::Tensor& v, at::Tensor& u, at::Tensor& w, at::Tensor& beta,
                          std::optional<at::Tensor>& gate, const std::string& compiled_dims, cudaStream_t stream,
                          std::optional<at::Tensor>& cu_seqlens, std::optional<at::Tensor>& chunk_indices);

void bf16_chunked_seq_state_update(at::Tensor& k, at::Tensor& u, at::Tensor& w,
                                   std::optional<at::Tensor>& initial_state, at::Tensor& state,
                                   std::optional<at::Tensor>& final_state, std::optional<at::Tensor>& gate,
                                   const std::string& compiled_dims, cudaStream_t stream,
                                   std::optional<at::Tensor>& cu_seqlens, std::optional<at::Tensor>& cu_chunks,
                                   std::optional<int> total_chunks, uint32_t chunk_size);

void bf16_gdn_chunked_compute_O(at::Tensor& q, at::Tensor& state, at::Tensor& k, at::Tensor& u, at::Tensor& o,
                                std::optional<at::Tensor>& gate, std::optional<float> scale,
                                const std::string& compiled_dims, cudaStream_t stream,
                                std::optional<at::Tensor>& cu_seqlens, std::optional<at::Tensor>& chunk_indices,
                                std::optional<at::Tensor>& cu_chunks, std::optional<int> total_chunks,
                                uint32_t chunk_size);

void chunk_local_cumsum_bf16(at::Tensor& input, at::Tensor& output, int batch_size, int seq_len, int num_heads,
                             bool head_first, std::optional<at::Tensor>& cu_seqlens,
                             std::optional<at::Tensor>& chunk_indices, cudaStream_t stream);

at::Tensor transpose_to_mn_major(at::Tensor& input, cudaStream_t stream, uint32_t alignment = 16);

}  // namespace gdn_cuda
