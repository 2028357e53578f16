// pybind11 module `gdn_cuda`: the names, argument order, keywords and defaults of the reference's
// csrc/python_api.cpp:17-393, forwarding to namespace gdn_cuda (gdn_api.hpp) on the current torch stream.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include "gdn_api.hpp"

namespace py = pybind11;

// Every call runs on the device of its first tensor and on that device's current torch stream.
struct OnDevice {
    c10::cuda::CUDAGuard guard;
    explicit OnDevice(const at::Tensor& t) : guard(t.device()) {}
    cudaStream_t stream() const { return at::cuda::getCurrentCUDAStream().stream(); }
};

PYBIND11_MODULE(gdn_cuda, m) {
    m.doc() = "Gated DeltaNet kernels for B200 (sm_100a) behind the gdn_cuda API";

    m.def("init", &gdn_cuda::init, py::arg("library_root"), py::arg("cuda_home"),
          "Record the repository root and the CUDA toolkit root for the run-time kernel compiler.");

    m.def(
        "chunked_forward",
        [](at::Tensor& q, at::Tensor& k, at::Tensor& v, at::Tensor& beta, at::Tensor& gate, std::optional<float> scale,
           std::optional<at::Tensor> initial_state, std::optional<at::Tensor> cu_seqlens,
           std::optional<at::Tensor> chunk_indices, std::optional<at::Tensor> cu_chunks,
           std::optional<int> total_chunks, bool is_qk_norm) {
            OnDevice dev(q);
            return gdn_cuda::chunked_forward(q, k, v, beta, gate, scale, initial_state, cu_seqlens, chunk_indices,
                                             cu_chunks, total_chunks, dev.stream(), is_qk_norm);
        },
        py::arg("query"), py::arg("key"), py::arg("value"), py::arg("beta"), py::arg("gate"),
        py::arg("scale") = py::none(), py::arg("initial_state") = py::none(), py::arg("cu_seqlens") = py::none(),
        py::arg("chunk_indices") = py::none(), py::arg("cu_chunks") = py::none(), py::arg("total_chunks") = py::none(),
        py::kw_only(), py::arg("is_qk_norm") = false,
        "Chunked (64-token) prefill.  query/key (B,T,kh,d)|(N,kh,d), value (B,T,vh,d)|(N,vh,d), beta bf16 and gate "
        "fp32 (raw log-decay) (B,T,vh)|(N,vh), initial_state (B|S,vh,d,d) bf16.  Returns (output, final_state).");

    m.def(
        "recurrent_forward",
        [](at::Tensor& q, at::Tensor& k, at::Tensor& v, std::optional<at::Tensor> initial_state,
           std::optional<at::Tensor> beta, std::optional<at::Tensor> gate, std::optional<at::Tensor> cu_seqlens,
           std::optional<at::Tensor> num_accepted_tokens, int inference_mode, bool is_qk_norm, std::optional<float> scale,
           std::optional<std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor>> gating, bool inplace_state,
           std::optional<at::Tensor> state_indices) {
            OnDevice dev(q);
            const auto mode = static_cast<gdn_cuda::InferenceMode>(inference_mode);
            if (!gating.has_value() && !beta.has_value()) throw std::runtime_error("beta is required");
            gdn_cuda::RecurrentExtensions ext;
            ext.inplace_state = inplace_state;
            ext.state_indices = state_indices;
            return gdn_cuda::recurrent_forward_ext(q, k, v, initial_state, beta, gate, gating, cu_seqlens, num_accepted_tokens,
                                                   mode, dev.stream(), is_qk_norm, scale, ext);
        },
        py::arg("query"), py::arg("key"), py::arg("value"), py::arg("initial_state") = py::none(), py::arg("beta"),
        py::arg("gate"), py::arg("cu_seqlens") = py::none(), py::arg("num_accepted_tokens") = py::none(),
        py::arg("inference_mode") = 0, py::arg("is_qk_norm") = false, py::arg("scale") = py::none(), py::kw_only(),
        py::arg("gating") = py::none(), py::arg("inplace_state") = false, py::arg("state_indices") = py::none(),
        "Token recurrence for decode / speculative verify.  Returns (output, new_state); new_state holds one state "
        "per token when inference_mode == SpecVerify.");

    m.def(
        "causal_conv1d",
        [](at::Tensor& x, at::Tensor& weight, std::optional<at::Tensor> bias, std::optional<at::Tensor> initial_state,
           std::optional<at::Tensor> cu_seqlens, bool activation, std::optional<at::Tensor> final_state,
           bool return_final_state) -> py::object {
            OnDevice dev(x);
            auto r = gdn_cuda::causal_conv1d(x, weight, bias, initial_state, cu_seqlens, activation, final_state,
                                             return_final_state, dev.stream());
            if (r.second.has_value()) return py::cast(std::make_pair(r.first, *r.second));
            return py::cast(r.first);
        },
        py::arg("x"), py::arg("weight"), py::arg("bias") = py::none(), py::arg("initial_state") = py::none(),
        py::arg("cu_seqlens") = py::none(), py::arg("activation") = true, py::arg("final_state") = py::none(),
        py::arg("return_final_state") = false,
        "Depthwise causal convolution along the token axis (+ SiLU) over (B,T,C) or packed (N,C); returns y, or "
        "(y, final_state) when a final state is asked for.  Not part of the reference's module.");

    m.def(
        "gated_rmsnorm",
        [](at::Tensor& x, at::Tensor& z, at::Tensor& weight, float eps) {
            OnDevice dev(x);
            return gdn_cuda::gated_rmsnorm(x, z, weight, eps, dev.stream());
        },
        py::arg("x"), py::arg("z"), py::arg("weight"), py::arg("eps") = 1e-6f,
        "y = x * rsqrt(mean(x^2) + eps) * weight * silu(z) over the last axis.  Not part of the reference's module.");

    m.def(
        "fused_gdn_gating",
        [](at::Tensor& A_log, at::Tensor& dt_bias, at::Tensor& a, at::Tensor& b, bool is_var_len) {
            OnDevice dev(a);
            return gdn_cuda::fused_gdn_gating(A_log, dt_bias, a, b, is_var_len, dev.stream());
        },
        py::arg("A_log"), py::arg("dt_bias"), py::arg("a"), py::arg("b"), py::arg("is_var_len") = false,
        "(beta, gate) = (sigmoid(b), -exp(A_log) * softplus(a + dt_bias)).");

    m.def(
        "bf16_gdn_compute_u_w",
        [](at::Tensor& k, at::Tensor& v, at::Tensor& u, at::Tensor& w, at::Tensor& beta, std::optional<at::Tensor> gate,
           const std::string& compiled_dims, std::optional<at::Tensor> cu_seqlens,
           std::optional<at::Tensor> chunk_indices) {
            OnDevice dev(k);
            gdn_cuda::bf16_gdn_compute_u_w(k, v, u, w, beta, gate, compiled_dims, dev.stream(), cu_seqlens,
                                           chunk_indices);
        },
        py::arg("k"), py::arg("v"), py::arg("u"), py::arg("w"), py::arg("beta"), py::arg("gate") = py::none(),
        py::arg("compiled_dims") = "t", py::arg("cu_seqlens") = py::none(), py::arg("chunk_indices") = py::none(),
        "Low-level WY/UT transform; writes u and w.");

    m.def(
        "bf16_gdn_recurrent",
        [](at::Tensor& q, at::Tensor& k, at::Tensor& v, std::optional<at::Tensor> initial_state, at::Tensor& final_state,
           at::Tensor& out, std::optional<at::Tensor> gate, at::Tensor& beta, const std::string& compiled_dims,
           std::optional<at::Tensor> cu_seqlens, std::optional<at::Tensor> num_accepted_tokens, bool store_step_state,
           bool is_qk_norm, float scale) {
            OnDevice dev(q);
            gdn_cuda::bf16_gdn_recurrent(q, k, v, initial_state, final_state, out, gate, beta, compiled_dims, dev.stream(),
                                         cu_seqlens, num_accepted_tokens, store_step_state, is_qk_norm, scale);
        },
        py::arg("q"), py::arg("k"), py::arg("v"), py::arg("initial_state"), py::arg("final_state"), py::arg("out"),
        py::arg("gate"), py::arg("beta"), py::arg("compiled_dims") = "t", py::arg("cu_seqlens") = py::none(),
        py::arg("num_accepted_tokens") = py::none(), py::arg("store_step_state") = false, py::arg("is_qk_norm") = false,
        py::arg("scale") = 1.0f,
        "The recurrence on caller-provided tensors (the C++ gdn_cuda::bf16_gdn_recurrent); writes out and final_state.");

    m.def(
        "bf16_chunked_seq_state_update",
        [](at::Tensor& k, at::Tensor& u, at::Tensor& w, std::optional<at::Tensor>& initial_state, at::Tensor& state,
           std::optional<at::Tensor>& final_state, std::optional<at::Tensor> gate, const std::string& compiled_dims,
           std::optional<at::Tensor> cu_seqlens, std::optional<at::Tensor> cu_chunks, std::optional<int> total_chunks,
           uint32_t chunk_size) {
            OnDevice dev(k);
            gdn_cuda::bf16_chunked_seq_state_update(k, u, w, initial_state, state, final_state, gate, compiled_dims,
                                                    dev.stream(), cu_seqlens, cu_chunks, total_chunks, chunk_size);
        },
        py::arg("k"), py::arg("u"), py::arg("w"), py::arg("initial_state"), py::arg("state"), py::arg("final_state"),
        py::arg("gate") = py::none(), py::arg("compiled_dims") = "t", py::arg("cu_seqlens") = py::none(),
        py::arg("cu_chunks") = py::none(), py::arg("total_chunks") = py::none(), py::arg("chunk_size") = 64u,
        "Low-level chunk-to-chunk state pass; writes state, final_state and overwrites u with U_new.");

    m.def(
        "bf16_gdn_chunked_compute_O",
        [](at::Tensor& q, at::Tensor& state, at::Tensor& k, at::Tensor& u, at::Tensor& o, std::optional<at::Tensor> gate,
           std::optional<float> scale, const std::string& compiled_dims, std::optional<at::Tensor> cu_seqlens,
           std::optional<at::Tensor> chunk_indices, std::optional<at::Tensor> cu_chunks, uint32_t chunk_size) {
            OnDevice dev(q);
            gdn_cuda::bf16_gdn_chunked_compute_O(q, state, k, u, o, gate, scale, compiled_dims, dev.stream(),
                                                 cu_seqlens, chunk_indices, cu_chunks, std::nullopt, chunk_size);
        },
        py::arg("q"), py::arg("state"), py::arg("k"), py::arg("u"), py::arg("o"), py::arg("gate") = py::none(),
        py::arg("scale") = py::none(), py::arg("compiled_dims") = "t", py::arg("cu_seqlens") = py::none(),
        py::arg("chunk_indices") = py::none(), py::arg("cu_chunks") = py::none(), py::arg("chunk_size") = 64u,
        "Low-level output stage; writes o.");

    m.def(
        "chunk_local_cumsum_bf16",
        [](at::Tensor& input, at::Tensor& output, int batch_size, int seq_len, int num_heads, bool head_first,
           std::optional<at::Tensor> cu_seqlens, std::optional<at::Tensor> chunk_indices) {
            OnDevice dev(input);
            gdn_cuda::chunk_local_cumsum_bf16(input, output, batch_size, seq_len, num_heads, head_first, cu_seqlens,
                                              chunk_indices, dev.stream());
        },
        py::arg("input"), py::arg("output"), py::arg("batch_size"), py::arg("seq_len"), py::arg("num_heads"),
        py::arg("head_first") = false, py::arg("cu_seqlens") = py::none(), py::arg("chunk_indices") = py::none(),
        "Chunk-local inclusive cumsum (bf16 or fp32 in, fp32 out).");

    m.def(
        "transpose_to_mn_major",
        [](at::Tensor& input, uint32_t alignment) {
            OnDevice dev(input);
            return gdn_cuda::transpose_to_mn_major(input, dev.stream(), alignment);
        },
        py::arg("input"), py::arg("alignment") = 16u, "Transpose the last two dims to a stride(-2) == 1 layout.");

    py::enum_<gdn_cuda::InferenceMode>(m, "InferenceMode")
        .value("Prefill", gdn_cuda::InferenceMode::Prefill)
        .value("Decode", gdn_cuda::InferenceMode::Decode)
        .value("SpecVerify", gdn_cuda::InferenceMode::SpecVerify)
        .export_values();
}
