// `namespace gdn_cuda` implemented on the C ABI (include/gdn_b200.h).  Every function keeps the
// argument meaning of the reference's csrc/apis/gdn_forward.cpp; what it does is: check,
// allocate outputs / workspace with torch, fill the C structs, call, throw on a non-zero status.
#include "gdn_api.hpp"

#include <ATen/ops/constant_pad_nd.h>
#include <gdn_b200.h>

#include <cmath>
#include <stdexcept>

namespace gdn_cuda {
namespace {

constexpr int64_t kPrefillDim = 128;  // head dimension the tensor-core prefill kernels are built for

void require(bool cond, const std::string& msg) {
    if (!cond) throw std::runtime_error(msg);
}
void check(int rc, const char* what) {
    if (rc != GDN_OK) throw std::runtime_error(std::string(what) + " failed: " + gdn_last_error());
}
void cuda_bf16(const at::Tensor& t, const char* name) {
    require(t.is_cuda(), std::string(name) + " must be a CUDA tensor");
    require(t.scalar_type() == at::kBFloat16, std::string(name) + " must be bf16");
}
int dtype_tag(const at::Tensor& t) {
    if (t.scalar_type() == at::kBFloat16) return GDN_BF16;
    if (t.scalar_type() == at::kFloat) return GDN_F32;
    throw std::runtime_error("unsupported dtype (bf16 or fp32 expected)");
}
GdnTokenTensor tok(const at::Tensor& t, bool packed) {
    require(t.stride(-1) == 1, "head dimension must be contiguous");
    if (packed) {
        require(t.dim() == 3, "packed tensors are rank 3 (tokens, heads, dim)");
        return GdnTokenTensor{t.data_ptr(), 0, t.stride(0), t.stride(1)};
    }
    require(t.dim() == 4, "padded tensors are rank 4 (batch, tokens, heads, dim)");
    return GdnTokenTensor{t.data_ptr(), t.stride(0), t.stride(1), t.stride(2)};
}
GdnTokenScalar sca(const std::optional<at::Tensor>& o, bool packed, int64_t tokens) {
    if (!o.has_value()) return GdnTokenScalar{nullptr, 0, 0, 0, 0};
    at::Tensor t = o.value();
    if (t.size(-2) != tokens) t = t.narrow(-2, 0, tokens);  // MN-major views carry a padded token axis
    if (packed) {
        require(t.dim() == 2, "packed beta/gate are rank 2 (tokens, heads)");
        return GdnTokenScalar{t.data_ptr(), dtype_tag(t), 0, t.stride(0), t.stride(1)};
    }
    require(t.dim() == 3, "padded beta/gate are rank 3 (batch, tokens, heads)");
    return GdnTokenScalar{t.data_ptr(), dtype_tag(t), t.stride(0), t.stride(1), t.stride(2)};
}
GdnState st(const std::optional<at::Tensor>& o) {
    if (!o.has_value()) return GdnState{nullptr, 0, 0};
    const at::Tensor& t = o.value();
    require(t.stride(-1) == 1 && t.stride(-2) == t.size(-1), "state (dv, dk) block must be contiguous");
    return GdnState{t.data_ptr(), t.stride(0), t.stride(1)};
}
const int32_t* i32(const std::optional<at::Tensor>& o, const char* name) {
    if (!o.has_value()) return nullptr;
    require(o->is_cuda() && o->scalar_type() == at::kInt && o->is_contiguous(),
            std::string(name) + " must be a contiguous int32 CUDA tensor");
    return o->data_ptr<int32_t>();
}
// The prefill kernels read token tensors through TMA: 16-byte aligned base, contiguous head dim, every other
// stride a multiple of 8 elements.  A view that does not qualify is compacted (a copy), anything else passes.
at::Tensor tma_ready(const at::Tensor& t) {
    bool ok = t.stride(-1) == 1 && reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0;
    for (int64_t i = 0; ok && i + 1 < t.dim(); ++i) ok = t.stride(i) % 8 == 0;
    return ok ? t : t.contiguous();
}
at::Tensor pad_last(const at::Tensor& t, int64_t to) {
    return t.size(-1) == to ? t : at::constant_pad_nd(t, {0, to - t.size(-1)}, 0);
}
at::Tensor pad_state(const at::Tensor& t, int64_t dv, int64_t dk) {
    if (t.size(-1) == dk && t.size(-2) == dv) return t;
    return at::constant_pad_nd(t, {0, dk - t.size(-1), 0, dv - t.size(-2)}, 0);
}
int64_t align64(int64_t d) { return (d + 63) / 64 * 64; }

GdnShape make_shape(const at::Tensor& q, const at::Tensor& v, const std::optional<at::Tensor>& cu_seqlens,
                    const std::optional<at::Tensor>& chunk_indices, const std::optional<at::Tensor>& cu_chunks,
                    int total_chunks) {
    GdnShape s{};
    const bool packed = cu_seqlens.has_value();
    s.batch = static_cast<int32_t>(packed ? cu_seqlens->numel() - 1 : q.size(0));
    s.seq_len = static_cast<int32_t>(packed ? 0 : q.size(1));
    s.total_tokens = packed ? q.size(0) : q.size(0) * q.size(1);
    s.num_k_heads = static_cast<int32_t>(q.size(-2));
    s.num_v_heads = static_cast<int32_t>(v.size(-2));
    s.head_dim_k = static_cast<int32_t>(q.size(-1));
    s.head_dim_v = static_cast<int32_t>(v.size(-1));
    s.cu_seqlens = i32(cu_seqlens, "cu_seqlens");
    s.chunk_indices = i32(chunk_indices, "chunk_indices");
    s.cu_chunks = i32(cu_chunks, "cu_chunks");
    s.total_chunks = total_chunks;
    return s;
}

}  // namespace

void init(const std::string& library_root, const std::string& cuda_home) {
    check(gdn_init(library_root.c_str(), cuda_home.c_str()), "init");
}

std::pair<at::Tensor, at::Tensor> chunked_forward(at::Tensor& query, at::Tensor& key, at::Tensor& value,
                                                  at::Tensor& beta, at::Tensor& gate, std::optional<float> scale,
                                                  std::optional<at::Tensor>& initial_state,
                                                  std::optional<at::Tensor>& cu_seqlens,
                                                  std::optional<at::Tensor>& chunk_indices,
                                                  std::optional<at::Tensor>& cu_chunks,
                                                  std::optional<int> total_chunks, cudaStream_t stream,
                                                  bool is_qk_norm) {
    cuda_bf16(query, "query");
    cuda_bf16(key, "key");
    cuda_bf16(value, "value");
    const bool packed = cu_seqlens.has_value();
    const int64_t d = query.size(-1);
    require(key.size(-1) == d && value.size(-1) == d, "chunked kernels need dk == dv");
    require(d > 0 && d <= 256, "chunked_forward supports head dims up to 256");
    // up to 128: the tensor-core kernels, which compute on 128 columns; a head dim that is a multiple of 8 goes
    // in as it is (the library's tensor maps supply the zero columns), any other is zero-padded to 128 here.
    // 129..256: the library runs the token recurrence on 192 or 256 columns instead
    const int64_t D = d <= kPrefillDim ? (d % 8 == 0 ? d : kPrefillDim) : (d + 63) / 64 * 64;
    at::Tensor q = tma_ready(pad_last(query, D)), k = tma_ready(pad_last(key, D)), v = tma_ready(pad_last(value, D));
    std::optional<at::Tensor> s_in;
    if (initial_state.has_value()) {
        cuda_bf16(*initial_state, "initial_state");
        at::Tensor t = pad_state(*initial_state, D, D);
        if (!(t.stride(-1) == 1 && t.stride(-2) == D)) t = t.contiguous();
        s_in = t;
    }
    int tc = 0;
    if (packed) {
        require(chunk_indices.has_value() && cu_chunks.has_value(),
                "packed mode needs cu_seqlens, chunk_indices and cu_chunks");
        tc = total_chunks.has_value() ? total_chunks.value() : static_cast<int>(chunk_indices->numel() / 2);
    }
    GdnChunkedArgs a{};
    a.shape = make_shape(q, v, cu_seqlens, chunk_indices, cu_chunks, tc);
    at::Tensor out = at::empty_like(v);
    at::Tensor fin = at::empty({a.shape.batch, v.size(-2), D, D}, v.options());
    const int64_t tokens = packed ? q.size(0) : q.size(1);
    a.q = tok(q, packed);
    a.k = tok(k, packed);
    a.v = tok(v, packed);
    a.out = tok(out, packed);
    a.beta = sca(beta, packed, tokens);
    a.gate = sca(gate, packed, tokens);
    a.initial_state = st(s_in);
    a.final_state = st(fin);
    a.scale = scale.value_or(1.0f / std::sqrt(static_cast<float>(d)));
    const size_t ws_bytes = gdn_chunked_forward_workspace_bytes(&a.shape);
    at::Tensor ws = at::empty({static_cast<int64_t>(ws_bytes)}, v.options().dtype(at::kByte));
    a.workspace = ws.data_ptr();
    a.workspace_bytes = ws_bytes;
    a.stage_events = nullptr;
    a.is_qk_norm = is_qk_norm ? 1 : 0;
    check(gdn_chunked_forward(&a, stream), "chunked_forward");
    if (d != D) {
        out = out.narrow(-1, 0, d);
        fin = fin.narrow(-1, 0, d).narrow(-2, 0, d);
    }
    return {out, fin};
}

namespace {
struct Gating {
    at::Tensor A_log, dt_bias, a, b;
};
std::pair<at::Tensor, at::Tensor> recurrent_impl(at::Tensor& query, at::Tensor& key, at::Tensor& value,
                                                 std::optional<at::Tensor>& initial_state,
                                                 const std::optional<at::Tensor>& beta, const std::optional<at::Tensor>& gate,
                                                 const Gating* gating, std::optional<at::Tensor>& cu_seqlens,
                                                 std::optional<at::Tensor>& num_accepted_tokens,
                                                 InferenceMode inference_mode, cudaStream_t stream, bool is_qk_norm,
                                                 std::optional<float> scale, const RecurrentExtensions& ext = {}) {
    cuda_bf16(query, "query");
    cuda_bf16(key, "key");
    cuda_bf16(value, "value");
    const bool packed = cu_seqlens.has_value();
    const bool store_steps = inference_mode == InferenceMode::SpecVerify;
    const int64_t d = query.size(-1), dv_in = value.size(-1);
    require(key.size(-1) == d, "query and key head dims differ");
    const int64_t d_al = align64(d), dv_al = align64(dv_in);
    require(d_al <= 256 && dv_al <= 256, "head dims above 256 are not supported");
    at::Tensor q = pad_last(query, d_al), k = pad_last(key, d_al), v = pad_last(value, dv_al);
    // the state: bf16, or fp32 when the caller's initial state is fp32 (it then stays fp32); updated where it
    // lies when the caller asks for that or passes a pool of states with one slot index per sequence
    const bool in_place = ext.inplace_state || ext.state_indices.has_value();
    std::optional<at::Tensor> s_in;
    auto state_opts = v.options();
    if (initial_state.has_value()) {
        const at::Tensor& s0 = *initial_state;
        require(s0.is_cuda() && (s0.scalar_type() == at::kBFloat16 || s0.scalar_type() == at::kFloat),
                "initial_state must be a bf16 or fp32 CUDA tensor");
        state_opts = s0.options();
        at::Tensor t = pad_state(s0, dv_al, d_al);
        if (!(t.stride(-1) == 1 && t.stride(-2) == d_al)) t = t.contiguous();
        // a padded or compacted copy would never reach the caller's tensor
        require(!in_place || t.data_ptr() == s0.data_ptr(),
                "inplace_state / state_indices need head dims that are multiples of 64 and contiguous (dv, dk) blocks");
        s_in = t;
    }
    GdnRecurrentArgs a{};
    a.shape = make_shape(q, v, cu_seqlens, std::nullopt, std::nullopt, 0);
    const int64_t vh = v.size(-2);
    at::Tensor out = at::empty_like(v);
    at::Tensor s_out;
    if (store_steps) {
        require(!ext.state_indices.has_value(), "state_indices cannot be combined with per-token states");
        s_out = packed ? at::empty({q.size(0), vh, dv_al, d_al}, state_opts)
                       : at::empty({q.size(0), q.size(1), vh, dv_al, d_al}, state_opts);
        a.state_out = GdnState{s_out.data_ptr(), vh * dv_al * d_al, dv_al * d_al};
    } else if (in_place) {
        require(s_in.has_value(), "inplace_state / state_indices need an initial_state");
        s_out = *s_in;
        a.state_out = st(s_out);
    } else {
        s_out = at::empty({a.shape.batch, vh, dv_al, d_al}, state_opts);
        a.state_out = st(s_out);
    }
    a.state_dtype = state_opts.dtype() == at::kFloat ? GDN_F32 : GDN_BF16;
    if (ext.state_indices.has_value()) {
        require(ext.state_indices->numel() == a.shape.batch, "state_indices needs one entry per sequence");
        a.state_indices = i32(ext.state_indices, "state_indices");
    }
    const int64_t tokens = packed ? q.size(0) : q.size(1);
    a.q = tok(q, packed);
    a.k = tok(k, packed);
    a.v = tok(v, packed);
    a.out = tok(out, packed);
    at::Tensor Ac, dc;  // keep the contiguous copies alive until the launch
    if (gating) {
        require(gating->a.scalar_type() == gating->b.scalar_type() && gating->a.scalar_type() == gating->A_log.scalar_type() &&
                    gating->a.scalar_type() == gating->dt_bias.scalar_type(),
                "A_log, dt_bias, a, b must share a dtype");
        require(gating->A_log.numel() >= vh && gating->dt_bias.numel() >= vh, "A_log and dt_bias need one entry per head");
        Ac = gating->A_log.contiguous();
        dc = gating->dt_bias.contiguous();
        a.gating_a = sca(gating->a, packed, tokens);
        a.gating_b = sca(gating->b, packed, tokens);
        a.A_log = Ac.data_ptr();
        a.dt_bias = dc.data_ptr();
    } else {
        require(beta.has_value(), "beta is required");
        a.beta = sca(beta, packed, tokens);
        a.gate = sca(gate, packed, tokens);
    }
    a.state_in = st(s_in);
    a.num_accepted_tokens = i32(num_accepted_tokens, "num_accepted_tokens");
    a.scale = scale.value_or(1.0f / std::sqrt(static_cast<float>(d)));
    a.is_qk_norm = is_qk_norm ? 1 : 0;
    a.store_step_state = store_steps ? 1 : 0;
    check(gdn_recurrent_forward(&a, stream), "recurrent_forward");
    if (dv_al != dv_in) out = out.narrow(-1, 0, dv_in);
    if (d_al != d || dv_al != dv_in) s_out = s_out.narrow(-1, 0, d).narrow(-2, 0, dv_in);
    return {out, s_out};
}
}  // namespace

std::pair<at::Tensor, at::Tensor> recurrent_forward(at::Tensor& query, at::Tensor& key, at::Tensor& value,
                                                    std::optional<at::Tensor>& initial_state, at::Tensor& beta,
                                                    at::Tensor& gate, std::optional<at::Tensor>& cu_seqlens,
                                                    std::optional<at::Tensor>& num_accepted_tokens,
                                                    InferenceMode inference_mode, cudaStream_t stream,
                                                    bool is_qk_norm, std::optional<float> scale) {
    return recurrent_impl(query, key, value, initial_state, beta, gate.defined() ? std::optional<at::Tensor>(gate) : std::nullopt,
                          nullptr, cu_seqlens, num_accepted_tokens, inference_mode, stream, is_qk_norm, scale);
}

std::pair<at::Tensor, at::Tensor> recurrent_forward_fused_gating(
    at::Tensor& query, at::Tensor& key, at::Tensor& value, std::optional<at::Tensor>& initial_state, at::Tensor& A_log,
    at::Tensor& dt_bias, at::Tensor& a, at::Tensor& b, std::optional<at::Tensor>& cu_seqlens,
    std::optional<at::Tensor>& num_accepted_tokens, InferenceMode inference_mode, cudaStream_t stream, bool is_qk_norm,
    std::optional<float> scale) {
    Gating g{A_log, dt_bias, a, b};
    return recurrent_impl(query, key, value, initial_state, std::nullopt, std::nullopt, &g, cu_seqlens, num_accepted_tokens,
                          inference_mode, stream, is_qk_norm, scale);
}

std::pair<at::Tensor, at::Tensor> recurrent_forward_ext(at::Tensor& query, at::Tensor& key, at::Tensor& value,
                                                        std::optional<at::Tensor>& initial_state,
                                                        std::optional<at::Tensor>& beta, std::optional<at::Tensor>& gate,
                                                        std::optional<std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor>>& gating,
                                                        std::optional<at::Tensor>& cu_seqlens,
                                                        std::optional<at::Tensor>& num_accepted_tokens,
                                                        InferenceMode inference_mode, cudaStream_t stream, bool is_qk_norm,
                                                        std::optional<float> scale, const RecurrentExtensions& ext) {
    if (gating.has_value()) {
        require(!beta.has_value() && !gate.has_value(), "pass either gating=(A_log, dt_bias, a, b) or beta/gate, not both");
        Gating g{std::get<0>(*gating), std::get<1>(*gating), std::get<2>(*gating), std::get<3>(*gating)};
        return recurrent_impl(query, key, value, initial_state, std::nullopt, std::nullopt, &g, cu_seqlens, num_accepted_tokens,
                              inference_mode, stream, is_qk_norm, scale, ext);
    }
    return recurrent_impl(query, key, value, initial_state, beta, gate, nullptr, cu_seqlens, num_accepted_tokens,
                          inference_mode, stream, is_qk_norm, scale, ext);
}

std::pair<at::Tensor, std::optional<at::Tensor>> causal_conv1d(at::Tensor& x, at::Tensor& weight,
                                                               std::optional<at::Tensor>& bias,
                                                               std::optional<at::Tensor>& initial_state,
                                                               std::optional<at::Tensor>& cu_seqlens, bool activation,
                                                               std::optional<at::Tensor>& final_state,
                                                               bool return_final_state, cudaStream_t stream) {
    cuda_bf16(x, "x");
    cuda_bf16(weight, "weight");
    require(x.stride(-1) == 1, "channels must be contiguous");
    require(weight.dim() == 2 && x.size(-1) == weight.size(0), "weight must be (channels, width)");
    const bool packed = cu_seqlens.has_value();
    const int64_t C = weight.size(0), W = weight.size(1);
    require(packed ? x.dim() == 2 : x.dim() == 3, packed ? "packed input is (tokens, channels)" : "padded input is (batch, tokens, channels)");
    const int64_t batch = packed ? cu_seqlens->numel() - 1 : x.size(0);
    at::Tensor y = at::empty(x.sizes(), x.options());
    at::Tensor w = weight.contiguous(), b, s_in;
    if (bias.has_value()) {
        cuda_bf16(*bias, "bias");
        b = bias->contiguous();
    }
    if (initial_state.has_value()) {
        cuda_bf16(*initial_state, "initial_state");
        require(initial_state->dim() == 3 && initial_state->size(0) == batch && initial_state->size(1) == W - 1 &&
                    initial_state->size(2) == C,
                "initial_state must be (sequences, W-1, C) bf16");
        s_in = initial_state->contiguous();
    }
    std::optional<at::Tensor> s_out = final_state;
    if (!s_out.has_value() && return_final_state) s_out = at::empty({batch, W - 1, C}, x.options());
    if (s_out.has_value())
        require(s_out->is_contiguous() && s_out->dim() == 3 && s_out->size(0) == batch && s_out->size(1) == W - 1 &&
                    s_out->size(2) == C && s_out->scalar_type() == at::kBFloat16,
                "final_state must be contiguous (sequences, W-1, C) bf16");
    GdnConvArgs a{};
    a.x = x.data_ptr();
    a.y = y.data_ptr();
    a.weight = w.data_ptr();
    a.bias = b.defined() ? b.data_ptr() : nullptr;
    a.state_in = s_in.defined() ? s_in.data_ptr() : nullptr;
    a.state_out = s_out.has_value() ? s_out->data_ptr() : nullptr;
    a.x_stride_batch = packed ? 0 : x.stride(0);
    a.x_stride_token = packed ? x.stride(0) : x.stride(1);
    a.y_stride_batch = packed ? 0 : y.stride(0);
    a.y_stride_token = packed ? y.stride(0) : y.stride(1);
    a.batch = static_cast<int32_t>(batch);
    a.seq_len = packed ? 0 : static_cast<int32_t>(x.size(1));
    a.total_tokens = packed ? x.size(0) : x.size(0) * x.size(1);
    a.cu_seqlens = i32(cu_seqlens, "cu_seqlens");
    a.channels = static_cast<int32_t>(C);
    a.width = static_cast<int32_t>(W);
    a.silu = activation ? 1 : 0;
    check(gdn_causal_conv1d(&a, stream), "causal_conv1d");
    return {y, s_out};
}

at::Tensor gated_rmsnorm(at::Tensor& x, at::Tensor& z, at::Tensor& weight, float eps, cudaStream_t stream) {
    cuda_bf16(x, "x");
    cuda_bf16(z, "z");
    cuda_bf16(weight, "weight");
    require(x.sizes() == z.sizes() && x.size(-1) == weight.numel(),
            "x and z must have the same shape, weight one entry per column");
    const int64_t D = x.size(-1);
    at::Tensor x2 = x.contiguous().view({-1, D}), z2 = z.contiguous().view({-1, D}), w = weight.contiguous();
    at::Tensor y = at::empty(x2.sizes(), x.options());
    check(gdn_gated_rmsnorm(x2.data_ptr(), z2.data_ptr(), y.data_ptr(), w.data_ptr(), x2.size(0), static_cast<int32_t>(D),
                            x2.stride(0), z2.stride(0), y.stride(0), eps, stream),
          "gated_rmsnorm");
    return y.view(x.sizes());
}

void bf16_gdn_recurrent(at::Tensor& q, at::Tensor& k, at::Tensor& v, std::optional<at::Tensor>& initial_state,
                        at::Tensor& final_state, at::Tensor& out, std::optional<at::Tensor>& gate, at::Tensor& beta,
                        const std::string& /*compiled_dims*/, cudaStream_t stream, std::optional<at::Tensor>& cu_seqlens,
                        std::optional<at::Tensor>& num_accepted_tokens, bool store_step_state, bool is_qk_norm,
                        float scale) {
    cuda_bf16(q, "q");
    cuda_bf16(k, "k");
    cuda_bf16(v, "v");
    cuda_bf16(out, "out");
    cuda_bf16(final_state, "final_state");
    const bool packed = cu_seqlens.has_value();
    const int64_t dk = q.size(-1), dv = v.size(-1), vh = v.size(-2);
    require(k.size(-1) == dk, "q and k head dims differ");
    require(dk % 64 == 0 && dv % 64 == 0 && dk <= 256 && dv <= 256,
            "bf16_gdn_recurrent works on the caller's tensors: head dims must be multiples of 64 up to 256");
    require(out.sizes() == v.sizes(), "out must be shaped like v");
    require(final_state.is_contiguous() && final_state.size(-1) == dk && final_state.size(-2) == dv,
            "final_state must be contiguous (..., dv, dk)");
    GdnRecurrentArgs a{};
    a.shape = make_shape(q, v, cu_seqlens, std::nullopt, std::nullopt, 0);
    const int64_t tokens = packed ? q.size(0) : q.size(1);
    const int64_t want = store_step_state ? a.shape.total_tokens : a.shape.batch;
    require(final_state.numel() == want * vh * dv * dk,
            store_step_state ? "final_state must hold one state per token" : "final_state must hold one state per sequence");
    a.q = tok(q, packed);
    a.k = tok(k, packed);
    a.v = tok(v, packed);
    a.out = tok(out, packed);
    a.beta = sca(beta, packed, tokens);
    a.gate = sca(gate, packed, tokens);
    a.state_in = st(initial_state);
    a.state_out = GdnState{final_state.data_ptr(), vh * dv * dk, dv * dk};
    a.num_accepted_tokens = i32(num_accepted_tokens, "num_accepted_tokens");
    a.scale = scale;
    a.is_qk_norm = is_qk_norm ? 1 : 0;
    a.store_step_state = store_step_state ? 1 : 0;
    check(gdn_recurrent_forward(&a, stream), "bf16_gdn_recurrent");
}

std::pair<at::Tensor, at::Tensor> fused_gdn_gating(at::Tensor& A_log, at::Tensor& dt_bias, at::Tensor& a,
                                                   at::Tensor& b, bool /*is_var_len*/, cudaStream_t stream) {
    require(a.is_cuda() && b.is_cuda() && A_log.is_cuda() && dt_bias.is_cuda(), "inputs must be CUDA tensors");
    require(a.scalar_type() == b.scalar_type() && a.scalar_type() == A_log.scalar_type() &&
                a.scalar_type() == dt_bias.scalar_type(),
            "A_log, dt_bias, a, b must share a dtype");
    const int64_t vh = a.size(-1);
    require(A_log.numel() >= vh && dt_bias.numel() >= vh, "A_log and dt_bias need one entry per head");
    at::Tensor ac = a.contiguous(), bc = b.contiguous(), Ac = A_log.contiguous(), dc = dt_bias.contiguous();
    at::Tensor beta = at::empty_like(bc), gate = at::empty_like(ac);
    check(gdn_fused_gating(Ac.data_ptr(), dc.data_ptr(), ac.data_ptr(), bc.data_ptr(), beta.data_ptr(),
                           gate.data_ptr(), ac.numel() / vh, static_cast<int32_t>(vh), dtype_tag(ac), dtype_tag(gate),
                           stream),
          "fused_gdn_gating");
    return {beta, gate};
}

void bf16_gdn_compute_u_w(at::Tensor& k, at::Tensor& v, at::Tensor& u, at::Tensor& w, at::Tensor& beta,
                          std::optional<at::Tensor>& gate, const std::string& /*compiled_dims*/, cudaStream_t stream,
                          std::optional<at::Tensor>& cu_seqlens, std::optional<at::Tensor>& chunk_indices) {
    cuda_bf16(k, "k");
    cuda_bf16(v, "v");
    cuda_bf16(u, "u");
    cuda_bf16(w, "w");
    const int64_t d = k.size(-1);
    require(d > 0 && d <= kPrefillDim && v.size(-1) == d, "low-level chunked kernels need dk = dv <= 128");
    if (d != kPrefillDim) {
        // the kernels are built for head dim 128: run on zero-padded copies (exact) and copy the results back
        at::Tensor kp = pad_last(k, kPrefillDim), vp = pad_last(v, kPrefillDim);
        at::Tensor up = at::empty_like(vp), wp = at::empty_like(vp);
        bf16_gdn_compute_u_w(kp, vp, up, wp, beta, gate, "t", stream, cu_seqlens, chunk_indices);
        u.copy_(up.narrow(-1, 0, d));
        w.copy_(wp.narrow(-1, 0, d));
        return;
    }
    const bool packed = cu_seqlens.has_value();
    const int64_t tokens = packed ? k.size(0) : k.size(1);
    GdnComputeUWArgs a{};
    a.shape = make_shape(k, v, cu_seqlens, chunk_indices, std::nullopt,
                         chunk_indices.has_value() ? static_cast<int>(chunk_indices->numel() / 2) : 0);
    a.k = tok(k, packed);
    a.v = tok(v, packed);
    a.u = tok(u, packed);
    a.w = tok(w, packed);
    a.beta = sca(beta, packed, tokens);
    a.gate_cumsum = sca(gate, packed, tokens);
    check(gdn_compute_u_w(&a, stream), "bf16_gdn_compute_u_w");
}

void bf16_chunked_seq_state_update(at::Tensor& k, at::Tensor& u, at::Tensor& w,
                                   std::optional<at::Tensor>& initial_state, at::Tensor& state,
                                   std::optional<at::Tensor>& final_state, std::optional<at::Tensor>& gate,
                                   const std::string& /*compiled_dims*/, cudaStream_t stream,
                                   std::optional<at::Tensor>& cu_seqlens, std::optional<at::Tensor>& cu_chunks,
                                   std::optional<int> total_chunks, uint32_t chunk_size) {
    require(chunk_size == 64, "only chunk_size 64 is supported");
    cuda_bf16(k, "k");
    cuda_bf16(u, "u");
    cuda_bf16(w, "w");
    cuda_bf16(state, "state");
    require(state.is_contiguous(), "state must be contiguous");
    const int64_t d = k.size(-1);
    require(d > 0 && d <= kPrefillDim && u.size(-1) == d, "low-level chunked kernels need dk = dv <= 128");
    if (d != kPrefillDim) {
        // as the reference's wrapper does (csrc/apis/gdn_forward.cpp:252-302): zero-padded copies, results copied back
        const int64_t D = kPrefillDim;
        at::Tensor kp = pad_last(k, D), up = pad_last(u, D), wp = pad_last(w, D);
        std::vector<int64_t> shp(state.sizes().begin(), state.sizes().end());
        shp[shp.size() - 1] = D;
        shp[shp.size() - 2] = D;
        at::Tensor sp = at::empty(shp, state.options());
        std::optional<at::Tensor> ip, fp;
        if (initial_state.has_value()) ip = pad_state(*initial_state, D, D).contiguous();
        if (final_state.has_value()) {
            std::vector<int64_t> fs(final_state->sizes().begin(), final_state->sizes().end());
            fs[fs.size() - 1] = D;
            fs[fs.size() - 2] = D;
            fp = at::empty(fs, state.options());
        }
        bf16_chunked_seq_state_update(kp, up, wp, ip, sp, fp, gate, "t", stream, cu_seqlens, cu_chunks, total_chunks, chunk_size);
        u.copy_(up.narrow(-1, 0, d));
        state.copy_(sp.narrow(-1, 0, d).narrow(-2, 0, d));
        if (final_state.has_value()) final_state->copy_(fp->narrow(-1, 0, d).narrow(-2, 0, d));
        return;
    }
    const bool packed = cu_seqlens.has_value();
    const int64_t tokens = packed ? k.size(0) : k.size(1);
    GdnSeqStateArgs a{};
    a.shape = make_shape(k, u, cu_seqlens, std::nullopt, cu_chunks,
                         packed ? (total_chunks.has_value() ? total_chunks.value() : static_cast<int>(state.size(0))) : 0);
    a.k = tok(k, packed);
    a.u = tok(u, packed);
    a.w = tok(w, packed);
    a.gate_cumsum = sca(gate, packed, tokens);
    a.initial_state = st(initial_state);
    a.final_state = st(final_state);
    a.chunk_states = state.data_ptr();
    check(gdn_seq_state_update(&a, stream), "bf16_chunked_seq_state_update");
}

void bf16_gdn_chunked_compute_O(at::Tensor& q, at::Tensor& state, at::Tensor& k, at::Tensor& u, at::Tensor& o,
                                std::optional<at::Tensor>& gate, std::optional<float> scale,
                                const std::string& /*compiled_dims*/, cudaStream_t stream,
                                std::optional<at::Tensor>& cu_seqlens, std::optional<at::Tensor>& chunk_indices,
                                std::optional<at::Tensor>& cu_chunks, std::optional<int> /*total_chunks*/,
                                uint32_t chunk_size) {
    require(chunk_size == 64, "only chunk_size 64 is supported");
    cuda_bf16(q, "q");
    cuda_bf16(k, "k");
    cuda_bf16(u, "u");
    cuda_bf16(o, "o");
    cuda_bf16(state, "state");
    require(state.is_contiguous(), "state must be contiguous");
    const int64_t d = q.size(-1);
    require(d > 0 && d <= kPrefillDim && u.size(-1) == d, "low-level chunked kernels need dk = dv <= 128");
    if (d != kPrefillDim) {
        const int64_t D = kPrefillDim;
        at::Tensor qp = pad_last(q, D), kp = pad_last(k, D), up = pad_last(u, D);
        at::Tensor sp = pad_state(state, D, D).contiguous();
        at::Tensor op = at::empty_like(up);
        std::optional<float> sc = scale.value_or(1.0f / std::sqrt(static_cast<float>(d)));
        bf16_gdn_chunked_compute_O(qp, sp, kp, up, op, gate, sc, "t", stream, cu_seqlens, chunk_indices, cu_chunks,
                                   std::nullopt, chunk_size);
        o.copy_(op.narrow(-1, 0, d));
        return;
    }
    const bool packed = cu_seqlens.has_value();
    const int64_t tokens = packed ? q.size(0) : q.size(1);
    GdnComputeOArgs a{};
    a.shape = make_shape(q, u, cu_seqlens, chunk_indices, cu_chunks,
                         chunk_indices.has_value() ? static_cast<int>(chunk_indices->numel() / 2) : 0);
    a.q = tok(q, packed);
    a.k = tok(k, packed);
    a.u_new = tok(u, packed);
    a.out = tok(o, packed);
    a.gate_cumsum = sca(gate, packed, tokens);
    a.chunk_states = state.data_ptr();
    a.scale = scale.value_or(1.0f / std::sqrt(static_cast<float>(q.size(-1))));
    check(gdn_compute_o(&a, stream), "bf16_gdn_chunked_compute_O");
}

void chunk_local_cumsum_bf16(at::Tensor& input, at::Tensor& output, int batch_size, int seq_len, int num_heads,
                             bool head_first, std::optional<at::Tensor>& cu_seqlens,
                             std::optional<at::Tensor>& chunk_indices, cudaStream_t stream) {
    require(input.is_cuda() && output.is_cuda(), "tensors must be CUDA tensors");
    require(output.scalar_type() == at::kFloat, "output must be fp32");
    require(input.is_contiguous() && output.is_contiguous(), "input and output must be contiguous");
    check(gdn_chunk_local_cumsum(input.data_ptr(), output.data_ptr<float>(), dtype_tag(input), batch_size, seq_len,
                                 num_heads, head_first ? 1 : 0, i32(cu_seqlens, "cu_seqlens"),
                                 i32(chunk_indices, "chunk_indices"),
                                 chunk_indices.has_value() ? static_cast<int>(chunk_indices->numel() / 2) : 0, stream),
          "chunk_local_cumsum_bf16");
}

at::Tensor transpose_to_mn_major(at::Tensor& input, cudaStream_t stream, uint32_t alignment) {
    require(input.is_cuda() && input.dim() >= 2, "input must be a CUDA tensor of rank >= 2");
    require(input.scalar_type() == at::kFloat || input.scalar_type() == at::kBFloat16, "only fp32 and bf16 are supported");
    const int64_t es = input.element_size();
    require(alignment % es == 0, "alignment must be a multiple of the element size");
    at::Tensor x = input.contiguous();
    const int64_t mn = x.size(-2), k = x.size(-1), per = alignment / es;
    const int64_t mn_al = (mn + per - 1) / per * per;
    std::vector<int64_t> shape(x.sizes().begin(), x.sizes().end() - 2);
    int64_t groups = 1;
    for (int64_t v : shape) groups *= v;
    shape.push_back(k);
    shape.push_back(mn_al);
    at::Tensor store = at::empty(shape, x.options());
    check(gdn_transpose_mn_major(x.data_ptr(), store.data_ptr(), static_cast<int32_t>(es), groups, mn, k, mn_al, stream),
          "transpose_to_mn_major");
    return store.transpose(-1, -2);
}

}  // namespace gdn_cuda
