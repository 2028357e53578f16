// C-ABI entry points of the chunked-prefill path (see include/gdn_b200.h): tensor-map
// construction, argument checks and launches of the tcgen05 kernels.
#include "heuristics.hpp"
#include "host_common.hpp"
#include "kernels/prefill_fused.cuh"
#include "kernels/prefill_o.cuh"
#include "kernels/prefill_seq.cuh"
#include "kernels/prefill_segments.cuh"
#include "kernels/prefill_uw.cuh"
#include "kernels/prefill_zp.cuh"
#include "tma_host.hpp"

using namespace gdn;

namespace {

constexpr int kD = 128;  // head dimension the tensor-core kernels are built for

int require_d128(const GdnShape& s, const char* who) {
    if (s.head_dim_k != kD || s.head_dim_v != kD)
        return fail(GDN_ERR_UNSUPPORTED,
                    "%s: the chunked kernels are built for dk = dv = 128 (got %d, %d); pad the head "
                    "dimension with zeros (the Python and C++ wrappers do)",
                    who, s.head_dim_k, s.head_dim_v);
    return GDN_OK;
}

// 4-D map over a token tensor: (dim, head, token, batch), box 64 x 1 x 64 x 1, 128-byte swizzle.
// `dim` below 128 (a multiple of 8): loads fill the columns past it with zeros and stores leave them out,
// so a kernel built for 128 sees a zero-padded head without a padded copy in memory.
int make_token_map(CUtensorMap* out, const GdnTokenTensor& t, const GdnShape& s, int heads, const char* name, int dim = kD) {
    const bool packed = s.cu_seqlens != nullptr;
    const uint64_t tokens = packed ? static_cast<uint64_t>(s.total_tokens) : static_cast<uint64_t>(s.seq_len);
    const uint64_t batch = packed ? 1 : static_cast<uint64_t>(s.batch);
    uint64_t dims[4] = {static_cast<uint64_t>(dim), static_cast<uint64_t>(heads), tokens, batch};
    uint64_t sb = static_cast<uint64_t>(t.stride_batch) * 2;
    if (packed || sb == 0) sb = std::max<uint64_t>(16, tokens * static_cast<uint64_t>(t.stride_token) * 2);
    uint64_t strides[3] = {static_cast<uint64_t>(t.stride_head) * 2, static_cast<uint64_t>(t.stride_token) * 2, sb};
    if (heads == 1 && strides[0] == 0) strides[0] = static_cast<uint64_t>(dim) * 2;
    uint32_t box[4] = {64, 1, 64, 1};
    if (tokens == 0) return fail(GDN_ERR_INVALID, "%s: no tokens", name);
    if (!make_tmap_bf16(out, t.ptr, 4, dims, strides, box, true))
        return fail(GDN_ERR_CUDA, "could not encode the TMA descriptor of %s (strides %llu/%llu/%llu bytes)", name,
                    (unsigned long long)strides[0], (unsigned long long)strides[1], (unsigned long long)strides[2]);
    return GDN_OK;
}

ScalarView scalar_view(const GdnTokenScalar& t) {
    ScalarView v;
    v.ptr = t.ptr;
    v.is_f32 = t.dtype == GDN_F32;
    v.sb = t.stride_batch;
    v.st = t.stride_token;
    v.sh = t.stride_head;
    return v;
}
TokenView token_view(const GdnTokenTensor& t) {
    TokenView v;
    v.ptr = static_cast<__nv_bfloat16*>(t.ptr);
    v.sb = t.stride_batch;
    v.st = t.stride_token;
    v.sh = t.stride_head;
    return v;
}
ChunkMap chunk_map(const GdnShape& s) {
    ChunkMap m;
    m.cu_seqlens = s.cu_seqlens;
    m.chunk_indices = s.chunk_indices;
    m.cu_chunks = s.cu_chunks;
    m.seq_len = s.seq_len;
    m.chunks_per_seq = (s.seq_len + kChunk - 1) / kChunk;
    return m;
}
int num_chunks(const GdnShape& s) {
    return s.cu_seqlens ? s.total_chunks : s.batch * ((s.seq_len + kChunk - 1) / kChunk);
}
// States are read and written with 16-byte accesses.
int check_state(const GdnState& t, const char* name) {
    if (!t.ptr) return GDN_OK;
    GDN_REQUIRE(aligned16(t.ptr) && t.stride_seq % 8 == 0 && t.stride_head % 8 == 0,
                "%s must be 16-byte aligned with strides that are multiples of 8 elements", name);
    return GDN_OK;
}
int check_scalar(const GdnTokenScalar& t, const char* name, bool required) {
    if (!t.ptr) {
        GDN_REQUIRE(!required, "%s is NULL", name);
        return GDN_OK;
    }
    GDN_REQUIRE(t.dtype == GDN_BF16 || t.dtype == GDN_F32, "%s dtype must be bf16 or f32", name);
    return GDN_OK;
}

template <typename K>
int set_smem(K kernel, int bytes) {
    GDN_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    return GDN_OK;
}

int launch_uw(const GdnShape& s, const GdnTokenTensor& k, const GdnTokenTensor& v, const GdnTokenTensor& u,
              const GdnTokenTensor& w, const GdnTokenScalar& beta, const GdnTokenScalar& gate, bool gate_is_raw,
              DeviceInfo* d, cudaStream_t st) {
    const int nc = num_chunks(s);
    if (nc == 0) return GDN_OK;
    GDN_REQUIRE(s.num_v_heads <= 65535, "too many heads");
    CUtensorMap tmK, tmV, tmUo, tmWo;
    if (int rc = make_token_map(&tmK, k, s, s.num_k_heads, "k")) return rc;
    if (int rc = make_token_map(&tmV, v, s, s.num_v_heads, "v")) return rc;
    if (int rc = make_token_map(&tmUo, u, s, s.num_v_heads, "u")) return rc;
    if (int rc = make_token_map(&tmWo, w, s, s.num_v_heads, "w")) return rc;
    UWParams p{};
    p.map = chunk_map(s);
    p.beta = scalar_view(beta);
    p.gate = scalar_view(gate);
    p.gate_is_raw = gate_is_raw;
    p.u = token_view(u);
    p.w = token_view(w);
    p.kh = s.num_k_heads;
    p.vh = s.num_v_heads;
    p.num_chunks = nc;
    p.status = d->status;
    constexpr int smem = UWSmem<kD>::kBytes;
    const int grid = uw_grid(static_cast<long long>(nc) * s.num_v_heads, d->sms);
    if (int rc = set_smem(gdn_uw_kernel<kD>, smem)) return rc;
    gdn_uw_kernel<kD><<<grid, 128, smem, st>>>(tmK, tmV, tmUo, tmWo, p);
    GDN_CUDA(cudaGetLastError());
    return GDN_OK;
}

// Chunk-parallel stage of the whole-layer path: Z and PT of every (chunk, v-head) into `blocks`.
int launch_zp(const GdnShape& s, const GdnTokenTensor& q, const GdnTokenTensor& k, const GdnTokenScalar& beta,
              const GdnTokenScalar& gate, void* blocks, float* norms, float p_scale, DeviceInfo* d, cudaStream_t st) {
    const int nc = num_chunks(s);
    if (nc == 0) return GDN_OK;
    CUtensorMap tmK, tmQ;
    if (int rc = make_token_map(&tmK, k, s, s.num_k_heads, "k", s.head_dim_k)) return rc;
    if (int rc = make_token_map(&tmQ, q, s, s.num_k_heads, "q", s.head_dim_k)) return rc;
    ZPParams p{};
    p.map = chunk_map(s);
    p.beta = scalar_view(beta);
    p.gate = scalar_view(gate);
    p.blocks = static_cast<uint8_t*>(blocks);
    p.p_scale = p_scale;
    p.norms = norms;
    p.kh = s.num_k_heads;
    p.vh = s.num_v_heads;
    p.num_chunks = nc;
    p.status = d->status;
    constexpr int smem = ZPSmem::kBytes;
    const int grid = zp_grid(static_cast<long long>(nc) * s.num_k_heads, d->sms);
    // launched as a programmatic dependent of the preceding work in the stream (the kernel waits before its
    // first global read): its launch and set-up overlap that work's tail
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(zp::kThreads);
    cfg.dynamicSmemBytes = static_cast<size_t>(smem);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (norms) {
        if (int rc = set_smem(gdn_zp_kernel<true>, smem)) return rc;
        GDN_CUDA(cudaLaunchKernelEx(&cfg, gdn_zp_kernel<true>, tmK, tmQ, p));
    } else {
        if (int rc = set_smem(gdn_zp_kernel<false>, smem)) return rc;
        GDN_CUDA(cudaLaunchKernelEx(&cfg, gdn_zp_kernel<false>, tmK, tmQ, p));
    }
    return GDN_OK;
}

template <bool O, bool H, bool UN>
int launch_seq_t(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmW, const CUtensorMap& tmU,
                 const SeqParams& p, dim3 grid, cudaStream_t st) {
    constexpr int smem = SeqSmem::kBytes;
    if (int rc = set_smem(gdn_seq_kernel<O, H, UN>, smem)) return rc;
    gdn_seq_kernel<O, H, UN><<<grid, 256, smem, st>>>(tmQ, tmK, tmW, tmU, p);
    GDN_CUDA(cudaGetLastError());
    return GDN_OK;
}

}  // namespace

extern "C" {

int gdn_compute_u_w(const GdnComputeUWArgs* a, gdn_stream_t stream) {
    GDN_REQUIRE(a != nullptr, "gdn_compute_u_w: args is NULL");
    if (int rc = check_shape(a->shape, true)) return rc;
    if (int rc = require_d128(a->shape, "gdn_compute_u_w")) return rc;
    if (int rc = check_token_tensor(a->k, "k", kD)) return rc;
    if (int rc = check_token_tensor(a->v, "v", kD)) return rc;
    if (int rc = check_token_tensor(a->u, "u", kD)) return rc;
    if (int rc = check_token_tensor(a->w, "w", kD)) return rc;
    if (int rc = check_scalar(a->beta, "beta", true)) return rc;
    if (int rc = check_scalar(a->gate_cumsum, "gate", false)) return rc;
    DeviceInfo* d = nullptr;
    if (int rc = get_device_info(&d)) return rc;
    return launch_uw(a->shape, a->k, a->v, a->u, a->w, a->beta, a->gate_cumsum, false, d,
                     static_cast<cudaStream_t>(stream));
}

int gdn_seq_state_update(const GdnSeqStateArgs* a, gdn_stream_t stream) {
    GDN_REQUIRE(a != nullptr, "gdn_seq_state_update: args is NULL");
    const GdnShape& s = a->shape;
    if (int rc = check_shape(s, false)) return rc;
    if (int rc = require_d128(s, "gdn_seq_state_update")) return rc;
    if (int rc = check_token_tensor(a->k, "k", kD)) return rc;
    if (int rc = check_token_tensor(a->u, "u", kD)) return rc;
    if (int rc = check_token_tensor(a->w, "w", kD)) return rc;
    if (int rc = check_scalar(a->gate_cumsum, "gate", false)) return rc;
    if (int rc = check_state(a->initial_state, "initial_state")) return rc;
    if (int rc = check_state(a->final_state, "final_state")) return rc;
    GDN_REQUIRE(a->chunk_states != nullptr, "gdn_seq_state_update: chunk_states is NULL");
    GDN_REQUIRE(aligned16(a->chunk_states), "chunk_states must be 16-byte aligned");
    GDN_REQUIRE(!s.cu_seqlens || s.cu_chunks, "gdn_seq_state_update: packed mode needs cu_chunks");
    GDN_REQUIRE(s.num_v_heads <= 65535, "too many heads");
    DeviceInfo* d = nullptr;
    if (int rc = get_device_info(&d)) return rc;
    CUtensorMap tmK, tmW, tmU;
    if (int rc = make_token_map(&tmK, a->k, s, s.num_k_heads, "k")) return rc;
    if (int rc = make_token_map(&tmW, a->w, s, s.num_v_heads, "w")) return rc;
    if (int rc = make_token_map(&tmU, a->u, s, s.num_v_heads, "u")) return rc;
    SeqParams p{};
    p.map = chunk_map(s);
    p.gate = scalar_view(a->gate_cumsum);
    p.gate_is_raw = 0;
    p.u_out = token_view(a->u);
    p.state_in = static_cast<const __nv_bfloat16*>(a->initial_state.ptr);
    p.si_ss = a->initial_state.stride_seq;
    p.si_sh = a->initial_state.stride_head;
    p.state_out = static_cast<__nv_bfloat16*>(a->final_state.ptr);
    p.so_ss = a->final_state.stride_seq;
    p.so_sh = a->final_state.stride_head;
    p.chunk_states = static_cast<__nv_bfloat16*>(a->chunk_states);
    p.kh = s.num_k_heads;
    p.vh = s.num_v_heads;
    p.scale = 1.f;
    p.status = d->status;
    return launch_seq_t<false, true, true>(tmK, tmK, tmW, tmU, p, dim3(s.batch, s.num_v_heads),
                                           static_cast<cudaStream_t>(stream));
}

int gdn_compute_o(const GdnComputeOArgs* a, gdn_stream_t stream) {
    GDN_REQUIRE(a != nullptr, "gdn_compute_o: args is NULL");
    const GdnShape& s = a->shape;
    if (int rc = check_shape(s, true)) return rc;
    if (int rc = require_d128(s, "gdn_compute_o")) return rc;
    if (int rc = check_token_tensor(a->q, "q", kD)) return rc;
    if (int rc = check_token_tensor(a->k, "k", kD)) return rc;
    if (int rc = check_token_tensor(a->u_new, "u", kD)) return rc;
    if (int rc = check_token_tensor(a->out, "o", kD)) return rc;
    if (int rc = check_scalar(a->gate_cumsum, "gate", false)) return rc;
    GDN_REQUIRE(a->chunk_states != nullptr && aligned16(a->chunk_states), "gdn_compute_o: chunk_states must be a 16-byte aligned pointer");
    GDN_REQUIRE(s.num_v_heads <= 65535, "too many heads");
    const int nc = num_chunks(s);
    if (nc == 0) return GDN_OK;
    const long long units = static_cast<long long>(nc) * s.num_v_heads;
    GDN_REQUIRE(units * 128 < (1ll << 31), "gdn_compute_o: too many (chunk, head) units");
    DeviceInfo* d = nullptr;
    if (int rc = get_device_info(&d)) return rc;
    CUtensorMap tmQ, tmK, tmU, tmH, tmO;
    if (int rc = make_token_map(&tmQ, a->q, s, s.num_k_heads, "q")) return rc;
    if (int rc = make_token_map(&tmK, a->k, s, s.num_k_heads, "k")) return rc;
    if (int rc = make_token_map(&tmU, a->u_new, s, s.num_v_heads, "u")) return rc;
    if (int rc = make_token_map(&tmO, a->out, s, s.num_v_heads, "o")) return rc;
    {
        uint64_t dims[2] = {128, static_cast<uint64_t>(units) * 128};
        uint64_t strides[1] = {256};
        uint32_t box[2] = {64, 128};
        if (!make_tmap_bf16(&tmH, a->chunk_states, 2, dims, strides, box, true))
            return fail(GDN_ERR_CUDA, "could not encode the TMA descriptor of the chunk states");
    }
    OParams p{};
    p.map = chunk_map(s);
    p.gate = scalar_view(a->gate_cumsum);
    p.out = token_view(a->out);
    p.kh = s.num_k_heads;
    p.vh = s.num_v_heads;
    p.scale = a->scale;
    p.status = d->status;
    constexpr int smem = OSmem::kBytes;
    if (int rc = set_smem(gdn_o_kernel, smem)) return rc;
    gdn_o_kernel<<<dim3(nc, s.num_v_heads), 128, smem, static_cast<cudaStream_t>(stream)>>>(tmQ, tmK, tmU, tmH, tmO, p);
    GDN_CUDA(cudaGetLastError());
    return GDN_OK;
}

// Head dims above the 128 the tensor-core kernels are built for (192 and 256, which the
// reference's chunked kernels accept: sm90_bf16_gdn_compute_u_w.cuh:169) take the token-recurrent
// kernel: the same layer semantics with the state kept in fp32 from the first token to the last,
// no scratch, one launch.  Slower per token than the chunked kernels, but exact and on the GPU.
static bool wide_heads(const GdnShape& s) { return s.head_dim_k > kD || s.head_dim_v > kD; }

static int chunked_forward_wide(const GdnChunkedArgs* a, gdn_stream_t stream) {
    const GdnShape& s = a->shape;
    GDN_REQUIRE(s.head_dim_k == s.head_dim_v && s.head_dim_k % 64 == 0 && s.head_dim_k <= 256,
                "gdn_chunked_forward: head dims above 128 must be dk = dv = 192 or 256 (got %d, %d); pad with zeros",
                s.head_dim_k, s.head_dim_v);
    GDN_REQUIRE(a->final_state.ptr != nullptr, "gdn_chunked_forward: head dims above 128 need a final_state buffer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    void* const* ev = a->stage_events;
    if (ev) {
        GDN_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(ev[0]), st));
        GDN_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(ev[1]), st));
    }
    GdnRecurrentArgs r{};
    r.shape = s;
    r.q = a->q;
    r.k = a->k;
    r.v = a->v;
    r.out = a->out;
    r.beta = a->beta;
    r.gate = a->gate;
    r.state_in = a->initial_state;
    r.state_out = a->final_state;
    r.scale = a->scale;
    r.is_qk_norm = a->is_qk_norm;
    if (int rc = gdn_recurrent_forward(&r, stream)) return rc;
    if (ev) GDN_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(ev[2]), st));
    return GDN_OK;
}

// Launch of the state kernel right after the chunk-parallel kernel in the same stream, with
// programmatic stream serialization: its CTAs may be placed (each takes a whole SM) and set up while
// that kernel drains; the kernel waits (grid_dep_wait) before it reads that kernel's results.
static cudaError_t launch_fused_after_zp(dim3 grid, int smem, cudaStream_t st, const CUtensorMap& tmQ, const CUtensorMap& tmK,
                                         const CUtensorMap& tmV, const CUtensorMap& tmO, const FusedParams& p) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(fused::kThreads);
    cfg.dynamicSmemBytes = static_cast<size_t>(smem);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gdn_fused_seq_kernel, tmQ, tmK, tmV, tmO, p);
}

// Workspace layout of gdn_chunked_forward: [Z, PT blocks][q/k norm factors][segment states | sequence order]
static size_t ws_blocks_bytes(size_t chunks, int vh) { return (chunks * static_cast<size_t>(vh) * kZPBlockBytes + 255) / 256 * 256; }
static size_t ws_norms_bytes(size_t chunks, int kh) { return (chunks * static_cast<size_t>(kh) * 128 * sizeof(float) + 255) / 256 * 256; }

// The segment plan of a problem (heuristics.hpp); num_segments == 1: not segmented.
static SegmentPlan segment_plan_of(const GdnShape& s) {
    if (s.cu_seqlens) return prefill_segments_packed(s.batch, s.num_v_heads, s.total_chunks > 0 ? s.total_chunks : 0);
    SegmentPlan plan = prefill_segments(static_cast<long long>(s.batch) * s.num_v_heads, (s.seq_len + kChunk - 1) / kChunk, false);
    plan.slots = s.batch * plan.num_segments;
    return plan;
}

size_t gdn_chunked_forward_workspace_bytes(const GdnShape* s) {
    if (!s) return 0;
    if (wide_heads(*s)) return 0;
    const size_t chunks = s->cu_seqlens ? static_cast<size_t>(s->total_chunks > 0 ? s->total_chunks : 0)
                                        : static_cast<size_t>(s->batch) * static_cast<size_t>((s->seq_len + kChunk - 1) / kChunk);
    // one block of Z (64 x 128 bf16) and PT (64 x 64 bf16) per (chunk, v-head); for a
    // segmented run (few long sequences) three fp32 states per v-head and segment slot on top
    size_t bytes = ws_blocks_bytes(chunks, s->num_v_heads) + ws_norms_bytes(chunks, s->num_k_heads) + 256;
    const SegmentPlan plan = segment_plan_of(*s);
    if (plan.num_segments > 1)
        bytes += static_cast<size_t>(plan.slots) * s->num_v_heads * 3 * kD * kD * sizeof(float) + 256;
    else if (s->cu_seqlens && s->batch > 1 && s->batch <= kMaxOrderedSeqs)
        bytes += (static_cast<size_t>(s->batch) * sizeof(int) + 255) / 256 * 256;  // sequences by length
    return bytes;
}

int gdn_chunked_forward(const GdnChunkedArgs* a, gdn_stream_t stream) {
    GDN_REQUIRE(a != nullptr, "gdn_chunked_forward: args is NULL");
    const GdnShape& s = a->shape;
    if (int rc = check_shape(s, true)) return rc;
    if (wide_heads(s)) return chunked_forward_wide(a, stream);
    // The kernels are built for dk = dv = 128.  A smaller head dim that is a multiple of 8 (the 16-byte
    // rule of the copies) runs on them as it is: the tensor maps deliver zero columns past it and the state
    // is read and written with a column predicate, which is the zero-padded problem without padded copies.
    const int hd = s.head_dim_k;
    if (s.head_dim_k != s.head_dim_v || hd % 8 != 0)
        return fail(GDN_ERR_UNSUPPORTED,
                    "gdn_chunked_forward: head dims must be dk = dv, a multiple of 8 up to 128, or 192 / 256 (got %d, %d); "
                    "pad the head dimension with zeros (the Python and C++ wrappers do)", s.head_dim_k, s.head_dim_v);
    if (int rc = check_token_tensor(a->q, "q", hd)) return rc;
    if (int rc = check_token_tensor(a->k, "k", hd)) return rc;
    if (int rc = check_token_tensor(a->v, "v", hd)) return rc;
    if (int rc = check_token_tensor(a->out, "out", hd)) return rc;
    if (int rc = check_scalar(a->beta, "beta", true)) return rc;
    if (int rc = check_scalar(a->gate, "gate", false)) return rc;
    if (int rc = check_state(a->initial_state, "initial_state")) return rc;
    if (int rc = check_state(a->final_state, "final_state")) return rc;
    GDN_REQUIRE(s.num_v_heads <= 65535, "too many heads");
    const size_t need = gdn_chunked_forward_workspace_bytes(&s);
    if (!a->workspace || a->workspace_bytes < need || (reinterpret_cast<uintptr_t>(a->workspace) & 255u))
        return fail(GDN_ERR_WORKSPACE, "gdn_chunked_forward: workspace of %zu bytes (256-byte aligned) required, got %zu",
                    need, a->workspace_bytes);
    DeviceInfo* d = nullptr;
    if (int rc = get_device_info(&d)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    const bool packed = s.cu_seqlens != nullptr;
    void* const* ev = a->stage_events;
    if (ev) GDN_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(ev[0]), st));
    GDN_REQUIRE(!packed || s.cu_chunks, "gdn_chunked_forward: packed mode needs cu_chunks");
    if (num_chunks(s) == 0) {
        if (ev) {
            GDN_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(ev[1]), st));
            GDN_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(ev[2]), st));
        }
        return GDN_OK;
    }
    uint8_t* const ws = static_cast<uint8_t*>(a->workspace);
    const size_t nchunks = static_cast<size_t>(num_chunks(s));
    float* const norms = a->is_qk_norm ? reinterpret_cast<float*>(ws + ws_blocks_bytes(nchunks, s.num_v_heads)) : nullptr;
    uint8_t* const ws_extra = ws + ws_blocks_bytes(nchunks, s.num_v_heads) + ws_norms_bytes(nchunks, s.num_k_heads);
    // Both kernels are prepared before the first is launched, so that the state kernel is in the stream
    // when the chunk-parallel kernel starts to drain.
    auto run_zp = [&]() -> int {
        if (int rc = launch_zp(s, a->q, a->k, a->beta, a->gate, a->workspace, norms, a->scale, d, st)) return rc;
        if (ev) GDN_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(ev[1]), st));
        return GDN_OK;
    };
    {
        CUtensorMap tmQ, tmK, tmV, tmO;
        if (int rc = make_token_map(&tmQ, a->q, s, s.num_k_heads, "q", hd)) return rc;
        if (int rc = make_token_map(&tmK, a->k, s, s.num_k_heads, "k", hd)) return rc;
        if (int rc = make_token_map(&tmV, a->v, s, s.num_v_heads, "v", hd)) return rc;
        if (int rc = make_token_map(&tmO, a->out, s, s.num_v_heads, "out", hd)) return rc;
        FusedParams p{};
        p.d = hd;
        p.map = chunk_map(s);
        p.gate = scalar_view(a->gate);
        p.out = token_view(a->out);
        p.state_in = static_cast<const __nv_bfloat16*>(a->initial_state.ptr);
        p.si_ss = a->initial_state.stride_seq;
        p.si_sh = a->initial_state.stride_head;
        p.state_out = static_cast<__nv_bfloat16*>(a->final_state.ptr);
        p.so_ss = a->final_state.stride_seq;
        p.so_sh = a->final_state.stride_head;
        p.kh = s.num_k_heads;
        p.vh = s.num_v_heads;
        p.scale = a->scale;
        p.status = d->status;
        p.blocks = static_cast<const uint8_t*>(a->workspace);
        p.norms = norms;
        constexpr int smem = FusedSmem::kBytes;
        if (int rc = set_smem(gdn_fused_seq_kernel, smem)) return rc;
        const long long chains = static_cast<long long>(s.batch) * s.num_v_heads;
        const SegmentPlan plan = segment_plan_of(s);
        if (plan.num_segments <= 1 && packed && s.batch > 1 && s.batch <= kMaxOrderedSeqs && chains > d->sms) {
            // more chains than SMs and unequal lengths: dispatch the longest sequences first
            int* order = reinterpret_cast<int*>(ws_extra);
            gdn_seq_order_kernel<<<(s.batch + 127) / 128, 128, 0, st>>>(s.cu_seqlens, s.batch, order);
            GDN_CUDA(cudaGetLastError());
            p.seq_order = order;
            if (int rc = run_zp()) return rc;
            GDN_CUDA(launch_fused_after_zp(dim3(s.num_v_heads, s.batch), smem, st, tmQ, tmK, tmV, tmO, p));
        } else if (plan.num_segments <= 1) {
            if (int rc = run_zp()) return rc;
            GDN_CUDA(launch_fused_after_zp(dim3(s.batch, s.num_v_heads), smem, st, tmQ, tmK, tmV, tmO, p));
        } else {
            // composite transitions of all segments, their start states, then all segments at once
            float* seg_mn = reinterpret_cast<float*>(ws_extra);
            const size_t seg_units = static_cast<size_t>(plan.slots) * s.num_v_heads;
            float* seg_start = seg_mn + seg_units * 2 * kD * kD;
            p.seg_chunks = plan.seg_chunks;
            p.num_segments = plan.num_segments;
            p.num_seqs = s.batch;
            p.seg_mn = seg_mn;
            p.seg_start = seg_start;
            p.mode = 1;
            if (int rc = set_smem(gdn_seg_combine_kernel, SegCombineSmem::kBytes)) return rc;
            if (int rc = run_zp()) return rc;
            GDN_CUDA(launch_fused_after_zp(dim3(plan.slots, s.num_v_heads, 2), smem, st, tmQ, tmK, tmV, tmO, p));
            SegCombineParams cp{};
            cp.seg_mn = seg_mn;
            cp.seg_start = seg_start;
            cp.state_in = p.state_in;
            cp.si_ss = p.si_ss;
            cp.si_sh = p.si_sh;
            cp.d = hd;
            cp.vh = s.num_v_heads;
            cp.num_segments = plan.num_segments;
            cp.map = p.map;
            cp.seg_chunks = plan.seg_chunks;
            cp.status = d->status;
            {
                // a programmatic dependent of the composite-transition launch (it waits before its first global access)
                cudaLaunchConfig_t cfg{};
                cfg.gridDim = dim3(static_cast<unsigned>(chains), kD / SegCombineSmem::R);
                cfg.blockDim = dim3(128);
                cfg.dynamicSmemBytes = SegCombineSmem::kBytes;
                cfg.stream = st;
                cudaLaunchAttribute attr[1];
                attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
                attr[0].val.programmaticStreamSerializationAllowed = 1;
                cfg.attrs = attr;
                cfg.numAttrs = 1;
                GDN_CUDA(cudaLaunchKernelEx(&cfg, gdn_seg_combine_kernel, cp));
            }
            p.mode = 2;
            GDN_CUDA(launch_fused_after_zp(dim3(plan.slots, s.num_v_heads), smem, st, tmQ, tmK, tmV, tmO, p));
        }
    }
    if (ev) GDN_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(ev[2]), st));
    return GDN_OK;
}

// ------------------------------------------------------------------ prefill on built-in scratch
// Scratch for callers that cannot allocate device memory (see include/gdn_b200.h).  The array
// lives in the library image; in host code its name is only a handle for the runtime, so the
// device address is looked up once per device and that address is what the kernels receive.
static __device__ __align__(256) unsigned char g_static_scratch[GDN_STATIC_SCRATCH_BYTES];
static void* g_static_scratch_addr[64] = {};
static std::mutex g_static_scratch_mutex;

int gdn_chunked_forward_static_scratch(const GdnChunkedArgs* a, gdn_stream_t stream) {
    GDN_REQUIRE(a != nullptr, "gdn_chunked_forward_static_scratch: args is NULL");
    if (int rc = check_shape(a->shape, true)) return rc;
    const size_t need = gdn_chunked_forward_workspace_bytes(&a->shape);
    if (need > GDN_STATIC_SCRATCH_BYTES)
        return fail(GDN_ERR_WORKSPACE,
                    "gdn_chunked_forward_static_scratch: this problem needs %zu bytes of scratch but the built-in "
                    "array holds %u (384 bytes per token and v-head); use gdn_chunked_forward with a "
                    "caller-provided workspace",
                    need, GDN_STATIC_SCRATCH_BYTES);
    int dev = 0;
    GDN_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(GDN_ERR_UNSUPPORTED, "device index %d out of range", dev);
    void* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
        if (!g_static_scratch_addr[dev]) {
            // first call on this device (it is the current one): resolve the device address
            void* p = nullptr;
            GDN_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
            if (!p) return fail(GDN_ERR_CUDA, "built-in scratch array has no device address");
            g_static_scratch_addr[dev] = p;
        }
        scratch = g_static_scratch_addr[dev];
    }
    GdnChunkedArgs b = *a;
    b.workspace = scratch;
    b.workspace_bytes = GDN_STATIC_SCRATCH_BYTES;
    return gdn_chunked_forward(&b, stream);
}

}  // extern "C"
