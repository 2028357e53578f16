// C-ABI entry points of libgdn_b200.so: runtime, helper kernels and the recurrent
// (decode / speculative-verify) path.  The chunked-prefill entry points live in
// gdn_prefill.cu.  See include/gdn_b200.h for the contract of each function.
#include "heuristics.hpp"
#include "host_common.hpp"
#include "jit/jit.hpp"
#include "kernels/helpers.cuh"
#include "kernels/layer_adjacent.cuh"
#include "kernels/recurrent.cuh"

#include <atomic>

namespace gdn {

static __device__ int g_status_word;

static std::mutex g_dev_mutex;
static DeviceInfo g_devices[64];
static std::string g_library_root, g_cuda_home;
// Environment switches of the recurrent path, read when the library is first used and again by
// every gdn_init() (never on the launch path): GDN_REC_RING_MIN (tuning aid: token count above
// which the multi-token instance is used), GDN_JIT_RECURRENT (test aid: force the run-time compiler).
static std::atomic<int> g_ring_min{-1}, g_force_jit{-1};
static void read_env_switches() {
    g_ring_min.store(jit::env_int("GDN_REC_RING_MIN", kRecTokRingMin));
    g_force_jit.store(jit::env_int("GDN_JIT_RECURRENT", 0));
}

int get_device_info(DeviceInfo** out) {
    int dev = 0;
    GDN_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(GDN_ERR_UNSUPPORTED, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    DeviceInfo& d = g_devices[dev];
    if (!d.valid) {
        GDN_CUDA(cudaDeviceGetAttribute(&d.major, cudaDevAttrComputeCapabilityMajor, dev));
        GDN_CUDA(cudaDeviceGetAttribute(&d.minor, cudaDevAttrComputeCapabilityMinor, dev));
        GDN_CUDA(cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev));
        if (d.major != 10)
            return fail(GDN_ERR_UNSUPPORTED,
                        "device %d is sm_%d%d; this library only has sm_100a kernels", dev, d.major,
                        d.minor);
        void* p = nullptr;
        GDN_CUDA(cudaGetSymbolAddress(&p, g_status_word));
        d.status = static_cast<int*>(p);
        d.valid = true;
    }
    *out = &d;
    return GDN_OK;
}

const std::string& library_root() { return g_library_root; }
const std::string& cuda_home() { return g_cuda_home; }

}  // namespace gdn

using namespace gdn;

// ------------------------------------------------------------------ self-test of the bounded waits
// One warp waits, with the given cycle limit, on an mbarrier that nothing ever arrives on.  The
// wait gives up, the kernel records status 7 and returns: the same path a product kernel takes
// when a copy or an MMA never completes, exercised without any fault.
__global__ void gdn_selftest_wait_kernel(long long limit_cycles, int* status) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        ptx::mbar_init(&bar, 1);
        ptx::mbar_fence_init();
    }
    __syncthreads();
    const bool ok = ptx::mbar_wait_limit(&bar, 0, &abort_flag, limit_cycles);
    __syncthreads();
    if (threadIdx.x == 0 && (!ok || abort_flag) && status) atomicExch(status, 7);
}

// ------------------------------------------------------------------ recurrent
// Launch with programmatic stream serialization: the kernel's CTAs may be placed while the preceding work in the
// stream drains; every kernel launched this way waits (griddepcontrol.wait) before its first global access.
template <typename P>
static cudaError_t launch_dependent(void (*kernel)(P), dim3 grid, int threads, size_t smem, cudaStream_t st, const P& params) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, params);
}

template <int DK, bool kRing, bool kLean = false, bool kF32 = false>
static int launch_recurrent_t(const RecurrentParams& p, int sms, cudaStream_t st) {
    constexpr int smem = recurrent_smem_bytes<DK, kRing, kF32>();
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set[dev]) {
        GDN_CUDA(cudaFuncSetAttribute(gdn_recurrent_kernel<DK, kRing, kLean, kF32>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        attr_set[dev] = true;
    }
    const int per_sm = recurrent_ctas_per_sm<DK, kRing, kF32>();
    const long long grid = std::min<long long>(p.num_tiles, static_cast<long long>(sms) * per_sm);
    GDN_CUDA(launch_dependent(gdn_recurrent_kernel<DK, kRing, kLean, kF32>, dim3(static_cast<unsigned>(grid)), kRecThreads, smem, st, p));
    return GDN_OK;
}

// `ring`: long runs of tokens (more than kRecTokRingMin per sequence on average) take the instance
// with the multi-token ring; speculative verify keeps the decode instance; plain single-token decode
// from a given state (`lean`) takes the decode instance with its run-time tests compiled away.
template <int DK>
static int launch_recurrent(const RecurrentParams& p, int sms, cudaStream_t st, bool ring, bool lean) {
    if (ring) return launch_recurrent_t<DK, true>(p, sms, st);
    if (lean) return launch_recurrent_t<DK, false, true>(p, sms, st);
    return launch_recurrent_t<DK, false>(p, sms, st);
}

// Head dimensions without a prebuilt kernel (or every call when GDN_JIT_RECURRENT=1) go through
// the run-time compiler: a three-line translation unit instantiates the kernel body for DK.
static int launch_recurrent_jit(const RecurrentParams& p, int dk, int sms, cudaStream_t st, bool ring) {
    const RecurrentConfig cfg = recurrent_config(dk, p.num_tiles, sms, ring);
    char src[512];
    snprintf(src, sizeof(src),
             "#include \"kernels/recurrent.cuh\"\n"
             "extern \"C\" __global__ void __launch_bounds__(%d, %d) gdn_recurrent_jit(const gdn::RecurrentParams p) {\n"
             "    gdn::gdn_recurrent_body<%d, %s>(p);\n}\n",
             kRecThreads, cfg.ctas_per_sm, dk, ring ? "true" : "false");
    jit::LoadedKernel k;
    std::string err;
    if (int rc = jit::get_kernel("recurrent_dk" + std::to_string(dk) + (ring ? "_ring" : ""), src, "gdn_recurrent_jit", &k, &err))
        return fail(rc, "%s", err.c_str());
    GDN_CUDA(cudaFuncSetAttribute(reinterpret_cast<const void*>(k.kernel), cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  cfg.smem_bytes));
    RecurrentParams pc = p;
    void* args[] = {&pc};
    GDN_CUDA(cudaLaunchKernel(reinterpret_cast<const void*>(k.kernel), dim3(static_cast<unsigned>(cfg.grid)),
                              dim3(kRecThreads), args, cfg.smem_bytes, st));
    return GDN_OK;
}

extern "C" {

int gdn_init(const char* library_root, const char* cuda_home) {
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    g_library_root = library_root ? library_root : "";
    g_cuda_home = cuda_home ? cuda_home : "";
    jit::set_roots(g_library_root, g_cuda_home);
    read_env_switches();
    return GDN_OK;
}

const char* gdn_last_error(void) { return last_error_ref().c_str(); }

int gdn_version(void) { return 100; }

int gdn_device_status(int device, int* status_out) {
    GDN_REQUIRE(status_out != nullptr, "status_out is NULL");
    int cur = 0;
    GDN_CUDA(cudaGetDevice(&cur));
    if (device != cur) GDN_CUDA(cudaSetDevice(device));
    DeviceInfo* d = nullptr;
    int rc = get_device_info(&d);
    if (rc == GDN_OK) {
        cudaError_t e = cudaDeviceSynchronize();
        if (e == cudaSuccess) e = cudaMemcpy(status_out, d->status, sizeof(int), cudaMemcpyDeviceToHost);
        if (e == cudaSuccess) e = cudaMemset(d->status, 0, sizeof(int));
        if (e != cudaSuccess) rc = fail(GDN_ERR_CUDA, "reading status word: %s", cudaGetErrorString(e));
    }
    if (device != cur) cudaSetDevice(cur);
    return rc;
}

int gdn_selftest_bounded_wait(int64_t limit_cycles, gdn_stream_t stream) {
    GDN_REQUIRE(limit_cycles > 0 && limit_cycles <= 1000000000ll,
                "gdn_selftest_bounded_wait: limit must be between 1 and 1e9 cycles (got %lld)", (long long)limit_cycles);
    DeviceInfo* d = nullptr;
    if (int rc = get_device_info(&d)) return rc;
    gdn_selftest_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(limit_cycles, d->status);
    GDN_CUDA(cudaGetLastError());
    return GDN_OK;
}

// ------------------------------------------------------------------ helpers
int gdn_fused_gating(const void* A_log, const void* dt_bias, const void* a, const void* b,
                     void* beta, void* gate, int64_t num_tokens, int32_t num_v_heads,
                     int32_t dtype, int32_t gate_dtype, gdn_stream_t stream) {
    GDN_REQUIRE(A_log && dt_bias && a && b && beta && gate, "gdn_fused_gating: NULL pointer");
    GDN_REQUIRE(num_tokens >= 0 && num_v_heads > 0, "gdn_fused_gating: bad sizes");
    GDN_REQUIRE(dtype == GDN_BF16 || dtype == GDN_F32, "gdn_fused_gating: dtype must be bf16 or f32");
    GDN_REQUIRE(gate_dtype == GDN_BF16 || gate_dtype == GDN_F32, "gdn_fused_gating: bad gate dtype");
    DeviceInfo* d = nullptr;
    if (int rc = get_device_info(&d)) return rc;
    const long long total = static_cast<long long>(num_tokens) * num_v_heads;
    if (total == 0) return GDN_OK;
    const int blocks = static_cast<int>(std::min<long long>((total + 255) / 256, d->sms * 16ll));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    using bf = __nv_bfloat16;
    if (dtype == GDN_F32 && gate_dtype == GDN_F32)
        gdn_gating_kernel<float, float><<<blocks, 256, 0, st>>>((const float*)A_log, (const float*)dt_bias, (const float*)a, (const float*)b, (float*)beta, (float*)gate, total, num_v_heads);
    else if (dtype == GDN_BF16 && gate_dtype == GDN_BF16)
        gdn_gating_kernel<bf, bf><<<blocks, 256, 0, st>>>((const bf*)A_log, (const bf*)dt_bias, (const bf*)a, (const bf*)b, (bf*)beta, (bf*)gate, total, num_v_heads);
    else if (dtype == GDN_BF16 && gate_dtype == GDN_F32)
        gdn_gating_kernel<bf, float><<<blocks, 256, 0, st>>>((const bf*)A_log, (const bf*)dt_bias, (const bf*)a, (const bf*)b, (bf*)beta, (float*)gate, total, num_v_heads);
    else
        return fail(GDN_ERR_UNSUPPORTED, "gdn_fused_gating: f32 inputs with bf16 gate is not built");
    GDN_CUDA(cudaGetLastError());
    return GDN_OK;
}

int gdn_chunk_local_cumsum(const void* input, float* output, int32_t in_dtype, int32_t batch,
                           int64_t seq_len, int32_t num_heads, int32_t token_major,
                           const int32_t* cu_seqlens, const int32_t* chunk_indices,
                           int32_t total_chunks, gdn_stream_t stream) {
    GDN_REQUIRE(input && output, "gdn_chunk_local_cumsum: NULL pointer");
    GDN_REQUIRE(in_dtype == GDN_BF16 || in_dtype == GDN_F32, "gdn_chunk_local_cumsum: bad dtype");
    GDN_REQUIRE(batch > 0 && seq_len >= 0 && num_heads > 0, "gdn_chunk_local_cumsum: bad sizes");
    int chunks_per_seq = 0, nchunks = 0;
    if (cu_seqlens) {
        GDN_REQUIRE(chunk_indices != nullptr, "gdn_chunk_local_cumsum: packed mode needs chunk_indices");
        GDN_REQUIRE(total_chunks >= 0, "gdn_chunk_local_cumsum: bad total_chunks");
        nchunks = total_chunks;
    } else {
        chunks_per_seq = static_cast<int>((seq_len + 63) / 64);
        nchunks = chunks_per_seq * batch;
    }
    if (nchunks == 0) return GDN_OK;
    DeviceInfo* d = nullptr;
    if (int rc = get_device_info(&d)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const long long items = static_cast<long long>(nchunks) * num_heads;
    using bf = __nv_bfloat16;
    if (token_major) {
        const unsigned blocks = static_cast<unsigned>((items + 127) / 128);
        if (in_dtype == GDN_F32)
            gdn_cumsum_token_major_kernel<float><<<blocks, 128, 0, st>>>((const float*)input, output, nchunks, chunks_per_seq, seq_len, num_heads, cu_seqlens, chunk_indices);
        else
            gdn_cumsum_token_major_kernel<bf><<<blocks, 128, 0, st>>>((const bf*)input, output, nchunks, chunks_per_seq, seq_len, num_heads, cu_seqlens, chunk_indices);
    } else {
        const unsigned blocks = static_cast<unsigned>((items + 3) / 4);
        if (in_dtype == GDN_F32)
            gdn_cumsum_time_major_kernel<float><<<blocks, 128, 0, st>>>((const float*)input, output, nchunks, chunks_per_seq, seq_len, num_heads, batch, cu_seqlens, chunk_indices);
        else
            gdn_cumsum_time_major_kernel<bf><<<blocks, 128, 0, st>>>((const bf*)input, output, nchunks, chunks_per_seq, seq_len, num_heads, batch, cu_seqlens, chunk_indices);
    }
    GDN_CUDA(cudaGetLastError());
    return GDN_OK;
}

int gdn_transpose_mn_major(const void* input, void* output, int32_t elem_size, int64_t groups,
                           int64_t mn, int64_t k, int64_t mn_aligned, gdn_stream_t stream) {
    GDN_REQUIRE(input && output, "gdn_transpose_mn_major: NULL pointer");
    GDN_REQUIRE(elem_size == 2 || elem_size == 4, "gdn_transpose_mn_major: element size must be 2 or 4");
    GDN_REQUIRE(groups >= 0 && mn >= 0 && k >= 0 && mn_aligned >= mn, "gdn_transpose_mn_major: bad sizes");
    GDN_REQUIRE(groups <= 65535 && (k + 31) / 32 <= 65535, "gdn_transpose_mn_major: too many groups or columns");
    if (groups == 0 || k == 0 || mn_aligned == 0) return GDN_OK;
    DeviceInfo* d = nullptr;
    if (int rc = get_device_info(&d)) return rc;
    dim3 grid(static_cast<unsigned>((mn_aligned + 31) / 32), static_cast<unsigned>((k + 31) / 32),
              static_cast<unsigned>(groups));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (elem_size == 4)
        gdn_transpose_kernel<uint32_t><<<grid, 256, 0, st>>>((const uint32_t*)input, (uint32_t*)output, mn, k, mn_aligned);
    else
        gdn_transpose_kernel<uint16_t><<<grid, 256, 0, st>>>((const uint16_t*)input, (uint16_t*)output, mn, k, mn_aligned);
    GDN_CUDA(cudaGetLastError());
    return GDN_OK;
}

int gdn_causal_conv1d(const GdnConvArgs* a, gdn_stream_t stream) {
    GDN_REQUIRE(a != nullptr, "gdn_causal_conv1d: args is NULL");
    GDN_REQUIRE(a->x && a->y && a->weight, "gdn_causal_conv1d: x, y and weight are required");
    GDN_REQUIRE(a->width >= 2 && a->width <= kConvMaxWidth, "gdn_causal_conv1d: width must be 2 .. 4 (got %d)", a->width);
    GDN_REQUIRE(a->channels > 0 && a->channels % 8 == 0, "gdn_causal_conv1d: channels must be a positive multiple of 8");
    GDN_REQUIRE(a->batch > 0, "gdn_causal_conv1d: batch must be positive");
    GDN_REQUIRE(aligned16(a->x) && aligned16(a->y) && a->x_stride_token % 8 == 0 && a->y_stride_token % 8 == 0 &&
                    a->x_stride_batch % 8 == 0 && a->y_stride_batch % 8 == 0,
                "gdn_causal_conv1d: x and y must be 16-byte aligned with strides that are multiples of 8 elements");
    GDN_REQUIRE(a->x_stride_token >= a->channels && a->y_stride_token >= a->channels, "gdn_causal_conv1d: token stride below channels");
    GDN_REQUIRE((!a->state_in || aligned16(a->state_in)) && (!a->state_out || aligned16(a->state_out)),
                "gdn_causal_conv1d: states must be 16-byte aligned");
    const bool packed = a->cu_seqlens != nullptr;
    const long long tokens = packed ? a->total_tokens : a->seq_len;
    GDN_REQUIRE(tokens >= 0, "gdn_causal_conv1d: negative token count");
    if (a->state_out && a->state_out == a->state_in)
        GDN_REQUIRE(packed ? a->total_tokens <= a->batch : a->seq_len <= kConvTokBlock,
                    "gdn_causal_conv1d: state_out may alias state_in only when no sequence spans more than one %d-token block",
                    kConvTokBlock);
    DeviceInfo* d = nullptr;
    if (int rc = get_device_info(&d)) return rc;
    if (tokens == 0 && !packed) return GDN_OK;
    ConvParams p{};
    p.x = static_cast<const __nv_bfloat16*>(a->x);
    p.y = static_cast<__nv_bfloat16*>(a->y);
    p.w = static_cast<const __nv_bfloat16*>(a->weight);
    p.bias = static_cast<const __nv_bfloat16*>(a->bias);
    p.state_in = static_cast<const __nv_bfloat16*>(a->state_in);
    p.state_out = static_cast<__nv_bfloat16*>(a->state_out);
    p.x_sb = a->x_stride_batch; p.x_st = a->x_stride_token; p.y_sb = a->y_stride_batch; p.y_st = a->y_stride_token;
    p.cu_seqlens = a->cu_seqlens;
    p.batch = a->batch; p.seq_len = a->seq_len; p.channels = a->channels; p.width = a->width; p.silu = a->silu;
    p.total_tokens = a->total_tokens;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const long long tblocks = (tokens + kConvTokBlock - 1) / kConvTokBlock;
    GDN_REQUIRE(tblocks <= 65535 && a->batch <= 65535, "gdn_causal_conv1d: too many token blocks or sequences for one launch");
    if (tblocks > 0) {
        dim3 grid(static_cast<unsigned>((a->channels / 8 + 127) / 128), static_cast<unsigned>(tblocks), packed ? 1u : static_cast<unsigned>(a->batch));
        switch (a->width) {
            case 2: GDN_CUDA(launch_dependent(gdn_causal_conv1d_kernel<2>, grid, 128, 0, st, p)); break;
            case 3: GDN_CUDA(launch_dependent(gdn_causal_conv1d_kernel<3>, grid, 128, 0, st, p)); break;
            default: GDN_CUDA(launch_dependent(gdn_causal_conv1d_kernel<4>, grid, 128, 0, st, p)); break;
        }
    }
    if (packed && p.state_out && p.state_in && p.state_out != p.state_in) {
        gdn_conv_state_passthrough_kernel<<<a->batch, 128, 0, st>>>(p);
        GDN_CUDA(cudaGetLastError());
    }
    return GDN_OK;
}

int gdn_gated_rmsnorm(const void* x, const void* z, void* y, const void* weight, int64_t rows, int32_t dim,
                      int64_t x_row_stride, int64_t z_row_stride, int64_t y_row_stride, float eps, gdn_stream_t stream) {
    GDN_REQUIRE(x && z && y && weight, "gdn_gated_rmsnorm: NULL pointer");
    GDN_REQUIRE(rows >= 0 && dim > 0 && dim % 8 == 0 && dim <= 1024, "gdn_gated_rmsnorm: dim must be a multiple of 8 up to 1024");
    GDN_REQUIRE(aligned16(x) && aligned16(z) && aligned16(y) && aligned16(weight) && x_row_stride % 8 == 0 && z_row_stride % 8 == 0 &&
                    y_row_stride % 8 == 0 && x_row_stride >= dim && z_row_stride >= dim && y_row_stride >= dim,
                "gdn_gated_rmsnorm: pointers must be 16-byte aligned, row strides multiples of 8 and at least dim");
    DeviceInfo* d = nullptr;
    if (int rc = get_device_info(&d)) return rc;
    if (rows == 0) return GDN_OK;
    NormParams p{static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(z), static_cast<__nv_bfloat16*>(y),
                 static_cast<const __nv_bfloat16*>(weight), rows, x_row_stride, z_row_stride, y_row_stride, dim, eps};
    // lanes per row: the smallest power of two (4 .. 32) whose 16-byte pieces cover the row in one pass
    int lpr = 4;
    while (lpr < 32 && lpr * 8 < dim) lpr *= 2;
    const long long rows_per_block = 8ll * (32 / lpr) * (lpr == 32 ? 1 : 2);  // 8 warps, rows in flight per lane group as in the kernel
    const long long blocks = (rows + rows_per_block - 1) / rows_per_block;
    GDN_REQUIRE(blocks < (1ll << 31), "gdn_gated_rmsnorm: too many rows");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (lpr) {
        case 4: GDN_CUDA(launch_dependent(gdn_gated_rmsnorm_kernel<4>, dim3(static_cast<unsigned>(blocks)), 256, 0, st, p)); break;
        case 8: GDN_CUDA(launch_dependent(gdn_gated_rmsnorm_kernel<8>, dim3(static_cast<unsigned>(blocks)), 256, 0, st, p)); break;
        case 16: GDN_CUDA(launch_dependent(gdn_gated_rmsnorm_kernel<16>, dim3(static_cast<unsigned>(blocks)), 256, 0, st, p)); break;
        default: GDN_CUDA(launch_dependent(gdn_gated_rmsnorm_kernel<32>, dim3(static_cast<unsigned>(blocks)), 256, 0, st, p)); break;
    }
    return GDN_OK;
}

int gdn_recurrent_forward(const GdnRecurrentArgs* a, gdn_stream_t stream) {
    GDN_REQUIRE(a != nullptr, "gdn_recurrent_forward: args is NULL");
    if (int rc = check_shape(a->shape, false)) return rc;
    const GdnShape& s = a->shape;
    GDN_REQUIRE(s.head_dim_k % 64 == 0 && s.head_dim_k <= 512,
                "gdn_recurrent_forward: dk must be a multiple of 64 up to 512 (got %d)", s.head_dim_k);
    GDN_REQUIRE(s.head_dim_v % 32 == 0, "gdn_recurrent_forward: dv must be a multiple of 32 (got %d)", s.head_dim_v);
    if (int rc = check_token_tensor(a->q, "q", s.head_dim_k)) return rc;
    if (int rc = check_token_tensor(a->k, "k", s.head_dim_k)) return rc;
    if (int rc = check_token_tensor(a->v, "v", s.head_dim_v)) return rc;
    if (int rc = check_token_tensor(a->out, "out", s.head_dim_v)) return rc;
    const bool fused_gating = a->gating_a.ptr != nullptr;
    if (fused_gating) {
        GDN_REQUIRE(a->gating_b.ptr && a->A_log && a->dt_bias, "gdn_recurrent_forward: fused gating needs a, b, A_log and dt_bias");
        GDN_REQUIRE((a->gating_a.dtype == GDN_BF16 || a->gating_a.dtype == GDN_F32) && a->gating_b.dtype == a->gating_a.dtype,
                    "gdn_recurrent_forward: gating inputs must share one dtype, bf16 or f32");
    } else {
        GDN_REQUIRE(a->beta.ptr != nullptr, "gdn_recurrent_forward: beta is NULL");
        GDN_REQUIRE(a->beta.dtype == GDN_BF16 || a->beta.dtype == GDN_F32, "beta dtype must be bf16 or f32");
        GDN_REQUIRE(!a->gate.ptr || a->gate.dtype == GDN_BF16 || a->gate.dtype == GDN_F32, "gate dtype must be bf16 or f32");
    }
    GDN_REQUIRE(a->state_out.ptr != nullptr, "gdn_recurrent_forward: state_out is NULL");
    GDN_REQUIRE(aligned16(a->state_out.ptr) && a->state_out.stride_seq % 8 == 0 && a->state_out.stride_head % 8 == 0,
                "state_out must be 16-byte aligned with strides that are multiples of 8");
    if (a->state_in.ptr) {
        GDN_REQUIRE(aligned16(a->state_in.ptr) && a->state_in.stride_seq % 8 == 0 && a->state_in.stride_head % 8 == 0,
                    "state_in must be 16-byte aligned with strides that are multiples of 8");
        GDN_REQUIRE(!(a->store_step_state && a->state_in.ptr == a->state_out.ptr),
                    "state_out may not alias state_in when step states are stored");
    }
    GDN_REQUIRE(a->state_dtype == GDN_BF16 || a->state_dtype == GDN_F32, "gdn_recurrent_forward: state_dtype must be bf16 or f32");
    GDN_REQUIRE(!(a->state_indices && a->store_step_state), "gdn_recurrent_forward: state_indices cannot be combined with step states");
    GDN_REQUIRE(!(a->state_indices && !a->state_in.ptr), "gdn_recurrent_forward: state_indices needs a state_in pool");
    DeviceInfo* d = nullptr;
    if (int rc = get_device_info(&d)) return rc;

    RecurrentParams p{};
    p.q = (const __nv_bfloat16*)a->q.ptr; p.q_sb = a->q.stride_batch; p.q_st = a->q.stride_token; p.q_sh = a->q.stride_head;
    p.k = (const __nv_bfloat16*)a->k.ptr; p.k_sb = a->k.stride_batch; p.k_st = a->k.stride_token; p.k_sh = a->k.stride_head;
    p.v = (const __nv_bfloat16*)a->v.ptr; p.v_sb = a->v.stride_batch; p.v_st = a->v.stride_token; p.v_sh = a->v.stride_head;
    p.out = (__nv_bfloat16*)a->out.ptr; p.o_sb = a->out.stride_batch; p.o_st = a->out.stride_token; p.o_sh = a->out.stride_head;
    // with fused gating the kernel reads the raw projections b and a where it would read beta and the gate
    const GdnTokenScalar& sb = fused_gating ? a->gating_b : a->beta;
    const GdnTokenScalar& sg = fused_gating ? a->gating_a : a->gate;
    p.beta = sb.ptr; p.beta_f32 = sb.dtype == GDN_F32;
    p.beta_sb = sb.stride_batch; p.beta_st = sb.stride_token; p.beta_sh = sb.stride_head;
    p.gate = sg.ptr; p.gate_f32 = sg.dtype == GDN_F32;
    p.gate_sb = sg.stride_batch; p.gate_st = sg.stride_token; p.gate_sh = sg.stride_head;
    p.fused_gating = fused_gating;
    p.gating_param_f32 = fused_gating && a->gating_a.dtype == GDN_F32;
    p.A_log = a->A_log;
    p.dt_bias = a->dt_bias;
    p.state_in = a->state_in.ptr; p.si_ss = a->state_in.stride_seq; p.si_sh = a->state_in.stride_head;
    p.state_out = a->state_out.ptr; p.so_ss = a->state_out.stride_seq; p.so_sh = a->state_out.stride_head;
    p.cu_seqlens = s.cu_seqlens;
    p.num_accepted = a->num_accepted_tokens;
    p.state_idx = a->state_indices;
    p.batch = s.batch; p.seq_len = s.seq_len; p.kh = s.num_k_heads; p.vh = s.num_v_heads; p.dv = s.head_dim_v;
    p.scale = a->scale;
    p.is_qk_norm = a->is_qk_norm; p.store_step = a->store_step_state;
    p.num_tiles = static_cast<long long>(s.batch) * s.num_v_heads * (s.head_dim_v / kRecTileRows);
    GDN_REQUIRE(p.num_tiles < (1ll << 31), "gdn_recurrent_forward: too many state tiles");
    p.status = d->status;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    
    if (g_ring_min.load(std::memory_order_relaxed) < 0) read_env_switches();
    const int ring_min = g_ring_min.load(std::memory_order_relaxed);
    const int force_jit = g_force_jit.load(std::memory_order_relaxed);
    const bool ring = s.cu_seqlens ? (s.total_tokens > static_cast<long long>(ring_min) * s.batch)
                                   : (s.seq_len > ring_min);
    // Work units: the ring instance (long token runs) makes every 32-row tile a unit of its own; the decode
    // instance keeps the tiles of a (sequence, v-head) together, which shares the q/k normalisation and the
    // prepared tokens among them.  (Splitting the tiles of small decode batches over more CTAs as well was
    // tried: 3 % at B = 8, and the run-time unit decode it needs cost the large batches 2 %.)
    p.split_tiles = ring ? 1 : 0;
    if (force_jit && a->state_dtype != GDN_F32) return launch_recurrent_jit(p, s.head_dim_k, d->sms, st, ring);
    if (a->state_dtype == GDN_F32) {
        // fp32 states: the two head dims serving configurations use, on the decode and the multi-token instance
        if (s.head_dim_k == 128) return ring ? launch_recurrent_t<128, true, false, true>(p, d->sms, st) : launch_recurrent_t<128, false, false, true>(p, d->sms, st);
        if (s.head_dim_k == 64) return ring ? launch_recurrent_t<64, true, false, true>(p, d->sms, st) : launch_recurrent_t<64, false, false, true>(p, d->sms, st);
        return fail(GDN_ERR_UNSUPPORTED, "gdn_recurrent_forward: fp32 states are built for dk = 64 and 128 (got %d)", s.head_dim_k);
    }
    const bool lean = !s.cu_seqlens && s.seq_len == 1 && p.state_in != nullptr && !p.store_step && !p.state_idx;
    switch (s.head_dim_k) {
        case 64: return launch_recurrent<64>(p, d->sms, st, ring, lean);
        case 128: return launch_recurrent<128>(p, d->sms, st, ring, lean);
        case 192: return launch_recurrent<192>(p, d->sms, st, ring, lean);
        case 256: return launch_recurrent<256>(p, d->sms, st, ring, lean);
    }
    return launch_recurrent_jit(p, s.head_dim_k, d->sms, st, ring);  // 320 .. 512: compiled on first use
}

}  // extern "C"
