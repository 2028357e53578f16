// Host-side plumbing shared by the C-ABI entry points: thread-local error text, per-device
// facts (architecture check, SM count, status word address) and argument checks.
#pragma once
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include <algorithm>

#include <mutex>
#include <string>

#include "../../include/gdn_b200.h"

namespace gdn {

inline std::string& last_error_ref() {
    static thread_local std::string s;
    return s;
}

inline int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    last_error_ref() = buf;
    return code;
}

#define GDN_REQUIRE(cond, ...)                                   \
    do {                                                         \
        if (!(cond)) return ::gdn::fail(GDN_ERR_INVALID, __VA_ARGS__); \
    } while (0)

#define GDN_CUDA(call)                                                                         \
    do {                                                                                       \
        cudaError_t e__ = (call);                                                              \
        if (e__ != cudaSuccess)                                                                \
            return ::gdn::fail(GDN_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(e__)); \
    } while (0)

struct DeviceInfo {
    bool valid = false;
    int major = 0, minor = 0, sms = 0;
    int* status = nullptr;  // device address of the status word on that device
};

// Defined in gdn_b200.cu (needs the __device__ symbol).
int get_device_info(DeviceInfo** out);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int check_shape(const GdnShape& s, bool need_chunk_meta) {
    GDN_REQUIRE(s.batch > 0, "batch must be positive (got %d)", s.batch);
    GDN_REQUIRE(s.num_k_heads > 0 && s.num_v_heads > 0, "head counts must be positive");
    GDN_REQUIRE(s.num_v_heads % s.num_k_heads == 0,
                "num_v_heads (%d) must be a multiple of num_k_heads (%d)", s.num_v_heads,
                s.num_k_heads);
    GDN_REQUIRE(s.head_dim_k > 0 && s.head_dim_v > 0, "head dims must be positive");
    if (s.cu_seqlens) {
        GDN_REQUIRE(s.total_tokens >= 0, "total_tokens must be non-negative in packed mode");
        if (need_chunk_meta) {
            GDN_REQUIRE(s.total_chunks >= 0, "total_chunks must be given in packed mode");
            GDN_REQUIRE(s.total_chunks == 0 || s.chunk_indices != nullptr,
                        "chunk_indices is required in packed mode");
        }
    } else {
        GDN_REQUIRE(s.seq_len > 0, "seq_len must be positive (got %d)", s.seq_len);
    }
    return GDN_OK;
}

inline int check_token_tensor(const GdnTokenTensor& t, const char* name, int head_dim) {
    GDN_REQUIRE(t.ptr != nullptr, "%s is NULL", name);
    GDN_REQUIRE(aligned16(t.ptr), "%s must be 16-byte aligned", name);
    GDN_REQUIRE(t.stride_token % 8 == 0 && t.stride_head % 8 == 0 && t.stride_batch % 8 == 0,
                "%s strides must be multiples of 8 elements", name);
    GDN_REQUIRE(t.stride_head >= head_dim || t.stride_head == 0, "%s head stride below head dim", name);
    return GDN_OK;
}

}  // namespace gdn
