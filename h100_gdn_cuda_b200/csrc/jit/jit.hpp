// Run-time kernel compiler for sm_100a: source string -> cubin on disk -> loaded kernel.
// Stands in for the reference's JIT layer (csrc/jit/compiler.hpp:16-254, runtime.hpp:11-83,
// cache.hpp:5-37) with these differences: one target (sm_100a), kernels are found by a fixed
// extern "C" name (no binary inspection tools are run), NVRTC is loaded with dlopen so the
// library has no link-time dependency on it, modules are loaded through the CUDA runtime's
// library API, and every failure is a status code with a message.
//
// Cache layout (same scheme as the reference): $JIT_CACHE_DIR or ~/.gdn_b200/cache,
//   kernel.<name>.<hash>/kernel.cu, kernel.cubin
// where hash covers the name, the library version (a hash of every kernel header), the
// compiler signature, the flags and the source.  A cubin is written to a temporary file and
// renamed into place, so concurrent processes can share one cache directory.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

namespace gdn {
namespace jit {

uint64_t fnv1a64(const void* data, size_t n, uint64_t seed = 1469598103934665603ull);
std::string hex64(uint64_t v);

// Environment switches (names kept from the reference): JIT_CACHE_DIR, JIT_DEBUG, JIT_USE_NVRTC.
std::string env_str(const char* name, const std::string& dflt);
int env_int(const char* name, int dflt);

struct CompileResult {
    int status = 0;         // 0 or a GDN_ERR_* code
    std::string message;    // compiler log / reason on failure
    std::string cubin_path; // on success
    bool cache_hit = false;
};

// Paths given to gdn_init.
void set_roots(const std::string& library_root, const std::string& cuda_home);
std::string include_dir();    // <library_root>/h100_gdn_cuda_b200/csrc
std::string cuda_home();
std::string cache_root();     // creates the directory
uint64_t library_version();   // hash of the kernel headers under include_dir()/kernels

// Compile `source` (a complete translation unit that defines an extern "C" kernel) to a cubin
// for sm_100a, or find it in the cache.  Needs no GPU.
CompileResult compile(const std::string& name, const std::string& source);

// A loaded kernel (per device).
struct LoadedKernel {
    cudaLibrary_t library = nullptr;
    cudaKernel_t kernel = nullptr;
};

// Compile if needed, load on the current device if needed, return the kernel handle.
int get_kernel(const std::string& name, const std::string& source, const std::string& entry,
               LoadedKernel* out, std::string* error);

}  // namespace jit
}  // namespace gdn
