// Run-time kernel compiler (see jit/jit.hpp) and the C-ABI entry points that expose it.
#include <dirent.h>
#include <dlfcn.h>
#include <stdlib.h>
#include <string.h>
#include <sys/stat.h>
#include <sys/types.h>
#include <unistd.h>

#include <algorithm>
#include <fstream>
#include <sstream>

#include "host_common.hpp"
#include "jit/jit.hpp"

namespace gdn {
namespace jit {

namespace {
std::mutex g_mutex;
std::string g_library_root, g_cuda_home;
uint64_t g_library_version = 0;
bool g_version_valid = false;
std::map<std::string, LoadedKernel> g_loaded;  // key: "<device>:<cache key>"

bool file_exists(const std::string& p) {
    struct stat st;
    return stat(p.c_str(), &st) == 0;
}
bool mkdirs(const std::string& path) {
    std::string cur;
    for (size_t i = 0; i < path.size(); ++i) {
        cur.push_back(path[i]);
        if (path[i] == '/' || i + 1 == path.size()) {
            if (cur != "/" && !file_exists(cur) && mkdir(cur.c_str(), 0755) != 0 && !file_exists(cur)) return false;
        }
    }
    return true;
}
bool read_file(const std::string& p, std::string* out) {
    std::ifstream f(p, std::ios::binary);
    if (!f) return false;
    std::stringstream ss;
    ss << f.rdbuf();
    *out = ss.str();
    return true;
}
bool write_file(const std::string& p, const std::string& data) {
    std::ofstream f(p, std::ios::binary | std::ios::trunc);
    if (!f) return false;
    f.write(data.data(), static_cast<std::streamsize>(data.size()));
    return static_cast<bool>(f);
}
void list_files(const std::string& dir, std::vector<std::string>* out) {
    DIR* d = opendir(dir.c_str());
    if (!d) return;
    while (dirent* e = readdir(d)) {
        const std::string n = e->d_name;
        if (n == "." || n == "..") continue;
        const std::string p = dir + "/" + n;
        struct stat st;
        if (stat(p.c_str(), &st) != 0) continue;
        if (S_ISDIR(st.st_mode))
            list_files(p, out);
        else
            out->push_back(p);
    }
    closedir(d);
}
const char* kFlags = "-arch=sm_100a -O3 -std=c++17 -lineinfo --expt-relaxed-constexpr";
}  // namespace

uint64_t fnv1a64(const void* data, size_t n, uint64_t h) {
    const unsigned char* p = static_cast<const unsigned char*>(data);
    for (size_t i = 0; i < n; ++i) {
        h ^= p[i];
        h *= 1099511628211ull;
    }
    return h;
}
std::string hex64(uint64_t v) {
    char b[17];
    snprintf(b, sizeof(b), "%016llx", static_cast<unsigned long long>(v));
    return b;
}
std::string env_str(const char* name, const std::string& dflt) {
    const char* v = getenv(name);
    return (v && *v) ? std::string(v) : dflt;
}
int env_int(const char* name, int dflt) {
    const char* v = getenv(name);
    return (v && *v) ? atoi(v) : dflt;
}

void set_roots(const std::string& library_root, const std::string& cuda_home_) {
    std::lock_guard<std::mutex> lock(g_mutex);
    g_library_root = library_root;
    g_cuda_home = cuda_home_;
    g_version_valid = false;
}
std::string include_dir() {
    std::lock_guard<std::mutex> lock(g_mutex);
    return g_library_root.empty() ? std::string() : g_library_root + "/h100_gdn_cuda_b200/csrc";
}
std::string cuda_home() {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_cuda_home.empty()) return g_cuda_home;
    return env_str("CUDA_HOME", env_str("CUDA_HOME_PATH", "/usr/local/cuda"));
}
std::string cache_root() {
    std::string root = env_str("JIT_CACHE_DIR", "");
    if (root.empty()) root = env_str("HOME", "/tmp") + "/.gdn_b200/cache";
    mkdirs(root);
    return root;
}
uint64_t library_version() {
    const std::string inc = include_dir();
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_version_valid) return g_library_version;
    uint64_t h = fnv1a64("gdn_b200", 8);
    if (!inc.empty()) {
        std::vector<std::string> files;
        list_files(inc + "/kernels", &files);
        std::sort(files.begin(), files.end());
        for (const std::string& f : files) {
            std::string data;
            if (read_file(f, &data)) {
                h = fnv1a64(f.data() + inc.size(), f.size() - inc.size(), h);
                h = fnv1a64(data.data(), data.size(), h);
            }
        }
    }
    g_library_version = h;
    g_version_valid = true;
    return h;
}

// ---------------------------------------------------------------- NVRTC through dlopen
namespace {
struct Nvrtc {
    void* handle = nullptr;
    int (*createProgram)(void**, const char*, const char*, int, const char* const*, const char* const*) = nullptr;
    int (*destroyProgram)(void**) = nullptr;
    int (*compileProgram)(void*, int, const char* const*) = nullptr;
    int (*getCUBINSize)(void*, size_t*) = nullptr;
    int (*getCUBIN)(void*, char*) = nullptr;
    int (*getProgramLogSize)(void*, size_t*) = nullptr;
    int (*getProgramLog)(void*, char*) = nullptr;
    int (*version)(int*, int*) = nullptr;
    bool ok = false;
};
Nvrtc* load_nvrtc(const std::string& home) {
    static Nvrtc n;
    static std::once_flag once;
    std::call_once(once, [&] {
        const char* names[] = {"libnvrtc.so.12", "libnvrtc.so"};
        for (const char* nm : names) {
            n.handle = dlopen((home + "/lib64/" + nm).c_str(), RTLD_NOW | RTLD_LOCAL);
            if (!n.handle) n.handle = dlopen(nm, RTLD_NOW | RTLD_LOCAL);
            if (n.handle) break;
        }
        if (!n.handle) return;
#define GDN_SYM(field, sym) *reinterpret_cast<void**>(&n.field) = dlsym(n.handle, sym)
        GDN_SYM(createProgram, "nvrtcCreateProgram");
        GDN_SYM(destroyProgram, "nvrtcDestroyProgram");
        GDN_SYM(compileProgram, "nvrtcCompileProgram");
        GDN_SYM(getCUBINSize, "nvrtcGetCUBINSize");
        GDN_SYM(getCUBIN, "nvrtcGetCUBIN");
        GDN_SYM(getProgramLogSize, "nvrtcGetProgramLogSize");
        GDN_SYM(getProgramLog, "nvrtcGetProgramLog");
        GDN_SYM(version, "nvrtcVersion");
#undef GDN_SYM
        n.ok = n.createProgram && n.destroyProgram && n.compileProgram && n.getCUBINSize && n.getCUBIN &&
               n.getProgramLogSize && n.getProgramLog;
    });
    return n.ok ? &n : nullptr;
}

std::string compiler_signature(bool use_nvrtc, const std::string& home) {
    if (use_nvrtc) {
        Nvrtc* n = load_nvrtc(home);
        int ma = 0, mi = 0;
        if (n && n->version) n->version(&ma, &mi);
        return "nvrtc-" + std::to_string(ma) + "." + std::to_string(mi);
    }
    return "nvcc@" + home;
}

int compile_nvrtc(const std::string& source, const std::string& inc, const std::string& home, std::string* cubin,
                  std::string* log) {
    Nvrtc* n = load_nvrtc(home);
    if (!n) {
        *log = "libnvrtc could not be loaded";
        return GDN_ERR_UNSUPPORTED;
    }
    void* prog = nullptr;
    if (n->createProgram(&prog, source.c_str(), "kernel.cu", 0, nullptr, nullptr) != 0) {
        *log = "nvrtcCreateProgram failed";
        return GDN_ERR_CUDA;
    }
    const std::string i1 = "-I" + inc, i2 = "-I" + home + "/include";
    const char* opts[] = {"-arch=sm_100a", "-std=c++17", "-lineinfo", "-default-device", i1.c_str(), i2.c_str()};
    const int rc = n->compileProgram(prog, 6, opts);
    size_t ls = 0;
    n->getProgramLogSize(prog, &ls);
    if (ls > 1) {
        log->resize(ls);
        n->getProgramLog(prog, &(*log)[0]);
    }
    int status = GDN_OK;
    if (rc != 0) {
        status = GDN_ERR_CUDA;
    } else {
        size_t cs = 0;
        n->getCUBINSize(prog, &cs);
        cubin->resize(cs);
        n->getCUBIN(prog, &(*cubin)[0]);
    }
    n->destroyProgram(&prog);
    return status;
}

int compile_nvcc(const std::string& src_path, const std::string& out_path, const std::string& inc,
                 const std::string& home, std::string* log) {
    const std::string nvcc = home + "/bin/nvcc";
    if (!file_exists(nvcc)) {
        *log = "nvcc not found at " + nvcc;
        return GDN_ERR_UNSUPPORTED;
    }
    const std::string cmd = nvcc + " -cubin " + kFlags + " -I" + inc + " -o " + out_path + " " + src_path + " 2>&1";
    if (env_int("JIT_DEBUG", 0)) fprintf(stderr, "[gdn jit] %s\n", cmd.c_str());
    FILE* pipe = popen(cmd.c_str(), "r");
    if (!pipe) {
        *log = "could not start nvcc";
        return GDN_ERR_CUDA;
    }
    char buf[512];
    while (fgets(buf, sizeof(buf), pipe)) *log += buf;
    const int rc = pclose(pipe);
    return rc == 0 ? GDN_OK : GDN_ERR_CUDA;
}
}  // namespace

CompileResult compile(const std::string& name, const std::string& source) {
    CompileResult r;
    const std::string inc = include_dir();
    const std::string home = cuda_home();
    if (inc.empty() || !file_exists(inc + "/kernels")) {
        r.status = GDN_ERR_INVALID;
        r.message = "run-time compilation needs gdn_init(library_root, cuda_home) with the repository root "
                    "(kernel headers expected under <library_root>/h100_gdn_cuda_b200/csrc/kernels)";
        return r;
    }
    const bool use_nvrtc = env_int("JIT_USE_NVRTC", 1) != 0 && load_nvrtc(home) != nullptr;
    const std::string sig = compiler_signature(use_nvrtc, home);
    uint64_t h = fnv1a64(name.data(), name.size());
    const uint64_t ver = library_version();
    h = fnv1a64(&ver, sizeof(ver), h);
    h = fnv1a64(sig.data(), sig.size(), h);
    h = fnv1a64(kFlags, strlen(kFlags), h);
    h = fnv1a64(source.data(), source.size(), h);
    const std::string dir = cache_root() + "/kernel." + name + "." + hex64(h);
    const std::string cubin_path = dir + "/kernel.cubin";
    r.cubin_path = cubin_path;
    if (file_exists(cubin_path)) {
        r.cache_hit = true;
        return r;
    }
    if (!mkdirs(dir)) {
        r.status = GDN_ERR_CUDA;
        r.message = "cannot create cache directory " + dir;
        return r;
    }
    const std::string tag = std::to_string(getpid()) + "." + hex64(fnv1a64(&r, sizeof(void*), h));
    const std::string src_path = dir + "/kernel.cu";
    const std::string tmp_path = dir + "/kernel.cubin.tmp." + tag;
    if (!write_file(src_path + ".tmp." + tag, source) || rename((src_path + ".tmp." + tag).c_str(), src_path.c_str()) != 0) {
        r.status = GDN_ERR_CUDA;
        r.message = "cannot write " + src_path;
        return r;
    }
    std::string log;
    if (use_nvrtc) {
        std::string cubin;
        r.status = compile_nvrtc(source, inc, home, &cubin, &log);
        if (r.status == GDN_OK && !write_file(tmp_path, cubin)) {
            r.status = GDN_ERR_CUDA;
            log = "cannot write " + tmp_path;
        }
    } else {
        r.status = compile_nvcc(src_path, tmp_path, inc, home, &log);
    }
    if (env_int("JIT_DEBUG", 0) && !log.empty()) fprintf(stderr, "[gdn jit] %s (%s): %s\n", name.c_str(), sig.c_str(), log.c_str());
    if (r.status != GDN_OK) {
        r.message = "compiling " + name + " with " + sig + " failed: " + log;
        unlink(tmp_path.c_str());
        return r;
    }
    if (rename(tmp_path.c_str(), cubin_path.c_str()) != 0) {
        r.status = GDN_ERR_CUDA;
        r.message = "cannot move the cubin into " + cubin_path;
        unlink(tmp_path.c_str());
    }
    return r;
}

int get_kernel(const std::string& name, const std::string& source, const std::string& entry, LoadedKernel* out,
               std::string* error) {
    CompileResult c = compile(name, source);
    if (c.status != GDN_OK) {
        *error = c.message;
        return c.status;
    }
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        *error = "cudaGetDevice failed";
        return GDN_ERR_CUDA;
    }
    const std::string key = std::to_string(dev) + ":" + c.cubin_path;
    std::lock_guard<std::mutex> lock(g_mutex);
    auto it = g_loaded.find(key);
    if (it != g_loaded.end()) {
        *out = it->second;
        return GDN_OK;
    }
    std::string cubin;
    if (!read_file(c.cubin_path, &cubin) || cubin.size() < 64) {
        // a truncated file in the cache: drop it so that the next call compiles again
        unlink(c.cubin_path.c_str());
        *error = "cached cubin " + c.cubin_path + " is unreadable or truncated (removed; call again)";
        return GDN_ERR_CUDA;
    }
    LoadedKernel k;
    cudaError_t e = cudaLibraryLoadData(&k.library, cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0);
    if (e == cudaSuccess) e = cudaLibraryGetKernel(&k.kernel, k.library, entry.c_str());
    if (e != cudaSuccess) {
        *error = std::string("loading ") + c.cubin_path + ": " + cudaGetErrorString(e);
        cudaGetLastError();
        return GDN_ERR_CUDA;
    }
    g_loaded[key] = k;
    *out = k;
    return GDN_OK;
}

}  // namespace jit
}  // namespace gdn

using namespace gdn;

extern "C" {

int gdn_jit_compile(const char* name, const char* source, char* cubin_path_out, size_t cubin_path_cap,
                    int* cache_hit_out) {
    GDN_REQUIRE(name && source, "gdn_jit_compile: NULL argument");
    jit::CompileResult r = jit::compile(name, source);
    if (r.status != GDN_OK) return fail(r.status, "%s", r.message.c_str());
    if (cubin_path_out && cubin_path_cap > 0) {
        strncpy(cubin_path_out, r.cubin_path.c_str(), cubin_path_cap - 1);
        cubin_path_out[cubin_path_cap - 1] = 0;
    }
    if (cache_hit_out) *cache_hit_out = r.cache_hit ? 1 : 0;
    return GDN_OK;
}

}  // extern "C"
