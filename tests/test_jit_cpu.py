"""Run-time kernel compiler, CPU side: compiling needs no GPU, so hashing, caching, both
compilers, failure reporting and concurrent use of one cache directory are tested here."""
import ctypes as C
import multiprocessing as mp
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")

TRIVIAL = 'extern "C" __global__ void k(float* x) { x[threadIdx.x] += %d.f; }\n'
RECURRENT = ('#include "kernels/recurrent.cuh"\n'
             'extern "C" __global__ void __launch_bounds__(128, 2) gdn_recurrent_jit(const gdn::RecurrentParams p) {\n'
             '    gdn::gdn_recurrent_body<320>(p);\n}\n')


def _lib():
    from h100_gdn_cuda_b200 import build, _cabi
    build.build()
    lib = _cabi.load()
    assert lib.gdn_init(ROOT.encode(), CUDA_HOME.encode()) == 0
    return lib


def _compile(lib, name, src):
    path = C.create_string_buffer(1024)
    hit = C.c_int(-1)
    rc = lib.gdn_jit_compile(name.encode(), src.encode(), path, 1024, C.byref(hit))
    return rc, path.value.decode(), hit.value


@pytest.fixture()
def cache(tmp_path, monkeypatch):
    monkeypatch.setenv("JIT_CACHE_DIR", str(tmp_path))
    return tmp_path


@pytest.mark.parametrize("use_nvrtc", ["1", "0"])
def test_compile_then_cache_hit(cache, monkeypatch, use_nvrtc):
    monkeypatch.setenv("JIT_USE_NVRTC", use_nvrtc)
    lib = _lib()
    rc, path, hit = _compile(lib, "trivial", TRIVIAL % 1)
    assert rc == 0, lib.gdn_last_error()
    assert hit == 0 and os.path.getsize(path) > 500 and path.startswith(str(cache))
    assert os.path.exists(os.path.join(os.path.dirname(path), "kernel.cu"))
    rc, path2, hit = _compile(lib, "trivial", TRIVIAL % 1)
    assert rc == 0 and hit == 1 and path2 == path
    # another source -> another cache entry
    rc, path3, hit = _compile(lib, "trivial", TRIVIAL % 2)
    assert rc == 0 and hit == 0 and path3 != path


def test_compilers_have_separate_entries(cache, monkeypatch):
    lib = _lib()
    monkeypatch.setenv("JIT_USE_NVRTC", "1")
    _, p1, _ = _compile(lib, "trivial", TRIVIAL % 3)
    monkeypatch.setenv("JIT_USE_NVRTC", "0")
    _, p2, _ = _compile(lib, "trivial", TRIVIAL % 3)
    assert p1 != p2


@pytest.mark.parametrize("use_nvrtc", ["1", "0"])
def test_library_kernel_compiles(cache, monkeypatch, use_nvrtc):
    """The translation unit the library generates for a head dimension without a prebuilt kernel."""
    monkeypatch.setenv("JIT_USE_NVRTC", use_nvrtc)
    lib = _lib()
    rc, path, hit = _compile(lib, "recurrent_dk320", RECURRENT)
    assert rc == 0, lib.gdn_last_error().decode()
    assert os.path.getsize(path) > 5000


def test_compile_error_is_reported(cache):
    lib = _lib()
    rc, _, _ = _compile(lib, "broken", "this is not CUDA\n")
    assert rc != 0
    msg = lib.gdn_last_error().decode()
    assert "broken" in msg and "error" in msg.lower()
    # nothing half-written is left where a cubin would be found
    for root, _, files in os.walk(str(cache)):
        assert "kernel.cubin" not in files


def test_unwritable_cache_dir(monkeypatch, tmp_path):
    ro = tmp_path / "ro"
    ro.mkdir()
    os.chmod(ro, 0o500)
    if os.access(str(ro), os.W_OK):  # running as root: permissions do not bind
        blocker = tmp_path / "file"
        blocker.write_text("x")
        monkeypatch.setenv("JIT_CACHE_DIR", str(blocker / "sub"))
    else:
        monkeypatch.setenv("JIT_CACHE_DIR", str(ro / "sub"))
    lib = _lib()
    rc, _, _ = _compile(lib, "trivial", TRIVIAL % 4)
    assert rc != 0 and b"cache" in lib.gdn_last_error()


def test_needs_init(cache):
    from h100_gdn_cuda_b200 import build, _cabi
    build.build()
    lib = _cabi.load()
    assert lib.gdn_init(b"/nonexistent", CUDA_HOME.encode()) == 0
    rc, _, _ = _compile(lib, "trivial", TRIVIAL % 5)
    assert rc == -1 and b"gdn_init" in lib.gdn_last_error()
    assert lib.gdn_init(ROOT.encode(), CUDA_HOME.encode()) == 0


def _race(args):
    cache_dir, n = args
    os.environ["JIT_CACHE_DIR"] = cache_dir
    lib = _lib()
    rc, path, hit = _compile(lib, "race", TRIVIAL % 7)
    return rc, path, os.path.getsize(path) if rc == 0 else 0


def test_two_processes_share_a_cache(tmp_path):
    ctx = mp.get_context("spawn")
    with ctx.Pool(2) as pool:
        res = pool.map(_race, [(str(tmp_path), i) for i in range(2)])
    assert all(r[0] == 0 for r in res)
    assert res[0][1] == res[1][1] and res[0][2] == res[1][2] > 500
    leftovers = [f for f in os.listdir(os.path.dirname(res[0][1])) if ".tmp." in f]
    assert leftovers == []
