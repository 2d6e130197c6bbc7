"""Builds the package's native code in-tree, at first use, and finds it again afterwards.

Three kinds of library:
  * kernel libraries: CUDA sources under csrc/kernels compiled by nvcc for sm_100a only into a
    shared object of `extern "C"` launchers (loaded with ctypes);
  * the host library: C++17 sources under csrc/host (cache manager, batch builder, scheduler)
    compiled by g++ into a pybind11 module;
  * the reference library: plain C++ twins of the kernels under csrc/ref (scalar loops on host
    memory), which only the tests load.

A library's file name carries a hash of its sources and flags, so an up-to-date build is found
without compiling and a stale one is never loaded. Objects are built in parallel; while a build
runs, a line is printed every few seconds. The build folder is csrc/_build next to this file; if
that is not writable a per-user folder under the system temp dir is used.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, List

HERE = os.path.dirname(os.path.abspath(__file__))
KERNEL_DIR = os.path.join(HERE, "kernels")
HOST_DIR = os.path.join(HERE, "host")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wextra", "-Wno-unused-parameter"]

# name -> CUDA sources. "core" is what every model and precision needs; "tensorcore" holds the
# tcgen05/TMA kernels that only the bfloat16 path uses.
KERNEL_LIBRARIES: Dict[str, List[str]] = {
    "core": ["status.cu", "elementwise.cu", "gemm_simt.cu", "rope_kv.cu", "attention_simt.cu", "sampling.cu"],
    "tensorcore": ["status.cu", "gemm_tc.cu", "gemm_decode.cu", "attention_mma.cu", "attention_tc.cu", "attention_decode.cu"],
}
HOST_SOURCES = ["cache_manager.cpp", "scheduler.cpp", "bindings.cpp"]
REF_DIR = os.path.join(HERE, "ref")
REF_SOURCES = ["kernels_ref.cpp"]  # plain C++ twins of the kernels: what the kernel tests compare with


class BuildError(RuntimeError):
    pass


def _log(msg: str) -> None:
    print(f"[llmengine build] {msg}", file=sys.stderr, flush=True)


def _find_nvcc() -> str:
    for cand in (os.environ.get("LLMENGINE_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise BuildError("nvcc not found (looked at $LLMENGINE_NVCC, PATH and /usr/local/cuda/bin/nvcc); "
                     "the CUDA kernels cannot be built")


def _build_dir() -> str:
    d = os.path.join(HERE, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"llmengine_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _hash(paths: List[str], flags: List[str], extra: List[str]) -> str:
    h = hashlib.sha256()
    for p in sorted(paths + extra):
        h.update(os.path.basename(p).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:16]


def _run(cmd: List[str], what: str) -> None:
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise BuildError(f"building {what} failed:\n{' '.join(cmd)}\n{r.stdout}")


class _Ticker:
    """Prints a line every few seconds while a build runs."""

    def __init__(self, what: str):
        self.what, self.t0, self.stop = what, time.time(), threading.Event()
        self.thread = threading.Thread(target=self._loop, daemon=True)

    def _loop(self):
        while not self.stop.wait(5.0):
            _log(f"still compiling {self.what} ... {time.time() - self.t0:.0f}s")

    def __enter__(self):
        _log(f"compiling {self.what} (first use; the result is kept)")
        self.thread.start()
        return self

    def __exit__(self, *a):
        self.stop.set()
        _log(f"{self.what}: done in {time.time() - self.t0:.1f}s")


def _compile_and_link(compiler: List[str], srcs: List[str], obj_flags: List[str], link_flags: List[str],
                      out_path: str, what: str) -> None:
    bdir = os.path.dirname(out_path)
    tag = os.path.basename(out_path)
    objs = [os.path.join(bdir, f"{tag}.{os.path.basename(s)}.{os.getpid()}.o") for s in srcs]
    try:
        with _Ticker(what):
            with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 1)) as ex:
                jobs = [ex.submit(_run, compiler + obj_flags + ["-c", s, "-o", o], os.path.basename(s))
                        for s, o in zip(srcs, objs)]
                for j in jobs:
                    j.result()
            tmp = out_path + f".tmp{os.getpid()}"
            _run(compiler + link_flags + objs + ["-o", tmp], what)
            os.replace(tmp, out_path)  # atomic: a concurrent builder sees a whole file or none
    finally:
        for o in objs:
            if os.path.exists(o):
                os.remove(o)


def _drop_stale(build_dir: str, prefix: str, keep: str) -> None:
    """Removes earlier builds of the same library (other hashes)."""
    for f in os.listdir(build_dir):
        full = os.path.join(build_dir, f)
        if f.startswith(prefix) and full != keep and ".tmp" not in f:
            try:
                shutil.rmtree(full) if os.path.isdir(full) else os.remove(full)
            except OSError:
                pass


def kernel_library_path(name: str, build: bool = True) -> str:
    """Path of the built kernel library `name`; compiles it first if needed and allowed."""
    if name not in KERNEL_LIBRARIES:
        raise BuildError(f"unknown kernel library '{name}'")
    srcs = [os.path.join(KERNEL_DIR, s) for s in KERNEL_LIBRARIES[name]]
    headers = [os.path.join(KERNEL_DIR, f) for f in os.listdir(KERNEL_DIR) if f.endswith((".cuh", ".h"))]
    digest = _hash(srcs, NVCC_FLAGS, headers)
    out = os.path.join(_build_dir(), f"libllmengine_{name}_{digest}.so")
    if os.path.isfile(out):
        return out
    if not build:
        raise BuildError(f"kernel library '{name}' is not built")
    nvcc = _find_nvcc()
    _compile_and_link([nvcc], srcs, NVCC_FLAGS + ["-I", KERNEL_DIR], ["-shared"] + NVCC_FLAGS,
                      out, f"CUDA kernels '{name}' for sm_100a")
    _drop_stale(os.path.dirname(out), f"libllmengine_{name}_", out)
    return out


def host_module_path(build: bool = True) -> str:
    import pybind11
    srcs = [os.path.join(HOST_DIR, s) for s in HOST_SOURCES]
    headers = [os.path.join(HOST_DIR, f) for f in os.listdir(HOST_DIR) if f.endswith((".hpp", ".h"))]
    ext = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    flags = CXX_FLAGS + ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"], "-I", HOST_DIR]
    digest = _hash(srcs, CXX_FLAGS + [ext, pybind11.__version__], headers)  # no absolute paths in the hash
    d = os.path.join(_build_dir(), f"host_{digest}")
    out = os.path.join(d, "_llmengine_host" + ext)
    if os.path.isfile(out):
        return out
    if not build:
        raise BuildError("host library is not built")
    os.makedirs(d, exist_ok=True)
    cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
    if not cxx:
        raise BuildError("no C++ compiler found (g++)")
    _compile_and_link([cxx], srcs, flags, ["-shared"], out, "host runtime (C++)")
    _drop_stale(os.path.dirname(d), "host_", d)
    return out


def reference_library_path(build: bool = True) -> str:
    """Path of the plain C++ twins of the kernels (a shared library of `extern "C"` functions on host
    memory, loaded with ctypes by the tests); compiled first if needed and allowed."""
    srcs = [os.path.join(REF_DIR, s) for s in REF_SOURCES]
    flags = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-fno-fast-math", "-Wall", "-Wextra"]
    out = os.path.join(_build_dir(), f"libllmengine_ref_{_hash(srcs, flags, [])}.so")
    if os.path.isfile(out):
        return out
    if not build:
        raise BuildError("the reference library is not built")
    cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
    if not cxx:
        raise BuildError("no C++ compiler found (g++)")
    _compile_and_link([cxx], srcs, flags, ["-shared"], out, "plain C++ twins of the kernels")
    _drop_stale(os.path.dirname(out), "libllmengine_ref_", out)
    return out


def build_all() -> Dict[str, str]:
    """Builds every library; returns name -> path."""
    out = {"host": host_module_path(), "ref": reference_library_path()}
    for name in KERNEL_LIBRARIES:
        out[name] = kernel_library_path(name)
    return out


if __name__ == "__main__":
    for k, v in build_all().items():
        print(k, v)
