"""Compiles the CUDA sources of this folder for sm_100a and loads the result.

The kernels are plain ``extern "C"`` launchers that take raw device pointers and
a stream, so they compile with ``nvcc`` alone (no framework headers, a few
seconds per file) and are called through ``ctypes``.  The shared object is built
on first use, in ``csrc/_build/`` when that folder can be written and in a
per-user temporary folder otherwise, and is keyed by a hash of the sources and
flags, so an edited source rebuilds and an unchanged one does not.

There is no fallback: if ``nvcc`` is missing or a source does not compile, the
import of ``csrc.ops`` fails with the compiler's output.
"""
from __future__ import annotations

import concurrent.futures
import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time

_HERE = os.path.dirname(os.path.abspath(__file__))
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]
LIB_NAME = "libvcb_kernels.so"
_lib = None


class BuildError(RuntimeError):
    pass


def sources():
    return sorted(f for f in os.listdir(_HERE) if f.endswith(".cu"))


def _headers():
    return sorted(f for f in os.listdir(_HERE) if f.endswith((".cuh", ".h")))


def _find_nvcc() -> str:
    cand = [os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"]
    for c in cand:
        if c and os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise BuildError("nvcc not found (looked at $NVCC, PATH and /usr/local/cuda/bin/nvcc); "
                     "the engine's kernels cannot be built and there is no fallback")


def _source_hash() -> str:
    h = hashlib.sha256()
    for f in sources() + _headers():
        h.update(f.encode())
        with open(os.path.join(_HERE, f), "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _build_root() -> str:
    env = os.environ.get("VLLM_CPP_B200_BUILD_DIR")
    if env:
        os.makedirs(env, exist_ok=True)
        return env
    in_tree = os.path.join(_HERE, "_build")
    try:
        os.makedirs(in_tree, exist_ok=True)
        probe = os.path.join(in_tree, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return in_tree
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"vllm_cpp_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _say(msg: str) -> None:
    print(f"[vllm_cpp_b200 build] {msg}", file=sys.stderr, flush=True)


def _compile_one(nvcc: str, src: str, obj: str, extra) -> str:
    cmd = [nvcc] + NVCC_FLAGS + list(extra) + ["-I", _HERE, "-c", os.path.join(_HERE, src), "-o", obj]
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise BuildError(f"nvcc failed on {src}:\n{' '.join(cmd)}\n{p.stdout}")
    return p.stdout


def build(verbose: bool = False, ptxas_info: bool = False) -> str:
    """Build the shared object if it is not there yet; return its path."""
    root = _build_root()
    out_dir = os.path.join(root, _source_hash())
    lib_path = os.path.join(out_dir, LIB_NAME)
    if os.path.isfile(lib_path):
        return lib_path
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(root, ".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if os.path.isfile(lib_path):
                return lib_path
            nvcc = _find_nvcc()
            srcs = sources()
            _say(f"compiling {len(srcs)} CUDA sources for sm_100a into {out_dir}")
            t0 = time.time()
            extra = ["-Xptxas", "-v"] if ptxas_info else []
            objs = [os.path.join(out_dir, s[:-3] + ".o") for s in srcs]
            with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
                futs = {ex.submit(_compile_one, nvcc, s, o, extra): s for s, o in zip(srcs, objs)}
                for n, fut in enumerate(concurrent.futures.as_completed(futs), 1):
                    log = fut.result()
                    _say(f"  [{n}/{len(srcs)}] {futs[fut]} done ({time.time() - t0:.0f}s)")
                    if (verbose or ptxas_info) and log.strip():
                        print(log, file=sys.stderr, flush=True)
            tmp = lib_path + f".tmp{os.getpid()}"
            cmd = [nvcc, "-shared", "-o", tmp] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
            p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            if p.returncode != 0:
                raise BuildError(f"link failed:\n{' '.join(cmd)}\n{p.stdout}")
            os.replace(tmp, lib_path)
            for o in objs:
                os.remove(o)
            _say(f"built {LIB_NAME} in {time.time() - t0:.0f}s")
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return lib_path


# ------------------------------------------------------------------------------------ the C++ host
_ROOT = os.path.dirname(os.path.dirname(_HERE))
HOST_SRC, HOST_INCLUDE = os.path.join(_ROOT, "src"), os.path.join(_ROOT, "include")
HOST_FLAGS = ["-std=c++17", "-O2", "-fPIC", "-Wall", "-fvisibility=hidden"]


def _host_sources():
    return sorted(f for f in os.listdir(HOST_SRC) if f.endswith(".cpp"))


def _host_hash(kernels: str) -> str:
    h = hashlib.sha256(os.path.basename(os.path.dirname(kernels)).encode())
    for folder, _, files in sorted(os.walk(HOST_SRC)) + sorted(os.walk(HOST_INCLUDE)):
        for f in sorted(files):
            h.update(f.encode())
            with open(os.path.join(folder, f), "rb") as fh:
                h.update(fh.read())
    h.update(" ".join(HOST_FLAGS).encode())
    return h.hexdigest()[:12]


def build_engine() -> dict:
    """Build the C++ host runtime (src/, include/vllm/) against the kernel library: the shared object
    ``libvcb_engine_<hash>.so`` with vllm::Engine and its C face, and the command line ``vllm_cli``, both
    beside the kernel library.  Returns {"lib": path, "cli": path}."""
    if not os.path.isdir(HOST_SRC) or not os.path.isdir(HOST_INCLUDE):
        raise BuildError(f"the C++ host's sources are not at {HOST_SRC} and {HOST_INCLUDE}")
    kernels = build()
    out_dir = os.path.dirname(kernels)
    tag = _host_hash(kernels)
    lib, cli = os.path.join(out_dir, f"libvcb_engine_{tag}.so"), os.path.join(out_dir, f"vllm_cli_{tag}")
    if os.path.isfile(lib) and os.path.isfile(cli):
        return {"lib": lib, "cli": cli}
    cxx = shutil.which("g++") or shutil.which("c++")
    if not cxx:
        raise BuildError("g++ not found: the C++ host cannot be built")
    cuda = os.path.dirname(os.path.dirname(_find_nvcc()))
    with open(os.path.join(_build_root(), ".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if os.path.isfile(lib) and os.path.isfile(cli):
                return {"lib": lib, "cli": cli}
            _say(f"compiling the C++ host ({len(_host_sources())} sources) into {out_dir}")
            t0 = time.time()
            common = HOST_FLAGS + ["-I", HOST_INCLUDE, "-I", HOST_SRC, "-I", os.path.join(cuda, "include")]
            link = ["-L", out_dir, "-l:" + LIB_NAME, "-L", os.path.join(cuda, "lib64"), "-lcublas", "-lcudart",
                    "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + os.path.join(cuda, "lib64")]
            lib_srcs = [os.path.join(HOST_SRC, f) for f in _host_sources() if f not in ("main.cpp", "sim_api.cpp")]
            for cmd in ([cxx, "-shared"] + common + lib_srcs + ["-o", lib + ".tmp"] + link,
                        [cxx] + common + [os.path.join(HOST_SRC, "main.cpp"), "-o", cli + ".tmp", "-L", out_dir,
                                          "-l:" + os.path.basename(lib), "-Wl,-rpath,$ORIGIN"] + link):
                if cmd[-1] is None:
                    continue
                p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
                if p.returncode != 0:
                    raise BuildError(f"the C++ host did not build:\n{' '.join(cmd)}\n{p.stdout}")
                if cmd[1] == "-shared":
                    os.replace(lib + ".tmp", lib)
            os.replace(cli + ".tmp", cli)
            _say(f"built the C++ host in {time.time() - t0:.0f}s")
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return {"lib": lib, "cli": cli}


def build_scheduler_sim() -> str:
    """The C++ cache manager and scheduler alone as a small library (src/cache.cpp + src/sim_api.cpp): no device
    is needed to build or to run it.  Tests step it beside the Python scheduler."""
    h = hashlib.sha256()
    for f in ("cache.cpp", "sim_api.cpp", "host.hpp"):
        with open(os.path.join(HOST_SRC, f), "rb") as fh:
            h.update(fh.read())
    for folder, _, files in sorted(os.walk(HOST_INCLUDE)):
        for f in sorted(files):
            with open(os.path.join(folder, f), "rb") as fh:
                h.update(fh.read())
    root = _build_root()
    lib = os.path.join(root, f"libvcb_scheduler_sim_{h.hexdigest()[:12]}.so")
    if os.path.isfile(lib):
        return lib
    cxx = shutil.which("g++") or shutil.which("c++")
    if not cxx:
        raise BuildError("g++ not found")
    cuda = os.path.dirname(os.path.dirname(_find_nvcc()))
    cmd = [cxx, "-shared"] + HOST_FLAGS + ["-I", HOST_INCLUDE, "-I", HOST_SRC, "-I", os.path.join(cuda, "include"),
                                          os.path.join(HOST_SRC, "cache.cpp"), os.path.join(HOST_SRC, "sim_api.cpp"),
                                          "-o", lib + f".tmp{os.getpid()}"]
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise BuildError(f"the scheduler library did not build:\n{' '.join(cmd)}\n{p.stdout}")
    os.replace(lib + f".tmp{os.getpid()}", lib)
    return lib


def load() -> ctypes.CDLL:
    """The loaded kernel library (built first if needed)."""
    global _lib
    if _lib is None:
        path = build()
        try:
            _lib = ctypes.CDLL(path)
        except OSError as e:
            raise BuildError(f"cannot load {path}: {e}") from None
    return _lib
