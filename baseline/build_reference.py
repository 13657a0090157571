#!/usr/bin/env python3
"""Builds the unmodified reference (jiamumuzhao/vllm-cpp) and this folder's driver into baseline/_ref/.

    python baseline/build_reference.py [--source /path/to/vllm-cpp]

The reference is a CMake C++/CUDA project with no Python packaging, so ``pip install`` cannot take
it; its own CMake build can, offline: ``-DVLLM_NETWORK_DEPS=OFF`` skips the downloaded dependencies
(spdlog, nlohmann_json, httplib, googletest), ``-DCMAKE_CUDA_ARCHITECTURES=100`` targets the B200.
The build type is RelWithDebInfo, not Release: the project's Release flags add ``-march=native``, and
the binary is built on one machine and run on another.  The result is ``baseline/_ref/build/libvllm.a``
(every source file of the reference, none changed) and ``baseline/_ref/ref_driver`` (ref_driver.cpp of
this folder linked against it).  ``baseline/_ref`` is not tracked.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
DRIVER = os.path.join(OUT, "ref_driver")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def default_source() -> str:
    """Where the reference's checkout lies: $VLLM_CPP_REFERENCE, else ``reference_path`` of BASELINE.json
    at the repository's root, else ``reference/`` beside the repository."""
    env = os.environ.get("VLLM_CPP_REFERENCE")
    if env:
        return env
    root = os.path.dirname(HERE)
    try:
        import json
        with open(os.path.join(root, "BASELINE.json")) as f:
            path = json.load(f).get("reference_path")
        if path:
            return path
    except (OSError, ValueError):
        pass
    return os.path.join(os.path.dirname(root), "reference")


def run(cmd, **kw):
    print("+ " + " ".join(cmd), file=sys.stderr, flush=True)
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, **kw)
    if p.returncode != 0:
        raise RuntimeError(f"{cmd[0]} failed ({p.returncode}):\n{p.stdout[-4000:]}")
    return p.stdout


def build(source: str) -> str:
    """Configure, build and link; returns the driver's path.  Raises RuntimeError with the tool's output."""
    if not os.path.isfile(os.path.join(source, "CMakeLists.txt")):
        raise RuntimeError(f"no checkout of the reference at {source}")
    cmake, nvcc = shutil.which("cmake"), os.path.join(CUDA, "bin", "nvcc")
    if not cmake or not os.path.isfile(nvcc):
        raise RuntimeError("cmake or nvcc not found")
    build_dir = os.path.join(OUT, "build")
    os.makedirs(build_dir, exist_ok=True)
    run([cmake, "-S", source, "-B", build_dir, "-DVLLM_NETWORK_DEPS=OFF", "-DCMAKE_CUDA_ARCHITECTURES=100",
         "-DCMAKE_BUILD_TYPE=RelWithDebInfo", f"-DCMAKE_CUDA_COMPILER={nvcc}"])
    run([cmake, "--build", build_dir, "--target", "vllm", "-j", str(min(16, os.cpu_count() or 4))])
    lib = os.path.join(build_dir, "libvllm.a")
    run(["g++", "-O2", "-std=c++17", "-I", os.path.join(source, "include"), "-I", os.path.join(CUDA, "include"),
         os.path.join(HERE, "ref_driver.cpp"), lib, "-L", os.path.join(CUDA, "lib64"),
         "-lcublas", "-lcublasLt", "-lcudart", "-lpthread", "-ldl", "-o", DRIVER + ".tmp"])
    os.replace(DRIVER + ".tmp", DRIVER)
    with open(os.path.join(OUT, "BUILT_FROM"), "w") as f:
        head = subprocess.run(["git", "-C", source, "rev-parse", "HEAD"], stdout=subprocess.PIPE,
                              stderr=subprocess.DEVNULL, text=True).stdout.strip()
        f.write(f"{source} {head}\n")
    return DRIVER


def driver_path(source: str = "") -> str:
    """The built driver; builds it first if it is missing and a checkout of the reference is at hand."""
    if os.path.isfile(DRIVER) and os.access(DRIVER, os.X_OK):
        return DRIVER
    return build(source or default_source())


def driver_env() -> dict:
    env = dict(os.environ)
    env["LD_LIBRARY_PATH"] = os.path.join(CUDA, "lib64") + os.pathsep + env.get("LD_LIBRARY_PATH", "")
    return env


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--source", default=default_source())
    print(build(ap.parse_args().source))
