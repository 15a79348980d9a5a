"""Builds the CUDA sources under ``csrc/`` into one shared library for sm_100a.

The library is built in-tree (``mimirmind_b200/_build/``) with plain ``nvcc`` the first
time it is needed and whenever a source or flag changed, so a fresh checkout works
without any install step.  If the package folder is not writable the build goes to a
per-user folder under the system temporary directory instead.  The reference compiles
each of its kernels at build time as well and loads them at start-up
(CMakeLists.txt:1013-1024; src/compute/cuda/GpuOps.cpp:60-113); it targets compute_80
PTX, this library targets sm_100a machine code only.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
import time
from typing import List

_PKG_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC_DIR = os.path.join(_PKG_DIR, "csrc")
LIB_NAME = "libmimirmind_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]
LINK_FLAGS = ["-shared"]


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for cand in (
        os.environ.get("MIMIRMIND_NVCC"),
        os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
        shutil.which("nvcc"),
        "/usr/local/cuda/bin/nvcc",
    ):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (set CUDA_HOME or MIMIRMIND_NVCC); the CUDA kernels cannot be built")


EXEC_DIR = os.path.join(CSRC_DIR, "exec")     # the native step executor: host code over the kernels' entry points


def _sources() -> List[str]:
    return sorted(f for f in os.listdir(CSRC_DIR) if f.endswith(".cu")) + \
        sorted("exec/" + f for f in os.listdir(EXEC_DIR) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(CSRC_DIR) if f.endswith((".cuh", ".h"))) + \
        sorted("exec/" + f for f in os.listdir(EXEC_DIR) if f.endswith(".h")) + ["host/runtime_api.h"]


def _obj(build_dir: str, src: str) -> str:
    return os.path.join(build_dir, src[:-3].replace("/", "_") + ".o")


def _digest(paths: List[str], extra: str) -> str:
    h = hashlib.sha256()
    h.update(extra.encode())
    for p in paths:
        h.update(p.encode())
        with open(os.path.join(CSRC_DIR, p), "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _writable_build_dir() -> str:
    in_tree = os.path.join(_PKG_DIR, "_build")
    try:
        os.makedirs(in_tree, exist_ok=True)
        probe = os.path.join(in_tree, f".probe_{os.getpid()}")
        with open(probe, "w") as f:
            f.write("x")
        os.remove(probe)
        return in_tree
    except OSError:
        pass
    alt = os.path.join(tempfile.gettempdir(), f"mimirmind_b200_build_{os.getuid()}")
    os.makedirs(alt, exist_ok=True)
    return alt


def _log(msg: str) -> None:
    print(f"[mimirmind_b200 build] {msg}", file=sys.stderr, flush=True)


def _compile_one(nvcc: str, src: str, obj: str) -> float:
    t0 = time.time()
    cmd = [nvcc] + NVCC_FLAGS + ["-I", CSRC_DIR, "-c", os.path.join(CSRC_DIR, src), "-o", obj]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"nvcc failed on {src}:\n{proc.stdout}\n{proc.stderr}")
    return time.time() - t0


def library_path(build_if_needed: bool = True, verbose: bool = True) -> str:
    """Path of the built library; compiles what is missing or stale first."""
    srcs = _sources()
    hdrs = _headers()
    flags = " ".join(NVCC_FLAGS + LINK_FLAGS + ["host-linked"])
    header_digest = _digest(hdrs, flags)
    build_dir = _writable_build_dir()
    manifest_path = os.path.join(build_dir, "manifest.json")
    lib_path = os.path.join(build_dir, LIB_NAME)
    try:
        with open(manifest_path) as f:
            manifest = json.load(f)
    except (OSError, ValueError):
        manifest = {}
    want = {s: _digest([s], header_digest) for s in srcs}
    stale = [s for s in srcs if manifest.get(s) != want[s] or not os.path.isfile(_obj(build_dir, s))]
    removed = [s for s in manifest if s not in want]
    if not stale and not removed and os.path.isfile(lib_path):
        return lib_path
    if not build_if_needed:
        raise BuildError(f"{lib_path} is missing or stale")
    nvcc = find_nvcc()
    if verbose:
        _log(f"compiling {len(stale)} of {len(srcs)} CUDA sources for sm_100a into {build_dir}")
    t0 = time.time()
    done = 0
    workers = min(len(stale), max(1, min(8, (os.cpu_count() or 2)))) or 1
    with concurrent.futures.ThreadPoolExecutor(max_workers=workers) as pool:
        futs = {pool.submit(_compile_one, nvcc, s, _obj(build_dir, s)): s for s in stale}
        for fut in concurrent.futures.as_completed(futs):
            secs = fut.result()
            done += 1
            if verbose:
                _log(f"  [{done}/{len(stale)}] {futs[fut]} ({secs:.1f} s, {time.time() - t0:.0f} s elapsed)")
    objs = [_obj(build_dir, s) for s in srcs]
    tmp_lib = lib_path + f".tmp{os.getpid()}"
    # the executor calls the host runtime (cache manager, scheduler), which lives in a library of its own beside this one
    host_dir = os.path.dirname(host_library_path(verbose=verbose))
    link = LINK_FLAGS + ["-L", host_dir, "-lmimirmind_host", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN", "-ldl"]
    proc = subprocess.run([nvcc] + link + ["-o", tmp_lib] + objs, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp_lib, lib_path)
    with open(manifest_path, "w") as f:
        json.dump(want, f, indent=1)
    if verbose:
        _log(f"built {LIB_NAME} in {time.time() - t0:.0f} s")
    return lib_path


HOST_DIR = os.path.join(CSRC_DIR, "host")
HOST_LIB_NAME = "libmimirmind_host.so"
HOST_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-Wl,-soname," + HOST_LIB_NAME]


def host_library_path(verbose: bool = True) -> str:
    """Path of the host runtime library (page allocator, cache manager, scheduler: ``csrc/host/*.cpp``, no CUDA),
    built with the host C++ compiler when missing or stale."""
    srcs = sorted(f for f in os.listdir(HOST_DIR) if f.endswith((".cpp", ".h")))
    h = hashlib.sha256(" ".join(HOST_FLAGS).encode())
    for name in srcs:
        with open(os.path.join(HOST_DIR, name), "rb") as f:
            h.update(name.encode())
            h.update(f.read())
    digest = h.hexdigest()
    build_dir = _writable_build_dir()
    lib_path = os.path.join(build_dir, HOST_LIB_NAME)
    stamp = lib_path + ".sha256"
    try:
        with open(stamp) as f:
            if f.read().strip() == digest and os.path.isfile(lib_path):
                return lib_path
    except OSError:
        pass
    cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++") or shutil.which("clang++")
    if not cxx:
        raise BuildError("no C++ compiler found (g++, c++ or clang++; or set CXX): the host runtime cannot be built")
    if verbose:
        _log(f"compiling the host runtime into {build_dir}")
    tmp_lib = lib_path + f".tmp{os.getpid()}"
    cpps = [os.path.join(HOST_DIR, n) for n in srcs if n.endswith(".cpp")]
    proc = subprocess.run([cxx] + HOST_FLAGS + ["-o", tmp_lib] + cpps, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"host runtime build failed:\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp_lib, lib_path)
    with open(stamp, "w") as f:
        f.write(digest)
    return lib_path


def build_all(verbose: bool = True) -> str:
    host_library_path(verbose=verbose)
    return library_path(build_if_needed=True, verbose=verbose)


if __name__ == "__main__":
    print(build_all())
