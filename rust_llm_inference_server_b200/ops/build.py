"""Builds the native libraries in-tree, at first use, and only when their sources changed.

Two libraries:
  * `librlis_kernels.so`: every CUDA kernel, compiled by nvcc for sm_100a only, exported as plain
    C symbols and called through ctypes (no dependency on a tensor library's headers, so a build
    takes seconds);
  * `_rlis_host`: the C++ cache manager and scheduler, bound with pybind11, compiled by g++.

The build folder is `csrc/_build/` inside the package; when that is not writable, a folder per
user under the system's temporary directory is used instead.  A progress line goes to stderr
every few seconds while a compiler runs.
"""

from __future__ import annotations

import fcntl
import glob
import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
import tempfile
import threading
import time

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(_PKG, "csrc")

NVCC_FLAGS = [
    "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "-shared", "--threads", "0",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall"]


class BuildError(RuntimeError):
    pass


def _build_dir() -> str:
    d = os.path.join(CSRC, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"rlis_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _digest(paths: list[str], flags: list[str]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(flags).encode())
    for p in sorted(paths):
        h.update(os.path.basename(p).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _find_nvcc() -> str:
    for cand in (os.environ.get("RLIS_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise BuildError("nvcc not found (set CUDA_HOME or RLIS_NVCC); the CUDA kernels cannot be built")


def _run(cmd: list[str], what: str) -> None:
    t0 = time.time()
    done = threading.Event()

    def tick():
        while not done.wait(5.0):
            print(f"[rlis build] compiling {what} ... {time.time() - t0:.0f}s", file=sys.stderr, flush=True)

    print(f"[rlis build] compiling {what}", file=sys.stderr, flush=True)
    th = threading.Thread(target=tick, daemon=True)
    th.start()
    try:
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    finally:
        done.set()
    if r.returncode != 0:
        raise BuildError(f"building {what} failed:\n$ {' '.join(cmd)}\n{r.stdout}")
    print(f"[rlis build] {what} built in {time.time() - t0:.1f}s", file=sys.stderr, flush=True)


def _ensure(out_name: str, sources: list[str], deps: list[str], make_cmd, what: str) -> str:
    bdir = _build_dir()
    out = os.path.join(bdir, out_name)
    stamp = out + ".sha256"
    want = _digest(sources + deps, make_cmd("OUT"))
    def fresh() -> bool:
        try:
            with open(stamp) as f:
                return os.path.isfile(out) and f.read().strip() == want
        except OSError:
            return False
    if fresh():
        return out
    with open(os.path.join(bdir, out_name + ".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if fresh():
                return out
            tmp = os.path.join(bdir, f".{os.getpid()}.{out_name}")
            _run(make_cmd(tmp), what)
            os.replace(tmp, out)
            with open(stamp, "w") as f:
                f.write(want)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return out


def kernel_sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "kernels", "*.cu")))


def build_kernels() -> str:
    """Compiles every `.cu` under csrc/kernels for sm_100a; returns the library's path."""
    srcs = kernel_sources()
    hdrs = sorted(glob.glob(os.path.join(CSRC, "kernels", "*.cuh")) +
                  glob.glob(os.path.join(CSRC, "kernels", "*.h")))
    if not srcs:
        raise BuildError(f"no kernel sources under {CSRC}/kernels")

    # RLIS_TIMELINE=1: a second library with the streaming products' timeline compiled in (a
    # measurement build; see stream_gemm_tcgen05.cu), beside the ordinary one
    timeline = os.environ.get("RLIS_TIMELINE", "0") not in ("", "0")
    flags = NVCC_FLAGS + (["-DRLIS_TIMELINE"] if timeline else [])

    def cmd(out):
        if out == "OUT":
            return flags
        return [_find_nvcc()] + flags + ["-o", out] + srcs

    name = "librlis_kernels_timeline.so" if timeline else "librlis_kernels.so"
    return _ensure(name, srcs, hdrs, cmd, "CUDA kernels (sm_100a)" + (" with the timeline" if timeline else ""))


def build_host() -> str:
    """Compiles the C++ cache manager and scheduler with their pybind11 bindings."""
    import pybind11

    srcs = sorted(glob.glob(os.path.join(CSRC, "host", "*.cpp")))
    hdrs = sorted(glob.glob(os.path.join(CSRC, "host", "*.h")))
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    inc = ["-I" + pybind11.get_include(), "-I" + sysconfig.get_paths()["include"]]

    def cmd(out):
        if out == "OUT":
            return CXX_FLAGS + [suffix]
        cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
        if not cxx:
            raise BuildError("no C++ compiler found (g++)")
        return [cxx] + CXX_FLAGS + inc + ["-o", out] + srcs

    return _ensure("_rlis_host" + suffix, srcs, hdrs, cmd, "host runtime (C++)")
