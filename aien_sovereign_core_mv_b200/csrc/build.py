"""Compiles the engine's native code in-tree and loads it.

Two artefacts, both under ``<package>/_build`` (or ``$AIEN_B200_BUILD_DIR``, or a per-user
folder in the temporary directory when the package folder is read-only):

* ``libaien_kernels.so``: every ``csrc/kernels/*.cu`` compiled by ``nvcc`` for sm_100a
  (``-gencode arch=compute_100a,code=sm_100a``), loaded with ``ctypes``;
* ``_aien_host*.so``: the C++ cache manager and scheduler (``csrc/host/*.cpp``) behind
  pybind11, compiled by ``g++``.

Nothing is fetched and nothing outside the build folder is written, so the first call works in
a fresh checkout for any user, with or without a home directory.  A content hash of the
sources and flags decides whether an artefact is rebuilt.  While compiling, a line is printed
to stderr every few seconds.  A missing compiler or a failed compile raises: there is no
fallback path.
"""
from __future__ import annotations

import ctypes
import glob
import hashlib
import importlib.util
import os
import shutil
import subprocess
import sys
import sysconfig
import tempfile
import time
from typing import List, Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
_PKG = os.path.dirname(_HERE)
KERNEL_DIR = os.path.join(_HERE, "kernels")
HOST_DIR = os.path.join(_HERE, "host")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "--expt-relaxed-constexpr", "--extended-lambda", "-Xcompiler", "-fPIC",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall"]
# AIEN_B200_HOST_SANITIZE=1 builds the host runtime with AddressSanitizer and UndefinedBehaviorSanitizer
# (any error aborts the process) under a name of its own beside the ordinary one.  The sanitizer runtime
# must come first in the process, with the C++ runtime beside it (Python itself links neither, and the
# sanitizer looks up __cxa_throw when it starts): run Python with LD_PRELOAD set to sanitizer_preload().  The
# reference checks its cache manager and scheduler the same way with Miri (tests/gates/sc-miri.gate).
SANITIZE_FLAGS = ["-O1", "-g", "-fno-omit-frame-pointer", "-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"]


def host_sanitized() -> bool:
    return os.environ.get("AIEN_B200_HOST_SANITIZE", "").strip() not in ("", "0")


def _sanitizing_compiler():
    """(compiler, path of its libasan.so) for the first C++ compiler at hand that ships the
    sanitizer runtime, or (None, None)."""
    for cxx in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"), "/usr/bin/g++"):
        if not cxx or not os.path.exists(cxx):
            continue
        try:
            out = subprocess.run([cxx, "-print-file-name=libasan.so"], capture_output=True, text=True, check=True).stdout.strip()
        except (OSError, subprocess.CalledProcessError):
            continue
        if os.path.isabs(out) and os.path.exists(out):
            return cxx, out
    return None, None


def sanitizer_runtime() -> Optional[str]:
    """Path of libasan.so, or None when no compiler here has one."""
    return _sanitizing_compiler()[1]


def sanitizer_preload() -> Optional[str]:
    """The value of LD_PRELOAD for a Python process that loads the sanitized host runtime:
    libasan.so and libstdc++.so of the compiler that builds it; None when there is none."""
    cxx, asan = _sanitizing_compiler()
    if not cxx:
        return None
    try:
        cpp = subprocess.run([cxx, "-print-file-name=libstdc++.so"], capture_output=True, text=True, check=True).stdout.strip()
    except (OSError, subprocess.CalledProcessError):
        return None
    return f"{asan} {cpp}" if os.path.isabs(cpp) and os.path.exists(cpp) else None


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[aien-b200 build] {msg}", file=sys.stderr, flush=True)


def build_dir() -> str:
    cand = os.environ.get("AIEN_B200_BUILD_DIR") or os.path.join(_PKG, "_build")
    try:
        os.makedirs(cand, exist_ok=True)
        probe = os.path.join(cand, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.unlink(probe)
        return cand
    except OSError:
        alt = os.path.join(tempfile.gettempdir(), f"aien_b200_build_{os.getuid()}")
        os.makedirs(alt, exist_ok=True)
        return alt


def find_nvcc() -> str:
    for cand in (
        os.environ.get("AIEN_B200_NVCC"),
        os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
        shutil.which("nvcc"),
        "/usr/local/cuda/bin/nvcc",
    ):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked at $AIEN_B200_NVCC, $CUDA_HOME/bin, PATH, /usr/local/cuda/bin)")


def _hash_sources(paths: List[str], flags: List[str]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(flags).encode())
    for p in sorted(paths):
        h.update(os.path.basename(p).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _run_parallel(cmds: List[List[str]], what: str, jobs: int) -> None:
    """Run commands with bounded parallelism, printing a progress line now and then."""
    pending = list(cmds)
    running = []
    start = last = time.time()
    done = 0
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    while pending or running:
        while pending and len(running) < jobs:
            cmd = pending.pop(0)
            running.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env)))
        still = []
        for cmd, proc in running:
            if proc.poll() is None:
                still.append((cmd, proc))
                continue
            out = proc.stdout.read().decode(errors="replace")
            if proc.returncode != 0:
                for _, other in running:
                    if other.poll() is None:
                        other.kill()
                raise BuildError(f"{what}: command failed ({proc.returncode}): {' '.join(cmd)}\n{out}")
            done += 1
        running = still
        now = time.time()
        if now - last >= 5.0:
            _say(f"{what}: {done}/{len(cmds)} done, {now - start:.0f} s")
            last = now
        if running:
            time.sleep(0.1)


def build_kernels(force: bool = False) -> str:
    """Compile every kernel source for sm_100a and link ``libaien_kernels.so``; returns its path."""
    out_dir = build_dir()
    sources = sorted(glob.glob(os.path.join(KERNEL_DIR, "*.cu")))
    headers = sorted(glob.glob(os.path.join(KERNEL_DIR, "*.cuh")) + glob.glob(os.path.join(KERNEL_DIR, "*.h")))
    if not sources:
        raise BuildError(f"no kernel sources under {KERNEL_DIR}")
    lib = os.path.join(out_dir, "libaien_kernels.so")
    stamp = lib + ".stamp"
    digest = _hash_sources(sources + headers, NVCC_FLAGS)
    if not force and os.path.exists(lib) and os.path.exists(stamp) and open(stamp).read().strip() == digest:
        return lib
    nvcc = find_nvcc()
    _say(f"compiling {len(sources)} CUDA sources for sm_100a into {out_dir} (first use; a minute or so)")
    objs, cmds = [], []
    for src in sources:
        obj = os.path.join(out_dir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        cmds.append([nvcc, *NVCC_FLAGS, "-I", KERNEL_DIR, "-c", src, "-o", obj])
    _run_parallel(cmds, "kernels", jobs=max(1, min(8, os.cpu_count() or 1)))
    tmp = lib + f".{os.getpid()}.tmp"
    _run_parallel([[nvcc, "-shared", "-o", tmp, *objs]], "link", jobs=1)
    os.replace(tmp, lib)
    with open(stamp, "w") as f:
        f.write(digest)
    _say("kernels ready")
    return lib


def _host_ext_name() -> str:
    return "_aien_host" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so")


def build_host(force: bool = False) -> str:
    """Compile the C++ cache manager and scheduler into a pybind11 module; returns its path."""
    out_dir = build_dir()
    sources = sorted(glob.glob(os.path.join(HOST_DIR, "*.cpp")))
    headers = sorted(glob.glob(os.path.join(HOST_DIR, "*.h")))
    flags = [f for f in CXX_FLAGS if f != "-O2"] + SANITIZE_FLAGS if host_sanitized() else CXX_FLAGS
    if host_sanitized():
        out_dir = os.path.join(out_dir, "sanitized")          # same module name, its own folder
        os.makedirs(out_dir, exist_ok=True)
    lib = os.path.join(out_dir, _host_ext_name())
    stamp = lib + ".stamp"
    digest = _hash_sources(sources + headers, flags)
    if not force and os.path.exists(lib) and os.path.exists(stamp) and open(stamp).read().strip() == digest:
        return lib
    cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
    if host_sanitized():
        cxx = _sanitizing_compiler()[0]
        if not cxx:
            raise BuildError("AIEN_B200_HOST_SANITIZE=1: no C++ compiler here ships the sanitizer runtime (libasan.so)")
    if not cxx:
        raise BuildError("no C++ compiler found (g++)")
    try:
        import pybind11
    except ImportError as e:
        raise BuildError(f"pybind11 headers are needed to build the host module: {e}") from None
    _say(f"compiling the host runtime (cache manager, scheduler) into {out_dir}")
    tmp = lib + f".{os.getpid()}.tmp"
    cmd = [cxx, *flags, "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"],
           "-I", HOST_DIR, *sources, "-o", tmp]
    _run_parallel([cmd], "host", jobs=1)
    os.replace(tmp, lib)
    with open(stamp, "w") as f:
        f.write(digest)
    return lib


_KERNELS: Optional[ctypes.CDLL] = None
_HOST = None


def load_kernels() -> ctypes.CDLL:
    global _KERNELS
    if _KERNELS is None:
        _KERNELS = ctypes.CDLL(build_kernels())
    return _KERNELS


def load_host():
    global _HOST
    if _HOST is None:
        path = build_host()
        spec = importlib.util.spec_from_file_location("_aien_host", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _HOST = mod
    return _HOST


def build_all(force: bool = False) -> None:
    build_host(force)
    build_kernels(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print(build_dir())
