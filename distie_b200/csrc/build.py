"""Builds the native pieces on first use and keeps them beside the sources.

Two kinds of pieces:

* CUDA units: groups of ``.cu`` files compiled by ``nvcc`` for sm_100a into one
  shared library each, with plain ``extern "C"`` launchers that
  :mod:`distie_b200.kernels.library` binds through ``ctypes``.  A unit is built when
  the first kernel of it is asked for, so a float32 run never compiles the units
  only bfloat16 serving uses.
* the C++ block pool with its pybind11 binding, compiled by ``g++``.

Built files go to ``_build/`` next to this file, or to a per-user folder under the
system's temporary directory when the package folder is not writable.  A stamp
with a hash of sources and flags decides whether a rebuild is needed.  While
compilers run, a line is printed to stderr every few seconds.
"""

from __future__ import annotations

import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
import tempfile
import time
from contextlib import contextmanager

HERE = os.path.dirname(os.path.abspath(__file__))

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-O3",
    "-std=c++17",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC",
]

CUDA_UNITS: dict[str, list[str]] = {
    # every model needs these
    "base": ["elementwise.cu", "attention_generic.cu", "attention_decode.cu", "sampling.cu"],
    # bfloat16 serving only: tensor-core attention for prompts, weight-streaming products for decoding
    "bf16": ["attention_prefill.cu", "attention_decode_mma.cu", "gemm_tcgen05.cu", "attention_prefill_tcgen05.cu"],
}
_HEADERS = ["common.cuh", "tcgen05.cuh", "no_alloc.h"]


class BuildError(RuntimeError):
    pass


def register_unit(name: str, sources: list[str]) -> None:
    CUDA_UNITS[name] = list(sources)


def _say(message: str) -> None:
    print(f"[distie_b200] {message}", file=sys.stderr, flush=True)


def build_dir() -> str:
    override = os.environ.get("DISTIE_BUILD_DIR")
    candidates = [override] if override else []
    candidates.append(os.path.join(HERE, "_build"))
    candidates.append(os.path.join(tempfile.gettempdir(), f"distie_b200_build_{os.getuid()}"))
    for path in candidates:
        try:
            os.makedirs(path, exist_ok=True)
            probe = os.path.join(path, f".probe_{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return path
        except OSError:
            continue
    raise BuildError("no writable folder for built kernels; set DISTIE_BUILD_DIR")


@contextmanager
def _locked(path: str):
    with open(path, "w") as handle:
        fcntl.flock(handle, fcntl.LOCK_EX)
        try:
            yield
        finally:
            fcntl.flock(handle, fcntl.LOCK_UN)


def _digest(paths: list[str], flags: list[str]) -> str:
    h = hashlib.sha256()
    for flag in flags:
        h.update(flag.encode())
    for path in paths:
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as handle:
            h.update(handle.read())
    return h.hexdigest()


def find_nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.exists(candidate):
            return candidate
    raise BuildError("nvcc not found: the engine needs the CUDA toolkit to build its kernels (set NVCC)")


def _run_all(commands: list[tuple[str, list[str]]], what: str) -> None:
    """Run the commands in parallel; print a line now and then; raise with the compiler's words."""
    started = time.time()
    running = [(label, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)) for label, cmd in commands]
    _say(f"compiling {what}: {', '.join(label for label, _ in running)}")
    last = started
    outputs: dict[str, str] = {}
    pending = list(running)
    while pending:
        still = []
        for label, proc in pending:
            try:
                out, _ = proc.communicate(timeout=0.2)
                outputs[label] = out
            except subprocess.TimeoutExpired:
                still.append((label, proc))
        pending = still
        if pending and time.time() - last >= 10:
            last = time.time()
            _say(f"still compiling {', '.join(label for label, _ in pending)} ({int(last - started)} s)")
    failed = [(label, proc) for label, proc in running if proc.returncode != 0]
    if failed:
        text = "\n".join(f"--- {label} ---\n{outputs.get(label, '')}" for label, _ in failed)
        raise BuildError(f"building {what} failed:\n{text}")
    _say(f"built {what} in {time.time() - started:.0f} s")


def build_cuda_unit(name: str, verbose_ptxas: bool = False) -> str:
    """Path of the unit's shared library, building it if sources or flags changed."""
    if name not in CUDA_UNITS:
        raise BuildError(f"unknown kernel unit {name!r}")
    out_dir = build_dir()
    sources = [os.path.join(HERE, s) for s in CUDA_UNITS[name]]
    headers = [os.path.join(HERE, h) for h in _HEADERS]
    flags = NVCC_FLAGS + (["-Xptxas", "-v"] if verbose_ptxas else [])
    digest = _digest(sources + headers, flags)
    lib = os.path.join(out_dir, f"libdistie_{name}.so")
    stamp = os.path.join(out_dir, f"libdistie_{name}.stamp")
    with _locked(os.path.join(out_dir, f".lock_{name}")):
        if os.path.exists(lib) and os.path.exists(stamp):
            with open(stamp) as handle:
                if handle.read().strip() == digest:
                    return lib
        nvcc = find_nvcc()
        objects = []
        commands = []
        for src in sources:
            obj = os.path.join(out_dir, f"{name}_{os.path.basename(src)}.o")
            objects.append(obj)
            commands.append((os.path.basename(src), [nvcc, *flags, "-I", HERE, "-c", src, "-o", obj]))
        _run_all(commands, f"kernel unit '{name}'")
        tmp = lib + f".tmp{os.getpid()}"
        link = subprocess.run(
            [nvcc, "-shared", "-o", tmp, *objects, "-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"],
            capture_output=True,
            text=True,
        )
        if link.returncode != 0:
            raise BuildError(f"linking kernel unit '{name}' failed:\n{link.stdout}{link.stderr}")
        os.replace(tmp, lib)
        with open(stamp, "w") as handle:
            handle.write(digest)
        for obj in objects:
            try:
                os.remove(obj)
            except OSError:
                pass
    return lib


def build_block_pool() -> str:
    """Path of the pybind11 module ``distie_b200_core`` (the C++ page-id pool)."""
    import pybind11

    out_dir = build_dir()
    sources = [os.path.join(HERE, "block_pool.cpp"), os.path.join(HERE, "block_pool_bindings.cpp")]
    headers = [os.path.join(HERE, "block_pool.h")]
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    lib = os.path.join(out_dir, "distie_b200_core" + suffix)
    stamp = os.path.join(out_dir, "distie_b200_core.stamp")
    flags = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden"]
    digest = _digest(sources + headers, flags + [suffix])
    with _locked(os.path.join(out_dir, ".lock_core")):
        if os.path.exists(lib) and os.path.exists(stamp):
            with open(stamp) as handle:
                if handle.read().strip() == digest:
                    return lib
        compiler = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
        if not compiler:
            raise BuildError("no C++ compiler found for the block pool (set CXX)")
        tmp = lib + f".tmp{os.getpid()}"
        cmd = [
            compiler,
            *flags,
            "-I",
            HERE,
            "-I",
            pybind11.get_include(),
            "-I",
            sysconfig.get_paths()["include"],
            *sources,
            "-o",
            tmp,
            "-pthread",
        ]
        _run_all([("block_pool.cpp", cmd)], "block pool")
        os.replace(tmp, lib)
        with open(stamp, "w") as handle:
            handle.write(digest)
    return lib


def build_all(verbose_ptxas: bool = False) -> dict[str, str]:
    """Everything: used by the repository's build check."""
    out = {"core": build_block_pool()}
    for name in CUDA_UNITS:
        out[name] = build_cuda_unit(name, verbose_ptxas)
    return out
