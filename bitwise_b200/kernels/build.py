"""Compiling the CUDA sources of ``csrc/`` for sm_100a into shared libraries, in-tree.

Each kernel set becomes one library named after a hash of its sources and flags, so a
stale library is never loaded.  A set is built the first time something needs it
(the 32-bit path never compiles the bfloat16 kernels and the other way round); the
build prints a line per file and a heartbeat while nvcc runs.  Libraries live in
``bitwise_b200/kernels/_build`` when that is writable, else in a per-user folder under
the system's temporary directory.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, List, Sequence

CSRC = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "csrc"))

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

# kernel set -> list of (source file, extra flags)
KERNEL_SETS: Dict[str, List[tuple]] = {
    "f32": [("common.cu", []), ("exact_f32.cu", ["-fmad=false"])],
    "bf16": [("common.cu", []), ("bf16_ops.cu", []), ("bf16_gemm.cu", []), ("bf16_gemm_tc.cu", []),
             ("bf16_gemm_rows.cu", [])],
    # compiled once per head size, with -DBW_HEAD_DIM=<n>
    "bf16_attn": [("common.cu", []), ("bf16_attention.cu", []), ("bf16_attention_tc.cu", [])],
}

# head sizes whose attention library a full build prepares (others are compiled when a model asks)
DEFAULT_HEAD_DIMS = (16, 32, 64, 128)


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    cands = []
    for env in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(env):
            cands.append(os.path.join(os.environ[env], "bin", "nvcc"))
    cands.append("/usr/local/cuda/bin/nvcc")
    w = shutil.which("nvcc")
    if w:
        cands.append(w)
    for c in cands:
        if os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise BuildError("nvcc not found (looked in $CUDA_HOME/bin, /usr/local/cuda/bin and PATH); "
                     "the CUDA kernels cannot be compiled")


def _build_root() -> str:
    here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_build")
    try:
        os.makedirs(here, exist_ok=True)
        probe = os.path.join(here, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return here
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"bitwise_b200-build-{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _set_sources(kind: str, defines: Sequence[str]):
    if kind not in KERNEL_SETS:
        raise BuildError(f"unknown kernel set {kind!r}")
    return [(os.path.join(CSRC, f), list(extra) + [f"-D{d}" for d in defines]) for f, extra in KERNEL_SETS[kind]]


def _digest(kind: str, defines: Sequence[str]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(ARCH_FLAGS + BASE_FLAGS + list(defines)).encode())
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cu", ".cuh", ".h")):
            h.update(f.encode())
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(fh.read())
    for f, extra in KERNEL_SETS[kind]:
        h.update((f + " ".join(extra)).encode())
    return h.hexdigest()[:12]


def library_file(kind: str, defines: Sequence[str] = ()) -> str:
    tag = "".join("_" + d.replace("=", "") for d in defines)
    return os.path.join(_build_root(), f"libbitwise_{kind}{tag}-{_digest(kind, defines)}.so")


def _say(msg: str, verbose: bool) -> None:
    if verbose:
        print(f"[bitwise_b200 build] {msg}", file=sys.stderr, flush=True)


def ensure_built(kind: str, defines: Sequence[str] = (), verbose: bool = True) -> str:
    """Return the path of the library of kernel set ``kind``, compiling it if needed."""
    out = library_file(kind, defines)
    if os.path.isfile(out):
        return out
    nvcc = find_nvcc()
    root = os.path.dirname(out)
    srcs = _set_sources(kind, defines)
    objdir = os.path.join(root, f"obj-{kind}-{os.getpid()}")
    os.makedirs(objdir, exist_ok=True)
    _say(f"compiling kernel set '{kind}' ({len(srcs)} files) for sm_100a with {nvcc}", verbose)
    t0 = time.time()
    stop = threading.Event()

    def heartbeat():
        while not stop.wait(10.0):
            _say(f"... still compiling '{kind}' ({time.time() - t0:.0f} s)", verbose)

    hb = threading.Thread(target=heartbeat, daemon=True)
    hb.start()

    def compile_one(item):
        src, extra = item
        obj = os.path.join(objdir, os.path.basename(src) + ".o")
        cmd = [nvcc, *ARCH_FLAGS, *BASE_FLAGS, *extra, "-I", CSRC, "-c", src, "-o", obj]
        _say("nvcc " + os.path.basename(src), verbose)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        return obj

    try:
        with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
            objs = list(ex.map(compile_one, srcs))
        tmp = out + f".tmp{os.getpid()}"
        cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", tmp, *objs]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"link of {out} failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, out)
    finally:
        stop.set()
        shutil.rmtree(objdir, ignore_errors=True)
    # libraries of older source states are of no use any more
    prefix = os.path.basename(out).rsplit("-", 1)[0] + "-"
    for f in os.listdir(root):
        if f.startswith(prefix) and f.endswith(".so") and os.path.join(root, f) != out:
            try:
                os.remove(os.path.join(root, f))
            except OSError:
                pass
    _say(f"built {os.path.basename(out)} in {time.time() - t0:.1f} s", verbose)
    return out


# ---- the host runtime (plain C++: page pools, cache manager, scheduler) ------------------
HOST_SOURCES = ("host_runtime.cpp",)
HOST_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden"]


def find_cxx() -> str:
    cands = [os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"), shutil.which("clang++")]
    for c in cands:
        if c and os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise BuildError("no C++ compiler found ($CXX, g++, c++, clang++): the host runtime cannot be compiled")


def host_library_file() -> str:
    h = hashlib.sha256()
    h.update(" ".join(HOST_FLAGS).encode())
    for f in HOST_SOURCES:
        h.update(f.encode())
        with open(os.path.join(CSRC, f), "rb") as fh:
            h.update(fh.read())
    return os.path.join(_build_root(), f"libbitwise_host-{h.hexdigest()[:12]}.so")


def ensure_host_built(verbose: bool = True) -> str:
    """Return the path of the host runtime's library, compiling it if needed (no CUDA involved)."""
    out = host_library_file()
    if os.path.isfile(out):
        return out
    cxx = find_cxx()
    _say(f"compiling the host runtime ({', '.join(HOST_SOURCES)}) with {cxx}", verbose)
    t0 = time.time()
    tmp = out + f".tmp{os.getpid()}"
    cmd = [cxx, *HOST_FLAGS, *[os.path.join(CSRC, f) for f in HOST_SOURCES], "-o", tmp]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"{cxx} failed on the host runtime:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, out)
    root = os.path.dirname(out)
    for f in os.listdir(root):
        if f.startswith("libbitwise_host-") and f.endswith(".so") and os.path.join(root, f) != out:
            try:
                os.remove(os.path.join(root, f))
            except OSError:
                pass
    _say(f"built {os.path.basename(out)} in {time.time() - t0:.1f} s", verbose)
    return out


def build_all(verbose: bool = True) -> List[str]:
    """Compile every kernel set (what a 'does it build' check wants)."""
    out = [ensure_host_built(verbose)]
    out += [ensure_built(k, (), verbose) for k in ("f32", "bf16")]
    out += [ensure_built("bf16_attn", (f"BW_HEAD_DIM={hd}",), verbose) for hd in DEFAULT_HEAD_DIMS]
    return out
