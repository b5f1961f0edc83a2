"""Building the native kernel library at first use.

The CUDA sources under `rvllm_b200/csrc` are compiled with nvcc for sm_100a into one
shared library, `_build/librvllm_b200_<hash>.so` beside the sources, where <hash>
covers the sources and the flags: a changed source gives a new file name, so a stale
library is never loaded.  When the package folder is not writable the library goes to
a per-user folder under the system's temporary directory.  Each source is compiled by
its own nvcc process, in parallel, and a line is printed as each one finishes.

(The reference compiles its kernels at start-up too, with NVRTC to PTX for whatever
device is present, src/cuda/context.rs:92-106; here the target is fixed.)
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
from concurrent.futures import ThreadPoolExecutor, as_completed
from typing import List

from ..errors import KernelError

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
# no --use_fast_math: the float32 path needs exact division, sqrt and expf
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
              "--expt-relaxed-constexpr", "--expt-extended-lambda"]

_lock = threading.Lock()
_variant_locks = {}


# Sources compiled on demand with a size baked in, each into a library of its own.
VARIANT_SOURCES = {"attention_mma.cu", "attention_tcgen05.cu"}


def sources() -> List[str]:
    return sorted(f for f in os.listdir(CSRC)
                  if f.endswith(".cu") and f not in VARIANT_SOURCES)


def find_nvcc() -> str:
    for cand in (os.environ.get("RVLLM_NVCC"), shutil.which("nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelError("cannot build the CUDA kernels: nvcc was not found "
                      "(looked at $RVLLM_NVCC, PATH and /usr/local/cuda/bin)")


def source_hash() -> str:
    h = hashlib.sha256()
    for name in sorted(os.listdir(CSRC)):
        if name.endswith((".cu", ".cuh", ".h")):
            h.update(name.encode())
            with open(os.path.join(CSRC, name), "rb") as f:
                h.update(f.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


_build_dir = None


def build_dir() -> str:
    """The in-tree `_build` folder, or a per-user temporary one when that cannot be
    written (a read-only checkout, another user's files)."""
    global _build_dir
    if _build_dir is None:
        _build_dir = _find_build_dir()
    return _build_dir


def _find_build_dir() -> str:
    in_tree = os.path.join(CSRC, "_build")
    try:
        os.makedirs(in_tree, exist_ok=True)
        probe = os.path.join(in_tree, f".write_{os.getpid()}_{threading.get_ident()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return in_tree
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"rvllm_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def library_path() -> str:
    return os.path.join(build_dir(), f"librvllm_b200_{source_hash()}.so")


def _say(msg: str, verbose: bool) -> None:
    if verbose:
        print(f"[rvllm_b200] {msg}", file=sys.stderr, flush=True)


def build(verbose: bool = True, force: bool = False) -> str:
    """Compile if needed; return the library's path."""
    with _lock:
        out = library_path()
        if os.path.isfile(out) and not force:
            return out
        nvcc = find_nvcc()
        srcs = sources()
        work = tempfile.mkdtemp(prefix="obj_", dir=os.path.dirname(out))
        t0 = time.time()
        _say(f"compiling {len(srcs)} CUDA sources for sm_100a (first use; about a minute)",
             verbose)

        def compile_one(name: str) -> str:
            obj = os.path.join(work, name[:-3] + ".o")
            cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", CSRC, "-c",
                   os.path.join(CSRC, name), "-o", obj]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise KernelError(f"nvcc failed on {name}:\n{r.stderr[-4000:]}")
            return obj

        objs = []
        try:
            with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
                futures = {pool.submit(compile_one, s): s for s in srcs}
                for fut in as_completed(futures):
                    objs.append(fut.result())
                    _say(f"  compiled {futures[fut]} ({len(objs)}/{len(srcs)}, "
                         f"{time.time() - t0:.0f} s)", verbose)
            tmp_out = out + f".{os.getpid()}.tmp"
            cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", tmp_out, *sorted(objs), "-lcudart"]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise KernelError(f"linking the kernel library failed:\n{r.stderr[-4000:]}")
            os.replace(tmp_out, out)
            for old in os.listdir(os.path.dirname(out)):       # libraries of older sources
                if old.startswith("librvllm_b200_") and old.endswith(".so") and \
                        old.count("_") == 2 and \
                        os.path.join(os.path.dirname(out), old) != out:
                    try:
                        os.remove(os.path.join(os.path.dirname(out), old))
                    except OSError:
                        pass
        finally:
            shutil.rmtree(work, ignore_errors=True)
        _say(f"built {os.path.basename(out)} in {time.time() - t0:.0f} s", verbose)
        return out


def build_variant(source: str, defines: dict, tag: str, verbose: bool = True) -> str:
    """Compile one of `VARIANT_SOURCES` with the given -D definitions into its own
    library `librvllm_b200_<tag>_<hash>.so`; returns its path."""
    with _lock:
        lock = _variant_locks.setdefault(tag, threading.Lock())
    with lock:
        h = hashlib.sha256()
        for name in (source, "common.cuh"):
            with open(os.path.join(CSRC, name), "rb") as f:
                h.update(f.read())
        flags = [f"-D{k}={v}" for k, v in sorted(defines.items())]
        h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + flags).encode())
        out = os.path.join(build_dir(), f"librvllm_b200_{tag}_{h.hexdigest()[:16]}.so")
        if os.path.isfile(out):
            return out
        nvcc = find_nvcc()
        t0 = time.time()
        _say(f"compiling {source} for {tag} (first use of this size)", verbose)
        tmp_out = out + f".{os.getpid()}.tmp"
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, *flags, "-I", CSRC, "-shared", "-o", tmp_out,
               os.path.join(CSRC, source), "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise KernelError(f"nvcc failed on {source} ({tag}):\n{r.stderr[-4000:]}")
        os.replace(tmp_out, out)
        prefix = f"librvllm_b200_{tag}_"
        for old in os.listdir(os.path.dirname(out)):
            if old.startswith(prefix) and old.endswith(".so") and \
                    os.path.join(os.path.dirname(out), old) != out:
                try:
                    os.remove(os.path.join(os.path.dirname(out), old))
                except OSError:
                    pass
        _say(f"built {os.path.basename(out)} in {time.time() - t0:.0f} s", verbose)
        return out
