"""The reference project's CUDA kernels, run on the CPU.

`load()` compiles `tests/ref_shim.cpp` with g++; that file `#include`s the kernel sources
straight from a checkout of ermolushka/rvllm (src/cuda/kernels/*.cu) and walks each
launch grid with loops.  The checkout is looked for in $RVLLM_REFERENCE_DIR, then in a
folder `reference` beside this repository.  Nothing of it is copied: without a checkout
(or without g++) `load()` returns None and the tests that need it fall back to the
recorded outputs under `tests/golden/`.

Each function below takes and returns float32 numpy arrays.
"""
import ctypes
import os
import shutil
import subprocess
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
KERNELS = ("short_conv.cu", "rope.cu", "silu_gate_multiply.cu", "rmsnorm.cu", "softmax.cu",
           "argmax.cu", "kv_write.cu", "kv_gather.cu", "embed_lookup.cu")


def reference_kernel_dir():
    cands = [os.environ.get("RVLLM_REFERENCE_DIR"),
             os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")]
    for root in cands:
        if not root:
            continue
        d = os.path.join(root, "src", "cuda", "kernels")
        if all(os.path.isfile(os.path.join(d, k)) for k in KERNELS):
            return d
    return None


_lib = None
_tried = False


def load():
    """The compiled shim as a `RefKernels`, or None when it cannot be built here."""
    global _lib, _tried
    if _tried:
        return _lib
    _tried = True
    d = reference_kernel_dir()
    gxx = shutil.which("g++")
    if d is None or gxx is None:
        return None
    out = os.path.join(tempfile.mkdtemp(prefix="rvllm_ref_shim_"), "ref_shim.so")
    cmd = [gxx, "-O1", "-shared", "-fPIC", "-x", "c++", "-I", d,
           os.path.join(HERE, "ref_shim.cpp"), "-o", out]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("the reference kernels did not compile as C++:\n" + proc.stderr)
    _lib = RefKernels(ctypes.CDLL(out))
    return _lib


def _f(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _u(a):
    return np.ascontiguousarray(a, dtype=np.uint32)


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


_U = ctypes.c_uint


class RefKernels:
    def __init__(self, lib):
        self.lib = lib

    def short_conv_bx(self, proj, hidden):
        """proj [rows, 3*hidden] -> bx [rows, hidden] (short_conv.cu:6-13)."""
        proj = _f(proj)
        rows = proj.shape[0]
        bx = np.empty((rows, hidden), np.float32)
        self.lib.run_short_conv_bx(_p(proj), _p(bx), _U(hidden), _U(rows * hidden))
        return bx

    def short_conv_filter_gate(self, window, filt, proj, batch, q_len):
        """window [batch, K-1+q_len, hidden], filt [hidden, K], proj [batch*q_len, 3*hidden]
        -> out [batch*q_len, hidden] (short_conv.cu:21-47)."""
        window, filt, proj = _f(window), _f(filt), _f(proj)
        hidden, taps = filt.shape
        out = np.empty((batch * q_len, hidden), np.float32)
        self.lib.run_short_conv_filter_gate(_p(window), _p(filt), _p(proj), _p(out), _U(batch),
                                            _U(q_len), _U(hidden), _U(taps))
        return out

    def rope(self, x, cos, sin):
        """x [rows, head_dim], cos/sin [rows, head_dim/2] (rope.cu:1-30)."""
        x, cos, sin = _f(x), _f(cos), _f(sin)
        out = np.empty_like(x)
        self.lib.run_rope(_p(x), _p(cos), _p(sin), _p(out), _U(x.shape[1]), _U(x.shape[0]))
        return out

    def silu_gate_multiply(self, gate, up):
        gate, up = _f(gate), _f(up)
        out = np.empty_like(gate)
        self.lib.run_silu_gate_multiply(_p(gate), _p(up), _p(out), _U(gate.size))
        return out

    def rmsnorm(self, x, weight, eps):
        x, weight = _f(x), _f(weight)
        out = np.empty_like(x)
        self.lib.run_rmsnorm(_p(x), _p(weight), _p(out), _U(x.shape[0]), _U(x.shape[1]),
                             ctypes.c_float(eps))
        return out

    def softmax(self, x):
        x = _f(x)
        out = np.empty_like(x)
        self.lib.run_softmax(_p(x), _p(out), _U(x.shape[0]), _U(x.shape[1]))
        return out

    def argmax(self, x):
        x = _f(x)
        out = np.empty(x.shape[0], np.uint32)
        self.lib.run_argmax(_p(x), _p(out), _U(x.shape[0]), _U(x.shape[1]))
        return out

    def kv_write(self, k, v, block_ids, offsets, cache_k, cache_v):
        """k, v [tokens, kv_heads, hd] into caches [blocks, block_size, kv_heads, hd], in
        place (kv_write.cu)."""
        k, v = _f(k), _f(v)
        block_ids, offsets = _u(block_ids), _u(offsets)
        assert cache_k.dtype == np.float32 and cache_k.flags.c_contiguous
        self.lib.run_kv_write(_p(k), _p(v), _p(block_ids), _p(offsets), _p(cache_k), _p(cache_v),
                              _U(k.shape[0]), _U(k.shape[1]), _U(k.shape[2]),
                              _U(cache_k.shape[1]))

    def kv_gather(self, cache, block_idx, ctx_len):
        """cache [blocks, block_size, kv_heads, hd], block_idx [batch, max_blocks] ->
        [batch, kv_heads, ctx_len, hd] (kv_gather.cu)."""
        block_idx = _u(block_idx)
        batch, max_blocks = block_idx.shape
        _, bs, nkv, hd = cache.shape
        out = np.empty((batch, nkv, ctx_len, hd), np.float32)
        self.lib.run_kv_gather(_p(cache), _p(block_idx), _p(out), _U(batch), _U(max_blocks),
                               _U(ctx_len), _U(bs), _U(nkv), _U(hd))
        return out

    def embed_lookup(self, ids, table):
        ids, table = _u(ids), _f(table)
        out = np.empty((ids.shape[0], table.shape[1]), np.float32)
        self.lib.run_embed_lookup(_p(ids), _p(table), _p(out), _U(ids.shape[0]),
                                  _U(table.shape[1]))
        return out
