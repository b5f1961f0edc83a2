"""The CUDA kernel set: ctypes bindings of the native library, with the interface the
parts call (`embed`, `add_rmsnorm`, `linear`, `qk_norm_rope_write`, `paged_attention`,
`short_conv`, `swiglu`, `add_bias`, `argmax`, `sample`).

Every kernel launches on torch's current stream, so captured graphs and ordinary
stream order both work.  Matrix products go to cuBLAS through `torch.mm`, as the
reference sends them to cuBLAS (src/cuda/cublas_ops.rs:44-92); with float32 operands
TF32 is switched off, so the float32 path is float32 throughout.  There is no CPU
path here: constructing `CudaOps` without a CUDA device or without the library raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from ..errors import KernelError
from .build import build, build_variant

_F32, _BF16 = 0, 1


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return _F32
    if dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {dtype}")


def _ptr(t):
    return c_void_p(0 if t is None else t.data_ptr())


class CudaOps:
    name = "cuda"

    def __init__(self, verbose_build: bool = True):
        if not torch.cuda.is_available():
            raise KernelError("rvllm_b200 needs a CUDA device: there is no CPU path")
        path = build(verbose=verbose_build)
        try:
            self.lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load the kernel library {path}: {e}") from None
        self.library_path = path
        self.launches = 0
        self.lib.rv_last_error.restype = ctypes.c_char_p
        self.lib.rv_paged_attention_decode_scratch_bytes.restype = c_longlong
        self.lib.rv_gemm_tiled_bytes.restype = c_longlong
        self._scratch = {}
        self._retired = []
        self._attn_libs = {}
        self._verbose_build = verbose_build
        # bfloat16 attention: "mma" = mma.sync tensor-core kernels (attention_mma.cu, head
        # sizes that are multiples of 16 up to 128), "simt" = the float32-arithmetic kernels;
        # prompt portions also "tcgen05" (attention_tcgen05.cu, head size 64) and "auto" =
        # tcgen05 where it applies, else mma
        self.prefill_attention = os.environ.get("RVLLM_PREFILL_ATTENTION", "auto")
        self.decode_attention = os.environ.get("RVLLM_DECODE_ATTENTION", "mma")
        # keys per block of the tensor-core decode kernel: 256 (four warps) or 128 (two)
        self.decode_split = int(os.environ.get("RVLLM_ATTN_DECODE_SPLIT", "256"))
        # "stream": one persistent block per SM whose warps each stream their work items'
        # tiles through a private ring; "block": one block per (request, head, split);
        # "auto": the stream kernel from `stream_min_items` work items of 256 keys on
        self.decode_kernel = os.environ.get("RVLLM_ATTN_DECODE_KERNEL", "auto")
        self.stream_min_items = int(os.environ.get("RVLLM_ATTN_STREAM_MIN_ITEMS", "384"))
        self._sm_count = torch.cuda.get_device_properties(
            torch.cuda.current_device()).multi_processor_count
        # bfloat16 products with at most `gemm_small_m` tokens go to the tcgen05
        # weight-streaming kernel (gemm_tcgen05.cu), whose weight copies start before the
        # previous kernel has finished; larger ones go to cuBLAS.  RVLLM_GEMM=cublas sends
        # everything to cuBLAS, =auto only the shapes with few output tiles and a long K.
        self.gemm_small_m = int(os.environ.get("RVLLM_GEMM_SMALL_M", "16"))
        self.gemm_mode = os.environ.get("RVLLM_GEMM", "tcgen05")
        self._gemm_state = {}
        self._tiled = {}
        self.gemm_tiled = os.environ.get("RVLLM_GEMM_TILED", "1") != "0"
        self.gemm_row_pad = int(os.environ.get("RVLLM_GEMM_ROW_PAD", "64"))
        # q/k norm + rotation + cache write inside the q|k|v product's epilogue (few bfloat16
        # tokens, head size 64); "0": always the separate kernel
        self.fuse_qkv_rope = os.environ.get("RVLLM_FUSE_QKV_ROPE", "1") == "1"
        self._check(self.lib.rv_gemm_tcgen05_init(), "gemm_tcgen05 set-up")
        # float32 products must be float32: no TF32, no reduced-precision accumulation
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
        self.launches = 0

    # ---- plumbing --------------------------------------------------------------------

    def _check(self, rc: int, what: str) -> None:
        self.launches += 1
        if rc != 0:
            raise KernelError(f"{what}: {self.lib.rv_last_error().decode()}")

    @staticmethod
    def _stream() -> c_void_p:
        # the current stream of the current device; the raw query is a fraction of a microsecond
        # where `torch.cuda.current_stream()` builds a Python object in some 15 (and a step of a
        # small model makes some 140 launches)
        raw = getattr(torch._C, "_cuda_getCurrentRawStream", None)
        if raw is not None:
            return c_void_p(raw(torch._C._cuda_getDevice()))
        return c_void_p(torch.cuda.current_stream().cuda_stream)

    @staticmethod
    def _need(t: torch.Tensor, what: str, dtype=None, contiguous=True):
        if not t.is_cuda:
            raise KernelError(f"{what} must be a CUDA tensor")
        if contiguous and not t.is_contiguous():
            raise KernelError(f"{what} must be contiguous")
        if dtype is not None and t.dtype != dtype:
            raise KernelError(f"{what} must be {dtype}, got {t.dtype}")

    # ---- embedding -------------------------------------------------------------------

    def embed(self, table, ids, out, scale=None):
        self._need(table, "embedding table")
        self._need(ids, "token ids", torch.int32)
        self._need(out, "embedding output", torch.float32)
        n, hidden = out.shape
        self._check(self.lib.rv_embed(_ptr(table), _code(table.dtype), _ptr(ids), _ptr(out),
                                      c_int(n), c_int(hidden), c_int(table.shape[0]),
                                      c_float(1.0 if scale is None else scale), self._stream()),
                    "embed")

    # ---- residual add + RMSNorm ------------------------------------------------------

    def add_rmsnorm(self, resid, delta, weight, eps, out, rows=None):
        """`resid` None: the rows of `delta` alone are normalised (no stream involved)."""
        if resid is not None:
            self._need(resid, "residual stream", torch.float32)
        elif delta is None or rows is not None:
            raise KernelError("add_rmsnorm: without a stream it takes rows to normalise, all of them")
        self._need(weight, "norm weight", torch.float32)
        self._need(out, "norm output")
        if delta is not None:
            self._need(delta, "pending sub-layer output")
            if resid is not None and delta.shape != resid.shape:
                raise KernelError("add_rmsnorm: the stream and the pending output differ in shape")
        if rows is not None:
            self._need(rows, "row list", torch.int32)
        n, hidden = out.shape
        if (resid if resid is not None else delta).shape[1] != hidden or weight.shape[0] != hidden:
            raise KernelError("add_rmsnorm: widths disagree")
        self._check(self.lib.rv_add_rmsnorm(
            _ptr(resid), _ptr(delta), _code(delta.dtype) if delta is not None else _F32,
            _ptr(weight), _ptr(out), _code(out.dtype), _ptr(rows), c_int(n), c_int(hidden),
            c_float(eps), self._stream()), "add_rmsnorm")

    # ---- matrix product (library) -------------------------------------------------------

    def _gemm_status(self, device):
        device = torch.device(device)
        if device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        st = self._gemm_state.get(device)
        if st is None:
            st = torch.zeros(1, dtype=torch.int32, device=device)
            self._gemm_state[device] = st
        return st

    def linear_tcgen05(self, x, w, out_dtype):
        """y = x . w^T for bfloat16 x [M <= 256, K] and w [N, K] on the tcgen05 kernel."""
        self._need(x, "activation rows", torch.bfloat16)
        self._need(w, "weight matrix", torch.bfloat16)
        m, k = x.shape
        n = w.shape[0]
        y = torch.empty((m, n), dtype=out_dtype, device=x.device)
        self._check(self.lib.rv_gemm_tcgen05(
            _ptr(x), _ptr(w), _ptr(y), _code(out_dtype), _ptr(self._gemm_status(x.device)),
            c_int(m), c_int(n), c_int(k), _ptr(self._tiled_weight(w)), self._stream()),
            "gemm_tcgen05")
        return y

    def _tiled_weight(self, w):
        """The weight matrix once more, laid out tile by tile for the streaming product
        (`rv_gemm_tile_weights`): made the first time a matrix is used with few tokens and
        kept as long as the matrix lives.  It doubles the memory of the matrices that decode
        steps multiply (2.3 GB at LFM2-1.2B sizes) and lets an SM copy a tile as one
        contiguous 16 KB instead of 128 strided rows.  RVLLM_GEMM_TILED=0: not made."""
        if not self.gemm_tiled:
            return None
        key = (w.data_ptr(), tuple(w.shape))
        hit = self._tiled.get(key)
        if hit is not None and hit[0]() is w:
            return hit[1]
        if torch.cuda.is_current_stream_capturing():
            return None                    # no allocation inside a capture: the box copies do
        n, k = w.shape
        nbytes = int(self.lib.rv_gemm_tiled_bytes(c_int(n), c_int(k)))
        tiled = torch.empty(nbytes, dtype=torch.uint8, device=w.device)
        self._check(self.lib.rv_gemm_tile_weights(_ptr(w), _ptr(tiled), c_int(n), c_int(k),
                                                  self._stream()), "gemm_tile_weights")
        import weakref
        # the copies of matrices that have died go first (a model that was unloaded)
        self._tiled = {kk: v for kk, v in self._tiled.items() if v[0]() is not None}
        self._tiled[key] = (weakref.ref(w), tiled)
        return tiled

    def status_word(self, device) -> torch.Tensor:
        """The int32 word in which kernels on `device` record a wait that ran out (0: none).
        A caller that already copies a step's result to the host can copy this word along
        and pass what it read to `raise_for_status`, which costs no synchronisation."""
        return self._gemm_status(device)

    def raise_for_status(self, code: int, device=None) -> None:
        if code != 0:
            if device is not None:
                self._gemm_status(device).zero_()
            raise KernelError(f"a kernel gave up waiting on an mbarrier (code {code}: 1-4 "
                              f"gemm_tcgen05, 12 decode attention, 21 prefill attention); its "
                              f"output is not valid")

    def check_status(self) -> None:
        """Raise if a kernel recorded that one of its bounded waits ran out (this
        synchronises with the device)."""
        for device, st in self._gemm_state.items():
            code = int(st.item())
            if code != 0:
                st.zero_()
                raise KernelError(f"a kernel gave up waiting on an mbarrier (code {code}: 1-4 "
                                  f"gemm_tcgen05, 12 decode attention, 21 prefill attention) on {device}; its "
                                  f"output is not valid")

    def _small_product(self, x, w, out_dtype) -> bool:
        """Whether x . w^T goes to the tcgen05 weight-streaming kernel."""
        return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
                and 0 < x.shape[0] <= self.gemm_small_m and self.gemm_mode != "cublas"
                and x.shape[1] % 8 == 0 and x.is_contiguous() and w.is_contiguous()
                and out_dtype in (torch.bfloat16, torch.float32)
                and (self.gemm_mode == "tcgen05"
                     or (w.shape[0] <= 18 * 128 and x.shape[1] >= 4096)))

    def linear_qk_norm_rope_write(self, x, w_qkv, num_heads, num_kv_heads, head_dim, q_weight,
                                  k_weight, eps, table, positions, slot_mapping, k_cache, v_cache,
                                  out_dtype=None):
        """q|k|v = x . w_qkv^T, then per-head q/k norm, rotation and the cache write; returns
        the [tokens, (heads + 2 kv heads) * head_dim] buffer whose query columns attention
        reads.  Few bfloat16 tokens with head size 64 and a cache to write: one kernel (the
        product's epilogue does the rest); otherwise the product and `qk_norm_rope_write`."""
        out_dtype = out_dtype or x.dtype
        if (self.fuse_qkv_rope and k_cache is not None and num_kv_heads > 0 and head_dim == 64
                and out_dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
                and w_qkv.shape[0] == (num_heads + 2 * num_kv_heads) * 64
                and x.shape[0] <= 16 and self._small_product(x, w_qkv, out_dtype)):
            m, k = x.shape
            n = w_qkv.shape[0]
            qkv = torch.empty((m, n), dtype=out_dtype, device=x.device)
            cos, sin = table if table is not None else (None, None)
            self._check(self.lib.rv_gemm_tcgen05_qkv(
                _ptr(x), _ptr(w_qkv), _ptr(qkv), _ptr(self._gemm_status(x.device)), c_int(m),
                c_int(n), c_int(k), c_int(num_heads), c_int(num_kv_heads), _ptr(q_weight),
                _ptr(k_weight), c_float(eps), _ptr(cos), _ptr(sin), _ptr(positions),
                _ptr(slot_mapping), _ptr(k_cache), _ptr(v_cache), _ptr(self._tiled_weight(w_qkv)),
                self._stream()), "gemm_tcgen05_qkv")
            return qkv
        qkv = self.linear(x, w_qkv, out_dtype=out_dtype)
        self.qk_norm_rope_write(qkv, num_heads, num_kv_heads, head_dim, q_weight, k_weight, eps,
                                table, positions, slot_mapping, k_cache, v_cache)
        return qkv

    def linear(self, x, w, bias=None, out_dtype=None):
        out_dtype = out_dtype or x.dtype
        if x.dtype != w.dtype:
            # a matrix kept in 32 bits is multiplied in 32 bits
            wide = torch.float32 if torch.float32 in (x.dtype, w.dtype) else x.dtype
            x, w = x.to(wide), w.to(wide)
        if x.shape[0] == 0:
            return torch.empty((0, w.shape[0]), dtype=out_dtype, device=x.device)
        if self._small_product(x, w, out_dtype):
            y = self.linear_tcgen05(x, w, out_dtype)
        else:
            # The library chooses an algorithm per shape, and a shape it has not met costs it
            # some 70 us on the host: a prompt portion of 301 tokens, then 302, ... would pay
            # that in every product of every step.  So it is shown row counts in multiples of
            # 64 (RVLLM_GEMM_ROW_PAD): the rows beyond the real ones are whatever the buffer
            # holds (`new_rows` leaves room for them) and their results are dropped.
            m = x.shape[0]
            xp = self._padded_rows(x)
            if out_dtype == x.dtype:
                y = torch.mm(xp, w.t())
            elif x.dtype == torch.bfloat16 and out_dtype == torch.float32:
                y = torch.mm(xp, w.t(), out_dtype=torch.float32)
            else:
                y = torch.mm(xp, w.t()).to(out_dtype)
            if y.shape[0] != m:
                y = y[:m]
        if bias is not None:
            self.add_bias(y, bias)
        return y

    def new_rows(self, n, width, dtype, device):
        """An uninitialised [n, width] buffer for activation rows whose storage is a multiple
        of the row padding long, so that a library product can take it as it is."""
        pad = self._row_pad(n)
        if pad <= 1 or n % pad == 0:
            return torch.empty((n, width), dtype=dtype, device=device)
        return torch.empty((-(-n // pad) * pad, width), dtype=dtype, device=device)[:n]

    def _row_pad(self, n: int) -> int:
        """Rows are padded to multiples of 64, of 32 up to 64 rows (a replayed decode step of 32
        requests is 1 % slower with 64 rows than with its own 32)."""
        return min(self.gemm_row_pad, 32) if n <= 64 else self.gemm_row_pad

    def _padded_rows(self, x):
        m, k = x.shape
        pad = self._row_pad(m)
        if pad <= 1 or m % pad == 0 or not x.is_contiguous():
            return x
        mp = -(-m // pad) * pad
        if x.storage_offset() == 0 and x.untyped_storage().nbytes() >= mp * k * x.element_size():
            return x.as_strided((mp, k), (k, 1))          # the buffer has the room (`new_rows`)
        xp = torch.empty((mp, k), dtype=x.dtype, device=x.device)
        xp[:m].copy_(x)
        return xp

    def add_bias(self, x, bias):
        self._need(x, "add_bias input")
        self._need(bias, "bias", torch.float32)
        self._check(self.lib.rv_add_bias(_ptr(x), _code(x.dtype), _ptr(bias), c_int(x.shape[0]),
                                         c_int(x.shape[1]), self._stream()), "add_bias")

    # ---- q/k norm + rotation + cache write -------------------------------------------

    def qk_norm_rope_write(self, qkv, num_heads, num_kv_heads, head_dim, q_weight, k_weight,
                           eps, table, positions, slot_mapping, k_cache, v_cache):
        self._need(qkv, "q|k|v rows")
        if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
            raise KernelError("qk_norm_rope_write: row width and head counts disagree")
        if k_cache is not None:
            self._need(k_cache, "key pages", qkv.dtype)
            self._need(v_cache, "value pages", qkv.dtype)
        cos, sin = table if table is not None else (None, None)
        self._check(self.lib.rv_qk_norm_rope_write(
            _ptr(qkv), _code(qkv.dtype), c_int(qkv.shape[1]), c_int(qkv.shape[0]),
            c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), _ptr(q_weight),
            _ptr(k_weight), c_float(eps), _ptr(cos), _ptr(sin), _ptr(positions),
            _ptr(slot_mapping), _ptr(k_cache), _ptr(v_cache), self._stream()),
            "qk_norm_rope_write")

    # ---- attention -------------------------------------------------------------------

    def _scratch_buffer(self, nbytes: int, device) -> torch.Tensor:
        """The split-KV scratch of `device`, at least `nbytes` long.  A captured launch
        sequence holds the raw address of the buffer it was captured with, so a buffer
        that is outgrown is never given back: it moves to `_retired` and stays valid for
        every graph that names it.  Growth doubles, so the retired ones together are
        smaller than the live one."""
        key = str(device)
        buf = self._scratch.get(key)
        if buf is None or buf.numel() < nbytes:
            size = max(nbytes, 1 << 20, 2 * buf.numel() if buf is not None else 0)
            if buf is not None:
                self._retired.append(buf)
            buf = torch.empty(size, dtype=torch.uint8, device=device)
            self._scratch[key] = buf
        return buf

    def attention_scratch_bytes(self, n_reqs: int, num_heads: int, head_dim: int,
                                max_ctx_len: int) -> int:
        """Bytes of split-KV scratch the decode attention kernels need at most for
        `n_reqs` single-token requests of up to `max_ctx_len` cached tokens (with the
        smallest split any of them uses, 128 keys)."""
        decode = int(self.lib.rv_paged_attention_decode_scratch_bytes(
            c_int(n_reqs), c_int(num_heads), c_int(head_dim), c_int(2 * max_ctx_len)))
        return max(decode, self._prefill_scratch_bytes(head_dim))

    def reserve_scratch(self, nbytes: int, device) -> None:
        """Size the scratch before any launch sequence is captured, so that it does not
        have to grow afterwards."""
        if nbytes > 0:
            self._scratch_buffer(nbytes, device)

    def _attn_lib(self, head_dim: int):
        """The tensor-core attention library for this head size, built at first use."""
        lib = self._attn_libs.get(head_dim)
        if lib is None:
            path = build_variant("attention_mma.cu", {"RV_HD": head_dim}, f"attn_hd{head_dim}",
                                 verbose=self._verbose_build)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelError(f"cannot load the kernel library {path}: {e}") from None
            getattr(lib, f"rv_attention_mma_last_error_hd{head_dim}").restype = ctypes.c_char_p
            self._attn_libs[head_dim] = lib
        return lib

    def _attn5_lib(self, head_dim: int):
        """The tcgen05 prefill attention library for this head size, built at first use."""
        key = ("tcgen05", head_dim)
        lib = self._attn_libs.get(key)
        if lib is None:
            path = build_variant("attention_tcgen05.cu", {"RV_HD": head_dim},
                                 f"attn5_hd{head_dim}", verbose=self._verbose_build)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelError(f"cannot load the kernel library {path}: {e}") from None
            getattr(lib, f"rv_attention_tcgen05_last_error_hd{head_dim}").restype = ctypes.c_char_p
            self._attn_libs[key] = lib
        return lib

    def _tcgen05_prefill_ok(self, qkv, out, num_heads, num_kv_heads, head_dim, page_size) -> bool:
        return (qkv.dtype == torch.bfloat16 and head_dim == 64
                and page_size in (8, 16, 32, 64) and num_heads // num_kv_heads <= 128
                and qkv.shape[1] % head_dim == 0 and qkv.data_ptr() % 16 == 0
                and out.data_ptr() % 16 == 0)

    def paged_attention_prefill_tcgen05(self, qkv, num_heads, num_kv_heads, head_dim, k_cache,
                                        v_cache, ctx, group, scale, window, out):
        """Requests [n_decode, n_reqs) -- the ones that bring more than one token -- on the
        tcgen05 kernel (bfloat16, head size 64)."""
        lib = self._attn5_lib(head_dim)
        nd = ctx.n_decode
        fn = getattr(lib, f"rv_paged_attention_prefill_tcgen05_hd{head_dim}")
        # scratch for the parts of a launch too small to fill the GPU (the kernel shares the key
        # tiles of its blocks out); never made or grown inside a stream capture
        need = self._prefill_scratch_bytes(head_dim)
        scratch = self._scratch.get(str(qkv.device))
        if scratch is None or scratch.numel() < need:
            scratch = (None if torch.cuda.is_current_stream_capturing()
                       else self._scratch_buffer(need, qkv.device))
        rc = fn(_ptr(qkv), c_int(qkv.shape[1]), c_int(qkv.shape[0]), _ptr(k_cache), _ptr(v_cache),
                c_longlong(k_cache.shape[0] * k_cache.shape[1]), _ptr(group.block_table),
                c_int(group.max_blocks), _ptr(ctx.q_start), _ptr(ctx.ctx_lens), _ptr(out),
                c_int(nd), c_int(ctx.n_reqs - nd), c_int(ctx.max_q_len), c_int(ctx.max_ctx_len),
                c_int(num_heads), c_int(num_kv_heads), c_int(group.page_size), c_float(scale),
                c_int(window if window else 0), _ptr(self._gemm_status(qkv.device)),
                _ptr(scratch), c_longlong(scratch.numel() if scratch is not None else 0),
                c_int(self._sm_count), self._stream())
        self.launches += 1
        if rc != 0:
            msg = getattr(lib, f"rv_attention_tcgen05_last_error_hd{head_dim}")().decode()
            raise KernelError(f"paged_attention_prefill_tcgen05: {msg}")

    def _prefill_scratch_bytes(self, head_dim: int) -> int:
        """What the tcgen05 prefill attention may use for the parts of shared-out blocks."""
        if head_dim != 64 or self.prefill_attention not in ("auto", "tcgen05"):
            return 0
        # rv_paged_attention_prefill_tcgen05_scratch_bytes: six parts an SM, each 128 rows of
        # 64 float32 values, an offset and a sum (the kernel fits its parts to what it is given)
        return 6 * self._sm_count * 128 * (64 * 4 + 8)

    def _check_attn(self, lib, head_dim: int, rc: int, what: str) -> None:
        self.launches += 1
        if rc != 0:
            msg = getattr(lib, f"rv_attention_mma_last_error_hd{head_dim}")().decode()
            raise KernelError(f"{what}: {msg}")

    @staticmethod
    def _mma_ok(dtype, head_dim: int) -> bool:
        return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 128

    def paged_attention(self, qkv, num_heads, num_kv_heads, head_dim, k_cache, v_cache,
                        ctx, group, scale, window, out):
        self._need(qkv, "query rows")
        self._need(out, "attention output", qkv.dtype)
        self._need(k_cache, "key pages", qkv.dtype)
        self._need(v_cache, "value pages", qkv.dtype)
        code = _code(qkv.dtype)
        win = c_int(window if window else 0)
        nd = ctx.n_decode
        mma = self._mma_ok(qkv.dtype, head_dim)
        if nd > 0:
            if mma and self.decode_attention == "mma":
                self.paged_attention_decode_mma(qkv, num_heads, num_kv_heads, head_dim, k_cache,
                                                v_cache, group.block_table, ctx.q_start,
                                                ctx.ctx_lens, nd, ctx.max_ctx_len,
                                                group.page_size, scale, window, out)
            else:
                self.paged_attention_decode(qkv, num_heads, num_kv_heads, head_dim, k_cache,
                                            v_cache, group.block_table, ctx.ctx_lens, nd,
                                            ctx.max_ctx_len, group.page_size, scale, window, out)
        if (ctx.n_tokens > nd and self.prefill_attention in ("auto", "tcgen05")
                and self._tcgen05_prefill_ok(qkv, out, num_heads, num_kv_heads, head_dim,
                                             group.page_size)):
            self.paged_attention_prefill_tcgen05(qkv, num_heads, num_kv_heads, head_dim, k_cache,
                                                 v_cache, ctx, group, scale, window, out)
        elif ctx.n_tokens > nd and mma and self.prefill_attention in ("auto", "mma", "tcgen05"):
            lib = self._attn_lib(head_dim)
            fn = getattr(lib, f"rv_paged_attention_prefill_mma_hd{head_dim}")
            self._check_attn(lib, head_dim, fn(
                _ptr(qkv), c_int(qkv.shape[1]), _ptr(k_cache), _ptr(v_cache),
                _ptr(group.block_table), c_int(group.max_blocks), _ptr(ctx.q_start),
                _ptr(ctx.ctx_lens), _ptr(out), c_int(nd), c_int(ctx.n_reqs - nd),
                c_int(ctx.max_q_len), c_int(num_heads), c_int(num_kv_heads),
                c_int(group.page_size), c_float(scale), win, self._stream()),
                "paged_attention_prefill_mma")
        elif ctx.n_tokens > nd:
            self._check(self.lib.rv_paged_attention_warp(
                _ptr(qkv), code, c_int(qkv.shape[1]), _ptr(k_cache), _ptr(v_cache),
                _ptr(group.block_table), c_int(group.max_blocks), _ptr(ctx.q_start),
                _ptr(ctx.ctx_lens), _ptr(ctx.token_req), _ptr(out), c_int(nd),
                c_int(ctx.n_tokens - nd), c_int(num_heads), c_int(num_kv_heads),
                c_int(head_dim), c_int(group.page_size), c_float(scale), win,
                self._stream()), "paged_attention")

    def paged_attention_decode(self, qkv, num_heads, num_kv_heads, head_dim, k_cache, v_cache,
                               block_table, ctx_lens, n_reqs, max_ctx_len, page_size, scale,
                               window, out, scratch=None):
        """Split-KV attention for requests [0, n_reqs) that bring one token each."""
        need = self.lib.rv_paged_attention_decode_scratch_bytes(
            c_int(n_reqs), c_int(num_heads), c_int(head_dim), c_int(max_ctx_len))
        if scratch is None:
            scratch = self._scratch_buffer(need, qkv.device)
        self._check(self.lib.rv_paged_attention_decode(
            _ptr(qkv), _code(qkv.dtype), c_int(qkv.shape[1]), _ptr(k_cache), _ptr(v_cache),
            _ptr(block_table), c_int(block_table.shape[1]), _ptr(ctx_lens), _ptr(out),
            _ptr(scratch), c_longlong(scratch.numel() * scratch.element_size()),
            c_int(n_reqs), c_int(max_ctx_len), c_int(num_heads), c_int(num_kv_heads),
            c_int(head_dim), c_int(page_size), c_float(scale), c_int(window if window else 0),
            self._stream()), "paged_attention_decode")

    def paged_attention_decode_mma(self, qkv, num_heads, num_kv_heads, head_dim, k_cache, v_cache,
                                   block_table, q_start, ctx_lens, n_reqs, max_ctx_len,
                                   page_size, scale, window, out, scratch=None):
        """Tensor-core split-KV attention (bfloat16) for requests [0, n_reqs) that bring one
        token each; the splits are combined by the merge kernel."""
        stream = (self.decode_kernel in ("stream", "auto") and head_dim == 64
                  and page_size in (8, 16, 32, 64))
        lib = self._attn_lib(head_dim)
        if stream and self.decode_kernel == "auto":
            items = (n_reqs * -(-max_ctx_len // 256) * num_kv_heads
                     * -(-(num_heads // num_kv_heads) // 16))
            stream = items >= self.stream_min_items
        if stream:
            split = getattr(lib, f"rv_paged_attention_decode_stream_split_hd{head_dim}")(
                c_int(n_reqs), c_int(max_ctx_len), c_int(num_heads), c_int(num_kv_heads),
                c_int(self._sm_count))
        else:
            split = self.decode_split
        need = self.lib.rv_paged_attention_decode_scratch_bytes(
            c_int(n_reqs), c_int(num_heads), c_int(head_dim), c_int(max_ctx_len * (256 // split)))
        if scratch is None:
            scratch = self._scratch_buffer(need, qkv.device)
        win = c_int(window if window else 0)
        if stream:
            fn = getattr(lib, f"rv_paged_attention_decode_stream_hd{head_dim}")
            self._check_attn(lib, head_dim, fn(
                _ptr(qkv), c_int(qkv.shape[1]), _ptr(k_cache), _ptr(v_cache),
                c_longlong(k_cache.shape[0] * k_cache.shape[1]), _ptr(block_table),
                c_int(block_table.shape[1]), _ptr(ctx_lens), _ptr(scratch),
                c_longlong(scratch.numel() * scratch.element_size()), c_int(n_reqs),
                c_int(max_ctx_len), c_int(num_heads), c_int(num_kv_heads), c_int(page_size),
                c_float(scale), win, c_int(split), c_int(self._sm_count),
                _ptr(self._gemm_status(qkv.device)), self._stream()),
                "paged_attention_decode_stream")
            self._check(self.lib.rv_paged_attention_merge(
                _ptr(scratch), _ptr(ctx_lens), _ptr(out), _code(out.dtype), c_int(n_reqs),
                c_int(max_ctx_len), c_int(num_heads), c_int(head_dim), win, c_int(split),
                self._stream()), "paged_attention_merge")
            return
        fn = getattr(lib, f"rv_paged_attention_decode_mma_hd{head_dim}")
        self._check_attn(lib, head_dim, fn(
            _ptr(qkv), c_int(qkv.shape[1]), _ptr(k_cache), _ptr(v_cache), _ptr(block_table),
            c_int(block_table.shape[1]), _ptr(q_start), _ptr(ctx_lens), _ptr(scratch),
            c_longlong(scratch.numel() * scratch.element_size()), c_int(n_reqs),
            c_int(max_ctx_len), c_int(num_heads), c_int(num_kv_heads), c_int(page_size),
            c_float(scale), win, c_int(split), self._stream()), "paged_attention_decode_mma")
        self._check(self.lib.rv_paged_attention_merge(
            _ptr(scratch), _ptr(ctx_lens), _ptr(out), _code(out.dtype), c_int(n_reqs),
            c_int(max_ctx_len), c_int(num_heads), c_int(head_dim), win, c_int(split),
            self._stream()), "paged_attention_merge")

    def paged_attention_general(self, qkv, num_heads, num_kv_heads, head_dim, k_cache, v_cache,
                                ctx, group, scale, window, out):
        """Every token through the one-warp-per-(token, head) kernel."""
        self._check(self.lib.rv_paged_attention_warp(
            _ptr(qkv), _code(qkv.dtype), c_int(qkv.shape[1]), _ptr(k_cache), _ptr(v_cache),
            _ptr(group.block_table), c_int(group.max_blocks), _ptr(ctx.q_start),
            _ptr(ctx.ctx_lens), _ptr(ctx.token_req), _ptr(out), c_int(0), c_int(ctx.n_tokens),
            c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(group.page_size),
            c_float(scale), c_int(window if window else 0), self._stream()), "paged_attention")

    # ---- gated short convolution -----------------------------------------------------

    def short_conv(self, proj, filt, in_bias, conv_bias, state, ctx, out):
        self._need(proj, "in_proj rows")
        self._need(filt, "filter", torch.float32)
        self._need(out, "short_conv output", proj.dtype)
        hidden, taps = filt.shape
        if proj.shape[1] != 3 * hidden:
            raise KernelError("short_conv: in_proj rows must be three times the filter's width")
        if state is not None:
            self._need(state, "convolution state", torch.float32)
        self._check(self.lib.rv_short_conv(
            _ptr(proj), _code(proj.dtype), _ptr(filt), _ptr(in_bias), _ptr(conv_bias),
            _ptr(state), _ptr(ctx.q_start), _ptr(ctx.state_slot), _ptr(ctx.start_pos), _ptr(out),
            c_int(ctx.n_reqs), c_int(ctx.max_q_len), c_int(hidden), c_int(taps),
            self._stream()), "short_conv")

    # ---- SwiGLU ----------------------------------------------------------------------

    def swiglu(self, gate_up, out):
        self._need(gate_up, "gate|up rows")
        self._need(out, "swiglu output", gate_up.dtype)
        if gate_up.shape[1] != 2 * out.shape[1]:
            raise KernelError("swiglu: input rows must be twice the output's width")
        self._check(self.lib.rv_swiglu(_ptr(gate_up), _ptr(out), _code(out.dtype),
                                       c_int(out.shape[0]), c_int(out.shape[1]), self._stream()),
                    "swiglu")

    # ---- sampling --------------------------------------------------------------------

    def argmax(self, logits):
        self._need(logits, "logits", torch.float32)
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
        scratch = torch.empty(logits.shape[0] * 64 * 2, dtype=torch.int32, device=logits.device)
        self._check(self.lib.rv_argmax(_ptr(logits), _ptr(out), _ptr(scratch),
                                       c_longlong(scratch.numel() * 4), c_int(logits.shape[0]),
                                       c_int(logits.shape[1]), self._stream()), "argmax")
        self.launches += 1
        return out

    def sample(self, logits, temperature, top_p, seed, counter):
        """Rows with temperature <= 0 are greedy."""
        self._need(logits, "logits", torch.float32)
        self._need(temperature, "temperatures", torch.float32)
        self._need(top_p, "top-p values", torch.float32)
        self._need(seed, "seeds", torch.int64)
        self._need(counter, "counters", torch.int64)
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
        self._check(self.lib.rv_sample(_ptr(logits), _ptr(temperature),
                                       _ptr(top_p), _ptr(seed), _ptr(counter), _ptr(out),
                                       c_int(logits.shape[0]), c_int(logits.shape[1]),
                                       self._stream()), "sample")
        return out
