"""A decode step as a list of operations that one resident kernel carries out.

`StepProgram` is the host side of `csrc/step_program.cu`.  The parts of a model describe
their share of a single-token step to it (`emit` methods in `rvllm_b200.parts`): products,
the elementwise operations between them, and calls of other kernels (attention) at which
the list is cut into stretches.  A stretch is one cooperative launch in which every SM
walks the list and the weights of the next products are copied while the current operation
still runs.  The program owns the buffers between its operations; the step's index arrays
(token ids, positions, slots) must live at fixed addresses, which is the case inside a
replayed step.

What flows between operations:

    Rows  bfloat16 rows [16, width] that a product reads.  Rows that came out of a norm carry
          the norm's division as a debt: the sums of squares by column slice, from which
          whoever consumes the product computes 1 / sqrt(mean square + eps) per token.
    Sums  a product's float32 partial sums [slices][16][n], which the next elementwise
          operation adds up as it reads them, times the debt of the rows that went in.

The reference runs the same step as some hundred cuBLAS calls and small kernels
(src/cuda/model.rs:560-790).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_void_p
from dataclasses import dataclass
from typing import Callable, List, Optional, Tuple

import torch

from ..errors import KernelError

TOKENS = 16          # token columns of the program's products
SLICE = 64           # columns per sum-of-squares slice


def enabled() -> bool:
    """RVLLM_STEP_PROGRAM=1 runs replayed steps of few tokens as a step program."""
    return os.environ.get("RVLLM_STEP_PROGRAM", "0") == "1"


@dataclass
class Debt:
    """A per-token factor 1 / sqrt(sum(ss) / dim + eps) still to be applied."""
    ss: torch.Tensor          # float32 [slices, 16]
    slices: int
    eps: float
    dim: int


@dataclass
class Rows:
    buf: torch.Tensor         # bfloat16 [16, width]
    width: int
    debt: Optional[Debt] = None


@dataclass
class Sums:
    part: torch.Tensor        # float32, at least [splits, 16, n]
    splits: int
    n: int
    debt: Optional[Debt] = None
    bias: Optional[torch.Tensor] = None       # float32 [n], added by the operation that reads the sums


@dataclass
class Embedding:
    """The stream's start: rows of the table, taken by the first norm's operation."""
    table: torch.Tensor
    scale: float
    token_ids: torch.Tensor


def _ptr(t):
    return c_void_p(0 if t is None else t.data_ptr())


class StepProgram:
    def __init__(self, ops, device, tokens: int, hidden: int):
        if not 1 <= tokens <= TOKENS:
            raise KernelError(f"a step program takes 1 to {TOKENS} tokens, got {tokens}")
        self.ops = ops
        self.lib = ops.lib
        self.device = device
        self.tokens = tokens
        self.hidden = hidden
        self.grid = int(self.lib.rv_step_program_grid())
        self.handle = None
        self.dry = True
        self.part_floats = 0
        self.part = None
        self.resid = None
        self._keep: List[torch.Tensor] = []
        self._plan: List[Tuple] = []           # ("run", first, count) | ("call", fn)
        self._open_from = 0
        self._n_ops = 0
        self.logits_out: Optional[torch.Tensor] = None
        self.stretches = 0

    # ---- building --------------------------------------------------------------------

    def begin(self, dry: bool) -> None:
        """Parts emit twice: a dry pass that only sizes the shared partial-sum buffer, then
        the pass that records the operations."""
        self.dry = dry
        self._keep = []
        self._plan = []
        self._open_from = 0
        self._n_ops = 0
        if not dry:
            self.part = torch.zeros(max(self.part_floats, 1), dtype=torch.float32, device=self.device)
            self.resid = torch.zeros((TOKENS, self.hidden), dtype=torch.float32, device=self.device)
            self.handle = c_void_p(self.lib.rv_step_program_create(
                _ptr(self.ops.status_word(self.device))))
            if not self.handle:
                raise KernelError("step program: out of memory")

    def _check(self, rc: int) -> None:
        if rc != 0:
            raise KernelError(self.lib.rv_last_error().decode())

    def buffer(self, width: int, dtype=torch.bfloat16) -> torch.Tensor:
        t = torch.zeros((TOKENS, width), dtype=dtype, device=self.device)
        self._keep.append(t)
        return t

    def rows_from(self, buf: torch.Tensor) -> Rows:
        return Rows(buf, buf.shape[1])

    def rows_from_width(self, width: int) -> Rows:
        """In the sizing pass, rows of a buffer that does not exist yet."""
        return Rows(None, width)

    def _count(self) -> None:
        self._n_ops += 1

    def gemm(self, rows: Rows, weight: torch.Tensor) -> Sums:
        """y = rows . weight^T, weight [n, width] bfloat16."""
        n, k = weight.shape
        if k != rows.width or weight.dtype != torch.bfloat16 or not weight.is_contiguous():
            raise KernelError("step program: a product needs a contiguous bfloat16 matrix as wide "
                              "as its rows")
        splits = int(self.lib.rv_step_program_splits(c_int(n), c_int(k), c_int(self.grid)))
        self.part_floats = max(self.part_floats, splits * TOKENS * n)
        if not self.dry:
            got = c_int(0)
            self._check(self.lib.rv_step_program_add_gemm(
                self.handle, _ptr(rows.buf), _ptr(weight), _ptr(self.part), c_int(self.tokens),
                c_int(n), c_int(k), ctypes.byref(got)))
            assert got.value == splits
            self._keep.append(weight)
        self._count()
        return Sums(self.part, splits, n, rows.debt)

    def _debt_args(self, debt: Optional[Debt]):
        if debt is None:
            return c_void_p(0), c_int(0), c_float(0.0), c_float(1.0)
        return _ptr(debt.ss), c_int(debt.slices), c_float(debt.eps), c_float(float(debt.dim))

    def add_norm(self, pending, weight: torch.Tensor, eps: float) -> Rows:
        """The stream takes `pending` (an `Embedding` or `Sums`); returns the stream times the
        norm's weight, owing the norm's division."""
        h = self.hidden
        slices = -(-h // SLICE)
        xw = ss = None
        if not self.dry:
            xw = self.buffer(h)
            ss = torch.zeros((slices, TOKENS), dtype=torch.float32, device=self.device)
            self._keep.append(ss)
            self._keep.append(weight)
            if isinstance(pending, Embedding):
                self._check(self.lib.rv_step_program_add_resid(
                    self.handle, _ptr(self.resid), c_void_p(0), c_int(0), c_void_p(0),
                    _ptr(pending.table), _ptr(pending.token_ids), c_float(pending.scale),
                    c_int(pending.table.shape[0]), _ptr(weight), _ptr(xw), _ptr(ss),
                    c_int(self.tokens), c_int(h)))
                self._keep.append(pending.table)
            else:
                if pending.n != h or pending.debt is not None:
                    raise KernelError("step program: only plain sums of the stream's width can "
                                      "be added to the stream")
                self._check(self.lib.rv_step_program_add_resid(
                    self.handle, _ptr(self.resid), _ptr(pending.part), c_int(pending.splits),
                    _ptr(pending.bias), c_void_p(0), c_void_p(0), c_float(1.0), c_int(0),
                    _ptr(weight), _ptr(xw), _ptr(ss), c_int(self.tokens), c_int(h)))
        self._count()
        return Rows(xw, h, Debt(ss, slices, eps, h))

    def conv(self, sums: Sums, filt, in_bias, conv_bias, state, ctx) -> Rows:
        hidden, taps = filt.shape
        out = None
        if not self.dry:
            out = self.buffer(hidden)
            d = self._debt_args(sums.debt)
            self._check(self.lib.rv_step_program_add_conv(
                self.handle, _ptr(sums.part), c_int(sums.splits), d[0], d[1], d[2], d[3],
                _ptr(filt), _ptr(in_bias), _ptr(conv_bias), _ptr(state), _ptr(ctx.state_slot),
                _ptr(ctx.start_pos), _ptr(out), c_int(self.tokens), c_int(hidden), c_int(taps)))
            self._keep += [t for t in (filt, in_bias, conv_bias) if t is not None]
        self._count()
        return Rows(out, hidden)

    def qk(self, sums: Sums, num_heads, num_kv_heads, head_dim, q_weight, k_weight, qk_eps, table,
           positions, slot_mapping, k_cache, v_cache) -> Optional[torch.Tensor]:
        """Query rows [16, (heads + 2 kv heads) * head_dim] (the key and value columns stay
        unwritten); keys and values go to their pages."""
        out = None
        if not self.dry:
            out = self.buffer(sums.n)
            cos, sin = table if table is not None else (None, None)
            d = self._debt_args(sums.debt)
            self._check(self.lib.rv_step_program_add_qk(
                self.handle, _ptr(sums.part), c_int(sums.splits), d[0], d[1], d[2], d[3],
                c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), _ptr(q_weight),
                _ptr(k_weight), c_float(qk_eps), _ptr(cos), _ptr(sin), _ptr(positions),
                _ptr(slot_mapping), _ptr(k_cache), _ptr(v_cache), _ptr(out), c_int(self.tokens)))
            self._keep += [t for t in (q_weight, k_weight, cos, sin) if t is not None]
        self._count()
        return out

    def swiglu(self, sums: Sums, ffn: int) -> Rows:
        out = None
        if not self.dry:
            out = self.buffer(ffn)
            d = self._debt_args(sums.debt)
            self._check(self.lib.rv_step_program_add_swiglu(
                self.handle, _ptr(sums.part), c_int(sums.splits), d[0], d[1], d[2], d[3],
                _ptr(out), c_int(self.tokens), c_int(ffn)))
        self._count()
        return Rows(out, ffn)

    def logits(self, sums: Sums) -> None:
        if not self.dry:
            self.logits_out = self.buffer(sums.n, torch.float32)
            d = self._debt_args(sums.debt)
            self._check(self.lib.rv_step_program_add_logits(
                self.handle, _ptr(sums.part), c_int(sums.splits), d[0], d[1], d[2], d[3],
                _ptr(self.logits_out), c_int(self.tokens), c_int(sums.n)))
        self._count()

    def call(self, fn: Callable[[], None]) -> None:
        """Cut the list here and run `fn` (which launches other kernels on the current stream)
        between the two stretches."""
        self._close_stretch()
        self._plan.append(("call", fn))

    def _close_stretch(self) -> None:
        if self._n_ops > self._open_from:
            self._plan.append(("run", self._open_from, self._n_ops - self._open_from))
            self._open_from = self._n_ops

    def finish(self) -> None:
        self._close_stretch()
        self._check(self.lib.rv_step_program_finish(self.handle))
        self.stretches = sum(1 for p in self._plan if p[0] == "run")

    # ---- running ---------------------------------------------------------------------

    def run(self) -> torch.Tensor:
        """Carry out the step on torch's current stream; float32 logits [16, vocab] (rows
        past the step's tokens are not meaningful)."""
        stream = c_void_p(torch.cuda.current_stream().cuda_stream)
        for p in self._plan:
            if p[0] == "run":
                self._check(self.lib.rv_step_program_run(self.handle, c_int(p[1]), c_int(p[2]), stream))
                self.ops.launches += 1
            else:
                p[1]()
        return self.logits_out

    def reset(self) -> None:
        """After a launch that recorded a failed wait: clear the meeting counters."""
        self._check(self.lib.rv_step_program_reset(
            self.handle, c_void_p(torch.cuda.current_stream().cuda_stream)))

    def __del__(self):
        h, self.handle = getattr(self, "handle", None), None
        if h:
            try:
                self.lib.rv_step_program_destroy(h)
            except Exception:
                pass
