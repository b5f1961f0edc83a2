"""The allocation-free decode attention entry point, called through its exported C
symbol, against the ordinary entry point.

`rv_paged_attention_decode_static` is for users of the native library who cannot
allocate device memory (see rvllm_b200/csrc/attention_decode_static.h): it keeps the
split partial results in a fixed 4 MiB array inside the library.  This test loads the
library with ctypes, as such a user would, and checks that two calls in a row (with
different inputs, so that the second call finds the first call's leftovers in the array)
give what `rv_paged_attention_decode` gives with a caller-owned scratch buffer, and that
a batch too large for the array is refused with a message instead of running.

The file's name makes pytest collect it last, so a run that stops at the first failure
has already run every other test.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr(t):
    return c_void_p(t.data_ptr())


def _case(seed, dtype, n_reqs, ctx_lens, nh, nkv, hd, ps):
    g = torch.Generator().manual_seed(seed)
    blocks = [-(-c // ps) for c in ctx_lens]
    pages = sum(blocks) + 2
    perm = torch.randperm(pages, generator=g).tolist()
    table = torch.full((n_reqs, max(blocks)), -1, dtype=torch.int32)
    k = 0
    for r in range(n_reqs):
        for b in range(blocks[r]):
            table[r, b] = perm[k]
            k += 1
    mk = lambda *s: torch.randn(*s, generator=g).to(dtype).cuda()
    return dict(q=mk(n_reqs, (nh + 2 * nkv) * hd), k=mk(pages, ps, nkv, hd),
                v=mk(pages, ps, nkv, hd), table=table.cuda(),
                ctx=torch.tensor(ctx_lens, dtype=torch.int32).cuda())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_scratch_matches_caller_scratch_twice(dtype):
    from rvllm_b200.kernels import cuda_ops
    ops = cuda_ops()
    lib = ctypes.CDLL(ops.library_path)         # the exported C symbols, nothing else
    lib.rv_last_error.restype = ctypes.c_char_p
    lib.rv_paged_attention_decode_static_need.restype = c_longlong
    nh, nkv, hd, ps = 6, 2, 64, 16
    code = 0 if dtype == torch.float32 else 1
    scale = 1.0 / math.sqrt(hd)
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    calls = [(21, [700, 1, 300, 257, 64]), (22, [90, 1025, 513, 16, 255])]
    for seed, ctx_lens in calls:
        n = len(ctx_lens)
        c = _case(seed, dtype, n, ctx_lens, nh, nkv, hd, ps)
        want = torch.empty(n, nh * hd, dtype=dtype, device="cuda")
        ops.paged_attention_decode(c["q"], nh, nkv, hd, c["k"], c["v"], c["table"], c["ctx"], n,
                                   max(ctx_lens), ps, scale, None, want)
        got = torch.full((n, nh * hd), float("nan"), dtype=dtype, device="cuda")
        rc = lib.rv_paged_attention_decode_static(
            _ptr(c["q"]), c_int(code), c_int(c["q"].shape[1]), _ptr(c["k"]), _ptr(c["v"]),
            _ptr(c["table"]), c_int(c["table"].shape[1]), _ptr(c["ctx"]), _ptr(got), c_int(n),
            c_int(max(ctx_lens)), c_int(nh), c_int(nkv), c_int(hd), c_int(ps), c_float(scale),
            c_int(0), stream)
        assert rc == 0, lib.rv_last_error().decode()
        torch.cuda.synchronize()
        tol = dict(atol=3e-6, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
        assert torch.isfinite(got.float()).all()
        assert torch.allclose(got.float(), want.float(), **tol)
        assert torch.equal(got, want)            # the same kernels in the same order


def test_static_scratch_refuses_what_does_not_fit():
    from rvllm_b200.kernels import cuda_ops
    ops = cuda_ops()
    lib = ctypes.CDLL(ops.library_path)
    lib.rv_last_error.restype = ctypes.c_char_p
    lib.rv_paged_attention_decode_static_need.restype = c_longlong
    limit = 4 << 20
    assert lib.rv_paged_attention_decode_static_need(c_int(8), c_int(32), c_int(64),
                                                     c_int(4096)) <= limit
    assert lib.rv_paged_attention_decode_static_need(c_int(64), c_int(32), c_int(64),
                                                     c_int(4096)) > limit
    dummy = torch.zeros(16, device="cuda")
    rc = lib.rv_paged_attention_decode_static(
        _ptr(dummy), c_int(1), c_int(64 * 48), _ptr(dummy), _ptr(dummy), _ptr(dummy), c_int(256),
        _ptr(dummy), _ptr(dummy), c_int(64), c_int(4096), c_int(32), c_int(8), c_int(64),
        c_int(16), c_float(0.125), c_int(0), c_void_p(0))
    assert rc != 0
    msg = lib.rv_last_error().decode()
    assert "fixed array" in msg and "4194304" in msg
