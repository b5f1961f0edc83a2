"""Plain references of the kernels, one function per kernel, on ordinary torch tensors.

Two uses.  The GPU tests compare each CUDA kernel with the function of the same name
here, at sizes other than the engine's.  And because `PlainOps` has the interface of
the product's kernel set, the CPU tests can drive the engine's host side (cache
manager, batch packing, step function, scheduler) through it without a GPU.  It is a
test double: the product never imports it and has no CPU path of its own.

Each function works in float32 (float64 where noted) whatever the storage dtype, and
loops over requests and tokens in the obvious way.
"""
from __future__ import annotations

import math

import torch


def _f(t):
    return t.to(torch.float32)


class PlainOps:
    name = "plain"

    # ---- embedding -------------------------------------------------------------------
    def embed(self, table, ids, out, scale=None):
        x = _f(table[ids.long()])
        out.copy_(x if scale is None else x * scale)

    # ---- residual add + RMSNorm ------------------------------------------------------
    def add_rmsnorm(self, resid, delta, weight, eps, out, rows=None):
        if resid is None:
            x = _f(delta)
        elif rows is None:
            if delta is not None:
                resid.add_(_f(delta))
            x = resid
        else:
            x = resid[rows.long()]
            if delta is not None:
                x = x + _f(delta[rows.long()])
        rms = (x.pow(2).mean(dim=-1, keepdim=True) + eps).sqrt()
        out.copy_((x / rms * _f(weight)).to(out.dtype))

    # ---- matrix product --------------------------------------------------------------
    def linear(self, x, w, bias=None, out_dtype=None):
        y = _f(x) @ _f(w).t()
        if bias is not None:
            y = y + _f(bias)
        return y.to(out_dtype or x.dtype)

    def new_rows(self, n, width, dtype, device):
        return torch.empty((n, width), dtype=dtype, device=device)

    def linear_qk_norm_rope_write(self, x, w_qkv, num_heads, num_kv_heads, head_dim, q_weight,
                                  k_weight, eps, table, positions, slot_mapping, k_cache, v_cache,
                                  out_dtype=None):
        qkv = self.linear(x, w_qkv, out_dtype=out_dtype or x.dtype)
        self.qk_norm_rope_write(qkv, num_heads, num_kv_heads, head_dim, q_weight, k_weight, eps,
                                table, positions, slot_mapping, k_cache, v_cache)
        return qkv

    def add_bias(self, x, bias):
        x.copy_((_f(x) + _f(bias)).to(x.dtype))

    # ---- q/k norm + rotation + cache write -------------------------------------------
    def qk_norm_rope_write(self, qkv, num_heads, num_kv_heads, head_dim, q_weight, k_weight,
                           eps, table, positions, slot_mapping, k_cache, v_cache):
        n = qkv.shape[0]
        hd, half = head_dim, head_dim // 2
        qd, kd = num_heads * hd, num_kv_heads * hd

        def norm_rotate(x, w):          # x: [n, heads, hd] float32
            if w is not None:
                x = x / (x.pow(2).mean(dim=-1, keepdim=True) + eps).sqrt() * _f(w)
            if table is not None:
                cos = table[0][positions.long()].unsqueeze(1)
                sin = table[1][positions.long()].unsqueeze(1)
                a, b = x[..., :half], x[..., half:]
                x = torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)
            return x

        q = norm_rotate(_f(qkv[:, :qd]).reshape(n, num_heads, hd), q_weight)
        qkv[:, :qd] = q.reshape(n, qd).to(qkv.dtype).clone()
        if num_kv_heads:
            k = norm_rotate(_f(qkv[:, qd:qd + kd]).reshape(n, num_kv_heads, hd), k_weight)
            v = qkv[:, qd + kd:qd + 2 * kd].reshape(n, num_kv_heads, hd)
            kc = k_cache.view(-1, num_kv_heads, hd)
            vc = v_cache.view(-1, num_kv_heads, hd)
            for t in range(n):
                s = int(slot_mapping[t])
                if s >= 0:
                    kc[s] = k[t].to(kc.dtype)
                    vc[s] = v[t].to(vc.dtype)

    # ---- attention over the pages ----------------------------------------------------
    def paged_attention(self, qkv, num_heads, num_kv_heads, head_dim, k_cache, v_cache,
                        ctx, group, scale, window, out):
        hd = head_dim
        G = num_heads // num_kv_heads
        ps = group.page_size
        q_start = ctx.q_start.tolist()
        ctx_lens = ctx.ctx_lens.tolist()
        for r in range(ctx.n_reqs):
            clen = ctx_lens[r]
            a, b = q_start[r], q_start[r + 1]
            if clen == 0:
                out[a:b] = 0
                continue
            table = group.block_table[r].tolist()
            for t in range(a, b):
                p = clen - (b - a) + (t - a)
                lo = 0 if window is None else max(0, p - window + 1)
                keys = list(range(lo, p + 1))
                idx = torch.tensor([table[j // ps] * ps + j % ps for j in keys])
                k = _f(k_cache.view(-1, num_kv_heads, hd)[idx])      # [keys, kv, hd]
                v = _f(v_cache.view(-1, num_kv_heads, hd)[idx])
                q = _f(qkv[t, :num_heads * hd]).reshape(num_heads, hd)
                for h in range(num_heads):
                    g = h // G
                    s = (k[:, g] @ q[h]) * scale
                    pr = torch.softmax(s, dim=0)
                    out[t, h * hd:(h + 1) * hd] = (pr @ v[:, g]).to(out.dtype)

    # ---- gated short convolution -----------------------------------------------------
    def short_conv(self, proj, filt, in_bias, conv_bias, state, ctx, out):
        hidden, taps = filt.shape
        q_start = ctx.q_start.tolist()
        slots = ctx.state_slot.tolist()
        start_pos = ctx.start_pos.tolist()
        p = _f(proj)
        if in_bias is not None:
            p = p + _f(in_bias)
        B, C, X = p[:, :hidden], p[:, hidden:2 * hidden], p[:, 2 * hidden:]
        bx = B * X
        for r in range(ctx.n_reqs):
            a, b = q_start[r], q_start[r + 1]
            slot = slots[r]
            if taps > 1 and slot >= 0 and start_pos[r] > 0:
                old = state[slot].clone()
            else:
                old = torch.zeros(taps - 1, hidden)
            rows = torch.cat([old, bx[a:b]], dim=0)
            n = b - a
            conv = torch.zeros(n, hidden)
            for k in range(taps):
                conv = conv + rows[k:k + n] * filt[:, k]
            if conv_bias is not None:
                conv = conv + _f(conv_bias)
            out[a:b] = (C[a:b] * conv).to(out.dtype)
            if taps > 1 and slot >= 0:
                state[slot] = rows[n:]

    # ---- SwiGLU activation -----------------------------------------------------------
    def swiglu(self, gate_up, out):
        f = out.shape[1]
        g, u = _f(gate_up[:, :f]), _f(gate_up[:, f:])
        out.copy_((g / (1.0 + torch.exp(-g)) * u).to(out.dtype))

    # ---- sampling --------------------------------------------------------------------
    def argmax(self, logits):
        out = torch.zeros(logits.shape[0], dtype=torch.int32)
        for m in range(logits.shape[0]):
            best, best_v = 0, float("-inf")
            for i, v in enumerate(logits[m].tolist()):
                if v > best_v:
                    best, best_v = i, v
            out[m] = best
        return out

    def sample(self, logits, temperature, top_p, seed, counter):
        out = torch.zeros(logits.shape[0], dtype=torch.int32)
        for m in range(logits.shape[0]):
            out[m] = sample_row(logits[m], float(temperature[m]), float(top_p[m]),
                                int(seed[m]), int(counter[m]))
        return out


# ---- the sampler's definition, restated --------------------------------------------

MASK64 = (1 << 64) - 1


def uniform(seed: int, counter: int) -> float:
    """The draw for (seed, counter): a splitmix64 finaliser over seed + (counter + 1) *
    the golden-ratio increment; the top 24 bits make a float in [0, 1)."""
    z = (seed + (counter + 1) * 0x9E3779B97F4A7C15) & MASK64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
    z = z ^ (z >> 31)
    return (z >> 40) / float(1 << 24)


def sample_row(logits, temperature: float, top_p: float, seed: int, counter: int) -> int:
    """Temperature and nucleus sampling of one row, in float64.

    temperature <= 0: first maximum.  Else p = softmax(logits / T); the nucleus is the
    set {p_i >= tau} for the largest tau whose set has mass >= top_p (ties with the last
    kept token are kept); the token is the first, in index order, whose cumulative
    kept mass reaches u * kept mass.
    """
    if temperature <= 0:
        return int(PlainOps().argmax(logits.unsqueeze(0))[0])
    z = logits.double() / temperature
    p = torch.exp(z - z.max())
    if top_p < 1.0:
        total = p.sum()
        order = torch.argsort(p, descending=True, stable=True)
        cum = torch.cumsum(p[order], 0)
        hit = (cum >= top_p * total).nonzero()
        cut = int(hit[0]) if len(hit) else len(p) - 1
        p = torch.where(p >= p[order[cut]], p, torch.zeros_like(p))
    r = uniform(seed, counter) * float(p.sum())
    cum = torch.cumsum(p, 0)
    hit = ((cum >= r) & (p > 0)).nonzero()
    return int(hit[0]) if len(hit) else int((p > 0).nonzero()[-1])
