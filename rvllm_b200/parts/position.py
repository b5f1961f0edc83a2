"""Position encodings for the attention mixer.

"rope": rotate-half rotation by angle pos * theta^(-2j/head_dim) for the pair
(j, j + head_dim/2) (the reference's `rope_cos_sin` and `rope_apply`,
src/model.rs:224-263).  Frequencies, angles, cosines and sines are float32, as in the
reference; the table is built once per (theta, head_dim, max_position) and indexed by
absolute position in the kernel, where the reference rebuilds it for every forward
call (src/model.rs:487-492).
"""
from __future__ import annotations

import torch

from .base import PositionEncoding, register_position
from .spec import PositionSpec

_TABLES = {}


class Rope(PositionEncoding):
    def __init__(self, spec: PositionSpec, device):
        if spec.head_dim % 2:
            raise ValueError(f"rope needs an even head size, got {spec.head_dim}")
        self.spec = spec
        key = (spec.theta, spec.head_dim, spec.max_position, str(device))
        if key not in _TABLES:
            half = spec.head_dim // 2
            j = torch.arange(half, dtype=torch.float32)
            freq = torch.pow(torch.tensor(spec.theta, dtype=torch.float32),
                             -2.0 * j / spec.head_dim)
            pos = torch.arange(spec.max_position, dtype=torch.float32).unsqueeze(1)
            angles = pos * freq.unsqueeze(0)
            _TABLES[key] = (angles.cos().to(device).contiguous(),
                            angles.sin().to(device).contiguous())
        self.cos, self.sin = _TABLES[key]

    def rotation_table(self):
        return self.cos, self.sin


class NoPosition(PositionEncoding):
    def __init__(self, spec: PositionSpec, device):
        self.spec = spec

    def rotation_table(self):
        return None


register_position("rope", Rope)
register_position("none", NoPosition)
