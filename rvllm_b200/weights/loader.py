"""Weights by tensor name, checked against what the model declares.

Every tensor the `ModelSpec` needs is looked up by its name, its shape compared with
the declared one, and all problems reported together in one `WeightsError`: missing
tensors, unexpected tensors, wrong shapes.  (The reference stops at the first:
`GGUF tensor "x" has shape [..], expected [..]`, src/weights.rs:322-331; a missing
tensor is named, src/weights.rs:750-753.)

Precision on the device.  With compute dtype bfloat16 a floating tensor is kept in
bfloat16 (float16 is narrowed to it) except that a tensor stored in 32 bits stays in
32 bits; with compute dtype float32 everything is widened to float32, which is exact
for bfloat16 and float16 files.  Integer tables become int32.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List

import torch

from ..errors import WeightsError
from ..parts.model import param_decls
from ..parts.spec import ModelSpec
from .safetensors_io import SafetensorsFile

SINGLE = "model.safetensors"
INDEX = "model.safetensors.index.json"


def open_folder(folder: str) -> List[SafetensorsFile]:
    single = os.path.join(folder, SINGLE)
    if os.path.isfile(single):
        return [SafetensorsFile(single)]
    index = os.path.join(folder, INDEX)
    if os.path.isfile(index):
        with open(index) as f:
            files = sorted(set(json.load(f)["weight_map"].values()))
        return [SafetensorsFile(os.path.join(folder, name)) for name in files]
    raise WeightsError(f"{folder}: no {SINGLE} (nor {INDEX}) in this model folder")


def device_dtype(stored: torch.dtype, compute: torch.dtype, integer: bool) -> torch.dtype:
    if integer:
        return torch.int32
    if compute == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return compute


def load_tensors(folder: str, spec: ModelSpec, compute_dtype: torch.dtype,
                 device) -> Dict[str, torch.Tensor]:
    """name -> tensor on `device`, for every tensor `spec` declares."""
    decls = param_decls(spec)
    files = open_folder(folder)
    where = {}
    for f in files:
        for name in f.names():
            where[name] = f
    missing = sorted(n for n in decls if n not in where)
    unexpected = sorted(n for n in where if n not in decls)
    wrong = []
    for name, decl in decls.items():
        if name not in where:
            continue
        shape = where[name].shape(name)
        if shape != tuple(decl.shape) and shape not in decl.alt_shapes:
            wrong.append(f"{name} has {list(shape)}, expected {list(decl.shape)}")
        elif decl.integer == where[name].dtype(name).is_floating_point:
            wrong.append(f"{name} is {where[name].dtype(name)}, expected "
                         f"{'an integer' if decl.integer else 'a floating'} type")
    if missing or unexpected or wrong:
        lines = [f"{folder}: the tensor file does not fit {spec.architecture}:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(sorted(wrong)))
        raise WeightsError("\n".join(lines))
    out = {}
    for name, decl in decls.items():
        t = where[name].tensor(name)
        target = device_dtype(t.dtype, compute_dtype, decl.integer)
        t = t.to(device=device, dtype=target).reshape(decl.shape)
        out[name] = t.contiguous() if t.device.type != "cpu" else t.clone()
    return out
