"""The random-weights mode: a model folder (config.json, model.safetensors) from a
configuration and a seed.

Distributions: matrices and the embedding N(0, 0.02); convolution filters N(0, 0.2);
norm weights 1 + N(0, 0.05); biases N(0, 0.02); a declaration may carry a mean and a
standard deviation of its own instead (`ParamDecl.mean`, `.std`).  Each tensor draws from its own
generator, keyed by the seed and the tensor's name, so a tensor's values do not
depend on which other tensors the model has.  Values are stored in the
configuration's `torch_dtype`.  (The reference has no such mode; its tests build
tiny models in memory, src/model.rs:981-1055, and write temporary GGUF files,
src/weights.rs:684-700.)
"""
from __future__ import annotations

import json
import os
import zlib
from typing import Dict

import torch

from ..config.registry import architecture
from ..parts.model import param_decls
from ..parts.spec import ParamDecl
from .loader import SINGLE
from .safetensors_io import write_streamed

_STD = {"linear": 0.02, "embedding": 0.02, "conv": 0.2, "norm": 0.05, "bias": 0.02}
_TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32,
                 "float16": torch.float16}


def random_tensor(name: str, decl: ParamDecl, seed: int, dtype: torch.dtype) -> torch.Tensor:
    gen = torch.Generator(device="cpu")
    gen.manual_seed((zlib.crc32(name.encode()) << 20) ^ (seed & 0xFFFFFFFFFFFF))
    if decl.integer:
        return torch.randint(0, 2 ** 15, decl.shape, generator=gen, dtype=torch.int32)
    if decl.init == "zeros":
        return torch.zeros(decl.shape, dtype=dtype)
    if decl.init not in _STD and (decl.init != "normal" or decl.std is None):
        raise ValueError(f"tensor {name!r}: unknown initialisation {decl.init!r} (a named "
                         f"one of {sorted(_STD)} or zeros, or \"normal\" with its own std)")
    std = decl.std if decl.std is not None else _STD[decl.init]
    mean = decl.mean if decl.mean is not None else (1.0 if decl.init == "norm" else 0.0)
    t = torch.randn(decl.shape, generator=gen, dtype=torch.float32) * std
    if mean != 0.0:
        t = t + mean
    return t.to(dtype)


def random_tensors(config, seed: int) -> Dict[str, torch.Tensor]:
    spec = architecture(config.architecture).build_spec(config)
    dtype = _TORCH_DTYPES[config.torch_dtype]
    return {n: random_tensor(n, d, seed, dtype) for n, d in param_decls(spec).items()}


def write_random_model(folder: str, config, seed: int) -> str:
    """Write config.json and model.safetensors for `config` into `folder`."""
    os.makedirs(folder, exist_ok=True)
    spec = architecture(config.architecture).build_spec(config)
    dtype = _TORCH_DTYPES[config.torch_dtype]
    decls = param_decls(spec)

    layout = [(n, tuple(d.shape), torch.int32 if d.integer else dtype)
              for n, d in decls.items()]
    write_streamed(os.path.join(folder, SINGLE), layout,
                   lambda n: random_tensor(n, decls[n], seed, dtype),
                   metadata={"format": "pt", "seed": str(seed)})
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config.to_dict(), f, indent=2)
    return folder
