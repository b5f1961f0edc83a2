"""From a model folder to a runnable model: config.json picks the architecture, the
architecture builds the `ModelSpec`, the loader reads the declared tensors, and the
generic `Model` is put together from the registered parts.  (The reference:
`Model::load`, src/weights.rs:300-448, then `Runtime::new`, src/runtime.rs:24-77.)
"""
from __future__ import annotations

import torch

from ..cache import CacheManager
from ..config.registry import architecture, load_config
from ..parts.model import Model
from ..weights.loader import load_tensors

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
          "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"compute dtype must be bfloat16 or float32, got {name}")
        return name
    if name not in DTYPES:
        raise ValueError(f"unknown dtype {name!r} (known: bfloat16, float32)")
    return DTYPES[name]


def load_model(folder: str, dtype="bfloat16", device="cuda", ops=None):
    """(model, config) for the folder.  `ops` defaults to the CUDA kernel set, whose
    import fails loudly when the native library cannot be built or loaded."""
    dtype = parse_dtype(dtype)
    config = load_config(folder)
    spec = architecture(config.architecture).build_spec(config)
    if ops is None:
        from ..kernels import cuda_ops
        ops = cuda_ops()
    tensors = load_tensors(folder, spec, dtype, device)
    model = Model(spec, tensors, ops, dtype)
    del tensors
    return model, config


def make_cache(model: Model, page_size: int, num_pages: int, max_requests: int) -> CacheManager:
    return CacheManager(model.cache_needs(), [c.cache_of for c in model.spec.order],
                        page_size, num_pages, max_requests, dtype=model.dtype,
                        device=model.device)
