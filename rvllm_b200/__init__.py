"""rvllm_b200: a small, whole LFM2 inference engine for one NVIDIA B200."""
from . import models  # noqa: F401  (registers the architectures)
from . import parts  # noqa: F401  (registers the built-in parts)
from .engine import GenerateOptions, Generator
from .sampling import SamplingParams

__version__ = "0.1.0"
__all__ = ["Generator", "GenerateOptions", "SamplingParams"]
