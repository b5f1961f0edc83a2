"""Error types shared by the package."""


class ConfigError(ValueError):
    """A config.json that cannot describe a model: a missing or mistyped key, or sizes
    that contradict each other."""


class WeightsError(ValueError):
    """A tensor file that does not fit the model: lists every missing tensor, every
    unexpected tensor and every wrong shape in one message."""


class KernelError(RuntimeError):
    """A kernel refused its arguments, or the native library is missing."""


class CacheError(RuntimeError):
    """The cache manager was asked for something it cannot give."""


class RequestError(ValueError):
    """A request the scheduler will never be able to run
    (the reference's RequestError, src/engine.rs:151-177)."""
