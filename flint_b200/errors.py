"""Error categories of the engine (the reference keeps one enum with the same
categories: crates/thuban_error/src/lib.rs:5-21)."""


class FlintError(Exception):
    """Base class of every error the engine raises on purpose."""


class ConfigError(FlintError, ValueError):
    """config.json is missing a key, has a wrong type or an unsupported value."""


class WeightError(FlintError, ValueError):
    """A checkpoint does not match the model: missing, unexpected or mis-shaped tensors."""


class ModelError(FlintError, RuntimeError):
    """A request to the model that it cannot serve (bad batch, unsupported size)."""


class CacheError(FlintError, RuntimeError):
    """The cache manager cannot serve a request (no pages, no slot, context limit)."""


class KernelError(FlintError, RuntimeError):
    """The CUDA extension is missing, failed to build, or refused a size."""
