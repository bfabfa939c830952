"""flint_b200: a small, whole LLM inference engine for one NVIDIA B200.

Everything between a request's tokens and its next token: typed configuration and an
architecture registry, safetensors weights by name, layers composed from parts, a
paged cache with block tables, one step function for mixed batches, a scheduler with
sampling, and hand-written sm_100a kernels underneath.
"""
from . import parts as _parts  # noqa: F401  (registers built-in parts)
from . import models as _models  # noqa: F401  (registers built-in architectures)
from .errors import CacheError, ConfigError, FlintError, KernelError, ModelError, WeightError  # noqa: F401

__version__ = "0.1.0"
