"""clockwork_b200: a single-GPU inference engine for the Qwen2.5 dense decoder on NVIDIA B200,
with the feature set of jasonjesuraja06/clockwork's engine (paged KV cache, radix prefix
cache, continuous batching with chunked prefill, greedy/temperature sampling)."""

__version__ = "0.1.0"

from . import models  # noqa: F401  (registers the architectures)
from .config import EngineConfig

__all__ = ["EngineConfig", "__version__"]
