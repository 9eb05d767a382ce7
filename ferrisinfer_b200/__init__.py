"""ferrisinfer_b200: a small, whole inference engine for the Qwen2 dense decoder on one B200.

    from ferrisinfer_b200 import Engine, SamplingParams
    engine = Engine("path/to/model")                      # config.json + model.safetensors
    out = engine.generate([[1, 2, 3]], SamplingParams.greedy(max_new_tokens=16))

Importing the package needs neither a GPU nor the compiled kernels; creating an ``Engine`` does.
"""

from .config import Qwen2Config, register_architecture, registered_architectures
from .engine.scheduler import FinishReason, SchedulerConfig
from .errors import (CacheError, ConfigError, FerrisError, KernelError, OutOfPages, SchedulerError, UnsupportedError,
                     WeightFileError, WeightLoadError)
from .sampling.params import SamplingParams

__version__ = "0.1.0"


def __getattr__(name):
    if name in ("Engine", "generate", "GenerationOutput", "TokenSample"):
        from .engine import engine as _engine

        return getattr(_engine, name)
    raise AttributeError(name)
