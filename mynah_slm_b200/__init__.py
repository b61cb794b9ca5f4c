"""mynah_slm_b200: a small, whole Qwen3-dense engine for one B200 (sm_100a).

From a model folder (config.json + safetensors) to generated token ids on one
GPU: typed configuration and architecture registry, weights bound by tensor
name, layers put together from parts, a paged key/value cache with
per-sequence state, one step function, a generation loop, sampling, a command
line, and a trace-replay program. The kernels are hand-written CUDA for
sm_100a; there is no CPU fallback.
"""
__version__ = "0.1.0"

from .config.keys import ConfigError
from .registry import known_architectures, parse_config, read_config_folder, register_architecture

__all__ = ["ConfigError", "known_architectures", "parse_config", "read_config_folder", "register_architecture",
           "LLM", "Engine", "StepEntry", "SamplingParams", "__version__"]


def __getattr__(name):
    # the device-side half is imported on first use, so that configuration and
    # weight handling work where there is no GPU
    if name in ("LLM",):
        from .engine.api import LLM
        return LLM
    if name in ("Engine", "StepEntry"):
        from .engine import engine as _e
        return getattr(_e, name)
    if name == "SamplingParams":
        from .sampling.sampler import SamplingParams
        return SamplingParams
    raise AttributeError(name)
