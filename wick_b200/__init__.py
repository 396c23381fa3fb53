"""wick_b200: a small model library with generation for one NVIDIA B200.

Everything between a request's token ids and its next token for the Qwen3 dense
decoder: typed configuration and architecture registry, safetensors weights (or
seeded random ones), layers assembled from registered parts, a paged cache with
a slot per sequence, one step function for batches of unequal sequences, a
generation loop, sampling, and hand-written CUDA kernels for sm_100a.

    import wick_b200 as wick
    eng = wick.Engine.from_dir("model-dir", dtype="bfloat16", max_tokens=8192)
    out = wick.generate(eng, [[1, 2, 3], [4, 5]], wick.GenOptions(max_tokens=16,
                        sampler=wick.SamplerConfig.greedy()))
"""
from .config.base import (ConfigError, ModelConfig, architecture_names, config_from_json, get_architecture,
                          load_config, register_architecture, Architecture)
from .config.qwen3 import Qwen3Config
from .models import qwen3 as _qwen3  # registers the architecture  # noqa: F401
from .models.model import Model
from .models.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .sampling.sampler import Rng, Sampler, SamplerConfig
from .engine.generate import GenOptions, GenResult, generate
from .weights.loader import WeightError, load_weights
from .weights.random_init import write_random_model
from .weights.safetensors_io import SafeTensorsDir, SafeTensorsError, write_safetensors


def __getattr__(name):
    # The engine needs CUDA; import it on first use so that configuration,
    # weights and the cache bookkeeping stay usable without a GPU.
    if name in ("Engine", "parse_dtype"):
        from .engine import engine as _e
        return getattr(_e, name)
    raise AttributeError(name)


__all__ = ["Architecture", "ConfigError", "Engine", "GenOptions", "GenResult", "LayerSpec", "Model", "ModelConfig",
           "ModelSpec", "PartSpec", "Qwen3Config", "Rng", "SafeTensorsDir", "SafeTensorsError", "Sampler",
           "SamplerConfig", "ScheduleEntry", "WeightError", "architecture_names", "config_from_json", "generate",
           "get_architecture", "load_config", "load_weights", "register_architecture", "write_random_model",
           "write_safetensors"]
