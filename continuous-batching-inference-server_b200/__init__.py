"""A single-GPU inference engine for NVIDIA B200 (sm_100a): TinyGPT (GPT-2 style) from a model
folder to generated tokens, with a paged cache, one step function for mixed batches, a
continuous-batching scheduler and hand-written CUDA kernels.

    import cbis_b200 as cb
    engine = cb.Engine("model_dir", dtype="bfloat16")
    outputs = engine.generate([[1, 2, 3]], cb.SamplingParams(max_new_tokens=16))
"""
from .config import (ConfigError, GPT2Config, LayerSpec, ModelSpec, PartSpec, config_from_dict,
                     known_architectures, load_config, register_architecture)
from .weights import InitScheme, WeightsError, write_model_folder

__version__ = "0.1.0"


def __getattr__(name):
    # The engine side imports lazily, so that configuration and weights work without building anything.
    if name in ("Engine", "SamplingParams", "build_model"):
        from .engine import api
        return getattr(api, name)
    if name in ("Model", "load_model"):
        from . import models
        return getattr(models, name)
    if name in ("StepEntry", "ModelRunner"):
        from . import engine
        return getattr(engine, name)
    if name == "CachePool":
        from .cache import CachePool
        return CachePool
    raise AttributeError(name)
