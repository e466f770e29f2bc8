"""mdma_b200: a small, whole Llama inference library for one B200.

Model folder (config.json + safetensors) or seeded random weights -> typed
configuration -> parts -> paged cache -> one step function -> generation.
"""
from .config import ConfigError, LlamaConfig, load_config
from .registry import (ARCHITECTURES, BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS,
                       POSITIONS, RegistryError)
from .weights import CheckpointError, WeightsError, write_random_model

__all__ = ["ARCHITECTURES", "BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS",
           "POSITIONS", "CheckpointError", "ConfigError", "LlamaConfig", "RegistryError",
           "WeightsError", "load_config", "write_random_model", "Engine", "StepEntry", "generate"]


def __getattr__(name):
    # The engine pulls in the CUDA side; keep plain imports (config, weights) light.
    if name in ("Engine", "StepEntry", "StepError", "MemoryBudgetError"):
        from . import engine
        return getattr(engine, name)
    if name in ("generate", "Generator", "SamplingParams", "Output"):
        from .engine import generate as _g
        return getattr(_g, name)
    raise AttributeError(name)
