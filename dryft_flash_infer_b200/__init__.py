"""dryft-flash-infer_b200: a small single-GPU model library with generation of its own,
written for NVIDIA B200 (sm_100a), for the Qwen3 dense decoder.

    from dryft_flash_infer_b200 import Engine
    engine = Engine("/path/to/model")                  # config.json + model.safetensors
    for tokens in engine.generate([[1, 2, 3], [4, 5]], max_new_tokens=16):
        ...
"""

from . import models  # noqa: F401
from .config import ConfigError, Qwen3Config, load_config, register_architecture
from .engine import Engine, EngineOptions, Request, StepEntry
from .sampling import SamplingParams
from .weights import WeightError, write_random_model

__all__ = ["Engine", "EngineOptions", "Request", "StepEntry", "SamplingParams", "ConfigError", "Qwen3Config",
           "load_config", "register_architecture", "WeightError", "write_random_model"]
