"""A small B200-native generation library for the dense Qwen3 decoder.

From a model folder (config.json + safetensors) to generated token ids on one GPU:

    import herbert_rs_b200 as hb
    engine = hb.Engine.from_folder("model_dir", dtype="bfloat16", max_tokens=8192)
    result = hb.generate(engine, [[1, 2, 3], [4, 5]], hb.GenerationOptions(max_tokens=16),
                         hb.SamplingParams(temperature=0.0))
    result.tokens            # one list of ids per prompt

Lower down: `engine.step(entries, want)` is the one step function (logits at wanted places).
"""

from . import models as _models  # registers the architectures  # noqa: F401
from . import parts as _parts  # registers the built-in parts  # noqa: F401
from .config import Qwen3Config, read_config_json
from .engine.backends import BACKENDS, available_backends_help, resolve_backend
from .engine.engine import Engine
from .engine.generate import (GenerationOptions, GenerationResult, GenerationStats,
                              detect_repetition_loop, generate)
from .engine.runtime import Runtime
from .models.decoder import DecoderModel
from .errors import (BackendError, CacheError, ConfigError, HerbertError, RequestError,
                     SafeTensorsError, WeightError)
from .registry import (architectures, build_part, config_from_json, register_architecture,
                       register_part)
from .sampling import SamplingParams
from .weights import load_model, random_model, write_random_model

__version__ = "0.1.0"

__all__ = [
    "Engine", "generate", "GenerationOptions", "GenerationResult", "GenerationStats", "SamplingParams",
    "Qwen3Config", "read_config_json", "Runtime", "DecoderModel", "load_model", "random_model", "write_random_model",
    "register_architecture", "register_part", "build_part", "config_from_json", "architectures",
    "BACKENDS", "available_backends_help", "resolve_backend", "detect_repetition_loop",
    "HerbertError", "ConfigError", "WeightError", "SafeTensorsError", "CacheError", "BackendError",
    "RequestError",
]
