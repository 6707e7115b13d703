"""A small, whole inference engine for one GPU (NVIDIA B200, sm_100a): from a model folder
(config.json, model.safetensors) to next-token logits and generated tokens.

    config/    typed configuration and the architecture registry
    weights/   safetensors by tensor name, random-weights mode
    parts/     mixers, feed-forwards, norms, position encodings, blocks
    models/    architectures as lists of layers made from parts
    cache/     pages, block tables, state slots
    engine/    the step function, the scheduler, generation
    sampling/  greedy, temperature, top-k, top-p, repetition penalty
    kernels/   loader of the CUDA kernels under csrc/
"""
from . import config, parts, models, cache  # noqa: F401
from .config import ConfigError, load_config, register_architecture
from .parts import register_part
from .models import build_model
from .engine import Engine, generate, load_runner
from .sampling import SamplingParams
from .weights import write_random_model

__all__ = ["ConfigError", "load_config", "register_architecture", "register_part", "build_model", "Engine",
           "generate", "load_runner", "SamplingParams", "write_random_model"]
