"""burn_transformers_b200: a small, whole GPT-2 inference library for one B200.

config.json + model.safetensors -> typed configuration -> parts -> paged cache -> step function ->
generation loop -> sampler, with hand-written CUDA kernels for sm_100a underneath.
"""
from . import models  # noqa: F401  (registers the architectures)
from .cache import CacheConfig
from .config import Gpt2Config, config_from_folder, register_architecture, supported_model_types
from .engine import Engine, StepEntry
from .errors import (BurnTransformersError, CacheError, CheckpointError, ConfigError, GenerationError, KernelError,
                     ShapeError, UnsupportedArchitecture)
from .weights import write_random_model
from .sampling import GenerationConfig, GeneratedSequence, FinishReason
from .auto import (AutoCausalLm, AutoLoadOptions, CausalGenerationOutput, CausalGenerationRequest, LoadedModel,
                   generate_causal, generate_causal_streaming)
from .engine.generate import generate, plan_batches

__all__ = ["CacheConfig", "Gpt2Config", "config_from_folder", "register_architecture", "supported_model_types",
           "Engine", "StepEntry", "BurnTransformersError", "CacheError", "CheckpointError", "ConfigError",
           "GenerationError", "KernelError", "ShapeError", "UnsupportedArchitecture", "write_random_model", "GenerationConfig", "GeneratedSequence", "FinishReason",
           "AutoCausalLm", "AutoLoadOptions", "CausalGenerationOutput", "CausalGenerationRequest", "LoadedModel",
           "generate_causal", "generate_causal_streaming", "generate", "plan_batches"]
