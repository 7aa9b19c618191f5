"""lumenllm_b200: a small, whole, single-GPU generation library for NVIDIA B200
(sm_100a), in the manner of demented484/LumenLLM: config.json and safetensors in,
tokens out, through hand-written CUDA kernels."""
from .config import ConfigError, Qwen3Config, config_from_dict, load_config
from .engine import (BuiltEngine, Engine, EngineConfig, GenerateOutput, GenerateRequest, StepEntry,
                     StepError, build)
from .ops.native import KernelError
from .sampling import SamplingConfig

__version__ = "0.1.0"
__all__ = ["ConfigError", "Qwen3Config", "config_from_dict", "load_config", "BuiltEngine", "Engine",
           "EngineConfig", "GenerateOutput", "GenerateRequest", "StepEntry", "StepError", "build",
           "SamplingConfig", "KernelError"]
