"""ghost-infer_b200: a small, whole model library for the Llama 3 dense decoder on one B200.

Everything between a request's tokens and its next token: typed configuration and a registry of
architectures, safetensors weights, layers put together from parts, a paged per-sequence cache, one
step function, a generation loop, sampling, and hand-written CUDA kernels for sm_100a.
"""
from .config import (ConfigError, LlamaConfig, UnknownArchitectureError, load_config, register_architecture,
                     registered_architectures)
from .config.llama_spec import build_llama_spec

register_architecture("LlamaForCausalLM", LlamaConfig.from_dict, build_llama_spec, replace=True)

from .engine import Engine, Model, StepEntry  # noqa: E402
from .api import LLM  # noqa: E402
from .sampling import SamplingParams  # noqa: E402

__all__ = ["ConfigError", "LlamaConfig", "UnknownArchitectureError", "load_config", "register_architecture",
           "registered_architectures", "Engine", "Model", "StepEntry", "LLM", "SamplingParams"]
__version__ = "0.1.0"
