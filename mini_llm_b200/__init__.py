"""mini_llm_b200: a small, whole inference engine for one B200 (sm_100a): GPT-2, Finuvik, Falisun, Mumopel and Kusirax.

Configuration and registry (``config``), safetensors weights (``weights``), model
parts and their assembly (``parts``, ``models``), paged cache manager (``cache``),
step function, scheduler and entry point (``engine``), sampling (``sampling``),
hand-written CUDA kernels (``csrc``, reached through ``ops``).
"""
from .config.base import (ConfigError, EngineConfig, config_from_dict, load_config, register_architecture,
                          registered_architectures)
from .parts import (attention, block, embedding, head, hyper, join, latent, mlp, moe, norm, positions,  # noqa: F401
                    projected, recurrent, ssm, wkv)                                                                # (register the parts)
from .parts.base import register_part
from .models import falisun, finuvik, gpt2, kusirax, mumopel  # noqa: F401  (register GPT2LMHeadModel, Finuvik, Falisun, Mumopel, Kusirax)
from .weights.random_init import write_random_model
from .sampling.params import SamplingParams
from .engine.request import Request, RequestState, Response


def __getattr__(name):
    if name == "LLM":          # needs CUDA at construction only; imported on demand
        from .engine.llm import LLM
        return LLM
    raise AttributeError(name)


__all__ = ["ConfigError", "EngineConfig", "config_from_dict", "load_config", "register_architecture",
           "registered_architectures", "register_part", "write_random_model", "SamplingParams", "Request",
           "RequestState", "Response", "LLM"]
__version__ = "0.1.0"
