"""bitwise_b200: a small, whole Llama inference engine for one B200.

The public names follow the reference's Python package (python/bitwise/__init__.py:3-10):
``Model``, ``Engine``, ``EngineConfig``, ``SamplingParams``.
"""
from .config import LlamaConfig, RopeScaling  # noqa: F401
from .model import Model  # noqa: F401
from .sampling.sampler import SamplingParams  # noqa: F401
from .engine.engine import Engine, EngineConfig, EngineStats, RequestResult, StepEvent  # noqa: F401

__all__ = ["Model", "Engine", "EngineConfig", "SamplingParams", "LlamaConfig", "RopeScaling", "EngineStats",
           "RequestResult", "StepEvent"]
