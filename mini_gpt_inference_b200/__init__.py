"""A small, whole inference engine for the GPT-2 style decoder, written for NVIDIA B200."""

__version__ = "0.1.0"

from .config import EngineConfig, GPTConfig, SamplingParams  # noqa: E402
from .engine import LLMEngine, Request, RequestOutput  # noqa: E402

__all__ = ["EngineConfig", "GPTConfig", "SamplingParams", "LLMEngine", "Request", "RequestOutput"]
