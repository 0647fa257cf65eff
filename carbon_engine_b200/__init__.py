"""carbon_engine_b200: a single-GPU inference engine for the Qwen3 dense architecture on B200.

``Engine`` is the entry point (tokens in, tokens out); ``SamplingParams`` its options.
"""
from .sampling.params import SamplingParams

__all__ = ["Engine", "SamplingParams"]
__version__ = "0.1.0"


def __getattr__(name):
    if name == "Engine":
        from .engine.engine import Engine
        return Engine
    raise AttributeError(name)
