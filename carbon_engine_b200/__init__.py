"""carbon_engine_b200: a single-GPU inference engine for the Qwen3 dense architecture on B200.

``Engine`` is the entry point (tokens in, tokens out), ``SamplingParams`` its options, and
``EngineHandle`` runs an engine on a thread of its own and streams tokens as events.
"""
from .sampling.params import SamplingParams

__all__ = ["Engine", "EngineHandle", "SamplingParams"]
__version__ = "0.1.0"


def __getattr__(name):
    if name == "Engine":
        from .engine.engine import Engine
        return Engine
    if name == "EngineHandle":
        from .engine.handle import EngineHandle
        return EngineHandle
    raise AttributeError(name)
