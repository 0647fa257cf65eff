"""Registries of part kinds, so that a configuration can choose each layer's mixer, feed-forward,
norm and position encoding by name, and so that new kinds can be added from outside the package.

A factory takes keyword parameters (sizes, constants, the tensor-name prefix) and returns the part.
"""
from __future__ import annotations

from typing import Callable, Dict

from .attention import PagedAttention
from .mlp import GatedMLP
from .norm import RMSNorm
from .rope import NoPositionEncoding, RotaryEmbedding

_KINDS: Dict[str, Dict[str, Callable]] = {"mixer": {}, "feed_forward": {}, "norm": {}, "position": {}}


def register_part(kind: str, name: str, factory: Callable, replace: bool = False) -> None:
    table = _KINDS[kind]
    if name in table and not replace:
        raise ValueError(f"{kind} '{name}' is already registered")
    table[name] = factory


def unregister_part(kind: str, name: str) -> None:
    _KINDS[kind].pop(name, None)


def build_part(kind: str, part: str, /, **params):
    try:
        factory = _KINDS[kind][part]
    except KeyError:
        raise ValueError(f"unknown {kind} '{part}' (registered: {', '.join(sorted(_KINDS[kind]))})") from None
    return factory(**params)


def register_mixer(name, factory, replace=False): register_part("mixer", name, factory, replace)
def register_feed_forward(name, factory, replace=False): register_part("feed_forward", name, factory, replace)
def register_norm(name, factory, replace=False): register_part("norm", name, factory, replace)
def register_position(name, factory, replace=False): register_part("position", name, factory, replace)


register_mixer("full_attention", lambda **kw: PagedAttention(**{**kw, "window": 0}))
register_mixer("sliding_attention", lambda **kw: PagedAttention(**kw))
register_feed_forward("gated_mlp", GatedMLP)
register_norm("rmsnorm", RMSNorm)
register_position("rotary", RotaryEmbedding)
register_position("none", lambda **kw: NoPositionEncoding())
