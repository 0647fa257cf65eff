"""Interfaces of the parts a decoder is put together from.

A layer is a block; a block arranges a mixer (attention here), a feed-forward and norms; a mixer
may use a position encoding.  Every part gets its sizes and constants as constructor parameters,
declares the tensors it needs by name and shape, and loads them from a name -> tensor function.  No
part knows which model it is in.  The reference assembles its layers the same way from
``Mixer``/``Ffn``/``Residual`` choices made per layer index (src/model/mod.rs:35-64, 68-73).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, List, Optional, Tuple, Union

import torch

#: How random weights are drawn for a tensor, by the ``init`` of its :class:`TensorSpec`: kind -> (mean,
#: standard deviation, kept in float32).  N(0, 0.02) for "linear" and "embedding", 1 + N(0, 0.1) for "norm"
#: (norm weights are small and are stored in 32-bit).  A part with other needs registers a kind of its own.
INIT_KINDS = {"linear": (0.0, 0.02, False), "embedding": (0.0, 0.02, False), "norm": (1.0, 0.1, True)}


def register_init_kind(name: str, mean: float, std: float, keep_float32: bool = False) -> None:
    INIT_KINDS[name] = (float(mean), float(std), bool(keep_float32))


@dataclass(frozen=True)
class TensorSpec:
    name: str
    shape: Tuple[int, ...]
    init: str = "linear"


@dataclass(frozen=True)
class PagedCacheSpec:
    """A mixer that stores per-token keys and values in pages.  window 0 keeps all keys.  ``page_size``
    None takes the engine's page size; caches with the same window and page size share their pages' ids."""
    kv_heads: int
    head_dim: int
    window: int = 0
    page_size: Optional[int] = None


@dataclass(frozen=True)
class StateCacheSpec:
    """A mixer that keeps a state of fixed size per request, indexed by the request's state slot.
    ``dtype`` None means the compute dtype."""
    shape: Tuple[int, ...]
    dtype: Optional[torch.dtype] = None


CacheSpec = Union[PagedCacheSpec, StateCacheSpec, None]
TensorGetter = Callable[[str], torch.Tensor]


class Part:
    """Anything with weights."""

    def tensor_specs(self) -> List[TensorSpec]:
        return []

    def load(self, get: TensorGetter, device: torch.device, dtype: torch.dtype) -> None:
        """Fetch the declared tensors with ``get(name)`` (CPU, as stored) and keep them on ``device``."""

    def children(self) -> List["Part"]:
        return []

    def ignorable_tensors(self) -> List[str]:
        """Names (shell patterns allowed) of tensors a checkpoint may carry for this part although the
        part does not use them: their presence is no error, they are not read."""
        return []

    def all_ignorable_tensors(self) -> List[str]:
        out = list(self.ignorable_tensors())
        for c in self.children():
            out.extend(c.all_ignorable_tensors())
        return out

    def step_bytes(self, tokens: int, element_size: int) -> int:
        """Bytes of activations this part allocates while a step of ``tokens`` tokens runs through it (its
        children's included), for sizing the cache beside them.  0: nothing worth counting."""
        return 0

    def all_tensor_specs(self) -> List[TensorSpec]:
        out = list(self.tensor_specs())
        for c in self.children():
            out.extend(c.all_tensor_specs())
        return out

    def load_all(self, get: TensorGetter, device: torch.device, dtype: torch.dtype) -> None:
        self.load(get, device, dtype)
        for c in self.children():
            c.load_all(get, device, dtype)


class Norm(Part):
    def forward(self, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
        """out[r] = norm(x[rows[r]] if rows is given else x[r]); x is the float32 residual stream."""
        raise NotImplementedError


class Mixer(Part):
    """Mixes information across the tokens of a sequence (attention, or anything with a cache)."""

    #: Mixers whose kernels need per-step tables of their own (tile lists, split counts) name a key
    #: here; the step function then calls :meth:`plan_step` once per step and key, whatever the
    #: number of layers that share it, and the mixers find the result in ``ctx.plans[plan_key]``.
    plan_key: Optional[str] = None

    def cache_spec(self) -> CacheSpec:
        return None

    def step_sections(self, max_tokens: int, max_seqs: int) -> List[Tuple[str, int]]:
        """(name, int32 count) of the sections this kind of mixer wants in the step's pinned buffer
        (uploaded with the step in one copy, at addresses that never change)."""
        return []

    def plan_step(self, ctx) -> Any:
        """Lay out what this kind of mixer's kernels need for the step described by ``ctx`` (host lists
        ``h_q_start``, ``h_ctx_before``, ``n_decode``; ``ctx.bufs.host_section(name)`` is the host side of
        a section asked for in :meth:`step_sections`, ``ctx.bufs.dev_section(name)`` its device side).
        Nothing may be launched or copied here: the step's one upload follows.  An attribute
        ``graph_key`` of the result becomes part of the key under which a decode step is captured as a
        CUDA graph (a grid size that changes with the contexts, for instance)."""
        return None

    def forward(self, ctx, h: torch.Tensor, x: torch.Tensor, cache) -> None:
        """Read the normed activations ``h`` [T, width] and ADD the result into the float32 residual
        stream ``x`` [T, width].  ``cache`` is this call's view of the cache (or None), ``ctx`` the
        step's :class:`carbon_engine_b200.engine.batch.StepContext`."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx, h: torch.Tensor, x: torch.Tensor) -> None:
        """Read ``h`` and ADD the result into the float32 residual stream ``x``."""
        raise NotImplementedError


class Block(Part):
    """One layer: an arrangement of norms, a mixer and a feed-forward around the residual stream."""

    mixer: Mixer

    def forward(self, ctx, x: torch.Tensor, cache) -> None:
        raise NotImplementedError


def to_device(t: torch.Tensor, device: torch.device, dtype: torch.dtype) -> torch.Tensor:
    """Copy a stored tensor to the device in ``dtype`` (via float32 when the stored type differs)."""
    t = t.to(device)
    if t.dtype != dtype:
        t = t.to(torch.float32).to(dtype)
    return t.contiguous()
