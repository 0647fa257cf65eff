"""Device storage behind the cache manager: key/value pools for paged caches, state tensors for
per-request state, and the device copies of the block tables.

The model's cache layout (one entry per cache of its layer schedule) decides what is allocated.
Paged caches with the same window and page size share a *group*: one pool of page ids and one block table, so a
page id addresses the same page in every cache of the group, as one slot id does in every layer
of the reference (src/model/mod.rs:443-461).  Each cache still has K and V tensors of its own,
shaped [num_pages, kv_heads, page_size, head_dim].  State caches are tensors
[max_requests, *shape] indexed by a request's state slot (src/model/mod.rs:468-478).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np
import torch

from .. import ops
from ..parts.base import PagedCacheSpec, StateCacheSpec
from ..parts.model import LayerCall
from .manager import CacheManager, GroupSpec


@dataclass
class LayerCacheView:
    """What a mixer sees of its cache in one call."""
    kind: str                                   # "paged", "state" or "none"
    group: int = -1
    page_size: int = 0
    k_pool: Optional[torch.Tensor] = None
    v_pool: Optional[torch.Tensor] = None
    state: Optional[torch.Tensor] = None        # [max_requests, *shape]
    writes: bool = True


class CacheStorage:
    def __init__(self, model, dtype: torch.dtype, device: torch.device, page_size: int, num_pages: int,
                 max_requests: int, max_seq_len: int, window_pages: Optional[int] = None, poison: bool = False):
        self.device, self.dtype, self.page_size = device, dtype, int(page_size)
        self.max_requests = int(max_requests)
        layout = model.cache_layout()
        # the block tables of all groups have one width: what the smallest page size needs
        smallest = min([page_size] + [s.page_size for _, s in layout if isinstance(s, PagedCacheSpec) and s.page_size])
        self.max_pages_per_request = (int(max_seq_len) + smallest - 1) // smallest
        group_of: Dict[tuple, int] = {}
        groups: List[GroupSpec] = []
        self._entries: Dict[int, LayerCacheView] = {}
        for cache_id, spec in layout:
            if isinstance(spec, PagedCacheSpec):
                ps = int(spec.page_size or page_size)
                if (spec.window, ps) not in group_of:
                    group_of[(spec.window, ps)] = len(groups)
                    n = num_pages if spec.window == 0 or window_pages is None else window_pages
                    # ``num_pages`` counts pages of the engine's size: a group with other pages holds as many tokens
                    groups.append(GroupSpec(ps, max(1, int(n) * int(page_size) // ps), int(spec.window)))
                g = group_of[(spec.window, ps)]
                shape = (groups[g].num_pages, spec.kv_heads, ps, spec.head_dim)
                k = torch.empty(shape, dtype=dtype, device=device)
                v = torch.empty(shape, dtype=dtype, device=device)
                if poison:          # stale reads then show up as NaN in the logits
                    k.fill_(float("nan")); v.fill_(float("nan"))
                else:
                    k.zero_(); v.zero_()
                self._entries[cache_id] = LayerCacheView("paged", g, ps, k, v)
            elif isinstance(spec, StateCacheSpec):
                st = torch.zeros((max_requests, *spec.shape), dtype=spec.dtype or dtype, device=device)
                self._entries[cache_id] = LayerCacheView("state", state=st)
            else:
                self._entries[cache_id] = LayerCacheView("none")
        self.groups = groups
        self.manager = CacheManager(groups, max_requests, self.max_pages_per_request)
        self.device_tables = [torch.full((max_requests, self.max_pages_per_request), -1, dtype=torch.int32, device=device)
                              for _ in groups]
        # per group and slot: how many leading table entries the device copy already has (kept up by the host
        # runtime's step layout, which gathers the entries a step adds; int64, C-contiguous: it holds a pointer to it)
        self._synced = np.zeros((max(len(groups), 1), max_requests), dtype=np.int64)

    def view(self, call: LayerCall) -> LayerCacheView:
        base = self._entries[call.cache]
        if call.writes:
            return base
        return LayerCacheView(base.kind, base.group, base.page_size, base.k_pool, base.v_pool, base.state, False)

    def paged_views(self) -> List[LayerCacheView]:
        return [e for e in self._entries.values() if e.kind == "paged"]

    def bytes_per_token(self) -> int:
        total = 0
        for e in self._entries.values():
            if e.kind == "paged":
                total += 2 * e.k_pool.shape[1] * e.k_pool.shape[3] * e.k_pool.element_size()
        return total

    def slot_opened(self, slot: int) -> None:
        """A new request took ``slot``: its table rows start over."""
        self._synced[:, slot] = 0

    def state_bytes(self) -> int:
        """Bytes of the fixed-size per-request state tensors (all slots)."""
        return sum(e.state.numel() * e.state.element_size() for e in self._entries.values() if e.kind == "state")

    def zero_state(self, slot: int) -> None:
        """Reset the fixed-size state of a slot for a new request."""
        for e in self._entries.values():
            if e.kind == "state":
                e.state[slot].zero_()
