"""Python face of the native cache manager (csrc/runtime/cache_manager.cpp).

A :class:`CacheManager` owns, for every group of layers, a pool of pages and a block table with one
row per state slot; a request holds a state slot and pages in every group.  The device-side
storage that pages and slots index (key/value pools, state tensors) is owned by
:class:`carbon_engine_b200.cache.storage.CacheStorage`; this class only does the bookkeeping.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Sequence

import numpy as np

from ..csrc.runtime_lib import runtime


class CacheError(RuntimeError):
    pass


class OutOfPages(CacheError):
    """A pool cannot give the pages asked for; nothing was changed."""


_MESSAGES = {
    -1: "every state slot is taken",
    -2: "the request is already open",
    -3: "no such request",
    -4: "out of pages",
    -5: "the request would need more pages than a block-table row holds",
    -6: "bad argument",
}


@dataclass(frozen=True)
class GroupSpec:
    """One group of layers with the same cache needs: all keys (window 0) or a window of them."""
    page_size: int
    num_pages: int
    window: int = 0


class CacheManager:
    def __init__(self, groups: Sequence[GroupSpec], max_requests: int, max_pages_per_request: int):
        self._lib = runtime()
        self.groups = list(groups)
        self.max_requests = int(max_requests)
        self.max_pages_per_request = int(max_pages_per_request)
        n = len(self.groups)
        arr = lambda xs: (ctypes.c_int * n)(*xs)
        self._h = self._lib.cm_create(n, arr([g.page_size for g in groups]), arr([g.num_pages for g in groups]),
                                      arr([g.window for g in groups]), self.max_requests, self.max_pages_per_request)
        if not self._h:
            raise CacheError(f"bad cache geometry: groups={groups}, max_requests={max_requests}, "
                             f"max_pages_per_request={max_pages_per_request}")
        self._tables = []
        for g in range(n):
            ptr = self._lib.cm_table(self._h, g)
            buf = (ctypes.c_int32 * (self.max_requests * self.max_pages_per_request)).from_address(
                ctypes.addressof(ptr.contents))
            self._tables.append(np.frombuffer(buf, dtype=np.int32).reshape(self.max_requests, self.max_pages_per_request))

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.cm_destroy(h)

    @property
    def handle(self):
        return self._h

    def _check(self, code: int, what: str) -> int:
        if code >= 0:
            return code
        if code == -4:
            raise OutOfPages(f"{what}: out of pages")
        raise CacheError(f"{what}: {_MESSAGES.get(code, code)}")

    def open(self, request_id: int) -> int:
        """Take a state slot for a new request and return it."""
        return self._check(self._lib.cm_open(self._h, request_id), f"open({request_id})")

    def reserve(self, request_id: int, new_len: int) -> None:
        """Make sure pages exist for positions below ``new_len`` in every group."""
        self._check(self._lib.cm_reserve(self._h, request_id, new_len), f"reserve({request_id}, {new_len})")

    def commit(self, request_id: int, new_len: int) -> None:
        """Positions below ``new_len`` are written; windowed groups give back pages now behind the window."""
        self._check(self._lib.cm_commit(self._h, request_id, new_len), f"commit({request_id}, {new_len})")

    def commit_many(self, request_ids: np.ndarray, new_lens: np.ndarray) -> None:
        """:meth:`commit` for several requests (int64 ids, int32 lengths) in one call."""
        n = len(request_ids)
        self._check(self._lib.cm_commit_many(self._h, request_ids.ctypes.data_as(ctypes.POINTER(ctypes.c_int64)),
                                             new_lens.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)), n), f"commit of {n} requests")

    def close(self, request_id: int) -> None:
        self._check(self._lib.cm_close(self._h, request_id), f"close({request_id})")

    def slot_of(self, request_id: int) -> int:
        return self._check(self._lib.cm_slot_of(self._h, request_id), f"slot_of({request_id})")

    def length_of(self, request_id: int) -> int:
        return self._check(self._lib.cm_length_of(self._h, request_id), f"length_of({request_id})")

    def reserved_of(self, request_id: int) -> int:
        """Positions the request holds pages for (at least its length)."""
        return self._check(self._lib.cm_reserved_of(self._h, request_id), f"reserved_of({request_id})")

    def has(self, request_id: int) -> bool:
        return self._lib.cm_slot_of(self._h, request_id) >= 0

    def free_pages(self, group: int = 0) -> int:
        return self._lib.cm_free_pages(self._h, group)

    def held_pages(self, request_id: int, group: int = 0) -> int:
        return self._check(self._lib.cm_held_pages(self._h, request_id, group), "held_pages")

    def free_slots(self) -> int:
        return self._lib.cm_free_slots(self._h)

    def open_requests(self) -> int:
        return self._lib.cm_open_requests(self._h)

    def pages_for_lifetime(self, group: int, total_len: int, max_chunk: int) -> int:
        return self._lib.cm_pages_for_lifetime(self._h, group, total_len, max_chunk)

    def pages_to_reserve(self, request_id: int, group: int, new_len: int) -> int:
        return self._check(self._lib.cm_pages_to_reserve(self._h, request_id, group, new_len), "pages_to_reserve")

    def table(self, group: int = 0) -> np.ndarray:
        """The group's block table as a live int32 view [max_requests, max_pages_per_request]."""
        return self._tables[group]

    def check(self) -> None:
        """Raise if a page is lost, held twice, or held by a slot nobody owns."""
        code = self._lib.cm_check(self._h)
        if code != 0:
            names = {1: "a page id out of range", 2: "a page held twice", 3: "a page in a table but marked free",
                     4: "a page lost (held by nobody)", 5: "held + free != pool size",
                     6: "a page in the row of an unowned slot", 7: "state slots lost"}
            raise CacheError(f"cache manager inconsistent: {names.get(code, code)}")
