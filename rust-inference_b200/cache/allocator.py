"""Host-side bookkeeping of the cache: which slots are live, which pages each
slot maps, how long each sequence is.  No device memory is touched here.

The bookkeeping itself is C++ (``csrc/host_cache.cpp``, built on first use and
loaded with ctypes); the classes here are its handles.  The paged design is
thanhauco/rust-inference's (src/kvcache.rs:12-61, 106-135): fixed pages of
``page_size`` tokens, a page table row per sequence with -1 for "unmapped",
pages handed out from a free list as a sequence grows (lowest page first).
Added to it: a row is a *slot* that is given out and taken back per sequence,
sequences grow by different amounts in one step, and a slot's pages return to
the free list when the slot is freed.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import numpy as np

from ..csrc import build as _build


class CacheError(RuntimeError):
    """Out of slots or pages, a sequence over its limit, or a misuse of a slot."""


_P, _I = ctypes.c_void_p, ctypes.c_int
_SIGNATURES = {
    "ri_slots_create": (_P, [_I]), "ri_slots_destroy": (None, [_P]), "ri_slots_alloc": (_I, [_P, _P]),
    "ri_slots_free": (_I, [_P, _I]), "ri_slots_is_live": (_I, [_P, _I]), "ri_slots_require_live": (_I, [_P, _I]),
    "ri_slots_live_count": (_I, [_P]), "ri_slots_check": (_I, [_P]),
    "ri_pages_create": (_P, [_I] * 5), "ri_pages_destroy": (None, [_P]), "ri_pages_table": (_P, [_P]),
    "ri_pages_free": (_I, [_P]), "ri_pages_len": (_I, [_P, _I]), "ri_pages_needed": (_I, [_P, _I, _I]),
    "ri_pages_extend": (_I, [_P, _I, _I, _P]), "ri_pages_release_behind_window": (_I, [_P, _I]),
    "ri_pages_release": (None, [_P, _I]), "ri_pages_check": (_I, [_P]), "ri_pages_take_dirty": (_I, [_P, _P, _I]),
    "ri_cache_create": (_P, [_I, _I, _I, _I, _I, _P]), "ri_cache_destroy": (None, [_P]),
    "ri_cache_slots": (_P, [_P]), "ri_cache_group": (_P, [_P, _I]), "ri_cache_alloc_slot": (_I, [_P, _P]),
    "ri_cache_free_slot": (_I, [_P, _I]), "ri_cache_length": (_I, [_P, _I, _P]),
    "ri_cache_extend": (_I, [_P, _I, _P, _P, _P]), "ri_cache_after_step": (None, [_P, _I, _P]),
    "ri_cache_free_pages": (_I, [_P, _I]), "ri_cache_check": (_I, [_P]),
}
_lib = None


def lib():
    """The host library, compiled at the first call."""
    global _lib
    if _lib is None:
        handle = _build.library("host_cache")
        for name, (res, args) in _SIGNATURES.items():
            f = getattr(handle, name)
            f.restype, f.argtypes = res, args
        _lib = handle
    return _lib


def _raise(rc: int) -> None:
    msg = lib().ri_last_error().decode(errors="replace")
    if rc == 1:
        raise CacheError(msg)
    raise AssertionError(msg)


def _ok(rc: int) -> None:
    if rc:
        _raise(rc)


class SlotAllocator:
    """Slots that are given out (lowest first) and taken back.  ``handle``: the
    slots of a whole cache, which that cache owns."""

    def __init__(self, num_slots: int, handle: Optional[int] = None):
        self.num_slots = num_slots
        self._owned = handle is None
        if handle is None:
            handle = lib().ri_slots_create(num_slots)
            if not handle:
                _raise(1)
        self._h = handle

    def __del__(self):
        if getattr(self, "_owned", False) and getattr(self, "_h", None) and _lib is not None:
            _lib.ri_slots_destroy(self._h)
            self._h = None

    def alloc(self) -> int:
        out = _I(0)
        _ok(lib().ri_slots_alloc(self._h, ctypes.byref(out)))
        return out.value

    def free(self, slot: int) -> None:
        _ok(lib().ri_slots_free(self._h, int(slot)))

    def require_live(self, slot: int) -> None:
        _ok(lib().ri_slots_require_live(self._h, int(slot)))

    def is_live(self, slot: int) -> bool:
        return bool(lib().ri_slots_is_live(self._h, int(slot)))

    @property
    def live_count(self) -> int:
        return lib().ri_slots_live_count(self._h)

    def check(self) -> None:
        """Every slot is either free or live, never both, never twice."""
        _ok(lib().ri_slots_check(self._h))


class PageTable:
    """Pages of one cache group: free list, the table [slots, max_pages_per_seq]
    (``table``: a numpy view of the C++ side's memory) and the number of tokens
    stored per slot.

    ``window`` > 0: only the last ``window`` keys are ever read again, so pages
    that lie wholly before them are released after every step.  ``handle``: a
    group of a whole cache, which that cache owns.
    """

    def __init__(self, num_slots: int, num_pages: int, max_pages_per_seq: int, page_size: int, window: int = 0,
                 handle: Optional[int] = None):
        self.num_slots, self.num_pages = num_slots, num_pages
        self.max_pages_per_seq, self.page_size, self.window = max_pages_per_seq, page_size, window
        self._owned = handle is None
        if handle is None:
            handle = lib().ri_pages_create(num_slots, num_pages, max_pages_per_seq, page_size, window)
            if not handle:
                _raise(1)
        self._h = handle
        ptr = ctypes.cast(lib().ri_pages_table(self._h), ctypes.POINTER(ctypes.c_int32))
        self.table = np.ctypeslib.as_array(ptr, shape=(num_slots, max_pages_per_seq))
        self._dirty_buf = np.empty(num_slots, dtype=np.int32)

    def __del__(self):
        if getattr(self, "_owned", False) and getattr(self, "_h", None) and _lib is not None:
            self.table = None
            _lib.ri_pages_destroy(self._h)
            self._h = None

    @property
    def free_pages(self) -> int:
        return lib().ri_pages_free(self._h)

    @property
    def max_seq_len(self) -> int:
        return self.max_pages_per_seq * self.page_size

    @property
    def lens(self) -> List[int]:
        f = lib().ri_pages_len
        return [f(self._h, s) for s in range(self.num_slots)]

    def pages_needed(self, slot: int, new_tokens: int) -> int:
        """Pages that ``extend(slot, new_tokens)`` would take from the free list."""
        return lib().ri_pages_needed(self._h, int(slot), int(new_tokens))

    def extend(self, slot: int, new_tokens: int) -> int:
        """Map pages for the next ``new_tokens`` positions of ``slot`` and advance
        its length; returns the length before.  Nothing changes if it fails."""
        before = _I(0)
        _ok(lib().ri_pages_extend(self._h, int(slot), int(new_tokens), ctypes.byref(before)))
        return before.value

    def release_behind_window(self, slot: int) -> int:
        """Give back the pages that no later query of ``slot`` can see (window groups)."""
        return lib().ri_pages_release_behind_window(self._h, int(slot))

    def release(self, slot: int) -> None:
        """Give back every page of ``slot`` and reset its length."""
        lib().ri_pages_release(self._h, int(slot))

    def take_dirty(self) -> np.ndarray:
        """The slots whose rows changed since the last call (their marks are cleared)."""
        n = lib().ri_pages_take_dirty(self._h, self._dirty_buf.ctypes.data, self.num_slots)
        return self._dirty_buf[:n]

    def check(self) -> None:
        """Every page is free or mapped exactly once."""
        _ok(lib().ri_pages_check(self._h))


class HostCache:
    """Slots, one ``PageTable`` per group of layers and the sequences' lengths, as one
    C++ object: a step's growth is one call."""

    def __init__(self, num_slots: int, num_pages: int, max_pages_per_seq: int, page_size: int, windows: Sequence[int]):
        w = np.asarray(list(windows), dtype=np.int32)
        self._h = lib().ri_cache_create(num_slots, num_pages, max_pages_per_seq, page_size, len(w), w.ctypes.data)
        if not self._h:
            _raise(1)
        self.slots = SlotAllocator(num_slots, handle=lib().ri_cache_slots(self._h))
        self.groups = [PageTable(num_slots, num_pages, max_pages_per_seq, page_size, int(win),
                                 handle=lib().ri_cache_group(self._h, g)) for g, win in enumerate(w)]
        self.num_pages = num_pages

    def __del__(self):
        if getattr(self, "_h", None) and _lib is not None:
            for g in getattr(self, "groups", []):
                g.table = None
            _lib.ri_cache_destroy(self._h)
            self._h = None

    def alloc_slot(self) -> int:
        out = _I(0)
        _ok(lib().ri_cache_alloc_slot(self._h, ctypes.byref(out)))
        return out.value

    def free_slot(self, slot: int) -> None:
        _ok(lib().ri_cache_free_slot(self._h, int(slot)))

    def length(self, slot: int) -> int:
        out = _I(0)
        _ok(lib().ri_cache_length(self._h, int(slot), ctypes.byref(out)))
        return out.value

    def extend(self, slots: Sequence[int], news: Sequence[int]) -> List[int]:
        """Either all of the step's growth happens or none; the lengths before."""
        s = np.asarray(slots, dtype=np.int32)
        n = np.asarray(news, dtype=np.int32)
        before = np.empty(len(s), dtype=np.int32)
        _ok(lib().ri_cache_extend(self._h, len(s), s.ctypes.data, n.ctypes.data, before.ctypes.data))
        return before.tolist()

    def after_step(self, slots: Sequence[int]) -> None:
        s = np.asarray(slots, dtype=np.int32)
        lib().ri_cache_after_step(self._h, len(s), s.ctypes.data)

    def free_pages(self) -> int:
        return lib().ri_cache_free_pages(self._h, self.num_pages)

    def check(self) -> None:
        _ok(lib().ri_cache_check(self._h))
