"""The step function: a batch of sequences, each bringing its next tokens.

``Engine.step`` takes, for every sequence of the batch, its cache slot and the
tokens it brings (a whole prompt, a piece of one, or one decoded token), runs
exactly those tokens as one packed batch against the cache that earlier steps
left, and returns float32 logits at the wanted places.  Sequences may bring
different numbers of tokens; nothing is padded, so padding cannot change a
result.  Positions come from the cache lengths, so a caller cannot give
positions that disagree with the cache (in the reference they are separate
arguments, thanhauco/rust-inference src/models/mod.rs:36-44).

Steps in which every sequence brings one token are replayed from a CUDA graph
per batch size: the step's small tables are copied to fixed device buffers and
the captured kernels read them from there.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Optional, Sequence, Union

import numpy as np
import torch

from .. import ops
from ..cache import Cache, CacheError, PAGE_SIZE
from ..csrc import build as _build
from ..parts.base import StepContext
from .model import Model


@dataclass
class Entry:
    """One sequence's share of a step: ``want`` lists the places among ``tokens``
    whose logits are asked for ("last", "all", or indices; may be empty)."""
    slot: int
    tokens: Sequence[int]
    want: Union[str, Sequence[int]] = "last"


class StepError(ValueError):
    pass


_P, _I, _L = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
_HOST_SIGNATURES = {
    "ri_step_check": (_I, [_I, _P, _P, _P, _L, _P, _P, _P, _P]),
    "ri_step_fill": (None, [_I, _P, _P, _P, _P, _P, _P, _L, _L, _P, _P, _P]),
    "ri_step_check_decode": (_I, [_I, _P, _L]),
    "ri_step_fill_decode": (None, [_I, _P, _P, _P, _I, _P, _P]),
}
_host_lib = None


def _host():
    """The C++ side of a step (csrc/host_step.cpp): the check of the entries and the tables."""
    global _host_lib
    if _host_lib is None:
        lib = _build.library("host_step")
        for name, (res, args) in _HOST_SIGNATURES.items():
            f = getattr(lib, name)
            f.restype, f.argtypes = res, args
        _host_lib = lib
    return _host_lib


def _i32(values) -> np.ndarray:
    return np.ascontiguousarray(values, dtype=np.int32)


class _Tables:
    """The int32 tables of a step in one device buffer (one copy from the host)."""

    def __init__(self, T: int, B: int, W: int, device):
        self.T, self.B, self.W = T, B, W
        sizes = (T, T, T, W, B, B + 1, B)
        self.offsets = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
        total = int(self.offsets[-1])
        self.pinned = device.type == "cuda"
        self.host = torch.empty(total, dtype=torch.int32, pin_memory=self.pinned)
        self.host_np = self.host.numpy()
        self.dev = torch.empty(total, dtype=torch.int32, device=device)
        self.event = torch.cuda.Event() if self.pinned else None
        self.used = False
        self.decode_constants = False

    def part(self, i: int, host: bool = False):
        lo, hi = int(self.offsets[i]), int(self.offsets[i + 1])
        return (self.host_np if host else self.dev)[lo:hi]

    def upload(self) -> None:
        self.dev.copy_(self.host, non_blocking=True)
        if self.event is not None:
            self.event.record()
        self.used = True

    def wait_host_free(self) -> None:
        if self.used and self.event is not None:
            self.event.synchronize()


class Engine:
    """A model with its cache.

    ``max_tokens``: tokens the cache holds over all live sequences (rounded up
    to whole pages per sequence); ``max_seqs``: slots; ``max_seq_len``: the
    longest a single sequence may get (default: what the model allows, capped by
    ``max_tokens``)."""

    def __init__(self, model: Model, max_tokens: int, max_seqs: int, max_seq_len: Optional[int] = None,
                 use_graphs: bool = True, page_size: int = PAGE_SIZE):
        self.model = model
        self.device = model.env.device
        self.dtype = model.env.dtype
        num_pages = max(1, -(-max_tokens // page_size))
        limit = model.spec.max_positions
        if max_seq_len is not None:
            limit = min(limit, max_seq_len)
        limit = min(limit, num_pages * page_size)
        self.max_seq_len = limit
        self.cache = Cache(model.cache_requests(), max(1, max_seqs), num_pages, max(1, -(-limit // page_size)),
                           self.dtype, self.device, page_size)
        model.prepare(self.cache.max_seq_len)
        self.use_graphs = use_graphs and self.device.type == "cuda" and model.graph_safe
        self._decode_tables = {}
        self._other_tables = {}
        self._graphs = {}
        self._warm = set()
        self.graph_replays = 0

    # ---- sequences ------------------------------------------------------------------------
    def new_sequence(self) -> int:
        return self.cache.alloc_slot()

    def release(self, slot: int) -> None:
        self.cache.free_slot(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    # ---- one step --------------------------------------------------------------------------
    def step(self, entries: Sequence[Entry]) -> torch.Tensor:
        """Run the step; float32 logits [wanted places in entry order, vocab] on the device.

        A step replayed from a graph returns the graph's own output buffer: the logits are
        valid until the next step of the same batch size runs; a caller that keeps them copies."""
        if not entries:
            raise StepError("a step needs at least one sequence")
        V = self.model.spec.vocab_size
        if all(len(e.tokens) == 1 and (e.want == "last" or (not isinstance(e.want, str) and list(e.want) == [0]))
               for e in entries):
            return self._step_one_token_each(entries, V)
        news, wants = [], []
        for e in entries:
            toks = np.asarray(e.tokens, dtype=np.int64).reshape(-1)
            news.append(toks)
            if isinstance(e.want, str):
                if e.want == "last":
                    w = [toks.size - 1]
                elif e.want == "all":
                    w = range(toks.size)
                else:
                    raise StepError(f"want must be 'last', 'all' or a list of places, got {e.want!r}")
            else:
                w = e.want
            wants.append(_i32(w).reshape(-1))
        B = len(entries)
        slots = _i32([int(e.slot) for e in entries])
        n_new, n_want = _i32([t.size for t in news]), _i32([w.size for w in wants])
        tokens = np.ascontiguousarray(np.concatenate(news))
        want_flat = np.ascontiguousarray(np.concatenate(wants))
        host = _host()
        T_, W_ = _L(0), _L(0)
        if host.ri_step_check(B, slots.ctypes.data, n_new.ctypes.data, tokens.ctypes.data, V, n_want.ctypes.data,
                              want_flat.ctypes.data, ctypes.byref(T_), ctypes.byref(W_)):
            raise StepError(host.ri_last_error().decode(errors="replace"))
        T, W = T_.value, W_.value
        before = _i32(self.cache.extend(list(zip(slots.tolist(), n_new.tolist()))))
        self.cache.upload()

        decode = T == B
        graphable = self.use_graphs and decode and bool((n_want == 1).all()) and bool((want_flat == 0).all())
        tables = self._tables_for(T, B, W, graphable)
        tables.wait_host_free()
        max_new, max_len = _I(0), _I(0)
        host.ri_step_fill(B, slots.ctypes.data, before.ctypes.data, n_new.ctypes.data, tokens.ctypes.data,
                          n_want.ctypes.data, want_flat.ctypes.data, T, W, tables.host_np.ctypes.data,
                          ctypes.byref(max_new), ctypes.byref(max_len))
        tables.decode_constants = False            # the general path writes every column
        tables.upload()
        after = before + n_new
        ctx = StepContext(
            tok_seq=tables.part(1), tok_pos=tables.part(2), seq_slot=tables.part(4), seq_start=tables.part(5),
            seq_len=tables.part(6), num_tokens=T, num_seqs=B, max_new=max_new.value, max_len=max_len.value,
            host_seq_slot=tuple(slots.tolist()), host_new=tuple(n_new.tolist()), host_len=tuple(after.tolist()))
        slots = slots.tolist()
        if W == 0:
            want_dev = tables.part(2)[:0]
        else:
            want_dev = tables.part(3)
        if graphable:
            logits = self._decode_step(tables, ctx, want_dev)
        else:
            logits = self.model.forward(tables.part(0), ctx, self.cache, want_dev)
        self.cache.after_step(slots)
        return logits

    def step_device_ids(self, slots: Sequence[int], ids: torch.Tensor) -> torch.Tensor:
        """A decode step whose token ids are on the device already (int32 [len(slots)], as the
        sampler left them): the host need not have seen them, so this step can be launched
        while the ids of the step before are still on their way to the host."""
        if ids.dtype != torch.int32 or ids.numel() != len(slots) or ids.device != self.device:
            raise StepError("step_device_ids: ids must be int32 on the engine's device, one per slot")
        return self._step_one_token_each(None, self.model.spec.vocab_size, slots=[int(s) for s in slots], ids_dev=ids)

    def _step_one_token_each(self, entries, V, slots=None, ids_dev=None) -> torch.Tensor:
        """The decode step: every sequence brings one token and wants its logits.  Same
        result as the general path, with the host work cut to a few array writes."""
        host = _host()
        toks = None
        if ids_dev is None:
            toks = np.ascontiguousarray([int(e.tokens[0]) for e in entries], dtype=np.int64)
            if host.ri_step_check_decode(len(toks), toks.ctypes.data, V):
                raise StepError(host.ri_last_error().decode(errors="replace"))
            slots = [int(e.slot) for e in entries]
        B = len(slots)
        before = _i32(self.cache.extend([(s, 1) for s in slots]))
        self.cache.upload()
        tables = self._tables_for(B, B, B, self.use_graphs)
        tables.wait_host_free()
        slots_np = _i32(slots)
        max_len = _I(0)
        host.ri_step_fill_decode(B, slots_np.ctypes.data, before.ctypes.data, None if toks is None else toks.ctypes.data,
                                 0 if tables.decode_constants else 1, tables.host_np.ctypes.data, ctypes.byref(max_len))
        tables.decode_constants = True
        after = (before + 1).tolist()
        tables.upload()
        if ids_dev is not None:
            tables.part(0).copy_(ids_dev)                 # device to device, after the upload in stream order
        ctx = StepContext(
            tok_seq=tables.part(1), tok_pos=tables.part(2), seq_slot=tables.part(4), seq_start=tables.part(5),
            seq_len=tables.part(6), num_tokens=B, num_seqs=B, max_new=1, max_len=max_len.value,
            host_seq_slot=tuple(slots), host_new=(1,) * B, host_len=tuple(after))
        if self.use_graphs:
            logits = self._decode_step(tables, ctx, tables.part(3))
        else:
            logits = self.model.forward(tables.part(0), ctx, self.cache, tables.part(3))
        self.cache.after_step(slots)
        return logits

    # ---- graphs for one-token steps ------------------------------------------------------------
    def _tables_for(self, T, B, W, graphable) -> _Tables:
        """Tables are kept per shape: pinned host memory is slow to allocate, and a captured
        step needs its tables at fixed addresses."""
        if graphable:
            t = self._decode_tables.get(B)
            if t is None:
                t = self._decode_tables[B] = _Tables(T, B, W, self.device)
            return t
        key = (T, B, W)
        t = self._other_tables.pop(key, None)
        if t is None:
            t = _Tables(T, B, W, self.device)
            if len(self._other_tables) >= 32:
                self._other_tables.pop(next(iter(self._other_tables)))
        self._other_tables[key] = t                       # most recently used last
        return t

    def _graph_key(self, ctx) -> tuple:
        return (ctx.num_seqs, ctx.len_bucket)

    def _decode_step(self, tables, ctx, want_dev):
        key = self._graph_key(ctx)
        rec = self._graphs.get(key)
        if rec is not None:
            rec[0].replay()
            self.graph_replays += 1
            ops.add_launches(rec[2])
            return rec[1]
        if key not in self._warm:
            # the first step of this shape runs eagerly: libraries set themselves up
            self._warm.add(key)
            return self.model.forward(tables.part(0), ctx, self.cache, want_dev)
        graph = torch.cuda.CUDAGraph()
        torch.cuda.synchronize(self.device)
        n0 = ops.launch_count()
        with torch.cuda.graph(graph):
            out = self.model.forward(tables.part(0), ctx, self.cache, want_dev)
        captured = ops.launch_count() - n0          # recorded, not run: they count at each replay
        ops.add_launches(-captured)
        self._graphs[key] = (graph, out, captured)
        graph.replay()
        self.graph_replays += 1
        ops.add_launches(captured)
        return out

    # ---- errors the kernels reported ------------------------------------------------------------
    def check_device_errors(self) -> None:
        if self.device.type != "cuda":
            return
        code = int(ops.error_flag(self.device).item())
        if code:
            ops.error_flag(self.device).zero_()
            raise RuntimeError(f"a kernel refused an index: {ops.ERROR_TEXT.get(code, code)}")
