"""What every part sees: the build environment, the step's context, and the
interfaces of the four kinds of part.

A part is built from its spec record and a :class:`BuildEnv` (compute dtype and
device), declares the tensors it wants (``param_infos``), receives them
(``load``) and then runs on packed tokens: activations are [tokens, features]
for all sequences of the step back to back, and a :class:`StepContext` says
which token belongs to which sequence, at which position, in which cache slot.

Hidden state between parts is a pair ``(resid, delta)``: the float32 residual
stream and the output of the last part in the compute dtype, not yet added.
A norm adds it while it reads it (one pass over the data instead of two).

Interfaces
----------
Norm            ``__call__(resid, delta=None, rows=None) -> normed``
PositionEncoding ``prepare(max_positions)``; either ``fused_table()`` (a float32
                [positions, rotary_dim/2, 2] cos/sin table that the attention
                kernel applies itself) or ``apply(q, k, ctx) -> (q, k)``
Mixer           ``cache_request() -> CacheRequest | None``;
                ``__call__(x, ctx, cache) -> y`` with ``cache`` the
                :class:`~..cache.LayerCache` of the schedule entry
FeedForward     ``__call__(x, ctx) -> y``
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional

import torch

from .registry import ParamInfo


@dataclass(frozen=True)
class BuildEnv:
    dtype: torch.dtype            # compute dtype: torch.float32 or torch.bfloat16
    device: torch.device


@dataclass
class StepContext:
    """The packed batch of one step.  Device tensors are int32.

    tok_seq[t]   index (within this step) of the sequence token t belongs to
    tok_pos[t]   position of token t in its sequence (= cache length before it)
    seq_slot[b]  cache slot of sequence b
    seq_start[b] first packed token of sequence b (length B+1)
    seq_len[b]   length of sequence b after this step
    """
    tok_seq: torch.Tensor
    tok_pos: torch.Tensor
    seq_slot: torch.Tensor
    seq_start: torch.Tensor
    seq_len: torch.Tensor
    num_tokens: int
    num_seqs: int
    max_new: int                  # most tokens any sequence brings in this step
    max_len: int                  # longest sequence after this step
    host_seq_slot: tuple = ()
    host_new: tuple = ()          # tokens each sequence brings
    host_len: tuple = ()          # lengths after this step

    @property
    def decode_only(self) -> bool:
        return self.max_new == 1

    @property
    def len_bucket(self) -> int:
        """``max_len`` rounded up to a multiple of 1024: what kernels size their grids
        and scratch memory by, so that a captured step stays valid while the
        sequences grow inside the bucket."""
        return -(-max(1, self.max_len) // 1024) * 1024


@dataclass(frozen=True)
class CacheRequest:
    """What a mixer needs stored per sequence.

    Keys and values: ``kv_heads`` x ``head_dim`` per token (0 for none), all of
    them (``window`` 0) or the last ``window``.  Fixed-size state:
    ``state_shape`` per sequence (empty for none), zeroed when a slot is given
    out."""
    kv_heads: int = 0
    head_dim: int = 0
    window: int = 0
    state_shape: tuple = ()
    state_dtype: torch.dtype = torch.float32


class Part:
    """Common base: parameters by local name.

    ``graph_safe``: one-token steps are captured into CUDA graphs and replayed.  A
    captured step repeats the same launches with the same host-side values, so a
    part may only be replayed if everything that changes from step to step reaches
    its kernels through device tensors (the context's int32 tables, the cache).  A
    part that reads ``ctx.host_*`` values, branches on them or indexes with them
    must leave this False; a model with such a part runs every step eagerly."""
    kind = "?"
    graph_safe = False

    def __init__(self, spec, env: BuildEnv):
        self.spec = spec
        self.env = env

    @classmethod
    def param_infos(cls, spec) -> Dict[str, ParamInfo]:
        return {}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Receives the declared tensors, already on the device and in the dtype of
        their role (matrix: compute dtype; gain: float32; table: int32)."""

    def weight_bytes(self) -> int:
        return 0

    def reads_first(self) -> Optional[torch.Tensor]:
        """The weight matrix [N, K] of the linear with which this part starts, if it starts
        with one: the norm before it may warm the cache for it (see ``Norm.takes_hint``)."""
        return None


class Norm(Part):
    """``takes_hint``: the norm's ``__call__`` has a fourth argument ``then``, the weight matrix
    that the following part reads first (a performance hint that changes no result)."""
    takes_hint = False

    def __call__(self, resid, delta=None, rows=None):
        raise NotImplementedError


class PositionEncoding(Part):
    def prepare(self, max_positions: int) -> None:
        pass

    def fused_table(self) -> Optional[torch.Tensor]:
        return None

    def apply(self, q, k, ctx: StepContext):
        return q, k


class Mixer(Part):
    def cache_request(self) -> Optional[CacheRequest]:
        return None

    def prepare(self, max_positions: int) -> None:
        pass

    def __call__(self, x, ctx: StepContext, cache):
        raise NotImplementedError


class FeedForward(Part):
    def __call__(self, x, ctx: StepContext):
        raise NotImplementedError
