"""Next-token selection: options, the random stream and the device sampler.

Options and their meaning are thanhauco/rust-inference's (src/sampling.rs:8-27):
temperature 0 means greedy, top_k 0 and top_p 1.0 switch those filters off,
repetition_penalty 1.0 switches the penalty off, seed 0x5EED.  The random
stream is its xorshift64* (src/sampling.rs:28-54).  The selection itself runs
on the device (``csrc/sampling.cu``); only the chosen ids come back.

The reference draws for one sequence from one stream.  A batch here gives every
request a stream of its own, seeded from (seed, request index), so what a
request draws does not depend on what it is batched with; request 0 has the
reference's stream.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..profiler import section

_MASK = (1 << 64) - 1


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    repetition_penalty: float = 1.0
    seed: int = 0x5EED

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    def validate(self) -> None:
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError("top_p must be in (0, 1]")
        if not (self.repetition_penalty > 0.0):
            raise ValueError("repetition_penalty must be positive")


class XorShiftRng:
    """splitmix64 of the seed, then xorshift64*; ``next_f32`` is uniform in [0, 1)."""

    def __init__(self, seed: int):
        z = (seed + 0x9E3779B97F4A7C15) & _MASK
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
        self.state = (z ^ (z >> 31)) | 1

    def next_u64(self) -> int:
        x = self.state
        x ^= x >> 12
        x = (x ^ (x << 25)) & _MASK
        x ^= x >> 27
        self.state = x
        return (x * 0x2545F4914F6CDD1D) & _MASK

    def next_f32(self) -> float:
        return float(np.float32(self.next_u64() >> 40) / np.float32(1 << 24))


def request_seed(seed: int, request_index: int) -> int:
    return (seed ^ ((request_index * 0x9E3779B97F4A7C15) & _MASK)) & _MASK


class _Staging:
    """Small host arrays on their way to the device without stalling the host.

    A copy from ordinary host memory waits for everything the stream holds, which would make
    the host wait for the whole step it has just launched.  So the arrays go through a ring of
    pinned buffers, each guarded by an event that says its last copy is done."""

    def __init__(self, device, entries: int = 12):
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.bufs: List[Optional[torch.Tensor]] = [None] * entries
        self.events = [None] * entries
        self.next = 0

    def put(self, arr: np.ndarray) -> torch.Tensor:
        arr = np.ascontiguousarray(arr)
        if not self.cuda:
            return torch.from_numpy(arr.copy())
        i = self.next
        self.next = (i + 1) % len(self.bufs)
        buf = self.bufs[i]
        if buf is None or buf.numel() < arr.nbytes:
            buf = self.bufs[i] = torch.empty(max(256, 2 * arr.nbytes), dtype=torch.uint8, pin_memory=True)
            self.events[i] = torch.cuda.Event()
        else:
            self.events[i].synchronize()                      # its last copy (several steps ago) is done
        host = buf[:arr.nbytes].view(_TORCH_OF[arr.dtype.type])
        host.numpy()[...] = arr.reshape(-1)
        dev = host.to(self.device, non_blocking=True).view(arr.shape)
        self.events[i].record()
        return dev


_TORCH_OF = {np.float32: torch.float32, np.int32: torch.int32, np.int64: torch.int64}


class Sampler:
    """Samples for the rows of one batch.  ``rows`` are the batch's own row numbers
    (0..n-1, fixed for a sequence's life); they index the random streams and the
    context maps of the repetition penalty."""

    def __init__(self, params: SamplingParams, vocab_size: int, device):
        params.validate()
        self.params = params
        self.vocab = vocab_size
        self.device = torch.device(device)
        self.rngs: List[XorShiftRng] = []
        self.seen: Optional[torch.Tensor] = None
        self._const = None
        self._staging = _Staging(self.device)

    @property
    def uses_context(self) -> bool:
        return self.params.repetition_penalty != 1.0

    def begin_batch(self, request_indices: Sequence[int], prompts: Sequence[Sequence[int]]) -> None:
        p = self.params
        n = len(request_indices)
        self.rngs = [XorShiftRng(request_seed(p.seed, i)) for i in request_indices]
        dev = self.device
        self._const = dict(
            temperature=torch.full((n,), float(p.temperature), dtype=torch.float32, device=dev),
            top_k=torch.full((n,), int(p.top_k), dtype=torch.int32, device=dev),
            top_p=torch.full((n,), float(p.top_p), dtype=torch.float32, device=dev),
            penalty=torch.full((n,), float(p.repetition_penalty), dtype=torch.float32, device=dev))
        if self.uses_context:
            self.seen = torch.zeros((n, self.vocab), dtype=torch.uint8, device=dev)
            rows = np.concatenate([np.full(len(pr), r, dtype=np.int32) for r, pr in enumerate(prompts)])
            toks = np.concatenate([np.asarray(pr, dtype=np.int32) for pr in prompts])
            self.note_tokens(rows, toks)
        else:
            self.seen = None

    def note_tokens(self, rows, tokens) -> None:
        """Tokens that entered the context of ``rows`` (needed by the repetition penalty);
        ``tokens`` may be a device tensor."""
        if self.seen is None or len(rows) == 0:
            return
        r = self._staging.put(np.asarray(rows, dtype=np.int32))
        if isinstance(tokens, torch.Tensor):
            t = tokens.to(device=self.device, dtype=torch.int32).contiguous()
        else:
            t = self._staging.put(np.asarray(tokens, dtype=np.int32))
        ops.mark_seen(self.seen, r, t)

    def sample(self, logits: torch.Tensor, rows: Sequence[int]) -> List[int]:
        """One token for each row of ``logits`` [len(rows), vocab], read back to the host."""
        return self.sample_device(logits, rows).tolist()

    def sample_device(self, logits: torch.Tensor, rows: Sequence[int]) -> torch.Tensor:
        """The same, left on the device (int32 [len(rows)]): the next step can be fed from it
        before the host has seen the ids."""
        with section("sampling"):
            return self._sample_device(logits, rows)

    def _sample_device(self, logits: torch.Tensor, rows: Sequence[int]) -> torch.Tensor:
        p = self.params
        n = len(rows)
        if p.greedy and not self.uses_context:
            return ops.argmax(logits)
        c = self._const
        contiguous = list(rows) == list(range(n))
        idx = None if contiguous else self._staging.put(np.asarray(rows, dtype=np.int64))

        def take(t):
            return t[:n] if contiguous else t[idx].contiguous()
        # the reference draws a number only when it does not take the greedy path
        u = [0.0 if p.greedy else self.rngs[r].next_f32() for r in rows]
        uniform = self._staging.put(np.asarray(u, dtype=np.float32))
        seen_rows = self._staging.put(np.asarray(rows, dtype=np.int32)) if self.seen is not None else None
        out = ops.sample(logits, take(c["temperature"]), uniform, top_k=take(c["top_k"]), top_p=take(c["top_p"]),
                         penalty=take(c["penalty"]), seen=self.seen, seen_rows=seen_rows,
                         uses_top_k=p.top_k > 0, uses_top_p=p.top_p < 1.0)
        return out
