"""The generation loop above the step function.

For one sequence the loop is thanhauco/rust-inference's (src/bin/runner.rs:264-314):
run the prompt, sample; then, until a stop token comes (it is not emitted) or
``max_new_tokens`` tokens are out (the first sampled token counts), feed the
last token and sample again.  Around that loop: requests are run in batches of
unequal prompts that start together; a sequence that ends leaves the batch and
gives its slot and pages back at once; when a batch is empty the next one
starts, on the same slots and pages, until no request is left.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field

import torch
from typing import Iterable, List, Optional, Sequence

from ..sampling import Sampler, SamplingParams
from .engine import Entry


@dataclass
class GenerationStats:
    prefill_tokens: int = 0
    prefill_s: float = 0.0
    decode_tokens: int = 0
    decode_steps: int = 0
    decode_s: float = 0.0
    batches: int = 0
    # one entry per decode step: (seconds from the end of the step before to this step's ids on the host, tokens)
    decode_step_s: List[tuple] = field(default_factory=list)


@dataclass
class GenerationResult:
    tokens: List[List[int]]
    finish_reasons: List[str]
    stats: GenerationStats = field(default_factory=GenerationStats)


@dataclass
class _Seq:
    request: int
    row: int
    slot: int
    prompt: Sequence[int]
    out: List[int] = field(default_factory=list)


class _Pending:
    """Sampled ids of a step on their way to the host (pinned buffer, event)."""

    def __init__(self, ids, seqs):
        self.ids, self.seqs = ids, seqs
        self.host = torch.empty(ids.shape, dtype=ids.dtype, pin_memory=True)
        self.host.copy_(ids, non_blocking=True)
        self.event = torch.cuda.Event()
        self.event.record()

    def wait(self):
        self.event.synchronize()
        return self.host.tolist()


def plan_batches(prompt_lens: Sequence[int], max_new_tokens: int, max_seqs: int, page_size: int, num_pages: int,
                 max_seq_len: int, batch_size: Optional[int] = None) -> List[List[int]]:
    """Cut the requests, in order, into batches that fit the cache: at most
    ``max_seqs`` (and ``batch_size``) sequences, and pages for every sequence's
    prompt plus what it may generate."""
    limit = min(max_seqs, batch_size) if batch_size else max_seqs
    batches, cur, cur_pages = [], [], 0
    for i, n in enumerate(prompt_lens):
        if n <= 0:
            raise ValueError(f"request {i} has an empty prompt")
        if n > max_seq_len:
            raise ValueError(f"request {i}: a prompt of {n} tokens exceeds the longest sequence the cache holds ({max_seq_len})")
        need = -(-min(n + max_new_tokens, max_seq_len) // page_size)
        if need > num_pages:
            raise ValueError(f"request {i} needs {need} pages, the cache has {num_pages}")
        if cur and (len(cur) >= limit or cur_pages + need > num_pages):
            batches.append(cur)
            cur, cur_pages = [], 0
        cur.append(i)
        cur_pages += need
    if cur:
        batches.append(cur)
    return batches


def generate(engine, prompts: Sequence[Sequence[int]], max_new_tokens: int = 64,
             sampling: Optional[SamplingParams] = None, stop_ids: Optional[Iterable[int]] = None,
             ignore_eos: bool = False, batch_size: Optional[int] = None, sampler=None,
             pipelined: Optional[bool] = None) -> GenerationResult:
    """Generate for every prompt; ``tokens[i]`` are the new tokens of request i.

    ``stop_ids`` default to the model's (config.json ``eos_token_id``); with
    ``ignore_eos`` they are not looked at.  A sequence also ends when it fills
    the longest sequence the cache holds.  ``pipelined`` chooses between the two
    loops below (default: the pipelined one on a GPU); both give the same tokens."""
    sampling = sampling or SamplingParams()
    spec = engine.model.spec
    stops = frozenset(spec.stop_ids if stop_ids is None else stop_ids)
    cache = engine.cache
    result = GenerationResult([[] for _ in prompts], ["" for _ in prompts])
    if max_new_tokens <= 0 or not prompts:
        result.finish_reasons = ["length"] * len(prompts)
        return result
    sampler = sampler or Sampler(sampling, spec.vocab_size, engine.device)
    batches = plan_batches([len(p) for p in prompts], max_new_tokens, cache.slots.num_slots, cache.page_size,
                           cache.num_pages, engine.max_seq_len, batch_size)
    stats = result.stats
    can_pipeline = hasattr(engine, "step_device_ids") and engine.device.type == "cuda"
    pipelined = can_pipeline if pipelined is None else (bool(pipelined) and can_pipeline)
    for batch in batches:
        stats.batches += 1
        live = [_Seq(req, row, engine.new_sequence(), prompts[req]) for row, req in enumerate(batch)]
        sampler.begin_batch(batch, [prompts[r] for r in batch])

        def finish(s, reason):
            result.tokens[s.request] = s.out
            result.finish_reasons[s.request] = reason
            engine.release(s.slot)
            s.slot = -1

        def accept(s, t):
            """Take the sampled token t for sequence s; True while s goes on."""
            if not ignore_eos and t in stops:
                finish(s, "stop")
                return False
            s.out.append(int(t))
            if len(s.out) >= max_new_tokens:
                finish(s, "length")
                return False
            if len(s.prompt) + len(s.out) > engine.max_seq_len:
                finish(s, "cache")
                return False
            return True

        def goes_on_after_one_more(s):
            """Whether s, if its pending token is no stop token, will be fed that token."""
            return len(s.out) + 1 < max_new_tokens and len(s.prompt) + len(s.out) + 1 <= engine.max_seq_len

        t0 = time.perf_counter()
        try:
            logits = engine.step([Entry(s.slot, s.prompt, "last") for s in live])
            if not pipelined:
                # ---- plain loop: sample, read the ids, decide, feed ------------------------------------
                first = True
                while True:
                    toks = sampler.sample(logits, [s.row for s in live])       # reads the ids back: a sync
                    now = time.perf_counter()
                    if first:
                        stats.prefill_s += now - t0
                        stats.prefill_tokens += sum(len(s.prompt) for s in live)
                        first = False
                    else:
                        stats.decode_s += now - t0
                        stats.decode_steps += 1
                        stats.decode_tokens += len(live)
                        stats.decode_step_s.append((now - t0, len(live)))
                    t0 = now
                    live = [s for s, t in zip(live, toks) if accept(s, t)]
                    if not live:
                        break
                    sampler.note_tokens([s.row for s in live], [s.out[-1] for s in live])
                    logits = engine.step([Entry(s.slot, [s.out[-1]], "last") for s in live])
            else:
                # ---- pipelined loop: the next step is fed from the device and launched before the
                # host reads the ids of this one.  Which sequences end by a stop token is known one
                # step late: such a sequence runs one step too many, whose token is thrown away.
                seqs = live
                handle = _Pending(sampler.sample_device(logits, [s.row for s in seqs]), seqs)
                handle.event.synchronize()            # the prompt step is timed on its own
                stats.prefill_s += time.perf_counter() - t0
                stats.prefill_tokens += sum(len(s.prompt) for s in seqs)
                t0 = time.perf_counter()
                first = True
                while handle is not None:
                    cont = [s for s in handle.seqs if s.slot >= 0 and goes_on_after_one_more(s)]
                    nxt = None
                    if cont:
                        ids = handle.ids
                        if len(cont) != len(handle.seqs):
                            where = {id(s): i for i, s in enumerate(handle.seqs)}
                            idx = torch.tensor([where[id(s)] for s in cont], dtype=torch.int64, device=ids.device)
                            ids = ids.index_select(0, idx)
                        sampler.note_tokens([s.row for s in cont], ids)
                        logits = engine.step_device_ids([s.slot for s in cont], ids)
                        nxt = _Pending(sampler.sample_device(logits, [s.row for s in cont]), cont)
                    toks = handle.wait()
                    if first:
                        first = False                 # the prompt step's ids: already counted
                    else:
                        now = time.perf_counter()
                        stats.decode_s += now - t0
                        stats.decode_steps += 1
                        n_live = sum(1 for s in handle.seqs if s.slot >= 0)
                        stats.decode_tokens += n_live
                        stats.decode_step_s.append((now - t0, n_live))
                        t0 = now
                    for s, t in zip(handle.seqs, toks):
                        if s.slot >= 0:               # else: it had ended, this was its step too many
                            accept(s, t)
                    handle = nxt
                live = []
        finally:
            for s in live:
                if s.slot >= 0:
                    engine.release(s.slot)
        engine.check_device_errors()
    return result
