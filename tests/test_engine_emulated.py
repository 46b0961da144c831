"""The engine's host logic on the CPU: packing, cache, slots, trace replay.

The CUDA kernels are replaced by the slow stand-ins of tests/emu_ops.py
(fixture ``emulated_ops``); everything else is the product's own code.  The
same traces run on the real kernels in tests/test_replay_gpu.py."""
import numpy as np
import pytest

import helpers as H
from tiny_configs import ALL


@pytest.mark.parametrize("name", ["A", "B"])
def test_replay_three_ways_matches_plain(tmp_path, emulated_ops, name):
    cfg, stored = ALL[name]
    d = H.make_model_dir(tmp_path, cfg, seed=11, stored=stored)
    rng = np.random.default_rng(5)
    reqs = H.random_requests(rng, cfg["vocab_size"], [5, 9, 13, 1, 40, 34, 70])
    want = H.plain_logits(d, reqs)
    for label, steps in (("whole", H.trace_whole(reqs)), ("tail", H.trace_tail(reqs, tail=32)),
                         ("batches", H.trace_batches(reqs, 3, [8, 3, 12, 0, 5]))):
        out = str(tmp_path / f"out_{label}")
        H.replay_inprocess(d, "float32", steps, out)
        rows = H.collect(steps, out, cfg["vocab_size"])
        assert len(rows) == sum(len(t) for t in reqs.values())
        H.assert_rows_close(rows, want, "float32", label)


def test_step_validation(tmp_path, emulated_ops):
    from rust_inference_b200.engine import Engine, Entry, Model, StepError
    from rust_inference_b200.cache import CacheError
    cfg, stored = ALL["A"]
    d = H.make_model_dir(tmp_path, cfg, seed=1, stored=stored)
    eng = Engine(Model.from_dir(d, "float32", "cpu"), max_tokens=128, max_seqs=2)
    s = eng.new_sequence()
    with pytest.raises(StepError):
        eng.step([Entry(s, [256])])                 # id outside the vocabulary
    with pytest.raises(StepError):
        eng.step([Entry(s, [])])
    with pytest.raises(StepError):
        eng.step([Entry(s, [1, 2], want=[2])])
    with pytest.raises(CacheError):
        eng.step([Entry(s, [1]), Entry(s, [2])])    # a slot twice in one step
    with pytest.raises(CacheError):
        eng.step([Entry(s, list(range(129)))])      # longer than the cache holds
    assert eng.length(s) == 0                        # failed steps left nothing behind
    out = eng.step([Entry(s, [1, 2, 3], want=[])])
    assert out.shape == (0, 256) and eng.length(s) == 3
    eng.cache.check()


def test_step_tables_match_a_plain_construction(tmp_path, emulated_ops):
    """The tables the C++ side writes for a step of unequal sequences (and for the decode steps after
    it, with and without ids on the host), against the same tables put together here in Python."""
    import torch
    from rust_inference_b200.engine import Engine, Entry, Model
    cfg, stored = ALL["A"]
    d = H.make_model_dir(tmp_path, cfg, seed=2, stored=stored)
    eng = Engine(Model.from_dir(d, "float32", "cpu"), max_tokens=512, max_seqs=4)
    seen = {}
    real_forward = eng.model.forward

    def spy(ids, ctx, cache, want_rows):
        seen.update(ids=ids.tolist(), tok_seq=ctx.tok_seq.tolist(), tok_pos=ctx.tok_pos.tolist(),
                    want=want_rows.tolist(), seq_slot=ctx.seq_slot.tolist(), seq_start=ctx.seq_start.tolist(),
                    seq_len=ctx.seq_len.tolist(), max_new=ctx.max_new, max_len=ctx.max_len, T=ctx.num_tokens)
        return real_forward(ids, ctx, cache, want_rows)

    eng.model.forward = spy
    rng = np.random.default_rng(0)
    slots = [eng.new_sequence() for _ in range(3)]
    lens = {s: 0 for s in slots}

    def expect(entries):
        ids, tok_seq, tok_pos, want, start = [], [], [], [], [0]
        for b, (s, toks, w) in enumerate(entries):
            want += [len(ids) + i for i in w]
            ids += toks
            tok_seq += [b] * len(toks)
            tok_pos += list(range(lens[s], lens[s] + len(toks)))
            lens[s] += len(toks)
            start.append(len(ids))
        return dict(ids=ids, tok_seq=tok_seq, tok_pos=tok_pos, want=want, seq_slot=[s for s, _, _ in entries],
                    seq_start=start, seq_len=[lens[s] for s, _, _ in entries],
                    max_new=max(len(t) for _, t, _ in entries), max_len=max(lens[s] for s, _, _ in entries), T=len(ids))

    first = [(slots[2], [int(t) for t in rng.integers(0, 256, 37)], [0, 36, 5]),
             (slots[0], [int(t) for t in rng.integers(0, 256, 1)], []),
             (slots[1], [int(t) for t in rng.integers(0, 256, 70)], list(range(70)))]
    eng.step([Entry(s, t, w) for s, t, w in first])
    assert seen == expect(first)
    for _ in range(3):                               # decode steps with the ids on the host ...
        nxt = [(s, [int(rng.integers(0, 256))], [0]) for s in (slots[1], slots[2])]
        eng.step([Entry(s, t) for s, t, _ in nxt])
        assert seen == expect(nxt)
    ids_dev = torch.tensor([7, 9, 11], dtype=torch.int32)    # ... and with the ids where the sampler left them
    eng.step_device_ids([slots[2], slots[0], slots[1]], ids_dev)
    assert seen == expect([(slots[2], [7], [0]), (slots[0], [9], [0]), (slots[1], [11], [0])])
    mixed = [(slots[0], [3, 4], [1]), (slots[1], [5], [0])]  # a step that is neither: the general path again
    eng.step([Entry(s, t, w) for s, t, w in mixed])
    assert seen == expect(mixed)
