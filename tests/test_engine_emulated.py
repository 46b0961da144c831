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
