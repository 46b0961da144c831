"""Trace replay on the GPU: the same requests whole, with the last 32 tokens one by
one, and in batches of unequal lengths (one batch after another, so that slots and
pages are used again), in float32 and in bfloat16, against the plain model."""
import numpy as np
import pytest

import helpers as H
from tiny_configs import ALL

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 9, 13, 1, 40, 34, 70, 100], "B": [1, 17, 33, 64, 65, 150, 2, 96], "C": [300, 47, 129, 33, 520],
           "D": [200, 65, 129, 1, 300, 40]}


@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    base = tmp_path_factory.mktemp("models")
    return {name: H.make_model_dir(base, cfg, seed=21 + i, stored=stored, name=name)
            for i, (name, (cfg, stored)) in enumerate(ALL.items())}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_replay_three_ways(tmp_path, model_dirs, name, dtype):
    cfg, _ = ALL[name]
    d = model_dirs[name]
    rng = np.random.default_rng(7)
    reqs = H.random_requests(rng, cfg["vocab_size"], LENGTHS[name])
    want = H.plain_logits(d, reqs, dtype)
    worst, by_cutting = {}, {}
    for label, steps in (("whole", H.trace_whole(reqs)), ("tail", H.trace_tail(reqs, tail=32)),
                         ("batches", H.trace_batches(reqs, 3, [8, 3, 12, 0, 33]))):
        out = str(tmp_path / f"out_{label}")
        H.replay_subprocess(d, dtype, steps, out)
        rows = H.collect(steps, out, cfg["vocab_size"])
        assert len(rows) == sum(len(t) for t in reqs.values())
        worst[label] = H.assert_rows_close(rows, want, dtype, f"{name} {dtype} {label}")
        by_cutting[label] = rows
    if dtype == "float32":
        H.assert_rows_identical(by_cutting, f"{name} float32")
    print(f"{name} {dtype}: worst error / bound = {worst}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["E", "F", "G", "H"])
def test_odd_sizes(tmp_path, name, dtype):
    """Sizes at the edges of what the kernels take, or beyond them where another kernel stands in (see
    tiny_configs.ODD): whole requests, the last 32 tokens one by one, and a batch that shrinks, against the plain
    model; in float32 the rows of the cuttings are the same bits."""
    from tiny_configs import ODD
    cfg, stored = ODD[name]
    d = H.make_model_dir(tmp_path, cfg, seed=40 + ord(name), stored=stored, name=name)
    reqs = H.random_requests(np.random.default_rng(ord(name)), cfg["vocab_size"], [70, 33, 1, 140, 65])
    want = H.plain_logits(d, reqs, dtype)
    by_cutting = {}
    for label, steps in (("whole", H.trace_whole(reqs)), ("tail", H.trace_tail(reqs, tail=32)),
                         ("batches", H.trace_batches(reqs, 5, [20, 3, 0, 40, 33]))):
        out = str(tmp_path / f"out_{label}")
        H.replay_inprocess(d, dtype, steps, out, device="cuda")
        by_cutting[label] = H.collect(steps, out, cfg["vocab_size"])
        H.assert_rows_close(by_cutting[label], want, dtype, f"odd sizes {name} {dtype} {label}")
    if dtype == "float32":
        H.assert_rows_identical(by_cutting, f"odd sizes {name}")
