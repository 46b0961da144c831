"""The layer shapes of the large models with one or two layers and a small vocabulary, replayed whole,
with the last 32 tokens one by one, and in a batch of unequal lengths, in float32 and in bfloat16,
against the plain model: Qwen3-8B (width 4096, 32 heads over 8 kv heads of 128, feed-forward 12288),
Qwen3-14B (width 5120, 40 heads over 8: five query heads per kv head, feed-forward 17408) and
Qwen3-32B (width 5120 under 64 heads of 128, so heads x head size is not the width; feed-forward 25600).

The tiny configurations cannot show what depends on the depth of a product (4096 and 12288 terms
per output: the order of the additions in the float32 linear, the stages a warp of the
weight-streaming linear walks, the split of K) or on four query heads per kv head of 128."""
import shutil

import numpy as np
import pytest

import helpers as H

pytestmark = pytest.mark.gpu


def _shapes(layers, hidden, heads, inter, vocab):
    return {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": layers,
            "hidden_size": hidden, "num_attention_heads": heads, "num_key_value_heads": 8, "head_dim": 128,
            "intermediate_size": inter, "vocab_size": vocab, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
            "tie_word_embeddings": False, "max_position_embeddings": 4096}


SHAPES = {"8B": _shapes(2, 4096, 32, 12288, 2003), "14B": _shapes(2, 5120, 40, 17408, 1501),
          "32B": _shapes(1, 5120, 64, 25600, 1009)}
LENGTHS = [70, 33, 97]


@pytest.fixture(scope="module", params=list(SHAPES))
def large(request, tmp_path_factory):
    cfg = SHAPES[request.param]
    d = H.make_model_dir(tmp_path_factory.mktemp("large" + request.param), cfg, seed=88, stored="bfloat16", name="large")
    reqs = H.random_requests(np.random.default_rng(3), cfg["vocab_size"], LENGTHS)
    # the weights are stored in bfloat16, so the plain model is the same for both dtypes of the engine
    yield cfg, d, reqs, H.plain_logits(d, reqs, "float32")
    shutil.rmtree(d, ignore_errors=True)          # a few GB of weights: not kept with the test's other files


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_three_ways_at_large_layer_shapes(tmp_path, large, dtype):
    LARGE_LAYERS, d, reqs, want = large
    worst, by_cutting = {}, {}
    for label, steps in (("whole", H.trace_whole(reqs)), ("tail", H.trace_tail(reqs, tail=32)),
                         ("batches", H.trace_batches(reqs, 3, [9, 32, 0]))):
        out = str(tmp_path / f"out_{label}")
        H.replay_inprocess(d, dtype, steps, out, device="cuda")
        rows = H.collect(steps, out, LARGE_LAYERS["vocab_size"])
        assert len(rows) == sum(LENGTHS)
        worst[label] = H.assert_rows_close(rows, want, dtype, f"large layers {dtype} {label}")
        by_cutting[label] = rows
    if dtype == "float32":
        H.assert_rows_identical(by_cutting, "large layers float32")
        shutil.rmtree(out, ignore_errors=True)
    print(f"large layers {dtype}: worst error / bound = {worst}")
