"""The layer shapes of the large models (Qwen3-8B: width 4096, 32 heads over 8 kv heads of 128,
feed-forward 12288) with two layers and a small vocabulary, replayed whole, with the last 32 tokens
one by one, and in a batch of unequal lengths, in float32 and in bfloat16, against the plain model.

The tiny configurations cannot show what depends on the depth of a product (4096 and 12288 terms
per output: the order of the additions in the float32 linear, the stages a warp of the
weight-streaming linear walks, the split of K) or on four query heads per kv head of 128."""
import numpy as np
import pytest

import helpers as H

pytestmark = pytest.mark.gpu

LARGE_LAYERS = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "intermediate_size": 12288, "vocab_size": 2003, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 4096,
}
LENGTHS = [70, 33, 97]


@pytest.fixture(scope="module")
def large(tmp_path_factory):
    d = H.make_model_dir(tmp_path_factory.mktemp("large"), LARGE_LAYERS, seed=88, stored="bfloat16", name="large")
    reqs = H.random_requests(np.random.default_rng(3), LARGE_LAYERS["vocab_size"], LENGTHS)
    # the weights are stored in bfloat16, so the plain model is the same for both dtypes of the engine
    return d, reqs, H.plain_logits(d, reqs, "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_three_ways_at_large_layer_shapes(tmp_path, large, dtype):
    d, reqs, want = large
    worst = {}
    for label, steps in (("whole", H.trace_whole(reqs)), ("tail", H.trace_tail(reqs, tail=32)),
                         ("batches", H.trace_batches(reqs, 3, [9, 32, 0]))):
        out = str(tmp_path / f"out_{label}")
        H.replay_inprocess(d, dtype, steps, out, device="cuda")
        rows = H.collect(steps, out, LARGE_LAYERS["vocab_size"])
        assert len(rows) == sum(LENGTHS)
        worst[label] = H.assert_rows_close(rows, want, dtype, f"large layers {dtype} {label}")
    print(f"large layers {dtype}: worst error / bound = {worst}")
