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
import plain_qwen3 as plain

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


# ---- the full width of Qwen3-8B with its real output head, without a file -------------------------------------
#
# 2 of the 36 layers, every other size as in Qwen3-8B (vocabulary 151,936 under a separate head of width 4,096).
# The engine's model is made on the device by the function that bench.py uses (Model.from_random); the plain
# model gets the same tensors from the host code of the same rule (value = f(seed, name, index)), the embedding
# only row by row for the ids in use.

FULL_8B = dict(_shapes(2, 4096, 32, 12288, 151936), num_hidden_layers=2)
FULL_SEED = 5


class _EmbeddingRows:
    """table[ids] and table.shape of the embedding, its rows made one at a time."""

    def __init__(self, name, vocab, width, round_bf16):
        self.name, self.shape, self.round_bf16 = name, (vocab, width), round_bf16

    def __getitem__(self, ids):
        import torch
        from rust_inference_b200.weights.random_init import random_tensor
        dt = torch.bfloat16 if self.round_bf16 else torch.float32
        rows = [random_tensor(FULL_SEED, self.name, (1, self.shape[1]), "matrix", dt, first_row=int(i)).float().numpy()[0]
                for i in np.asarray(ids).reshape(-1)]
        return np.stack(rows)


def _plain_weights_without_a_file(round_bf16):
    import torch
    from rust_inference_b200.config import config_from_dict
    from rust_inference_b200.engine.model import expected_tensors
    from rust_inference_b200.weights.random_init import random_tensor
    spec = config_from_dict(FULL_8B).to_spec()
    W = {}
    for name, info in expected_tensors(spec).items():
        if name == spec.embedding_name:
            W[name] = _EmbeddingRows(name, info.shape[0], info.shape[1], round_bf16)
            continue
        dt = torch.bfloat16 if (round_bf16 and info.role == "matrix") else torch.float32
        W[name] = random_tensor(FULL_SEED, name, info.shape, info.role, dt).float().numpy()
    return W


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_full_width_with_the_real_output_head(tmp_path, dtype):
    from rust_inference_b200.engine import Model
    reqs = H.random_requests(np.random.default_rng(4), FULL_8B["vocab_size"], LENGTHS)
    W = _plain_weights_without_a_file(round_bf16=(dtype == "bfloat16"))
    want = {rid: plain.forward_logits(FULL_8B, W, toks) for rid, toks in reqs.items()}
    del W
    model = Model.from_random(dict(FULL_8B), FULL_SEED, dtype=dtype, device="cuda:0")
    worst, by_cutting = {}, {}
    for label, steps in (("whole", H.trace_whole(reqs)), ("tail", H.trace_tail(reqs, tail=32)),
                         ("batches", H.trace_batches(reqs, 3, [9, 32, 0]))):
        out = str(tmp_path / f"out_{label}")
        H.replay_inprocess(None, dtype, steps, out, device="cuda", model=model)
        rows = H.collect(steps, out, FULL_8B["vocab_size"])
        assert len(rows) == sum(LENGTHS)
        worst[label] = H.assert_rows_close(rows, want, dtype, f"full width {dtype} {label}")
        by_cutting[label] = rows
        shutil.rmtree(out, ignore_errors=True)
    if dtype == "float32":
        H.assert_rows_identical(by_cutting, "full width float32")
    print(f"Qwen3-8B width, 2 of 36 layers, vocabulary 151,936, {dtype}: worst error / bound = {worst}")


# ---- all 36 layers of Qwen3-8B: the cuttings against each other -------------------------------------------------
#
# The plain model would need minutes on the CPU for this depth, so here the engine is compared with itself: in
# float32 the three cuttings must give the same bits (with 36 layers between a token and its logits, and the real
# head), and the bfloat16 engine must stay close to the float32 one (the reference accepts a cosine above 0.995
# between its bfloat16 GPU path and its float32 path: tests/cuda_parity.rs:154-166).

def test_all_36_layers_cuttings_agree(tmp_path):
    import torch
    from rust_inference_b200.engine import Model
    cfg = dict(FULL_8B, num_hidden_layers=36)
    reqs = H.random_requests(np.random.default_rng(6), cfg["vocab_size"], [70, 33, 97])
    cuttings = (("whole", H.trace_whole(reqs)), ("tail", H.trace_tail(reqs, tail=32)),
                ("batches", H.trace_batches(reqs, 3, [9, 32, 0])))
    rows = {}
    for dtype in ("float32", "bfloat16"):
        model = Model.from_random(dict(cfg), FULL_SEED, dtype=dtype, device="cuda:0")
        for label, steps in cuttings if dtype == "float32" else cuttings[:1]:
            out = str(tmp_path / f"out_{dtype}_{label}")
            H.replay_inprocess(None, dtype, steps, out, device="cuda", model=model)
            rows[(dtype, label)] = H.collect(steps, out, cfg["vocab_size"])
            shutil.rmtree(out, ignore_errors=True)
        del model
        torch.cuda.empty_cache()
    H.assert_rows_identical({label: rows[("float32", label)] for label, _ in cuttings}, "36 layers float32")
    f32, b16 = rows[("float32", "whole")], rows[("bfloat16", "whole")]
    worst_cos, worst_rel = 1.0, 0.0
    for key, a in f32.items():
        b = b16[key].astype(np.float64)
        a = a.astype(np.float64)
        worst_cos = min(worst_cos, float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b))))
        worst_rel = max(worst_rel, float(np.abs(a - b).max() / np.abs(a).max()))
        assert int(np.argmax(a)) == int(np.argmax(b)) or np.sort(a)[-1] - np.sort(a)[-2] < 0.05 * np.abs(a).max()
    print(f"36 layers: bfloat16 against float32 engine: worst cosine {worst_cos:.5f}, worst |diff| / max|logit| {worst_rel:.4f}")
    assert worst_cos > 0.995
