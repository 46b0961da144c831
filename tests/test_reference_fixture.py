"""thanhauco/rust-inference's own checked-in tiny model (tests/fixtures/tiny-qwen3 there: config.json,
a bfloat16 model.safetensors, the prompt with its greedy continuation in expected.json, and the
logits expected_prefill.f32 [11, 3072] / expected_decode.f32 [6, 3072]) read through this package.

The fixture is read from a checkout of the reference, never copied: its folder is
$RUST_INFERENCE_REFERENCE_DIR, or `reference` beside this repository; where neither exists the
tests are skipped.  The tolerance is the one of the reference's own parity test,
2e-4 * max|logit| + 1e-5 (tests/model_parity.rs:23-28 there).
"""
import json
import os

import numpy as np
import pytest

import helpers as H
import plain_qwen3 as plain

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("RUST_INFERENCE_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
FIX = os.path.join(REF, "tests", "fixtures", "tiny-qwen3")

pytestmark = pytest.mark.skipif(not os.path.exists(os.path.join(FIX, "expected_prefill.f32")),
                                reason="no checkout of the reference with its tiny-qwen3 fixture")


def _expected():
    with open(os.path.join(FIX, "expected.json")) as f:
        meta = json.load(f)
    with open(os.path.join(FIX, "config.json")) as f:
        vocab = json.load(f)["vocab_size"]
    pre = np.fromfile(os.path.join(FIX, "expected_prefill.f32"), dtype="<f4").reshape(-1, vocab).astype(np.float64)
    dec = np.fromfile(os.path.join(FIX, "expected_decode.f32"), dtype="<f4").reshape(-1, vocab).astype(np.float64)
    return meta["prompt"], meta["generated"], pre, dec


def _close(got, want, what):
    bound = 2e-4 * np.abs(want).max() + 1e-5
    err = np.abs(np.asarray(got, dtype=np.float64) - want).max()
    assert err <= bound, f"{what}: max error {err:.3e} > {bound:.3e}"


def test_plain_model_on_the_reference_fixture():
    prompt, generated, pre, dec = _expected()
    cfg, W = plain.load_model_dir(FIX)
    assert pre.shape[0] == len(prompt)
    _close(plain.forward_logits(cfg, W, prompt), pre, "prefill logits")
    # decode rows: the logits after each generated token but the last, by whole re-forwards
    whole = plain.forward_logits(cfg, W, prompt + generated[:-1])
    _close(whole[len(prompt):], dec, "decode logits")
    assert plain.generate_plain(cfg, W, prompt, len(generated), ignore_eos=True) == generated


def test_loader_and_engine_on_the_reference_fixture(tmp_path, emulated_ops):
    """The product's configuration, loader, cache and step function (kernels replaced by the slow
    stand-ins) on the reference's files: prompt whole, then its continuation token by token."""
    prompt, generated, pre, dec = _expected()
    steps = [{"step": 0, "entries": [{"id": "r", "tokens": prompt, "want": list(range(len(prompt)))}], "end": []}]
    for i, tok in enumerate(generated[:-1]):
        steps.append({"step": i + 1, "entries": [{"id": "r", "tokens": [tok], "want": [0]}],
                      "end": ["r"] if i == len(generated) - 2 else []})
    out = str(tmp_path / "out")
    H.replay_inprocess(FIX, "float32", steps, out)
    rows = H.collect(steps, out, pre.shape[1])
    got = np.stack([rows[("r", i)] for i in range(len(prompt) + len(generated) - 1)])
    _close(got[:len(prompt)], pre, "prefill logits through the engine")
    _close(got[len(prompt):], dec, "decode logits through the engine")


@pytest.mark.gpu
def test_generate_on_the_reference_fixture():
    """Greedy generation with the real kernels in float32 gives the reference's tokens (its margin
    between the best and the second logit is 0.06 at least)."""
    from rust_inference_b200 import generate
    prompt, generated, _, _ = _expected()
    assert generate(FIX, [prompt], len(generated), dtype="float32", ignore_eos=True) == [generated]
