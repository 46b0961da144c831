"""The plain model against the reference's own float64 model (tests/golden/), and
the plain sampler against the cases of the reference's unit tests."""
import hashlib
import json
import math
import os

import numpy as np
import pytest

import helpers as H
import plain_qwen3 as plain
from tiny_configs import ALL

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _digest(W):
    h = hashlib.sha256()
    for name in sorted(W):
        h.update(name.encode())
        h.update(np.ascontiguousarray(W[name], dtype=np.float64).tobytes())
    return h.hexdigest()


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_model_matches_reference_script(tmp_path, name):
    with open(os.path.join(GOLD, "golden.json")) as f:
        meta = json.load(f)[name]
    cfg, stored = ALL[name]
    d = H.make_model_dir(tmp_path, cfg, meta["seed"], stored=meta["stored"])
    pcfg, W = plain.load_model_dir(d)
    assert _digest(W) == meta["weights_sha256"], "the seeded weights changed: run tests/golden/make_golden.py again"
    want = np.load(os.path.join(GOLD, f"tiny_{name.lower()}_logits.npy")).astype(np.float64)
    got = plain.forward_logits(pcfg, W, meta["ids"])
    assert got.shape == want.shape
    # the golden file is float32: 6e-8 relative
    assert np.abs(got - want).max() <= 2e-7 * np.abs(want).max() + 1e-9


def test_plain_parts():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((3, 4, 16))
    # rope at position 0 is the identity and rotation keeps the norm (src/ops/rope.rs:85-111 there)
    cos, sin = plain.rope_cos_sin(np.array([0, 5, 12345]), 16, 1e6)
    y = plain.apply_rope(x, cos, sin)
    assert np.allclose(y[0], x[0])
    assert np.allclose(np.linalg.norm(y, axis=-1), np.linalg.norm(x, axis=-1))
    # rmsnorm of a constant row
    assert np.allclose(plain.rms_norm(np.full((1, 8), 2.0), np.ones(8), 0.0), 1.0)
    # attention: one key -> its value; window 1 -> own value
    q, k, v = rng.standard_normal((5, 4, 8)), rng.standard_normal((5, 2, 8)), rng.standard_normal((5, 2, 8))
    assert np.allclose(plain.causal_attention(q, k, v)[0], np.repeat(v[0], 2, axis=0))
    assert np.allclose(plain.causal_attention(q, k, v, window=1), np.repeat(v, 2, axis=1))
    assert plain.silu(0.0) == 0.0 and abs(plain.silu(1.0) - 1 / (1 + math.exp(-1))) < 1e-15
    assert plain.bf16_round(np.float32(1.00390625)) == np.float32(1.0)        # tie to even
    assert plain.bf16_round(np.float32(1.01171875)) == np.float32(1.015625)


def test_plain_sampler_reference_cases():
    """The cases of src/sampling.rs:145-187 of the reference."""
    rng = plain.PlainRng(0x5EED)
    assert plain.plain_sample([0.1, 3.0, 2.0], [], rng) == 1
    assert plain.plain_sample([0.1, 3.0, 2.0], [1], rng, repetition_penalty=2.0) == 2
    for _ in range(20):
        assert plain.plain_sample([0.5, 0.4, 0.6, 0.1], [], rng, temperature=1.0, top_k=1) == 2
    logits = [0.0, math.log(3.0)]
    a, b = plain.PlainRng(7), plain.PlainRng(7)
    picks = [plain.plain_sample(logits, [], a, temperature=1.0) for _ in range(4000)]
    assert abs(sum(picks) / 4000 - 0.75) < 0.03
    assert picks == [plain.plain_sample(logits, [], b, temperature=1.0) for _ in range(4000)]
    for _ in range(50):
        assert plain.plain_sample([3.0, 1.0, 0.5, 0.0], [], rng, temperature=1.0, top_p=0.5) == 0


def test_package_rng_is_the_plain_rng():
    from rust_inference_b200.sampling import XorShiftRng, request_seed
    for seed in (0, 7, 0x5EED, (1 << 64) - 1):
        a, b = XorShiftRng(seed), plain.PlainRng(seed)
        assert [a.next_u64() for _ in range(5)] == [b.next_u64() for _ in range(5)]
        assert a.next_f32() == float(b.next_f32())
    assert request_seed(0x5EED, 0) == 0x5EED
    assert len({request_seed(1, i) for i in range(100)}) == 100
