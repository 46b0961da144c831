#!/usr/bin/env python3
"""Makes tests/golden/*.npy: logits of thanhauco/rust-inference's own float64 model
(scripts/reference_qwen3.py, function `forward`) for the tiny random models of the
test suite.  The reference's script is imported from its checkout, not copied:

    python tests/golden/make_golden.py /path/to/rust-inference

It runs on the CPU with numpy only.  tests/test_plain.py compares the plain model
of tests/plain_qwen3.py with these files once; everything else in the suite is
compared with the plain model.  The weights are not stored: the test makes them
again from the seed and checks their digest against golden.json.
"""
import hashlib
import importlib.util
import json
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path[:0] = [os.path.dirname(os.path.dirname(HERE)), os.path.dirname(HERE)]

import plain_qwen3 as plain  # noqa: E402  (only its safetensors reader is used here)
from tiny_configs import ALL  # noqa: E402

CASES = {"A": dict(seed=101, tokens=13), "B": dict(seed=102, tokens=17)}


def digest(W):
    h = hashlib.sha256()
    for name in sorted(W):
        h.update(name.encode())
        h.update(np.ascontiguousarray(W[name], dtype=np.float64).tobytes())
    return h.hexdigest()


def reference_weights(cfg, W):
    """The dict layout that reference_qwen3.forward reads (scripts/reference_qwen3.py:157-187)."""
    layers = []
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        layers.append({
            "input_layernorm": W[p + "input_layernorm.weight"],
            "post_attention_layernorm": W[p + "post_attention_layernorm.weight"],
            "q_proj": W[p + "self_attn.q_proj.weight"], "k_proj": W[p + "self_attn.k_proj.weight"],
            "v_proj": W[p + "self_attn.v_proj.weight"], "o_proj": W[p + "self_attn.o_proj.weight"],
            "q_norm": W[p + "self_attn.q_norm.weight"], "k_norm": W[p + "self_attn.k_norm.weight"],
            "mlp": {k: W[p + f"mlp.{k}.weight"] for k in ("gate_proj", "up_proj", "down_proj")}})
    head = W["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else W["lm_head.weight"]
    return {"embed": W["model.embed_tokens.weight"], "layers": layers, "norm": W["model.norm.weight"], "lm_head": head}


def main(ref_root):
    spec = importlib.util.spec_from_file_location("reference_qwen3", os.path.join(ref_root, "scripts", "reference_qwen3.py"))
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    from rust_inference_b200.weights import write_random_model
    meta = {}
    for name, case in CASES.items():
        cfg, stored = ALL[name]
        with tempfile.TemporaryDirectory() as tmp:
            d = write_random_model(dict(cfg), case["seed"], os.path.join(tmp, "m"), dtype=stored)
            pcfg, W = plain.load_model_dir(d)
        ids = [int(t) for t in np.random.default_rng(case["seed"]).integers(0, cfg["vocab_size"], size=case["tokens"])]
        logits = ref.forward(dict(pcfg), reference_weights(pcfg, W), ids)
        np.save(os.path.join(HERE, f"tiny_{name.lower()}_logits.npy"), logits.astype(np.float32))
        meta[name] = {"seed": case["seed"], "ids": ids, "stored": stored, "weights_sha256": digest(W)}
        print(name, logits.shape, "max |logit|", float(np.abs(logits).max()))
    with open(os.path.join(HERE, "golden.json"), "w") as f:
        json.dump(meta, f, indent=1)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
