"""Plain, slow Qwen3-dense model in numpy float64: the yardstick of the test suite.

Whole sequences, no cache, one function for each part, nothing shared with the
package under test (it even reads safetensors files with a reader of its own).
Every function restates a formula of thanhauco/rust-inference and cites the
place (paths are relative to that project's root).  `tests/golden/` holds
logits that the reference's own float64 script produced for a tiny random
model; `tests/test_plain.py` checks this file against them.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np

F64 = np.float64


# ----------------------------------------------------------------------------
# number formats and files
# ----------------------------------------------------------------------------

def bf16_round(x):
    """Round float32 values to the nearest bfloat16 (ties to even), return float32.

    Same integer recipe as `f32_to_bf16`, src/dtype.rs:82-89.
    """
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return u.astype(np.uint32).view(np.float32).reshape(np.shape(x))


def read_safetensors(path):
    """name -> float64 / int64 array.  File layout: src/safetensors.rs:3-6, 56-74."""
    with open(path, "rb") as f:
        raw = f.read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    base = 8 + hlen
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        blob = raw[base + lo:base + hi]
        dt = info["dtype"]
        if dt == "F32":
            arr = np.frombuffer(blob, dtype="<f4").astype(F64)
        elif dt == "BF16":
            bits = np.frombuffer(blob, dtype="<u2").astype(np.uint32) << 16
            arr = bits.view(np.float32).astype(F64)
        elif dt == "I32":
            arr = np.frombuffer(blob, dtype="<i4").astype(np.int64)
        elif dt == "I64":
            arr = np.frombuffer(blob, dtype="<i8").astype(np.int64)
        else:
            raise ValueError(f"{name}: dtype {dt} not handled by the plain reader")
        out[name] = arr.reshape(info["shape"])
    return out


def load_model_dir(model_dir, round_to_bf16=False):
    """(config dict, weights dict) of a folder with config.json and model.safetensors.

    Tensor names are the ones src/models/qwen3.rs:157-188 fetches.
    `round_to_bf16` rounds the matrices (not the norm gains) to bfloat16 first,
    which is what a bfloat16 engine computes with (src/models/cuda.rs:34-58).
    """
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    tensors = read_safetensors(os.path.join(model_dir, "model.safetensors"))
    if round_to_bf16:
        for name, arr in tensors.items():
            if arr.ndim == 2:
                tensors[name] = bf16_round(arr.astype(np.float32)).astype(F64)
    return cfg, tensors


def head_dim_of(cfg):
    """`head_dim` defaults to hidden_size / heads: src/models/config.rs:75-77."""
    hd = cfg.get("head_dim")
    return int(hd) if hd else cfg["hidden_size"] // cfg["num_attention_heads"]


# ----------------------------------------------------------------------------
# parts
# ----------------------------------------------------------------------------

def embedding(ids, table):
    """h[t] = table[ids[t]], no scaling; ids must be < vocab: src/ops/embedding.rs:10-42."""
    ids = np.asarray(ids, dtype=np.int64)
    if ids.size and (ids.min() < 0 or ids.max() >= table.shape[0]):
        raise IndexError("token id out of range")
    return table[ids].astype(F64)


def rms_norm(x, gain, eps):
    """y = x * (1/sqrt(mean(x^2) + eps)) * gain over the last axis: src/ops/norm.rs:7-10, 25-30."""
    x = np.asarray(x, dtype=F64)
    inv = 1.0 / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + F64(eps))
    return x * inv * np.asarray(gain, dtype=F64)


def linear(x, w):
    """y = x W^T with W stored [out, in], no bias: src/ops/linear.rs:7-20."""
    return np.asarray(x, dtype=F64) @ np.asarray(w, dtype=F64).T


def rope_cos_sin(positions, head_dim, theta):
    """cos/sin tables [n, head_dim/2].

    inv_freq[i] = 1 / theta^(2i/head_dim) in float32 (theta itself is parsed as
    float32, src/models/config.rs:33-34), angle = float32(pos) * inv_freq[i] as a
    float32 product, the second half of the head repeats the first:
    src/ops/rope.rs:19-47.  cos and sin of that float32 angle are taken in float64.
    """
    half = head_dim // 2
    th = np.float32(theta)
    inv_freq = np.array(
        [np.float32(1.0) / np.power(th, np.float32(2 * i) / np.float32(head_dim), dtype=np.float32) for i in range(half)],
        dtype=np.float32,
    )
    ang = np.asarray(positions, dtype=np.float32)[:, None] * inv_freq[None, :]
    ang = ang.astype(np.float32).astype(F64)
    return np.cos(ang), np.sin(ang)


def apply_rope(x, cos, sin):
    """Rotate-half on x [n, heads, head_dim]:
    y[d] = x[d] cos[d] - x[d+half] sin[d];  y[d+half] = x[d+half] cos[d] + x[d] sin[d]
    (src/ops/rope.rs:52-79; both halves of the table are equal)."""
    half = x.shape[-1] // 2
    lo, hi = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return np.concatenate([lo * c - hi * s, hi * c + lo * s], axis=-1)


def causal_attention(q, k, v, window=0):
    """Grouped-query causal attention of one whole sequence.

    q [n, H, Dh], k and v [n, KV, Dh].  Query head h reads kv head h // (H/KV);
    query t sees keys 0..t; score = (q.k) / sqrt(Dh); softmax in one piece
    (the reference does it a page at a time with the same result):
    src/attention.rs:4-8, 26-29, 111-150.  `window` > 0 keeps only the last
    `window` keys (t-window+1..t); the reference has no window, the engine's
    attention part takes one as a parameter.
    """
    n, H, Dh = q.shape
    KV = k.shape[1]
    G = H // KV
    scale = 1.0 / math.sqrt(Dh)
    out = np.zeros((n, H, Dh), dtype=F64)
    for h in range(H):
        kh, vh = k[:, h // G, :], v[:, h // G, :]
        for t in range(n):
            first = max(0, t - window + 1) if window > 0 else 0
            s = (kh[first:t + 1] @ q[t, h]) * scale
            p = np.exp(s - s.max())
            out[t, h] = (p / p.sum()) @ vh[first:t + 1]
    return out


def attention_block(x, W, p, cfg, positions):
    """q/k/v projections, per-head RMSNorm of q and k, RoPE, attention, output
    projection, in that order: src/models/qwen3.rs:71-100."""
    n = x.shape[0]
    H, KV, Dh = cfg["num_attention_heads"], cfg["num_key_value_heads"], head_dim_of(cfg)
    eps = cfg.get("rms_norm_eps", 1e-6)
    q = linear(x, W[p + "q_proj.weight"]).reshape(n, H, Dh)
    k = linear(x, W[p + "k_proj.weight"]).reshape(n, KV, Dh)
    v = linear(x, W[p + "v_proj.weight"]).reshape(n, KV, Dh)
    q = rms_norm(q, W[p + "q_norm.weight"], eps)          # one gain vector for all heads,
    k = rms_norm(k, W[p + "k_norm.weight"], eps)          # src/models/qwen3.rs:86-89
    cos, sin = rope_cos_sin(positions, Dh, cfg.get("rope_theta", 1e6))
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    o = causal_attention(q, k, v).reshape(n, H * Dh)
    return linear(o, W[p + "o_proj.weight"])


def silu(t):
    """t / (1 + exp(-t)): src/ops/elementwise.rs:10-12."""
    return t / (1.0 + np.exp(-t))


def swiglu_mlp(x, W, p):
    """down(silu(gate x) * up x), no biases: src/models/qwen3.rs:103-118."""
    g = linear(x, W[p + "gate_proj.weight"])
    u = linear(x, W[p + "up_proj.weight"])
    return linear(silu(g) * u, W[p + "down_proj.weight"])


def decoder_layer(h, W, i, cfg, positions):
    """norm -> attention -> residual add -> norm -> MLP -> residual add:
    src/models/qwen3.rs:120-146."""
    p = f"model.layers.{i}."
    eps = cfg.get("rms_norm_eps", 1e-6)
    a = attention_block(rms_norm(h, W[p + "input_layernorm.weight"], eps), W, p + "self_attn.", cfg, positions)
    r = h + a
    y = swiglu_mlp(rms_norm(r, W[p + "post_attention_layernorm.weight"], eps), W, p + "mlp.")
    return r + y


def lm_head_weight(cfg, W):
    """Tied when the flag says so or when the tensor is absent: src/models/qwen3.rs:166-171."""
    if cfg.get("tie_word_embeddings", False) or "lm_head.weight" not in W:
        return W["model.embed_tokens.weight"]
    return W["lm_head.weight"]


def forward_logits(cfg, W, ids):
    """Logits [n, vocab] of one whole sequence, positions 0..n-1:
    src/models/qwen3.rs:255-287 with LogitsMode::All."""
    positions = np.arange(len(ids))
    h = embedding(ids, W["model.embed_tokens.weight"])
    for i in range(cfg["num_hidden_layers"]):
        h = decoder_layer(h, W, i, cfg, positions)
    h = rms_norm(h, W["model.norm.weight"], cfg.get("rms_norm_eps", 1e-6))
    return linear(h, lm_head_weight(cfg, W))


# ----------------------------------------------------------------------------
# sampling and generation
# ----------------------------------------------------------------------------

MASK64 = (1 << 64) - 1


class PlainRng:
    """splitmix64-mixed seed, xorshift64*, u = (x >> 40) / 2^24: src/sampling.rs:28-54."""

    def __init__(self, seed):
        z = (seed + 0x9E3779B97F4A7C15) & MASK64
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
        self.state = (z ^ (z >> 31)) | 1

    def next_u64(self):
        x = self.state
        x ^= x >> 12
        x = (x ^ (x << 25)) & MASK64
        x ^= x >> 27
        self.state = x
        return (x * 0x2545F4914F6CDD1D) & MASK64

    def next_f32(self):
        return np.float32(self.next_u64() >> 40) / np.float32(1 << 24)


def plain_argmax(row):
    """First index of the maximum: src/sampling.rs:132-140."""
    best = 0
    for i, x in enumerate(row):
        if x > row[best]:
            best = i
    return best


def plain_sample(logits, history, rng, temperature=0.0, top_k=0, top_p=1.0, repetition_penalty=1.0):
    """One draw, following src/sampling.rs:73-128 line by line in float32."""
    logits = np.array(logits, dtype=np.float32)
    if repetition_penalty != 1.0:
        pen = np.float32(repetition_penalty)
        for t in set(int(t) for t in history):
            if 0 <= t < len(logits):
                logits[t] = logits[t] / pen if logits[t] > 0 else logits[t] * pen
    if temperature <= 0.0:
        return int(np.argmax(logits))  # numpy also returns the first maximum
    cand = [(i, np.float32(l) / np.float32(temperature)) for i, l in enumerate(logits)]
    if 0 < top_k < len(cand):
        cand.sort(key=lambda c: -c[1])
        cand = cand[:top_k]
    cand.sort(key=lambda c: (-c[1], c[0]))
    mx = cand[0][1]
    probs = np.array([np.exp(np.float32(c[1] - mx)) for c in cand], dtype=np.float32)
    total = np.float32(0)
    for q in probs:
        total = np.float32(total + q)
    probs = (probs / total).astype(np.float32)
    if top_p < 1.0:
        acc, keep = np.float32(0), len(probs)
        for i, q in enumerate(probs):
            acc = np.float32(acc + q)
            if acc >= np.float32(top_p):
                keep = i + 1
                break
        probs = probs[:keep]
        total = np.float32(0)
        for q in probs:
            total = np.float32(total + q)
        probs = (probs / total).astype(np.float32)
    r = rng.next_f32()
    acc = np.float32(0)
    for c, q in zip(cand, probs):
        acc = np.float32(acc + q)
        if r < acc:
            return int(c[0])
    return int(cand[len(probs) - 1][0])


def generate_plain(cfg, W, prompt, max_new_tokens, stop_ids=(), ignore_eos=False, rng=None, **sampling):
    """One sequence: whole re-forward for every token (no cache), loop as in
    src/bin/runner.rs:264-314 — the stop token is not emitted, the first sampled
    token counts toward max_new_tokens."""
    rng = rng or PlainRng(sampling.pop("seed", 0x5EED))
    sampling.pop("seed", None)
    seq, out = list(prompt), []
    while len(out) < max_new_tokens:
        logits = forward_logits(cfg, W, seq)[-1]
        nxt = plain_sample(logits, seq, rng, **sampling)
        if not ignore_eos and nxt in stop_ids:
            break
        out.append(nxt)
        seq.append(nxt)
    return out
