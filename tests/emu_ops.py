"""Slow torch stand-ins for the CUDA kernels, for tests that run without a GPU.

They have the signatures of ``rust_inference_b200.ops`` and exist only so that
the host logic of the engine (packing, cache, slots, generation loop, trace
replay) can be exercised on the CPU.  They are no part of the product: the
package never imports this file, and on a GPU the tests use the real kernels.
"""
from __future__ import annotations

import math

import numpy as np
import torch

__all__ = ["embed", "rmsnorm", "add_rows", "silu_mul", "linear_swiglu", "linear", "qk_norm_rope_append", "attention", "argmax",
           "sample", "mark_seen"]


def embed(ids, table):
    return table[ids.long()].float()


def rmsnorm(resid, gain, eps, out_dtype, delta=None, rows=None, then=None):
    if rows is not None:
        x = resid[rows.long()]
        if delta is not None:
            x = x + delta[rows.long()].float()
    else:
        if delta is not None:
            resid += delta.float()
        x = resid
    inv = 1.0 / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return (x * inv * gain).to(out_dtype)


def add_rows(resid, delta):
    resid += delta.float()


def silu_mul(gate_up, block=None):
    rows, two = gate_up.shape
    inter = two // 2
    block = block or inter
    v = gate_up.float().view(rows, inter // block, 2, block)
    g, u = v[:, :, 0, :].reshape(rows, inter), v[:, :, 1, :].reshape(rows, inter)
    return ((g / (1.0 + torch.exp(-g))) * u).to(gate_up.dtype)


def linear_swiglu(x, w_gate_up, block):
    return silu_mul(linear(x, w_gate_up), block)


def linear(x, w, out_dtype=None):
    y = x.double() @ w.double().t()
    return y.to(out_dtype or x.dtype)


def qk_norm_rope_append(qkv, num_heads, num_kv_heads, head_dim, q_gain, k_gain, eps, rope_table, rotary_dim, k_pool,
                        v_pool, page_table, tok_seq, tok_pos, seq_slot, write_kv=True):
    T = qkv.shape[0]
    H, KV, Dh = num_heads, num_kv_heads, head_dim
    x = qkv.float().view(T, H + 2 * KV, Dh)
    q, k, v = x[:, :H], x[:, H:H + KV], x[:, H + KV:]

    def norm(t, gain):
        if gain is None:
            return t
        return t * (1.0 / torch.sqrt((t * t).mean(-1, keepdim=True) + eps)) * gain

    def rope(t):
        if rope_table is None:
            return t
        half = rotary_dim // 2
        cs = rope_table[tok_pos.long()]            # [T, half, 2]
        c, s = cs[:, None, :, 0], cs[:, None, :, 1]
        lo, hi, rest = t[..., :half], t[..., half:rotary_dim], t[..., rotary_dim:]
        return torch.cat([lo * c - hi * s, hi * c + lo * s, rest], dim=-1)

    q, k = rope(norm(q, q_gain)), rope(norm(k, k_gain))
    if write_kv:
        P = k_pool.shape[2]
        for t in range(T):
            pos = int(tok_pos[t])
            page = int(page_table[int(seq_slot[int(tok_seq[t])]), pos // P])
            assert page >= 0, "write to an unmapped page"
            k_pool[page, :, pos % P, :] = k[t].to(k_pool.dtype)
            v_pool[page, :, pos % P, :] = v[t].to(v_pool.dtype)
    return q.to(qkv.dtype).contiguous()


def attention(q, k_pool, v_pool, page_table, seq_slot, seq_start, seq_len, max_new, scale, window=0):
    T, H, Dh = q.shape
    KV, P = k_pool.shape[1], k_pool.shape[2]
    G = H // KV
    out = torch.zeros_like(q, dtype=torch.float32)
    for b in range(seq_slot.numel()):
        t0, t1, n = int(seq_start[b]), int(seq_start[b + 1]), int(seq_len[b])
        slot = int(seq_slot[b])
        for t in range(t0, t1):
            pos = n - (t1 - t0) + (t - t0)
            first = max(0, pos - window + 1) if window > 0 else 0
            idx = torch.arange(first, pos + 1)
            pages = page_table[slot, (idx // P).long()].long()
            assert (pages >= 0).all(), "read from an unmapped page"
            kk = k_pool[pages, :, (idx % P).long(), :].float()      # [n, KV, Dh]
            vv = v_pool[pages, :, (idx % P).long(), :].float()
            for h in range(H):
                s = (kk[:, h // G, :] @ q[t, h].float()) * scale
                p = torch.softmax(s, dim=0)
                out[t, h] = p @ vv[:, h // G, :]
    return out.to(q.dtype)


def argmax(logits):
    return torch.argmax(logits, dim=-1).to(torch.int32)      # torch returns the first maximum on the CPU


def sample(logits, temperature, uniform, top_k=None, top_p=None, penalty=None, seen=None, seen_rows=None,
           uses_top_k=True, uses_top_p=True):
    from plain_qwen3 import plain_sample

    class _Fixed:
        def __init__(self, u):
            self.u = u

        def next_f32(self):
            return np.float32(self.u)

    out = []
    for r in range(logits.shape[0]):
        hist = []
        pen = float(penalty[r]) if penalty is not None else 1.0
        if seen is not None and pen != 1.0:
            row = int(seen_rows[r]) if seen_rows is not None else r
            hist = torch.nonzero(seen[row]).flatten().tolist()
        out.append(plain_sample(logits[r].numpy(), hist, _Fixed(float(uniform[r])), temperature=float(temperature[r]),
                                top_k=int(top_k[r]) if top_k is not None else 0,
                                top_p=float(top_p[r]) if top_p is not None else 1.0, repetition_penalty=pen))
    return torch.tensor(out, dtype=torch.int32)


def mark_seen(seen, rows, tokens):
    seen[rows.long(), tokens.long()] = 1
