"""Causal grouped-query attention over the paged cache.

Order of work, as in thanhauco/rust-inference src/models/qwen3.rs:71-100:
q/k/v projections (one product with the stacked matrix), per-head RMSNorm of q
and k, position encoding, append k and v to the cache, attention over the
cache, output projection.  Norm, rotation and append are one kernel.

Sizes, the window, the scale, the per-head norm and the position encoding all
come from the spec; the part does not know which model it is in.
"""
from __future__ import annotations

import math

import torch

from .. import ops
from ..profiler import section
from .base import CacheRequest, Mixer, PositionEncoding
from .registry import ParamInfo, build_part, register_mixer


@register_mixer("attention")
class Attention(Mixer):
    graph_safe = True
    def __init__(self, spec, env):
        super().__init__(spec, env)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} heads are not a multiple of {spec.num_kv_heads} kv heads")
        if spec.qk_norm is not None and getattr(spec.qk_norm, "kind", None) != "rmsnorm":
            raise ValueError(f"the attention part norms its heads with RMSNorm inside its kernel; a per-head norm of kind "
                             f"{getattr(spec.qk_norm, 'kind', None)!r} is not built")
        self.position = build_part("position", spec.position, env)
        self.scale = spec.scale or 1.0 / math.sqrt(spec.head_dim)
        self.q_gain = self.k_gain = None

    @classmethod
    def param_infos(cls, spec):
        D, H, KV, Dh = spec.hidden_size, spec.num_heads, spec.num_kv_heads, spec.head_dim
        infos = {"q_proj.weight": ParamInfo((H * Dh, D)), "k_proj.weight": ParamInfo((KV * Dh, D)),
                 "v_proj.weight": ParamInfo((KV * Dh, D)), "o_proj.weight": ParamInfo((D, H * Dh))}
        if spec.qk_norm is not None:
            infos["q_norm.weight"] = ParamInfo((Dh,), "gain")
            infos["k_norm.weight"] = ParamInfo((Dh,), "gain")
        return infos

    def load(self, tensors):
        self.qkv = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]],
                             dim=0).contiguous()
        self.o = tensors["o_proj.weight"].contiguous()
        if self.spec.qk_norm is not None:
            self.q_gain, self.k_gain = tensors["q_norm.weight"], tensors["k_norm.weight"]

    def weight_bytes(self):
        return (self.qkv.numel() + self.o.numel()) * self.qkv.element_size()

    def reads_first(self):
        return self.qkv

    def cache_request(self):
        s = self.spec
        return CacheRequest(kv_heads=s.num_kv_heads, head_dim=s.head_dim, window=s.window)

    def prepare(self, max_positions):
        self.position.prepare(max_positions)

    def __call__(self, x, ctx, cache):
        s = self.spec
        with section("attn q/k/v proj"):
            qkv = ops.linear(x, self.qkv)
        table = self.position.fused_table()
        eps = s.qk_norm.eps if s.qk_norm is not None else 0.0
        meta = (ctx.tok_seq, ctx.tok_pos, ctx.seq_slot)
        with section("attn norm/rope/append"):
            if table is not None or type(self.position).apply is PositionEncoding.apply:
                # norm, rotation (by table, or none) and append in one kernel
                rot = getattr(s.position, "rot", 0) if table is not None else 0
                q = ops.qk_norm_rope_append(qkv, s.num_heads, s.num_kv_heads, s.head_dim, self.q_gain, self.k_gain, eps,
                                            table, rot, cache.k_pool, cache.v_pool, cache.page_table, *meta,
                                            write_kv=cache.writes)
            else:
                # a position encoding with a rule of its own: norm q and k, let it work on them, append
                T, H, KV, Dh = x.shape[0], s.num_heads, s.num_kv_heads, s.head_dim
                qw, kw = H * Dh, KV * Dh
                q = ops.qk_norm_rope_append(qkv[:, :qw].contiguous(), H, 0, Dh, self.q_gain, None, eps, None, 0,
                                            None, None, None, *meta, write_kv=False)
                k = ops.qk_norm_rope_append(qkv[:, qw:qw + kw].contiguous(), KV, 0, Dh, self.k_gain, None, eps, None, 0,
                                            None, None, None, *meta, write_kv=False)
                q, k = self.position.apply(q, k, ctx)
                if cache.writes:
                    kv = torch.cat([k.reshape(T, kw), qkv[:, qw + kw:]], dim=1).contiguous()
                    ops.qk_norm_rope_append(kv, 0, KV, Dh, None, None, eps, None, 0, cache.k_pool, cache.v_pool,
                                            cache.page_table, *meta, write_kv=True)
                q = q.contiguous()
        fast = ops.fast_attention_supported(q.dtype, s.head_dim, cache.page_size)
        with section("attention"):
            if fast and ctx.decode_only:
                out = ops.attention_decode(q, cache.k_pool, cache.v_pool, cache.page_table, ctx.seq_slot, ctx.seq_len,
                                           self.scale, s.window, ctx.len_bucket)
            elif fast:
                out = ops.attention_prefill(q, cache.k_pool, cache.v_pool, cache.page_table, ctx.seq_slot,
                                            ctx.seq_start, ctx.seq_len, ctx.max_new, self.scale, s.window)
            else:
                out = ops.attention(q, cache.k_pool, cache.v_pool, cache.page_table, ctx.seq_slot, ctx.seq_start,
                                    ctx.seq_len, ctx.max_new, self.scale, s.window)
        with section("attn o proj"):
            return ops.linear(out.view(x.shape[0], s.num_heads * s.head_dim), self.o)
