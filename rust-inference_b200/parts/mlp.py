"""SwiGLU feed-forward: down(silu(gate x) * up x), no biases
(thanhauco/rust-inference src/models/qwen3.rs:103-118).  The gate and up
matrices are stacked at load (rows alternating in blocks of 8 channels), so one matrix
product gives both, and for a few tokens its epilogue applies the gate as well."""
from __future__ import annotations

import torch

from .. import ops
from ..profiler import section
from .base import FeedForward
from .registry import ParamInfo, register_ffn


@register_ffn("swiglu")
class SwiGLU(FeedForward):
    graph_safe = True
    @classmethod
    def param_infos(cls, spec):
        D, I = spec.hidden_size, spec.intermediate_size
        return {"gate_proj.weight": ParamInfo((I, D)), "up_proj.weight": ParamInfo((I, D)),
                "down_proj.weight": ParamInfo((D, I))}

    def load(self, tensors):
        g, u = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        inter, width = g.shape
        # gate and up rows alternate in blocks of 8 (when the width allows it), so that a block of
        # 16 output rows of the product holds 8 channels' gate and up and can apply the gate itself
        self.block = 8 if inter % 8 == 0 else inter
        nb = inter // self.block
        self.gate_up = torch.stack([g.view(nb, self.block, width), u.view(nb, self.block, width)], dim=1) \
            .reshape(2 * inter, width).contiguous()
        self.down = tensors["down_proj.weight"].contiguous()

    def weight_bytes(self):
        return (self.gate_up.numel() + self.down.numel()) * self.gate_up.element_size()

    def reads_first(self):
        return self.gate_up

    def __call__(self, x, ctx):
        with section("mlp gate/up"):
            z = ops.linear_swiglu(x, self.gate_up, self.block)
        with section("mlp down"):
            return ops.linear(z, self.down)
