"""SwiGLU feed-forward: down(silu(gate x) * up x), no biases
(thanhauco/rust-inference src/models/qwen3.rs:103-118).  The gate and up
matrices are stacked at load, so one matrix product gives both."""
from __future__ import annotations

import torch

from .. import ops
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
        self.gate_up = torch.cat([tensors["gate_proj.weight"], tensors["up_proj.weight"]], dim=0).contiguous()
        self.down = tensors["down_proj.weight"].contiguous()

    def weight_bytes(self):
        return (self.gate_up.numel() + self.down.numel()) * self.gate_up.element_size()

    def __call__(self, x, ctx):
        return ops.linear(ops.silu_mul(ops.linear(x, self.gate_up)), self.down)
