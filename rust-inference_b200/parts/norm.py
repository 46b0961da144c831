"""RMSNorm: y = x * (1 / sqrt(mean(x^2) + eps)) * gain, all in float32
(thanhauco/rust-inference src/ops/norm.rs:7-62).  Reads the float32 residual
stream, adds the pending output of the previous part on the way if there is
one, and writes the normed rows in the compute dtype."""
from __future__ import annotations

from .. import ops
from ..profiler import section
from .base import Norm
from .registry import ParamInfo, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    graph_safe = True
    takes_hint = True

    @classmethod
    def param_infos(cls, spec):
        return {"weight": ParamInfo((spec.size,), "gain")}

    def load(self, tensors):
        self.gain = tensors["weight"]

    def weight_bytes(self):
        return self.gain.numel() * 4

    def __call__(self, resid, delta=None, rows=None, then=None):
        with section("rmsnorm"):
            return ops.rmsnorm(resid, self.gain, self.spec.eps, self.env.dtype, delta=delta, rows=rows, then=then)
