"""A layer: the arrangement of a mixer, a feed-forward and their norms.

"prenorm": each sub-layer reads the normed residual stream and its output is
added to the stream (thanhauco/rust-inference src/models/qwen3.rs:120-146).
The addition is left pending and done by the next norm while it reads the
stream, wherever that norm is: in this block or the next, or the model's final
norm.
"""
from __future__ import annotations

from .registry import build_part


class Block:
    def __init__(self, spec, env):
        if spec.arrangement != "prenorm":
            raise ValueError(f"arrangement {spec.arrangement!r} is not known")
        self.spec = spec
        self.mixer_norm = build_part("norm", spec.mixer_norm, env)
        self.mixer = build_part("mixer", spec.mixer, env)
        self.ffn_norm = build_part("norm", spec.ffn_norm, env)
        self.ffn = build_part("ffn", spec.ffn, env)

    def parts(self):
        """(name in ``LayerSpec.names``, part, family, spec record)"""
        s = self.spec
        return (("mixer_norm", self.mixer_norm, "norm", s.mixer_norm), ("mixer", self.mixer, "mixer", s.mixer),
                ("ffn_norm", self.ffn_norm, "norm", s.ffn_norm), ("ffn", self.ffn, "ffn", s.ffn))

    def __call__(self, resid, delta, ctx, cache):
        x = _norm(self.mixer_norm, resid, delta, self.mixer)
        a = self.mixer(x, ctx, cache)
        x = _norm(self.ffn_norm, resid, a, self.ffn)
        return resid, self.ffn(x, ctx)


def _norm(norm, resid, delta, reader):
    if norm.takes_hint:
        return norm(resid, delta, None, reader.reads_first())
    return norm(resid, delta)
