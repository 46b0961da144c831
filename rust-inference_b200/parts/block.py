"""A layer: the arrangement of a mixer, a feed-forward and their norms.

"prenorm": each sub-layer reads the normed residual stream and its output is
added to the stream (thanhauco/rust-inference src/models/qwen3.rs:120-146).
The addition is left pending and done by the next norm while it reads the
stream, wherever that norm is: in this block or the next, or the model's final
norm.

An arrangement is a class registered with ``@register_block(kind)`` for the
``arrangement`` of its layer record.  It says which parts the layer has
(``slots``), builds them, and runs them::

    slots(spec) -> ((slot name, family, record), ...)        a class method; the slot name is what
                                                             ``spec.prefix(slot)`` maps to tensor names
    parts()     -> ((slot name, part, family, record), ...)  the built parts, same order
    mixer                                                    the part whose cache request sizes the layer's cache entry
    __call__(resid, delta, ctx, cache) -> (resid, delta)     the float32 stream and the output not yet added
"""
from __future__ import annotations

from .registry import build_part, part_class, register_block


class BlockBase:
    def __init__(self, spec, env):
        self.spec = spec
        self.env = env
        self._parts = tuple((name, build_part(family, record, env), family, record)
                            for name, family, record in self.slots(spec))
        for name, part, _, _ in self._parts:
            setattr(self, name, part)

    @classmethod
    def slots(cls, spec):
        raise NotImplementedError

    def parts(self):
        return self._parts

    def __call__(self, resid, delta, ctx, cache):
        raise NotImplementedError


@register_block("prenorm")
class PreNormBlock(BlockBase):
    @classmethod
    def slots(cls, spec):
        return (("mixer_norm", "norm", spec.mixer_norm), ("mixer", "mixer", spec.mixer),
                ("ffn_norm", "norm", spec.ffn_norm), ("ffn", "ffn", spec.ffn))

    def __call__(self, resid, delta, ctx, cache):
        x = norm_before(self.mixer_norm, resid, delta, self.mixer)
        a = self.mixer(x, ctx, cache)
        x = norm_before(self.ffn_norm, resid, a, self.ffn)
        return resid, self.ffn(x, ctx)


def norm_before(norm, resid, delta, reader):
    """``norm(resid + delta)`` for the part ``reader``; a norm that takes hints is told which matrix is read next."""
    if norm.takes_hint:
        return norm(resid, delta, None, reader.reads_first())
    return norm(resid, delta)


def build_block(spec, env):
    """The block of a layer record: the class registered for its ``arrangement``."""
    return part_class("block", spec)(spec, env)
