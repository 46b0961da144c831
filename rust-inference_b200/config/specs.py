"""Descriptions of a model as data: which parts, with which sizes, in which order.

An architecture (see ``models/``) turns its ``config.json`` into a
:class:`ModelSpec`.  Everything below the architecture works from these
records only: the part factories in ``parts/`` build one object per record,
the cache reads the mixers' storage needs from them, and the engine runs the
``schedule``.  No record knows which model it belongs to, and no size lives
anywhere but here.

A record names its part by ``kind``; ``parts.registry`` maps kinds to classes,
so a new mixer, feed-forward, norm or position encoding is a new record class
plus a registered part class, with no change to existing files.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class RMSNormSpec:
    """y = x / sqrt(mean(x^2) + eps) * gain over ``size`` elements."""
    size: int
    eps: float
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class RopeSpec:
    """Rotate-half rotary encoding of the first ``rotary_dim`` elements of a head.

    ``theta`` is the base; angles are float32(position) * float32(inv_freq) and
    ``scaling`` multiplies cos and sin (1.0 for the "default" rope type).
    """
    head_dim: int
    theta: float
    rotary_dim: int = 0          # 0 means the whole head
    scaling: float = 1.0
    kind: str = "rope"

    @property
    def rot(self) -> int:
        return self.rotary_dim or self.head_dim


@dataclass(frozen=True)
class NoPositionSpec:
    """No position encoding inside the mixer."""
    kind: str = "none"


@dataclass(frozen=True)
class AttentionSpec:
    """Causal grouped-query attention over a key/value cache.

    ``qk_norm`` is the per-head norm applied to queries and keys before the
    position encoding (None for none); ``window`` > 0 limits a query to the last
    ``window`` keys; ``scale`` 0 means 1/sqrt(head_dim).
    """
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    position: object = NoPositionSpec()
    qk_norm: Optional[RMSNormSpec] = None
    window: int = 0
    scale: float = 0.0
    kind: str = "attention"


@dataclass(frozen=True)
class SwiGLUSpec:
    """down(silu(gate x) * up x), no biases."""
    hidden_size: int
    intermediate_size: int
    kind: str = "swiglu"


@dataclass(frozen=True)
class EmbeddingSpec:
    """h[t] = table[ids[t]], no scaling."""
    vocab_size: int
    hidden_size: int
    kind: str = "embedding"


@dataclass(frozen=True)
class HeadSpec:
    """logits = x W^T in float32, no bias, no soft-cap; W may be the embedding table (tied)."""
    vocab_size: int
    hidden_size: int
    kind: str = "linear"


@dataclass(frozen=True)
class LayerSpec:
    """One block: two sub-layers, each a norm followed by a part, each added to
    the residual stream (``arrangement`` "prenorm").

    ``names`` maps the block's four parts to the prefixes their tensors carry in
    the checkpoint, e.g. {"mixer": "model.layers.0.self_attn."}.

    A layer with another arrangement is another record class: it needs
    ``arrangement`` (the kind its block class is registered for) and
    ``prefix(part)``; which parts it has is for its block class to say.
    """
    mixer: object
    ffn: object
    mixer_norm: object
    ffn_norm: object
    names: Tuple[Tuple[str, str], ...] = ()
    arrangement: str = "prenorm"

    def prefix(self, part: str) -> str:
        return dict(self.names)[part]


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer.  ``layer`` indexes ``ModelSpec.layers``;
    ``cache`` names the cache entry (an index into the list of cache entries)
    that this execution reads, and ``writes`` says whether it also appends to
    it.  Two entries may name the same layer (weights shared) or the same cache
    (a layer that reads what another layer wrote)."""
    layer: int
    cache: int
    writes: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: object
    tie_embeddings: bool
    max_positions: int
    embedding_name: str = "model.embed_tokens.weight"
    head_name: str = "lm_head.weight"
    final_norm_prefix: str = "model.norm."
    stop_ids: Tuple[int, ...] = ()
    # a head tensor that is absent from the checkpoint means tied embeddings
    head_optional: bool = True
    # records of the embedding and of the output head (None: the plain table and the plain linear head);
    # the tensor "weight" of each carries ``embedding_name`` / ``head_name``, further tensors the same
    # name with "weight" replaced by theirs
    embedding: object = None
    head: object = None

    def embedding_record(self):
        return self.embedding or EmbeddingSpec(self.vocab_size, self.hidden_size)

    def head_record(self):
        return self.head or HeadSpec(self.vocab_size, self.hidden_size)

    def cache_entries(self):
        """For every cache entry, the layer whose mixer decides its storage: the
        (first) scheduled execution that writes it."""
        owners = {}
        for e in self.schedule:
            if e.writes and e.cache not in owners:
                owners[e.cache] = e.layer
        for e in self.schedule:
            if e.cache not in owners:
                raise ValueError(f"schedule reads cache {e.cache} that no layer writes")
        n = max(owners) + 1 if owners else 0
        if sorted(owners) != list(range(n)):
            raise ValueError("cache indices of the schedule must be 0..n-1 without gaps")
        return [owners[i] for i in range(n)]
