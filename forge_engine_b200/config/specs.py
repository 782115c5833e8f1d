"""Typed descriptions of the parts a model is assembled from.

A *spec* is plain frozen data: every size and constant a part needs, nothing about
the model it sits in.  An architecture (see ``models/``) turns its ``config.json``
into a ``ModelSpec``; ``parts.build`` turns specs into parts.  A new kind of part
brings its own spec dataclass with a unique ``kind`` string and registers a builder
for it (``parts.registry``); nothing in this file has to change for that.
"""

from __future__ import annotations

from dataclasses import dataclass, field


@dataclass(frozen=True)
class NormSpec:
    """RMS normalisation over the last ``size`` elements."""

    size: int
    eps: float
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class RotarySpec:
    """Rotary position encoding: pairs element j with j + rotary_dim/2.

    ``theta`` is the base; ``rotary_dim`` is the number of leading elements of a
    head that are rotated (the whole head for Qwen3).
    """

    head_dim: int
    theta: float
    rotary_dim: int
    kind: str = "rope"


@dataclass(frozen=True)
class NoPositionSpec:
    """No position encoding: queries and keys are used as they come."""

    kind: str = "none"


@dataclass(frozen=True)
class AttentionSpec:
    """Causal grouped-query attention.

    ``window`` is None for full attention, else the number of most recent keys
    (the query's own included) a query may look at.
    """

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    qk_norm: bool
    qk_norm_eps: float
    bias: bool
    scale: float
    position: object
    window: int | None = None
    kind: str = "gqa_attention"


@dataclass(frozen=True)
class GatedMLPSpec:
    """down(act(gate(x)) * up(x)) without biases."""

    hidden_size: int
    intermediate_size: int
    activation: str = "silu"
    kind: str = "gated_mlp"


@dataclass(frozen=True)
class LayerSpec:
    """One block: which norm, mixer and feed-forward it has and how they are wired.

    ``arrangement`` "pre_norm": h += mixer(norm1(h)); h += ffn(norm2(h)).
    ``names`` maps the roles (input_norm, mixer, post_norm, ffn) to the tensor-name
    prefix of this layer's weights in a checkpoint.
    """

    input_norm: object
    mixer: object
    post_norm: object
    ffn: object
    names: dict = field(default_factory=dict, hash=False, compare=False)
    arrangement: str = "pre_norm"


@dataclass(frozen=True)
class RunSpec:
    """One entry of the order in which layers run.

    ``layer`` indexes ``ModelSpec.layers`` (a layer may appear in several runs).
    ``cache_of`` is None when the run keeps a cache of its own, else the index of
    an earlier *run* whose cache it reads without writing.
    """

    layer: int
    cache_of: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    """Everything needed to assemble a decoder-only language model from parts."""

    vocab_size: int
    hidden_size: int
    layers: tuple
    schedule: tuple
    final_norm: object
    tie_embeddings: bool
    max_positions: int
    eos_token_ids: tuple = ()
    embed_name: str = "model.embed_tokens.weight"
    final_norm_name: str = "model.norm"
    head_name: str = "lm_head.weight"
