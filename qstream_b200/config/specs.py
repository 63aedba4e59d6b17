"""Typed descriptions of the parts a model is put together from.

A spec says which part to build (`kind`, looked up in the part registries), with
which sizes and constants, and under which checkpoint names its tensors lie
(`names`: the part's own tensor name -> the name in the safetensors file).  A spec
holds no weights and no code.  An architecture's configuration produces one
`ModelSpec`; nothing below it knows the architecture's name.

Any object with a `kind` attribute may serve as a spec of a part registered under
that kind, so a new part brings its own spec class.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Mapping, Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    """LayerNorm: mean and biased variance over `size`, eps inside the root,
    weight and (if `bias`) bias (QStream src/kernels_scalar.c:151-171)."""
    size: int
    eps: float
    bias: bool = True
    kind: str = "layernorm"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class PositionSpec:
    """Rotary position encoding on the first `rotary_dim` dims of each head,
    pairs (i, i+1) (QStream src/engine.c:205-234 with head_dim -> rotary_dim)."""
    rotary_dim: int
    base: float
    max_positions: int
    kind: str = "rotary_interleaved"


@dataclass(frozen=True)
class AttentionSpec:
    """Causal softmax attention over the sequence's cache.

    `window` = 0 reads all keys, w > 0 the last w (the query's own included).
    `shares_cache`: the layer projects queries only and reads the keys and values
    that another layer of the schedule wrote.
    """
    width: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    position: Optional[PositionSpec] = None
    window: int = 0
    qkv_bias: bool = False
    out_bias: bool = False
    shares_cache: bool = False
    kind: str = "attention"
    names: Mapping[str, str] = field(default_factory=dict)

    @property
    def scale(self) -> float:
        return self.head_dim ** -0.5


@dataclass(frozen=True)
class MlpSpec:
    """Dense feed-forward: up projection, activation, down projection
    (QStream src/engine.c:1150-1170), with biases if `bias`."""
    width: int
    inner: int
    activation: str
    bias: bool = True
    kind: str = "mlp"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class BlockSpec:
    """One layer: its norms, mixer and feed-forward, and how they are wired.

    arrangement "parallel": h = norm(x); x + mixer(h) + ffn(h)   (norms: "input")
    arrangement "sequential": x += mixer(norm_1(x)); x += ffn(norm_2(x))
                                                     (norms: "input", "post_mixer")
    """
    mixer: object
    ffn: object
    norms: Mapping[str, object]
    arrangement: str = "parallel"


@dataclass(frozen=True)
class LayerRun:
    """One entry of the schedule: run layer `layer` against cache entry `cache`.
    A layer may appear in several runs; two runs may name the same cache entry
    when the later one only reads it.  For a layer with several parts that use the
    cache, `cache` is a tuple with one entry id per such part."""
    layer: int
    cache: object


@dataclass(frozen=True)
class EmbeddingSpec:
    vocab_size: int
    width: int
    kind: str = "embedding"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class HeadSpec:
    """Output projection to the vocabulary, logits in 32-bit.  `tied` reuses the
    embedding table as its weight."""
    vocab_size: int
    width: int
    bias: bool = True
    tied: bool = False
    kind: str = "lm_head"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    width: int
    max_positions: int
    embedding: object
    layers: Tuple[BlockSpec, ...]
    schedule: Tuple[LayerRun, ...]
    final_norm: Optional[object]            # None: the head sees the last layer's output as it is
    head: object
    stop_tokens: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None

    def n_cache_entries(self) -> int:
        ids = [c for r in self.schedule for c in (r.cache if isinstance(r.cache, (tuple, list)) else (r.cache,))]
        return 1 + max(ids, default=-1)
