"""GPT-J's configuration, read from its own config.json keys.

QStream's converter reads llama-style keys (`hidden_size`, ... tools/convert_hf.py:
881-888) and so cannot read a GPT-J folder; this reads GPT-J's keys (`n_embd`,
`n_layer`, `n_head`, `rotary_dim`, `n_inner`, `activation_function`,
`layer_norm_epsilon`, `n_positions`, `vocab_size`) and checks them in the manner of
`qsf_validate_header` (src/format.c:37-96).  The tensor names are the GPT-J table of
tools/convert_hf.py:462-479.
"""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Optional

from ..errors import QsError, QStreamError
from .specs import (AttentionSpec, BlockSpec, EmbeddingSpec, HeadSpec, LayerRun,
                    MlpSpec, ModelSpec, NormSpec, PositionSpec)

ACTIVATIONS = ("gelu_new", "gelu")


def _bad(detail: str, code=QsError.INVALID_MODEL):
    return QStreamError(code, detail)


@dataclass(frozen=True)
class GptjConfig:
    n_layer: int
    n_embd: int
    n_head: int
    n_positions: int
    vocab_size: int
    rotary_dim: Optional[int] = None        # None: the whole head
    n_inner: Optional[int] = None           # None: 4 * n_embd (src/engine.c:36,514)
    activation_function: str = "gelu_new"
    layer_norm_epsilon: float = 1e-5
    rope_theta: float = 10000.0             # src/engine.c:872-873's default
    tie_word_embeddings: bool = False
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    torch_dtype: Optional[str] = None       # informational

    architecture = "GPTJForCausalLM"
    model_type = "gptj"

    # ----------------------------------------------------------------- reading
    @classmethod
    def from_dict(cls, d: dict) -> "GptjConfig":
        def need(key, *alts):
            for k in (key, *alts):
                if d.get(k) is not None:
                    return d[k]
            raise _bad(f"config.json: missing key '{key}'")

        def integer(name, v, optional=False):
            if v is None and optional:
                return None
            if isinstance(v, bool) or not isinstance(v, int):
                raise _bad(f"config.json: '{name}' must be an integer, got {v!r}")
            return v

        eps = d.get("layer_norm_epsilon", 1e-5)
        if isinstance(eps, bool) or not isinstance(eps, (int, float)):
            raise _bad(f"config.json: 'layer_norm_epsilon' must be a number, got {eps!r}")
        cfg = cls(
            n_layer=integer("n_layer", need("n_layer")),
            n_embd=integer("n_embd", need("n_embd")),
            n_head=integer("n_head", need("n_head")),
            n_positions=integer("n_positions", need("n_positions", "n_ctx")),
            vocab_size=integer("vocab_size", need("vocab_size")),
            rotary_dim=integer("rotary_dim", d.get("rotary_dim"), optional=True),
            n_inner=integer("n_inner", d.get("n_inner"), optional=True),
            activation_function=d.get("activation_function", "gelu_new"),
            layer_norm_epsilon=float(eps),
            rope_theta=float(d.get("rope_theta", 10000.0)),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            bos_token_id=integer("bos_token_id", d.get("bos_token_id"), optional=True),
            eos_token_id=integer("eos_token_id", d.get("eos_token_id"), optional=True),
            torch_dtype=d.get("torch_dtype", d.get("dtype")),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if not 1 <= self.n_layer <= 1000:
            raise _bad(f"n_layer={self.n_layer} out of range [1, 1000]")
        if self.n_embd < 1 or self.n_head < 1:
            raise _bad(f"n_embd={self.n_embd}, n_head={self.n_head} must be positive")
        if self.n_embd % self.n_head:
            raise _bad(f"n_embd={self.n_embd} not divisible by n_head={self.n_head}")
        r = self.rotary
        if r < 0 or r % 2 or r > self.head_dim:
            raise _bad(f"rotary_dim={r} must be even and within the head size {self.head_dim}")
        if self.n_positions < 1:
            raise _bad(f"n_positions={self.n_positions} must be positive")
        if self.vocab_size < 1:
            raise _bad(f"vocab_size={self.vocab_size} must be positive")
        if self.inner < 1:
            raise _bad(f"n_inner={self.n_inner} must be positive")
        if not self.layer_norm_epsilon > 0:
            raise _bad(f"layer_norm_epsilon={self.layer_norm_epsilon} must be positive")
        if not self.rope_theta > 0:
            raise _bad(f"rope_theta={self.rope_theta} must be positive")
        if self.activation_function not in ACTIVATIONS:
            raise _bad(f"activation_function '{self.activation_function}' is not one of "
                       f"{ACTIVATIONS}", QsError.UNSUPPORTED_ARCH)
        if self.tie_word_embeddings:
            raise _bad("tie_word_embeddings=true: GPT-J's head is untied", QsError.UNSUPPORTED_ARCH)
        for name in ("bos_token_id", "eos_token_id"):
            v = getattr(self, name)
            if v is not None and not 0 <= v < self.vocab_size:
                raise _bad(f"{name}={v} outside the vocabulary of {self.vocab_size}")

    # ----------------------------------------------------------------- derived
    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head

    @property
    def rotary(self) -> int:
        return self.head_dim if self.rotary_dim is None else self.rotary_dim

    @property
    def inner(self) -> int:
        return 4 * self.n_embd if self.n_inner is None else self.n_inner

    def to_dict(self) -> dict:
        d = asdict(self)
        d["architectures"] = [self.architecture]
        d["model_type"] = self.model_type
        return d

    # ----------------------------------------------------------------- the model
    def model_spec(self) -> ModelSpec:
        """Layer by layer: LayerNorm with bias, attention with partial interleaved
        rotary, an MLP, wired in parallel; one cache entry per layer."""
        D, H, dh = self.n_embd, self.n_head, self.head_dim
        position = PositionSpec(rotary_dim=self.rotary, base=self.rope_theta,
                                max_positions=self.n_positions)
        layers = []
        for i in range(self.n_layer):
            p = f"transformer.h.{i}."
            layers.append(BlockSpec(
                arrangement="parallel",
                norms={"input": NormSpec(size=D, eps=self.layer_norm_epsilon, bias=True, names={
                    "weight": p + "ln_1.weight", "bias": p + "ln_1.bias"})},
                mixer=AttentionSpec(
                    width=D, n_heads=H, n_kv_heads=H, head_dim=dh, position=position,
                    names={"q": p + "attn.q_proj.weight", "k": p + "attn.k_proj.weight",
                           "v": p + "attn.v_proj.weight", "out": p + "attn.out_proj.weight"}),
                ffn=MlpSpec(
                    width=D, inner=self.inner, activation=self.activation_function, bias=True,
                    names={"up": p + "mlp.fc_in.weight", "up_bias": p + "mlp.fc_in.bias",
                           "down": p + "mlp.fc_out.weight", "down_bias": p + "mlp.fc_out.bias"}),
            ))
        return ModelSpec(
            architecture=self.architecture,
            vocab_size=self.vocab_size, width=D, max_positions=self.n_positions,
            embedding=EmbeddingSpec(vocab_size=self.vocab_size, width=D,
                                    names={"weight": "transformer.wte.weight"}),
            layers=tuple(layers),
            schedule=tuple(LayerRun(layer=i, cache=i) for i in range(self.n_layer)),
            final_norm=NormSpec(size=D, eps=self.layer_norm_epsilon, bias=True, names={
                "weight": "transformer.ln_f.weight", "bias": "transformer.ln_f.bias"}),
            head=HeadSpec(vocab_size=self.vocab_size, width=D, bias=True, tied=False,
                          names={"weight": "lm_head.weight", "bias": "lm_head.bias"}),
            stop_tokens=() if self.eos_token_id is None else (self.eos_token_id,),
            bos_token_id=self.bos_token_id,
        )

    # Tensors a GPT-J checkpoint may carry that are buffers, not parameters.
    ignored_tensor_suffixes = (".attn.bias", ".attn.masked_bias")
