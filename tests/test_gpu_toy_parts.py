"""A feed-forward with routing and another position encoding, defined here and registered without
touching the library's files, in a toy architecture whose layers pick different parts.

- `HalfRotary`: rotates element i with element i + R/2 (not the neighbouring pair), through the
  `apply(q, k, step, ...)` interface: the attention part then only writes the cache.
- `RoutedFeedForward`: a router (32-bit logits), the two best experts of four per token, their outputs
  weighted by the softmax over the two logits.
Layer 0 is attention + dense MLP in the parallel arrangement, layer 1 attention + routed experts in the
sequential one.  A token whose second and third router logits lie closer than the arithmetic can tell
apart may go to another expert than in the plain model; such tokens (few, by the router's scale) are
left out of the comparison, and because the routed layer is the last one they disturb no other token."""
from dataclasses import dataclass, field
from typing import Mapping

import numpy as np
import pytest
import torch

import qstream_b200 as qs
import plain_gptj as P
from qstream_b200.config import (AttentionSpec, BlockSpec, EmbeddingSpec, HeadSpec, LayerRun, MlpSpec, ModelSpec,
                                 NormSpec, config_from_dict)
from qstream_b200.parts import Embedding, FeedForward, Head, PositionEncoding, add_residuals, linear, register
from qstream_b200.weights import TensorDecl

pytestmark = pytest.mark.gpu


@dataclass(frozen=True)
class HalfRotarySpec:
    rotary_dim: int
    base: float
    max_positions: int
    kind: str = "toy_half_rotary"


class HalfRotary(PositionEncoding):
    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        half = spec.rotary_dim // 2
        inv = spec.base ** (-(torch.arange(half, dtype=torch.float64) * 2.0) / spec.rotary_dim)
        ang = torch.arange(spec.max_positions, dtype=torch.float64)[:, None] * inv[None, :]
        self.cos = torch.cos(ang).float().to(runtime.device)
        self.sin = torch.sin(ang).float().to(runtime.device)

    def apply(self, q, k, step, n_heads, n_kv_heads, head_dim):
        pos = step.batch.tok_pos.clamp(min=0).long()           # rows of no sequence carry -1 and are never read
        cos, sin = self.cos[pos][:, None, :], self.sin[pos][:, None, :]
        half = self.spec.rotary_dim // 2
        for t, heads in ((q, n_heads), (k, n_kv_heads)):
            if t is None:
                continue
            v = t.view(t.shape[0], heads, head_dim)            # a view: the rotation happens in place
            a, b = v[..., :half].float(), v[..., half:2 * half].float()
            first, second = a * cos - b * sin, a * sin + b * cos           # both before either is written
            v[..., :half] = first.to(t.dtype)
            v[..., half:2 * half] = second.to(t.dtype)


@dataclass(frozen=True)
class RoutedSpec:
    width: int
    inner: int
    n_experts: int
    top_k: int
    kind: str = "toy_routed"
    names: Mapping[str, str] = field(default_factory=dict)


class RoutedFeedForward(FeedForward):
    @classmethod
    def declare(cls, spec):
        d = {"router": TensorDecl((spec.n_experts, spec.width))}
        for e in range(spec.n_experts):
            d[f"up{e}"] = TensorDecl((spec.inner, spec.width))
            d[f"down{e}"] = TensorDecl((spec.width, spec.inner))
        return d

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.router = tensors["router"].float()                # router logits in 32-bit
        self.up = [tensors[f"up{e}"] for e in range(spec.n_experts)]
        self.down = [tensors[f"down{e}"] for e in range(spec.n_experts)]

    def forward(self, h, step, residuals=()):
        logits = h.float() @ self.router.T                                   # [T, E]
        best, idx = torch.topk(logits, self.spec.top_k, dim=1)
        gate = torch.softmax(best, dim=1)                                    # over the chosen experts only
        out = torch.zeros(h.shape, dtype=torch.float32, device=h.device)
        for e in range(self.spec.n_experts):                                 # a toy: every expert sees every token
            y = linear(linear(h, self.up[e], None, "gelu_new"), self.down[e], out_dtype=torch.float32)
            w = (gate * (idx == e)).sum(dim=1, keepdim=True)                 # 0 for tokens that did not choose it
            out += w * y
        return add_residuals(out.to(h.dtype), residuals)


@dataclass(frozen=True)
class RoutedToyConfig:
    width: int
    n_head: int
    n_kv_head: int
    vocab_size: int
    n_positions: int
    rotary_dim: int
    architecture = "RoutedToyForCausalLM"
    model_type = "routed_toy"

    @classmethod
    def from_dict(cls, d):
        return cls(d["width"], d["n_head"], d["n_kv_head"], d["vocab_size"], d["n_positions"], d["rotary_dim"])

    def to_dict(self):
        return dict(width=self.width, n_head=self.n_head, n_kv_head=self.n_kv_head, vocab_size=self.vocab_size,
                    n_positions=self.n_positions, rotary_dim=self.rotary_dim, architectures=[self.architecture],
                    model_type=self.model_type)

    def model_spec(self):
        D, H, Hkv = self.width, self.n_head, self.n_kv_head
        dh = D // H
        pos = HalfRotarySpec(self.rotary_dim, 777.0, self.n_positions)

        def attn(p):
            return AttentionSpec(width=D, n_heads=H, n_kv_heads=Hkv, head_dim=dh, position=pos,
                                 names={"q": p + "q", "k": p + "k", "v": p + "v", "out": p + "o"})

        layers = (
            BlockSpec(arrangement="parallel", norms={"input": NormSpec(D, 1e-5, names={"weight": "l0.n.w", "bias": "l0.n.b"})},
                      mixer=attn("l0.attn."),
                      ffn=MlpSpec(D, 3 * D, "gelu", names={"up": "l0.ff.up", "up_bias": "l0.ff.up_b", "down": "l0.ff.down",
                                                           "down_bias": "l0.ff.down_b"})),
            BlockSpec(arrangement="sequential",
                      norms={"input": NormSpec(D, 1e-6, names={"weight": "l1.n1.w", "bias": "l1.n1.b"}),
                             "post_mixer": NormSpec(D, 1e-6, names={"weight": "l1.n2.w", "bias": "l1.n2.b"})},
                      mixer=attn("l1.attn."),
                      ffn=RoutedSpec(D, 2 * D, 4, 2, names={"router": "l1.moe.router", **{
                          f"{m}{e}": f"l1.moe.{e}.{m}" for e in range(4) for m in ("up", "down")}})))
        return ModelSpec(architecture=self.architecture, vocab_size=self.vocab_size, width=D, max_positions=self.n_positions,
                         embedding=EmbeddingSpec(self.vocab_size, D, names={"weight": "embed"}),
                         layers=layers, schedule=(LayerRun(0, 0), LayerRun(1, 1)),
                         final_norm=NormSpec(D, 1e-5, names={"weight": "norm.w", "bias": "norm.b"}),
                         head=HeadSpec(self.vocab_size, D, bias=True, names={"weight": "head.w", "bias": "head.b"}))


def half_rotary(x, positions, rotary_dim, base):
    """x [T, H, dh]: element i of the first half of the rotary part turns with element i + R/2."""
    half = rotary_dim // 2
    inv = base ** (-(np.arange(half) * 2.0) / rotary_dim)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * inv[None, :]
    cos, sin = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = x.copy()
    a, b = x[..., :half], x[..., half:2 * half]
    out[..., :half] = a * cos - b * sin
    out[..., half:2 * half] = a * sin + b * cos
    return out


def plain_routed_toy(cfg, w, tokens):
    """Logits [T, V] in float64 and, per token, the gap between its second and third router logit."""
    spec = cfg.model_spec()
    T = len(tokens)
    posn = np.arange(T)
    x = w["embed"][np.asarray(tokens)]
    margin = None

    def norm(v, ns):
        return P.layer_norm(v, w[ns.names["weight"]], w[ns.names["bias"]], ns.eps)

    def attention(h, ms):
        H, Hkv, dh = ms.n_heads, ms.n_kv_heads, ms.head_dim
        q = half_rotary((h @ w[ms.names["q"]].T).reshape(T, H, dh), posn, ms.position.rotary_dim, ms.position.base)
        k = half_rotary((h @ w[ms.names["k"]].T).reshape(T, Hkv, dh), posn, ms.position.rotary_dim, ms.position.base)
        v = (h @ w[ms.names["v"]].T).reshape(T, Hkv, dh)
        return P.causal_attention(q, k, v) @ w[ms.names["out"]].T

    def ffn(h, fs):
        nonlocal margin
        if fs.kind == "toy_routed":
            logits = h @ w[fs.names["router"]].T
            order = np.argsort(-logits, axis=1)
            srt = np.take_along_axis(logits, order, axis=1)
            margin = srt[:, fs.top_k - 1] - srt[:, fs.top_k]
            gate = P.softmax(srt[:, :fs.top_k])
            out = np.zeros_like(h)
            for t in range(T):
                for j in range(fs.top_k):
                    e = int(order[t, j])
                    out[t] += gate[t, j] * (P.gelu_new(h[t] @ w[fs.names[f"up{e}"]].T) @ w[fs.names[f"down{e}"]].T)
            return out
        u = h @ w[fs.names["up"]].T + w[fs.names["up_bias"]]
        return P.ACTIVATIONS[fs.activation](u) @ w[fs.names["down"]].T + w[fs.names["down_bias"]]

    for run in spec.schedule:
        b = spec.layers[run.layer]
        if b.arrangement == "parallel":
            h = norm(x, b.norms["input"])
            x = x + attention(h, b.mixer) + ffn(h, b.ffn)
        else:
            x = x + attention(norm(x, b.norms["input"]), b.mixer)
            x = x + ffn(norm(x, b.norms["post_mixer"]), b.ffn)
    return norm(x, spec.final_norm) @ w[spec.head.names["weight"]].T + w[spec.head.names["bias"]], margin


@pytest.fixture(scope="module")
def registered():
    register("position", "toy_half_rotary", HalfRotary)
    register("feed_forward", "toy_routed", RoutedFeedForward)
    qs.register_architecture(RoutedToyConfig, "routed_toy")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_routed_experts_and_another_rotation(tmp_path, registered, dtype):
    cfg = config_from_dict(dict(architectures=["RoutedToyForCausalLM"], width=96, n_head=6, n_kv_head=2, vocab_size=131,
                                n_positions=192, rotary_dim=12))
    assert isinstance(cfg, RoutedToyConfig)
    # a router that decides clearly: its rows are ten times the usual size
    folder = qs.write_model_folder(tmp_path / "routed", cfg, seed=9, dtype=dtype)
    raw = P.read_safetensors(folder / "model.safetensors")
    from qstream_b200.weights import write_safetensors
    tensors = {k: torch.from_numpy(np.asarray(v)).to(torch.bfloat16 if dtype == "bfloat16" else torch.float32)
               for k, v in raw.items()}
    tensors["l1.moe.router"] = (tensors["l1.moe.router"].float() * 10.0).to(tensors["l1.moe.router"].dtype)
    write_safetensors(folder / "model.safetensors", tensors)
    w = P.read_safetensors(folder / "model.safetensors")

    model = qs.load_model(folder, dtype=dtype, device="cuda")
    assert set(model.kv_needs()) == {0, 1} and not model.state_needs()
    engine = qs.Engine(model, max_tokens=64 * 8, max_batch=3)
    rng = np.random.default_rng(2)
    reqs = [[int(t) for t in rng.integers(0, 131, n)] for n in (150, 31, 77)]
    plain = [plain_routed_toy(cfg, w, r) for r in reqs]
    clear = 1e-3 if dtype == "float32" else 0.25                    # router logits are O(5) here
    keep = [m > clear for _, m in plain]
    assert sum(int(k.sum()) for k in keep) > 0.8 * sum(len(r) for r in reqs)
    atol, rtol = (3e-4, 1e-3) if dtype == "float32" else (8e-2, 5e-2)

    def check(got, i, positions):
        positions = np.asarray(positions)
        sel = keep[i][positions]
        np.testing.assert_allclose(np.asarray(got)[sel], plain[i][0][positions][sel], atol=atol, rtol=rtol,
                                   err_msg=f"request {i}")

    # whole, each alone
    for i, r in enumerate(reqs):
        s = engine.acquire()
        check(engine.step([s], [r], [list(range(len(r)))]).cpu().double().numpy(), i, range(len(r)))
        engine.release(s)

    # a batch of unequal prompts, then one token each; shorter requests end earlier; twice over the same slots
    for _ in range(2):
        heads = [90, 7, 40]
        slots = [engine.acquire() for _ in reqs]
        out = engine.step(slots, [r[:h] for r, h in zip(reqs, heads)], [[h - 1] for h in heads]).cpu().double().numpy()
        for i, h in enumerate(heads):
            check(out[i:i + 1], i, [h - 1])
        pos, live = list(heads), [0, 1, 2]
        while live:
            out = engine.step([slots[i] for i in live], [[reqs[i][pos[i]]] for i in live]).cpu().double().numpy()
            nxt = []
            for j, i in enumerate(live):
                check(out[j:j + 1], i, [pos[i]])
                pos[i] += 1
                if pos[i] < len(reqs[i]):
                    nxt.append(i)
                else:
                    engine.release(slots[i])
            live = nxt
        engine.cache.check()


# ----------------------------------------------------------------------------- another embedding, another head

@dataclass(frozen=True)
class PositionedEmbeddingSpec:
    vocab_size: int
    width: int
    max_positions: int
    scale: float
    kind: str = "toy_positioned_embedding"
    names: Mapping[str, str] = field(default_factory=dict)


class PositionedEmbedding(Embedding):
    """x[t] = scale * table[token[t]] + positions[pos[t]]: a learned position table and an embedding scale."""

    @classmethod
    def declare(cls, spec):
        return {"weight": TensorDecl((spec.vocab_size, spec.width)), "positions": TensorDecl((spec.max_positions, spec.width))}

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.weight, self.positions = tensors["weight"], tensors["positions"]

    def forward(self, step):
        b = step.batch
        x = self.weight[b.tokens.long()].float() * self.spec.scale + self.positions[b.tok_pos.clamp(min=0).long()].float()
        return x.to(self.runtime.dtype)


@dataclass(frozen=True)
class CappedHeadSpec:
    vocab_size: int
    width: int
    cap: float
    bias: bool = False
    tied: bool = True
    kind: str = "toy_capped_head"
    names: Mapping[str, str] = field(default_factory=dict)


class CappedHead(Head):
    """logits = cap * tanh(rows W^T / cap) with W the embedding table: a tied head with soft-capping."""

    def tie(self, embedding):
        self.weight = embedding.weight

    def forward(self, rows):
        z = linear(rows, self.weight, out_dtype=torch.float32)
        return self.spec.cap * torch.tanh(z / self.spec.cap)


@dataclass(frozen=True)
class CappedToyConfig:
    width: int
    n_head: int
    vocab_size: int
    n_positions: int
    architecture = "CappedToyForCausalLM"
    model_type = "capped_toy"

    @classmethod
    def from_dict(cls, d):
        return cls(d["width"], d["n_head"], d["vocab_size"], d["n_positions"])

    def to_dict(self):
        return dict(width=self.width, n_head=self.n_head, vocab_size=self.vocab_size, n_positions=self.n_positions,
                    architectures=[self.architecture], model_type=self.model_type)

    def model_spec(self):
        D, H = self.width, self.n_head
        layers = tuple(
            BlockSpec(arrangement="parallel", norms={"input": NormSpec(D, 1e-5, names={"weight": f"l{i}.n.w", "bias": f"l{i}.n.b"})},
                      mixer=AttentionSpec(width=D, n_heads=H, n_kv_heads=H, head_dim=D // H, position=None,
                                          names={"q": f"l{i}.q", "k": f"l{i}.k", "v": f"l{i}.v", "out": f"l{i}.o"}),
                      ffn=MlpSpec(D, 2 * D, "gelu_new", names={"up": f"l{i}.up", "up_bias": f"l{i}.up_b", "down": f"l{i}.down",
                                                               "down_bias": f"l{i}.down_b"}))
            for i in range(2))
        return ModelSpec(architecture=self.architecture, vocab_size=self.vocab_size, width=D, max_positions=self.n_positions,
                         embedding=PositionedEmbeddingSpec(self.vocab_size, D, self.n_positions, 3.0,
                                                           names={"weight": "embed", "positions": "positions"}),
                         layers=layers, schedule=(LayerRun(0, 0), LayerRun(1, 1)),
                         final_norm=None, head=CappedHeadSpec(self.vocab_size, D, cap=0.5))


def plain_capped_toy(cfg, w, tokens):
    spec = cfg.model_spec()
    T = len(tokens)
    x = 3.0 * w["embed"][np.asarray(tokens)] + w["positions"][:T]
    for i, b in enumerate(spec.layers):
        h = P.layer_norm(x, w[f"l{i}.n.w"], w[f"l{i}.n.b"], 1e-5)
        H, dh = b.mixer.n_heads, b.mixer.head_dim
        q, k, v = ((h @ w[f"l{i}.{n}"].T).reshape(T, H, dh) for n in "qkv")
        a = P.causal_attention(q, k, v) @ w[f"l{i}.o"].T
        m = P.gelu_new(h @ w[f"l{i}.up"].T + w[f"l{i}.up_b"]) @ w[f"l{i}.down"].T + w[f"l{i}.down_b"]
        x = x + a + m
    return 0.5 * np.tanh((x @ w["embed"].T) / 0.5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_another_embedding_and_another_head(tmp_path, dtype):
    """The embedding and the head are registered parts like the others: a position table with an embedding scale,
    and a tied head with soft-capping and no final norm, come from outside the library; attention runs without
    a position part.  Whole prompts, then tokens one by one, against the plain formulas."""
    register("embedding", "toy_positioned_embedding", PositionedEmbedding)
    register("head", "toy_capped_head", CappedHead)
    qs.register_architecture(CappedToyConfig, "capped_toy")
    cfg = config_from_dict(dict(architectures=["CappedToyForCausalLM"], width=64, n_head=4, vocab_size=97, n_positions=96))
    folder = qs.write_model_folder(tmp_path / "capped", cfg, seed=11, dtype=dtype, scales=qs.InitScales(0.05, 0.1, 0.02))
    w = P.read_safetensors(folder / "model.safetensors")
    assert set(w) >= {"embed", "positions"} and "head.w" not in w
    model = qs.load_model(folder, dtype=dtype, device="cuda")
    engine = qs.Engine(model, max_tokens=64 * 4, max_batch=2)
    assert not engine.captures_prefill                  # the toy parts do not claim to go by device metadata alone
    rng = np.random.default_rng(3)
    reqs = [[int(t) for t in rng.integers(0, 97, n)] for n in (70, 9)]
    atol = 2e-4 if dtype == "float32" else 2e-2
    slots = [engine.acquire(), engine.acquire()]
    heads = [60, 4]
    out = engine.step(slots, [r[:h] for r, h in zip(reqs, heads)], [list(range(h)) for h in heads]).cpu().double().numpy()
    np.testing.assert_allclose(out[:60], plain_capped_toy(cfg, w, reqs[0])[:60], atol=atol)
    np.testing.assert_allclose(out[60:], plain_capped_toy(cfg, w, reqs[1])[:4], atol=atol)
    assert np.abs(out).max() <= 0.5 + 1e-6 and np.abs(out).max() > 0.05
    for step in range(5):                                # both decode on: a captured decode step with the toy parts
        out = engine.step(slots, [[r[h + step]] for r, h in zip(reqs, heads)]).cpu().double().numpy()
        for i, (r, h) in enumerate(zip(reqs, heads)):
            np.testing.assert_allclose(out[i], plain_capped_toy(cfg, w, r)[h + step], atol=atol)
    engine.check_status()
