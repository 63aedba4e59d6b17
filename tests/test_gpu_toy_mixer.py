"""A toy mixer with state of its own, and a toy architecture around it, defined here and
registered without touching the library's files: built, stepped in every cutting, generated from.

The mixer keeps, per sequence, the running sum of its inputs (fixed-size state, no keys or
values): out[t] = W . mean(h[0..t]).  Its layers alternate with ordinary attention layers, one
layer's weights are run twice, and a late attention layer reads the cache that an earlier one
wrote - the schedule is data."""
from dataclasses import dataclass, field
from typing import Mapping

import numpy as np
import pytest
import torch

import qstream_b200 as qs
import plain_gptj as P
from qstream_b200.cache import StateNeed
from qstream_b200.config import (AttentionSpec, BlockSpec, EmbeddingSpec, HeadSpec, LayerRun, MlpSpec, ModelSpec,
                                 NormSpec, PositionSpec, config_from_dict)
from qstream_b200.engine.model import declared_tensors
from qstream_b200.parts import Mixer, Part, add_residuals, linear, register
from qstream_b200.parts.block import Arrangement
from qstream_b200.weights import TensorDecl

pytestmark = pytest.mark.gpu


@dataclass(frozen=True)
class RunningMeanSpec:
    width: int
    kind: str = "toy_running_mean"
    names: Mapping[str, str] = field(default_factory=dict)


class RunningMeanMixer(Mixer):
    """State: the sum of all inputs of the sequence so far, [width] in float32."""

    @classmethod
    def declare(cls, spec):
        return {"proj": TensorDecl((spec.width, spec.width))}

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.proj = tensors["proj"]

    def state_need(self):
        return StateNeed((self.spec.width,), torch.float32)

    def forward(self, h, step, cache_id, residuals=()):
        b = step.batch
        state = step.state(cache_id)                                    # [slots, width]
        T = h.shape[0]
        live = (b.tok_slot >= 0)
        slot = b.tok_slot.clamp(min=0).long()
        hf = h.float() * live[:, None]
        rows = torch.arange(T, device=h.device, dtype=torch.int32)
        seq = torch.searchsorted(b.seq_start[1:].contiguous(), rows, right=True).clamp(max=b.n_seq - 1)
        first = b.seq_start[seq.long()].long()                          # first row of each token's sequence
        cs = torch.cumsum(hf, 0)
        before = torch.where((first > 0)[:, None], cs[(first - 1).clamp(min=0)], torch.zeros_like(cs))
        total = state[slot] + cs - before                               # the sum up to and including this token
        state.index_add_(0, slot, hf)                                   # padding rows add zero
        mean = total / (b.tok_pos.float()[:, None] + 1.0)
        out = linear(mean.to(h.dtype), self.proj)
        return add_residuals(out, residuals)


@dataclass(frozen=True)
class ToyConfig:
    n_layer: int
    width: int
    n_head: int
    vocab_size: int
    n_positions: int
    eps: float = 1e-5
    architecture = "ToyForCausalLM"
    model_type = "toy"

    @classmethod
    def from_dict(cls, d):
        return cls(d["n_layer"], d["width"], d["n_head"], d["vocab_size"], d["n_positions"], d.get("eps", 1e-5))

    def to_dict(self):
        return dict(n_layer=self.n_layer, width=self.width, n_head=self.n_head, vocab_size=self.vocab_size,
                    n_positions=self.n_positions, eps=self.eps, architectures=[self.architecture],
                    model_type=self.model_type)

    def model_spec(self):
        D, H = self.width, self.n_head
        pos = PositionSpec(rotary_dim=D // H, base=10000.0, max_positions=self.n_positions)
        layers = []
        for i in range(self.n_layer):
            p = f"layers.{i}."
            if i % 2 == 0:
                mixer = RunningMeanSpec(width=D, names={"proj": p + "mix.proj"})
            else:
                mixer = AttentionSpec(width=D, n_heads=H, n_kv_heads=H, head_dim=D // H, position=pos,
                                      names={"q": p + "attn.q", "k": p + "attn.k", "v": p + "attn.v", "out": p + "attn.o"})
            layers.append(BlockSpec(
                arrangement="sequential",
                norms={"input": NormSpec(D, self.eps, names={"weight": p + "n1.w", "bias": p + "n1.b"}),
                       "post_mixer": NormSpec(D, self.eps, names={"weight": p + "n2.w", "bias": p + "n2.b"})},
                mixer=mixer,
                ffn=MlpSpec(D, 2 * D, "gelu_new", names={"up": p + "ff.up", "up_bias": p + "ff.up_b",
                                                          "down": p + "ff.down", "down_bias": p + "ff.down_b"})))
        # one more layer: attention that only reads the keys and values layer 1 wrote
        p = "reader."
        layers.append(BlockSpec(
            arrangement="parallel", norms={"input": NormSpec(D, self.eps, names={"weight": p + "n.w", "bias": p + "n.b"})},
            mixer=AttentionSpec(width=D, n_heads=H, n_kv_heads=H, head_dim=D // H, position=pos, shares_cache=True,
                                names={"q": p + "attn.q", "out": p + "attn.o"}),
            ffn=MlpSpec(D, D, "gelu", bias=False, names={"up": p + "ff.up", "down": p + "ff.down"})))
        # schedule: layers in order, layer 0 (state) and layer 1 (attention) once more with caches of
        # their own, then the reader on cache entry 1
        n = self.n_layer
        schedule = [LayerRun(i, i) for i in range(n)] + [LayerRun(0, n), LayerRun(1, n + 1), LayerRun(n, 1)]
        return ModelSpec(architecture=self.architecture, vocab_size=self.vocab_size, width=D,
                         max_positions=self.n_positions,
                         embedding=EmbeddingSpec(self.vocab_size, D, names={"weight": "embed"}),
                         layers=tuple(layers), schedule=tuple(schedule),
                         final_norm=NormSpec(D, self.eps, names={"weight": "norm.w", "bias": "norm.b"}),
                         head=HeadSpec(self.vocab_size, D, bias=False, tied=True, names={}))


def plain_toy(cfg: ToyConfig, w, tokens):
    """The toy model on a whole sequence, in float64 numpy."""
    spec = cfg.model_spec()
    T = len(tokens)
    posn = np.arange(T)
    x = w["embed"][np.asarray(tokens)]
    kept = {}

    def norm(v, ns):
        return P.layer_norm(v, w[ns.names["weight"]], w[ns.names["bias"]], ns.eps)

    def mixer(h, ms, cache_id):
        if ms.kind == "toy_running_mean":
            return (np.cumsum(h, 0) / (posn[:, None] + 1.0)) @ w[ms.names["proj"]].T
        H, dh = ms.n_heads, ms.head_dim
        q = P.rotary_interleaved((h @ w[ms.names["q"]].T).reshape(T, H, dh), posn, dh)
        if ms.shares_cache:
            k, v = kept[cache_id]
        else:
            k = P.rotary_interleaved((h @ w[ms.names["k"]].T).reshape(T, H, dh), posn, dh)
            v = (h @ w[ms.names["v"]].T).reshape(T, H, dh)
            kept[cache_id] = (k, v)
        return P.causal_attention(q, k, v) @ w[ms.names["out"]].T

    def ffn(h, fs):
        u = h @ w[fs.names["up"]].T + (w[fs.names["up_bias"]] if fs.bias else 0)
        return P.ACTIVATIONS[fs.activation](u) @ w[fs.names["down"]].T + (w[fs.names["down_bias"]] if fs.bias else 0)

    for run in spec.schedule:
        b = spec.layers[run.layer]
        if b.arrangement == "parallel":
            h = norm(x, b.norms["input"])
            x = x + mixer(h, b.mixer, run.cache) + ffn(h, b.ffn)
        else:
            x = x + mixer(norm(x, b.norms["input"]), b.mixer, run.cache)
            x = x + ffn(norm(x, b.norms["post_mixer"]), b.ffn)
    return norm(x, spec.final_norm) @ w["embed"].T


@pytest.fixture(scope="module")
def registered():
    register("mixer", "toy_running_mean", RunningMeanMixer)
    qs.register_architecture(ToyConfig, "toy")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_builds_loads_and_steps(tmp_path, registered, dtype):
    cfg = config_from_dict(dict(architectures=["ToyForCausalLM"], n_layer=3, width=64, n_head=2, vocab_size=97,
                                n_positions=160))
    assert isinstance(cfg, ToyConfig)
    folder = qs.write_model_folder(tmp_path / "toy", cfg, seed=4, dtype=dtype)      # through the files, like any model
    model = qs.load_model(folder, dtype=dtype, device="cuda")
    assert set(model.state_needs()) == {0, 2, 3} and set(model.kv_needs()) == {1, 4}
    engine = qs.Engine(model, max_tokens=64 * 8, max_batch=3)
    w = P.read_safetensors(folder / "model.safetensors")
    rng = np.random.default_rng(5)
    reqs = [[int(t) for t in rng.integers(0, 97, n)] for n in (70, 9, 130)]
    refs = [plain_toy(cfg, w, r) for r in reqs]
    atol = 2e-4 if dtype == "float32" else 6e-2

    # whole, each alone
    for r, ref in zip(reqs, refs):
        s = engine.acquire()
        got = engine.step([s], [r], [list(range(len(r)))]).cpu().double().numpy()
        engine.release(s)
        np.testing.assert_allclose(got, ref, atol=atol, rtol=1e-3 if dtype == "float32" else 5e-2)

    # a batch of unequal prompts, then token by token (captured graphs), shorter requests ending earlier;
    # twice, so that slots and their state are used again
    for _ in range(2):
        heads = [40, 3, 100]
        slots = [engine.acquire() for _ in reqs]
        out = engine.step(slots, [r[:h] for r, h in zip(reqs, heads)], [[h - 1] for h in heads]).cpu().double().numpy()
        for i, h in enumerate(heads):
            np.testing.assert_allclose(out[i], refs[i][h - 1], atol=atol, rtol=5e-2)
        pos, live = list(heads), [0, 1, 2]
        while live:
            out = engine.step([slots[i] for i in live], [[reqs[i][pos[i]]] for i in live]).cpu().double().numpy()
            nxt = []
            for j, i in enumerate(live):
                np.testing.assert_allclose(out[j], refs[i][pos[i]], atol=atol, rtol=5e-2, err_msg=f"request {i} at {pos[i]}")
                pos[i] += 1
                if pos[i] < len(reqs[i]):
                    nxt.append(i)
                else:
                    engine.release(slots[i])
            live = nxt
        engine.cache.check()

    res = qs.generate(engine, [r[:5] for r in reqs], max_new_tokens=4, sampling=qs.SamplingConfig.greedy(), stop_tokens=())
    if dtype == "float32":
        for r, got in zip(reqs, res.tokens):
            toks = r[:5]
            for g in got:
                assert g == int(np.argmax(plain_toy(cfg, w, toks)[-1]))
                toks.append(g)


def test_schedule_errors(registered):
    base = ToyConfig(3, 64, 2, 97, 160).model_spec()
    import dataclasses
    from qstream_b200.weights import random_tensors
    for bad, what in ((base.schedule + (LayerRun(1, 1),), "both write"),
                      ((LayerRun(3, 1),) + base.schedule, "before any layer wrote"),
                      (base.schedule + (LayerRun(9, 9),), "names layer")):
        spec = dataclasses.replace(base, schedule=tuple(bad))
        tensors = random_tensors(declared_tensors(spec), 0, torch.float32, "cuda")
        with pytest.raises(qs.QStreamError, match=what):
            qs.CausalLM(spec, tensors, "float32", "cuda")


# ----------------------------------------------------------------------------- a layer of another make

@dataclass(frozen=True)
class TwoMixerBlockSpec:
    """x + attention(norm x) + running_mean(norm x): two mixers that both use the cache, no feed-forward."""
    attention: object
    mean: object
    norm: object
    arrangement: str = "toy_two_mixers"


class TwoMixerBlock(Arrangement):
    @classmethod
    def part_specs(cls, spec):
        yield "mixer", spec.attention
        yield "mixer", spec.mean
        yield "norm", spec.norm

    @classmethod
    def build(cls, spec, make, runtime):
        self = cls.__new__(cls)
        Part.__init__(self, spec, {}, runtime)
        self.attention, self.mean, self.norm = make("mixer", spec.attention), make("mixer", spec.mean), make("norm", spec.norm)
        return self

    def cached_parts(self):
        return [self.attention, self.mean]

    def forward(self, x, step, cache_id):
        keys, state = cache_id                              # one cache entry per part that uses the cache
        h = self.norm.forward(x)
        a = self.attention.forward(h, step, keys)
        return self.mean.forward(h, step, state, residuals=(x, a))


@dataclass(frozen=True)
class TwoMixerConfig:
    width: int
    n_head: int
    vocab_size: int
    n_positions: int
    architecture = "TwoMixerForCausalLM"
    model_type = "two_mixer_toy"

    @classmethod
    def from_dict(cls, d):
        return cls(d["width"], d["n_head"], d["vocab_size"], d["n_positions"])

    def to_dict(self):
        return dict(width=self.width, n_head=self.n_head, vocab_size=self.vocab_size, n_positions=self.n_positions,
                    architectures=[self.architecture], model_type=self.model_type)

    def model_spec(self):
        D, H = self.width, self.n_head
        pos = PositionSpec(rotary_dim=D // H // 2, base=10000.0, max_positions=self.n_positions)
        layers = tuple(TwoMixerBlockSpec(
            attention=AttentionSpec(width=D, n_heads=H, n_kv_heads=H, head_dim=D // H, position=pos,
                                    names={"q": f"l{i}.q", "k": f"l{i}.k", "v": f"l{i}.v", "out": f"l{i}.o"}),
            mean=RunningMeanSpec(width=D, names={"proj": f"l{i}.mean"}),
            norm=NormSpec(D, 1e-5, names={"weight": f"l{i}.n.w", "bias": f"l{i}.n.b"})) for i in range(2))
        return ModelSpec(architecture=self.architecture, vocab_size=self.vocab_size, width=D, max_positions=self.n_positions,
                         embedding=EmbeddingSpec(self.vocab_size, D, names={"weight": "embed"}), layers=layers,
                         schedule=(LayerRun(0, (0, 1)), LayerRun(1, (2, 3))),
                         final_norm=NormSpec(D, 1e-5, names={"weight": "norm.w", "bias": "norm.b"}),
                         head=HeadSpec(self.vocab_size, D, bias=False, tied=True, names={}))


def plain_two_mixers(cfg, w, tokens):
    T = len(tokens)
    posn = np.arange(T)
    H, dh = cfg.n_head, cfg.width // cfg.n_head
    x = w["embed"][np.asarray(tokens)]
    for i in range(2):
        h = P.layer_norm(x, w[f"l{i}.n.w"], w[f"l{i}.n.b"], 1e-5)
        q = P.rotary_interleaved((h @ w[f"l{i}.q"].T).reshape(T, H, dh), posn, dh // 2)
        k = P.rotary_interleaved((h @ w[f"l{i}.k"].T).reshape(T, H, dh), posn, dh // 2)
        v = (h @ w[f"l{i}.v"].T).reshape(T, H, dh)
        a = P.causal_attention(q, k, v) @ w[f"l{i}.o"].T
        m = (np.cumsum(h, 0) / (posn[:, None] + 1.0)) @ w[f"l{i}.mean"].T
        x = x + a + m
    return P.layer_norm(x, w["norm.w"], w["norm.b"], 1e-5) @ w["embed"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_layer_with_two_mixers_and_no_feed_forward(tmp_path, registered, dtype):
    """What a layer is made of belongs to its arrangement: one registered here has two mixers that both use
    the cache (keys and values; a running sum) and no feed-forward, and each schedule run names two cache
    entries.  Nothing of the library changes."""
    register("arrangement", "toy_two_mixers", TwoMixerBlock)
    qs.register_architecture(TwoMixerConfig, "two_mixer_toy")
    cfg = config_from_dict(dict(architectures=["TwoMixerForCausalLM"], width=64, n_head=2, vocab_size=83, n_positions=128))
    folder = qs.write_model_folder(tmp_path / "two", cfg, seed=6, dtype=dtype)
    model = qs.load_model(folder, dtype=dtype, device="cuda")
    assert set(model.kv_needs()) == {0, 2} and set(model.state_needs()) == {1, 3}
    engine = qs.Engine(model, max_tokens=64 * 4, max_batch=2)
    w = P.read_safetensors(folder / "model.safetensors")
    rng = np.random.default_rng(7)
    reqs = [[int(t) for t in rng.integers(0, 83, n)] for n in (80, 21)]
    refs = [plain_two_mixers(cfg, w, r) for r in reqs]
    atol = 2e-4 if dtype == "float32" else 6e-2
    for _ in range(2):                                      # twice: slots, pages and state are used again
        slots = [engine.acquire(), engine.acquire()]
        heads = [66, 5]
        out = engine.step(slots, [r[:h] for r, h in zip(reqs, heads)], [list(range(h)) for h in heads]).cpu().double().numpy()
        np.testing.assert_allclose(out[:66], refs[0][:66], atol=atol, rtol=5e-2)
        np.testing.assert_allclose(out[66:], refs[1][:5], atol=atol, rtol=5e-2)
        for step in range(10):
            out = engine.step(slots, [[r[h + step]] for r, h in zip(reqs, heads)]).cpu().double().numpy()
            for i, (r, h) in enumerate(zip(reqs, heads)):
                np.testing.assert_allclose(out[i], refs[i][h + step], atol=atol, rtol=5e-2)
        for s in slots:
            engine.release(s)
        engine.cache.check()
    with pytest.raises(qs.QStreamError, match="cache entries"):
        import dataclasses
        from qstream_b200.weights import random_tensors
        spec = dataclasses.replace(cfg.model_spec(), schedule=(LayerRun(0, 0), LayerRun(1, (2, 3))))
        qs.CausalLM(spec, random_tensors(declared_tensors(spec), 0, torch.float32, "cuda"), "float32", "cuda")
