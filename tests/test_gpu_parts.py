"""Each part alone, built from its spec with tensors made in the test, against the plain functions."""
import numpy as np
import pytest
import torch

import plain_gptj as P
from qstream_b200.cache import SequenceCache
from qstream_b200.config import AttentionSpec, BlockSpec, MlpSpec, NormSpec, PositionSpec
from qstream_b200.engine.step import StepBatch, StepContext
from qstream_b200.parts import Runtime, build_block, part_class

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def f64(t):
    return t.detach().cpu().to(torch.float64).numpy()


def tol(dtype):
    return dict(atol=3e-5, rtol=1e-4) if dtype == "float32" else dict(atol=4e-2, rtol=3e-2)


def assert_rows_close(got, ref, dtype):
    """float32: element by element.  bfloat16: a block's output is a sum of terms that were each
    rounded to 8 bits, so the error is measured against the row's largest element (the rule of
    util.assert_logits_close)."""
    if dtype == "float32":
        np.testing.assert_allclose(got, ref, **tol(dtype))
    else:
        from util import assert_logits_close
        assert_logits_close(got, ref, dtype)


def make(role, spec, dtype, seed=0):
    """Build a part with random tensors; returns (part, {own name: float64 array})."""
    cls = part_class(role, spec.kind)
    g = torch.Generator().manual_seed(seed)
    tensors = {}
    for name, decl in cls.declare(spec).items():
        t = torch.randn(decl.shape, generator=g) * (0.3 if decl.role != "norm_weight" else 0.1)
        if decl.role == "norm_weight":
            t = t + 1
        tensors[name] = t.to(DT[dtype]).cuda()
    part = cls(spec, tensors, Runtime(DT[dtype], torch.device("cuda")))
    return part, {k: f64(v) for k, v in tensors.items()}


def step_for(cache, slots, new_tokens):
    """A step context for sequences that bring `new_tokens` tokens each (uploads metadata by hand)."""
    cache.prepare(slots, new_tokens)
    tok_slot, tok_pos, start = [], [], [0]
    for s, n in zip(slots, new_tokens):
        p0 = cache.length(s)
        tok_slot += [s] * n
        tok_pos += list(range(p0, p0 + n))
        start.append(start[-1] + n)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32).cuda()
    T = len(tok_slot)
    batch = StepBatch(n_seq=len(slots), n_tokens=T, n_want=0, tokens=i32([0] * T), tok_slot=i32(tok_slot),
                      tok_pos=i32(tok_pos), want_rows=i32([]), seq_slot=i32(slots), seq_start=i32(start),
                      seq_p0=i32([cache.length(s) for s in slots]), slots=list(slots), new_tokens=list(new_tokens),
                      p0=[cache.length(s) for s in slots], decode=all(n == 1 for n in new_tokens),
                      max_new=max(new_tokens), max_total=0)
    return StepContext(batch, cache, torch.zeros(1, dtype=torch.int32).cuda())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layernorm_part(dtype):
    for size, eps, bias in ((40, 1e-5, True), (136, 1e-2, False)):
        part, w = make("norm", NormSpec(size=size, eps=eps, bias=bias), dtype, seed=size)
        x = (torch.randn(5, size, generator=torch.Generator().manual_seed(1)) * 2).to(DT[dtype]).cuda()
        np.testing.assert_allclose(f64(part.forward(x)), P.layer_norm(f64(x), w["weight"], w.get("bias"), eps), **tol(dtype))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mlp_part(dtype):
    for width, inner, act, bias in ((48, 136, "gelu_new", True), (64, 72, "gelu", False)):
        part, w = make("feed_forward", MlpSpec(width=width, inner=inner, activation=act, bias=bias), dtype, seed=inner)
        g = torch.Generator().manual_seed(2)
        h = torch.randn(9, width, generator=g).to(DT[dtype]).cuda()
        r1 = torch.randn(9, width, generator=g).to(DT[dtype]).cuda()
        u = f64(h) @ w["up"].T + (w["up_bias"] if bias else 0)
        ref = P.ACTIVATIONS[act](u) @ w["down"].T + (w["down_bias"] if bias else 0)
        np.testing.assert_allclose(f64(part.forward(h, None)), ref, **tol(dtype))
        np.testing.assert_allclose(f64(part.forward(h, None, residuals=(r1, h))), ref + f64(r1) + f64(h), **tol(dtype))


def attention_reference(h, w, spec, n):
    T = h.shape[0]
    pos = np.arange(n)
    q = (h @ w["q"].T + w.get("q_bias", 0)).reshape(T, spec.n_heads, spec.head_dim)
    k = (h @ w["k"].T + w.get("k_bias", 0)).reshape(T, spec.n_kv_heads, spec.head_dim)
    v = (h @ w["v"].T + w.get("v_bias", 0)).reshape(T, spec.n_kv_heads, spec.head_dim)
    if spec.position is not None:
        q = P.rotary_interleaved(q, pos, spec.position.rotary_dim, spec.position.base)
        k = P.rotary_interleaved(k, pos, spec.position.rotary_dim, spec.position.base)
    o = P.causal_attention(q, k, v, spec.window)
    return o @ w["out"].T + w.get("out_bias", 0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv_heads,dh,rot,window,biases", [(4, 4, 16, 8, 0, False), (6, 2, 32, 32, 0, True),
                                                                 (2, 2, 48, 16, 50, False), (3, 1, 16, None, 0, False)])
def test_attention_part(dtype, heads, kv_heads, dh, rot, window, biases):
    """The mixer alone: a sequence given whole, then one cut into a prompt and single tokens, next to
    another sequence in the same steps; with grouped heads, biases, a window, another base, no rotary."""
    width, n = 72, 150
    pos = PositionSpec(rotary_dim=rot, base=500.0, max_positions=256) if rot else None
    spec = AttentionSpec(width=width, n_heads=heads, n_kv_heads=kv_heads, head_dim=dh, position=pos, window=window,
                         qkv_bias=biases, out_bias=biases)
    part, w = make("mixer", spec, dtype, seed=dh)
    cache = SequenceCache({0: part.kv_need()}, {}, 64 * 8, 4, 256, DT[dtype], "cuda")
    g = torch.Generator().manual_seed(7)
    h1 = (torch.randn(n, width, generator=g) * 0.5).to(DT[dtype]).cuda()
    h2 = (torch.randn(n, width, generator=g) * 0.5).to(DT[dtype]).cuda()
    ref1, ref2 = attention_reference(f64(h1), w, spec, n), attention_reference(f64(h2), w, spec, n)
    a, b = cache.acquire(), cache.acquire()
    # step 1: sequence 1 whole; sequence 2 its first 100
    ctx = step_for(cache, [a, b], [n, 100])
    out = part.forward(torch.cat([h1, h2[:100]]), ctx, 0)
    cache.commit([a, b], [n, 100])
    assert_rows_close(f64(out[:n]), ref1, dtype)          # the output projection sums bfloat16-rounded head outputs
    got2 = [out[n:]]
    cache.release(a)
    for t in range(100, n):                                 # sequence 2 goes on token by token
        ctx = step_for(cache, [b], [1])
        got2.append(part.forward(h2[t:t + 1], ctx, 0))
        cache.commit([b], [1])
    assert_rows_close(f64(torch.cat(got2)), ref2, dtype)
    assert int(ctx.status.item()) == 0
    cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("arrangement", ["parallel", "sequential"])
def test_block_arrangements(dtype, arrangement):
    width, n = 64, 20
    norms = {"input": NormSpec(size=width, eps=1e-5)}
    if arrangement == "sequential":
        norms["post_mixer"] = NormSpec(size=width, eps=1e-4, bias=False)
    spec = BlockSpec(arrangement=arrangement, norms=norms,
                     mixer=AttentionSpec(width=width, n_heads=2, n_kv_heads=2, head_dim=32,
                                         position=PositionSpec(rotary_dim=8, base=10000.0, max_positions=64)),
                     ffn=MlpSpec(width=width, inner=96, activation="gelu_new"))
    made = {}

    def tensors_of(part_spec, decls):
        g = torch.Generator().manual_seed(len(made) + 11)
        t = {}
        for name, d in decls.items():
            v = torch.randn(d.shape, generator=g) * 0.2 + (1 if d.role == "norm_weight" else 0)
            t[name] = v.to(DT[dtype]).cuda()
        made[id(part_spec)] = {k: f64(v) for k, v in t.items()}
        return t

    block = build_block(spec, tensors_of, Runtime(DT[dtype], torch.device("cuda")))
    cache = SequenceCache({0: block.mixer.kv_need()}, {}, 128, 2, 64, DT[dtype], "cuda")
    x = (torch.randn(n, width, generator=torch.Generator().manual_seed(3)) * 0.7).to(DT[dtype]).cuda()
    s = cache.acquire()
    out = block.forward(x, step_for(cache, [s], [n]), 0)
    xs = f64(x)
    wm, wf = made[id(spec.mixer)], made[id(spec.ffn)]
    ln = lambda v, ns: P.layer_norm(v, made[id(ns)]["weight"], made[id(ns)].get("bias"), ns.eps)
    ffn = lambda v: P.gelu_new(v @ wf["up"].T + wf["up_bias"]) @ wf["down"].T + wf["down_bias"]
    if arrangement == "parallel":
        h = ln(xs, norms["input"])
        ref = xs + attention_reference(h, wm, spec.mixer, n) + ffn(h)
    else:
        mid = xs + attention_reference(ln(xs, norms["input"]), wm, spec.mixer, n)
        ref = mid + ffn(ln(mid, norms["post_mixer"]))
    assert_rows_close(f64(out), ref, dtype)
