"""The plain implementation itself (no GPU): against QStream's own scalar kernels and sampler
(tests/golden/reference_ops.json, made by tests/golden/make_reference_ops.py), against
independent formulas, and for the properties the engine tests lean on."""
import json
import math
from pathlib import Path

import numpy as np
import pytest

import plain_gptj as P
from util import make_folder

GOLDEN = json.loads((Path(__file__).parent / "golden" / "reference_ops.json").read_text())


def test_layer_norm_matches_the_reference_kernel():
    for c in GOLDEN["layer_norm"]:
        y = P.layer_norm(np.array(c["x"]), np.array(c["w"]), np.array(c["b"]), c["eps"])
        np.testing.assert_allclose(y, c["y"], atol=2e-6, rtol=2e-6)


def test_gelu_softmax_match_the_reference_kernels():
    np.testing.assert_allclose(P.gelu_new(np.array(GOLDEN["gelu_tanh"]["x"])), GOLDEN["gelu_tanh"]["y"], atol=1e-6)
    np.testing.assert_allclose(P.softmax(np.array(GOLDEN["softmax"]["x"])), GOLDEN["softmax"]["y"], atol=1e-7)
    x = np.linspace(-4, 4, 33)
    assert np.abs(P.gelu_erf(x) - P.gelu_new(x)).max() < 2e-3          # two close but different functions
    assert np.abs(P.gelu_erf(x) - P.gelu_new(x)).max() > 1e-5


def test_rng_argmax_penalty_match_the_reference():
    for seed, draws in GOLDEN["rng"].items():
        r = P.XorShift128Plus(int(seed))
        assert [r.next_float() for _ in draws] == draws
    assert P.argmax_lowest(np.array([1.0, 5.0, 5.0, -2.0, 5.0])) == GOLDEN["argmax_tie"] == 1
    c = GOLDEN["repeat_penalty"]
    np.testing.assert_allclose(P.apply_repeat_penalty(np.array(c["x"]), c["recent"], c["penalty"]), c["y"], rtol=1e-6)


def test_filters_and_pipeline_match_the_reference():
    k = GOLDEN["top_k"]
    assert list(np.nonzero(np.isfinite(P.top_k_filter(np.array(k["x"]), k["k"])))[0]) == k["kept"]
    p = GOLDEN["top_p"]
    assert list(np.nonzero(np.isfinite(P.top_p_filter(np.array(p["x"]), p["p"])))[0]) == p["kept"]
    logits = np.array(GOLDEN["sample"]["logits"])
    for run in GOLDEN["sample"]["runs"]:
        rng = P.XorShift128Plus(run["seed"])
        got = []
        for _ in run["tokens"]:
            r = rng.next_float() if run["temperature"] >= 0.01 else 0.0
            got.append(P.sample(logits, run["temperature"], run["top_k"], run["top_p"], r))
        assert got == run["tokens"], run


def test_rotary_matches_the_reference_engine():
    """QStream's `apply_rope` (src/engine.c:205-234, run through a shim by the golden script) rotates the
    whole head with frequency base^(-i / head_dim): the plain rotation with rotary_dim = head_dim is the
    same function, and a partial rotation is that function on the first rotary_dim dims of a wider head.
    The reference rounds the frequency to 32 bits before it multiplies by the position, so the angles
    differ by up to position * 1e-7."""
    for c in GOLDEN["apply_rope"]:
        dh, pos = c["head_dim"], c["position"]
        tol = 2e-6 + 4e-7 * pos
        q = np.array(c["q"]).reshape(1, 2, dh)
        k = np.array(c["k"]).reshape(1, 1, dh)
        np.testing.assert_allclose(P.rotary_interleaved(q, [pos], dh).reshape(-1), c["q_out"], atol=tol, rtol=0)
        np.testing.assert_allclose(P.rotary_interleaved(k, [pos], dh).reshape(-1), c["k_out"], atol=tol, rtol=0)
        # partial: a head of 2 * dh dims of which the first dh are rotated
        wide = np.concatenate([q, 7.0 + q], axis=-1)
        out = P.rotary_interleaved(wide, [pos], dh)
        np.testing.assert_allclose(out[..., :dh].reshape(-1), c["q_out"], atol=tol, rtol=0)
        np.testing.assert_array_equal(out[..., dh:], wide[..., dh:])
    moved = [c for c in GOLDEN["apply_rope"] if c["position"] == 63 and c["head_dim"] == 32][0]
    assert np.abs(np.array(moved["q_out"]) - np.array(moved["q"])).max() > 0.1       # the case is not trivial


def test_rotary_is_a_rotation_of_pairs():
    rng = np.random.default_rng(0)
    v = rng.normal(size=(6, 2, 16))
    pos = np.array([0, 1, 2, 50, 51, 127])
    for R in (16, 8):
        out = P.rotary_interleaved(v, pos, R)
        z = v[..., 0:R:2] + 1j * v[..., 1:R:2]
        freq = 10000.0 ** (-np.arange(0, R, 2) / R)
        want = z * np.exp(1j * pos[:, None, None] * freq[None, None, :])
        np.testing.assert_allclose(out[..., 0:R:2], want.real, atol=1e-12)
        np.testing.assert_allclose(out[..., 1:R:2], want.imag, atol=1e-12)
        np.testing.assert_array_equal(out[..., R:], v[..., R:])             # dims beyond R untouched
    np.testing.assert_array_equal(P.rotary_interleaved(v, np.zeros(6), 16), v)


def test_attention_is_causal_and_windowed():
    rng = np.random.default_rng(1)
    q, k, v = (rng.normal(size=(9, 4, 8)) for _ in range(3))
    full = P.causal_attention(q, k, v)
    k2, v2 = k.copy(), v.copy()
    k2[5:], v2[5:] = 9.0, -9.0
    np.testing.assert_allclose(P.causal_attention(q, k2, v2)[:5], full[:5])          # later keys do not exist
    np.testing.assert_allclose(P.causal_attention(q, k, v)[0], v[0].reshape(-1))     # one key: its value
    np.testing.assert_allclose(P.causal_attention(q, k, v, window=1), v.reshape(9, -1))
    w3 = P.causal_attention(q, k, v, window=3)
    np.testing.assert_allclose(w3[:3], full[:3])
    assert np.abs(w3[8] - full[8]).max() > 1e-3
    grouped = P.causal_attention(q, k[:, :2], v[:, :2])                              # 4 query heads on 2 key heads
    np.testing.assert_allclose(grouped[:, 8:16], P.causal_attention(q[:, 1:2], k[:, :1], v[:, :1]))


def test_whole_model_is_causal_and_uses_every_part(tmp_path):
    folder, cfg = make_folder(tmp_path, "B", "float32")
    pcfg, w = P.load_model(folder)
    toks = [3, 1, 4, 1, 5, 9, 2, 6]
    full = P.logits_whole(pcfg, w, toks)
    assert full.shape == (8, 320)
    np.testing.assert_allclose(P.logits_whole(pcfg, w, toks[:5]), full[:5], atol=1e-12)   # a prefix's logits stay
    for name in ("lm_head.bias", "transformer.h.2.mlp.fc_out.bias", "transformer.h.0.ln_1.bias",
                 "transformer.h.1.attn.out_proj.weight", "transformer.ln_f.weight"):
        w2 = dict(w)
        w2[name] = w[name] + 0.1 * np.cos(np.arange(w[name].size)).reshape(w[name].shape)   # not a constant shift: LayerNorm would remove it
        assert np.abs(P.logits_whole(pcfg, w2, toks) - full).max() > 1e-6, name
    other = dict(pcfg, activation_function="gelu_new")
    assert np.abs(P.logits_whole(other, w, toks) - full).max() > 1e-7
    assert np.abs(P.logits_whole(dict(pcfg, rotary_dim=16), w, toks)[1:] - full[1:]).max() > 1e-7
    greedy = P.generate_greedy(pcfg, w, toks[:3], 4)
    assert len(greedy) == 4 and greedy[0] == int(np.argmax(full[2]))
