"""Helpers of the tests: the two tiny configurations, model folders, tolerances."""
from __future__ import annotations

import numpy as np

import qstream_b200 as qs
from qstream_b200.weights import InitScales

import plain_gptj as P

# Two tiny GPT-J configurations that differ in every size and option.
TINY_A = dict(n_layer=2, n_embd=64, n_head=4, n_positions=128, vocab_size=256, rotary_dim=8,
              n_inner=None, activation_function="gelu_new", layer_norm_epsilon=1e-5,
              bos_token_id=None, eos_token_id=None)
SCALES_A = InitScales(matrix_std=0.02, norm_spread=0.1, bias_std=0.02)
TINY_B = dict(n_layer=3, n_embd=96, n_head=3, n_positions=256, vocab_size=320, rotary_dim=32,
              n_inner=320, activation_function="gelu", layer_norm_epsilon=1e-6,
              bos_token_id=None, eos_token_id=None)
SCALES_B = InitScales(matrix_std=0.05, norm_spread=0.2, bias_std=0.01)
TINY = {"A": (TINY_A, SCALES_A, 0), "B": (TINY_B, SCALES_B, 1)}


def make_folder(tmp_path, which: str, dtype: str):
    cfg_dict, scales, seed = TINY[which]
    cfg = qs.GptjConfig.from_dict({**cfg_dict, "architectures": ["GPTJForCausalLM"]})
    folder = tmp_path / f"tiny_{which}_{dtype}"
    qs.write_model_folder(folder, cfg, seed, dtype, scales)
    return folder, cfg


def random_tokens(rng: np.random.Generator, n: int, vocab: int) -> list:
    return [int(t) for t in rng.integers(0, vocab, size=n)]


# Tolerances, fixed before the first run on a GPU and not widened since.
# float32 engine against the float64 plain model: rounding of 32-bit sums only.
F32_ATOL, F32_RTOL = 1e-5, 1e-4
# bfloat16 engine: every activation is rounded to 8 bits of mantissa (2^-9 relative) a
# dozen times per layer; the bound is relative to the largest logit of the row.
BF16_MAX_REL, BF16_MEAN_REL = 3e-2, 6e-3


def assert_logits_close(got: np.ndarray, ref: np.ndarray, dtype: str, what: str = ""):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    err = np.abs(got - ref)
    if dtype == "float32":
        bad = err > F32_ATOL + F32_RTOL * np.abs(ref)
        assert not bad.any(), (f"{what}: {bad.sum()} of {bad.size} logits differ; worst {err.max():.3e} "
                               f"at {np.unravel_index(err.argmax(), err.shape)}")
    else:
        scale = np.maximum(np.abs(ref).max(axis=-1, keepdims=True), 1e-3)
        rel = err / scale
        assert rel.max() <= BF16_MAX_REL, (f"{what}: worst error {rel.max():.3e} of the row's largest logit "
                                           f"at {np.unravel_index(rel.argmax(), rel.shape)}")
        assert rel.mean() <= BF16_MEAN_REL, f"{what}: mean error {rel.mean():.3e} of the row's largest logit"


def plain_logits(folder, tokens):
    cfg, w = P.load_model(folder)
    return P.logits_whole(cfg, w, tokens)
