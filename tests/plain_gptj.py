"""Plain, slow GPT-J for the tests: whole sequences, no cache, one function per part.

Written from the formulas of Ragu-123/Qstream's scalar engine (paths are those of
that project).  Where GPT-J needs something the reference engine does not do, the
function says so; those parts rest on the GPT-J architecture itself (parallel
residual, partial rotary, biases), not on reference code.  The whole-model result
therefore rests on the formulas; the per-part functions are compared once with the
reference's own scalar kernels by `tests/golden/make_reference_ops.py`.

This module shares no code with `qstream_b200`: it reads config.json and
model.safetensors itself, with numpy only.  All arithmetic is float64 unless
`dtype` says otherwise, so it is the "true" value both for the 32-bit and for the
bfloat16 engine.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np


# --------------------------------------------------------------------------- files

_ST_DTYPES = {"F32": np.float32, "F16": np.float16, "F64": np.float64,
              "I32": np.int32, "I64": np.int64}


def read_safetensors(path) -> dict[str, np.ndarray]:
    """Every tensor of a .safetensors file as float64 / int arrays.

    Same reading as the converter's TensorLoader: any float dtype becomes one
    working float type (tools/convert_hf.py:617-652).
    """
    raw = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    blob = memoryview(raw)[8 + hlen:]
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        a, b = meta["data_offsets"]
        buf = blob[a:b]
        if meta["dtype"] == "BF16":
            u16 = np.frombuffer(buf, dtype=np.uint16).astype(np.uint32) << 16
            arr = u16.view(np.float32).astype(np.float64)
        else:
            arr = np.frombuffer(buf, dtype=_ST_DTYPES[meta["dtype"]])
            if arr.dtype.kind == "f":
                arr = arr.astype(np.float64)
        out[name] = arr.reshape(meta["shape"])
    return out


def load_model(folder):
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    weights = read_safetensors(folder / "model.safetensors")
    return cfg, weights


# --------------------------------------------------------------------------- parts

def embedding(wte, tokens):
    """Row lookup, no position term, no scale (src/engine.c:710-765)."""
    return wte[np.asarray(tokens, dtype=np.int64)]


def layer_norm(x, w, b, eps):
    """Two-pass mean / biased variance, 1/sqrt(var+eps), *w, +b
    (src/kernels_scalar.c:151-171)."""
    mean = x.mean(axis=-1, keepdims=True)
    d = x - mean
    var = (d * d).mean(axis=-1, keepdims=True)
    y = d * (1.0 / np.sqrt(var + eps)) * w
    return y + b if b is not None else y


def linear(x, w, b=None):
    """y = x W^T (+ b), weight rows = outputs (include/qsf/kernels.h:53-58;
    bias is GPT-J's, the reference engine drops it, src/engine.c:1150-1170)."""
    y = x @ w.T
    return y + b if b is not None else y


def gelu_new(u):
    """tanh GELU with c = sqrt(2/pi) and 0.044715 (src/kernels_scalar.c:135-142)."""
    c = math.sqrt(2.0 / math.pi)
    return 0.5 * u * (1.0 + np.tanh(c * (u + 0.044715 * u * u * u)))


def gelu_erf(u):
    """Exact GELU, 0.5 u (1 + erf(u / sqrt 2)).  The reference maps 'gelu' to
    the tanh kernel (tools/convert_hf.py:75-79); GPT-J's 'gelu' is this one."""
    erf = np.vectorize(math.erf, otypes=[np.float64])
    return 0.5 * u * (1.0 + erf(u / math.sqrt(2.0)))


ACTIVATIONS = {"gelu_new": gelu_new, "gelu": gelu_erf}


def rotary_interleaved(v, positions, rotary_dim, base=10000.0):
    """Rotate pairs (i, i+1), i even, of the first `rotary_dim` dims of every head.

    Pairing and signs: src/engine.c:216-218; frequency 1/base^(i/R) with R the
    rotated width (src/engine.c:211 uses head_dim because it rotates the whole
    head; GPT-J rotates rotary_dim dims).  v: [T, H, dh]; positions: [T].
    """
    out = v.copy()
    i = np.arange(0, rotary_dim, 2, dtype=np.float64)
    freq = 1.0 / np.power(base, i / rotary_dim)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]
    cos = np.cos(ang)[:, None, :]
    sin = np.sin(ang)[:, None, :]
    a = v[..., 0:rotary_dim:2]
    b = v[..., 1:rotary_dim:2]
    out[..., 0:rotary_dim:2] = a * cos - b * sin
    out[..., 1:rotary_dim:2] = a * sin + b * cos
    return out


def softmax(s):
    """max-subtract, exp, divide by the sum (src/kernels_scalar.c:188-213)."""
    m = s.max(axis=-1, keepdims=True)
    e = np.exp(s - m)
    return e / e.sum(axis=-1, keepdims=True)


def causal_attention(q, k, v, window=0):
    """scores = q.k / sqrt(dh) over keys u <= t (src/engine.c:888-906), softmax
    (:910), weighted sum of v (:913-922), heads concatenated in head order.
    Query head j reads key head j // (H / Hkv) (src/engine.c:884,889).
    `window` > 0 keeps only keys u > t - window.  q: [T, H, dh]; k, v: [T, Hkv, dh].
    """
    T, H, dh = q.shape
    groups = H // k.shape[1]
    scale = 1.0 / math.sqrt(dh)
    out = np.zeros_like(q)
    t_idx = np.arange(T)
    allowed = t_idx[None, :] <= t_idx[:, None]
    if window > 0:
        allowed &= t_idx[None, :] > (t_idx[:, None] - window)
    for h in range(H):
        s = (q[:, h, :] @ k[:, h // groups, :].T) * scale
        s = np.where(allowed, s, -np.inf)
        out[:, h, :] = softmax(s) @ v[:, h // groups, :]
    return out.reshape(T, H * dh)


def attention_mixer(h, w, prefix, n_head, rotary_dim, positions, window=0):
    """q/k/v projections without bias (src/engine.c:841-867), rotary on q and k
    before the keys are kept (:871-880), attention, output projection (:926-934)."""
    T, D = h.shape
    dh = D // n_head
    q = linear(h, w[prefix + "q_proj.weight"]).reshape(T, n_head, dh)
    k = linear(h, w[prefix + "k_proj.weight"]).reshape(T, n_head, dh)
    v = linear(h, w[prefix + "v_proj.weight"]).reshape(T, n_head, dh)
    q = rotary_interleaved(q, positions, rotary_dim)
    k = rotary_interleaved(k, positions, rotary_dim)
    o = causal_attention(q, k, v, window)
    return linear(o, w[prefix + "out_proj.weight"])


def mlp(h, w, prefix, activation):
    """fc_in -> activation -> fc_out (src/engine.c:1150-1170), with GPT-J's biases."""
    u = linear(h, w[prefix + "fc_in.weight"], w[prefix + "fc_in.bias"])
    return linear(ACTIVATIONS[activation](u), w[prefix + "fc_out.weight"],
                  w[prefix + "fc_out.bias"])


def block(x, w, i, cfg, positions):
    """GPT-J's parallel residual: h = ln_1(x); x + attn(h) + mlp(h).  The
    reference engine runs the sequential two-norm form (src/engine.c:936-948,
    1173-1174); the parallel form is the architecture's."""
    p = f"transformer.h.{i}."
    h = layer_norm(x, w[p + "ln_1.weight"], w[p + "ln_1.bias"], cfg["layer_norm_epsilon"])
    a = attention_mixer(h, w, p + "attn.", cfg["n_head"], cfg["rotary_dim"], positions)
    m = mlp(h, w, p + "mlp.", cfg["activation_function"])
    return x + a + m


def output_head(x, w, cfg):
    """Final norm (src/engine.c:1191-1197) and untied head with bias (:1237-1241)."""
    z = layer_norm(x, w["transformer.ln_f.weight"], w["transformer.ln_f.bias"],
                   cfg["layer_norm_epsilon"])
    return linear(z, w["lm_head.weight"], w["lm_head.bias"])


def normalise_config(cfg):
    cfg = dict(cfg)
    cfg.setdefault("layer_norm_epsilon", 1e-5)
    cfg.setdefault("activation_function", "gelu_new")
    if cfg.get("rotary_dim") is None:
        cfg["rotary_dim"] = cfg["n_embd"] // cfg["n_head"]
    return cfg


def logits_whole(cfg, w, tokens):
    """Logits [T, V] of one whole sequence, float64."""
    cfg = normalise_config(cfg)
    positions = np.arange(len(tokens))
    x = embedding(w["transformer.wte.weight"], tokens)
    for i in range(cfg["n_layer"]):
        x = block(x, w, i, cfg, positions)
    return output_head(x, w, cfg)


# --------------------------------------------------------------------------- sampling

class XorShift128Plus:
    """SplitMix64-seeded xorshift128+ (src/sampling.c:13-38)."""
    M = (1 << 64) - 1

    def __init__(self, seed):
        s = []
        seed &= self.M
        for _ in range(2):
            seed = (seed + 0x9E3779B97F4A7C15) & self.M
            z = seed
            z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & self.M
            z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & self.M
            seed = z            # the reference feeds the mixed value on (sampling.c:15-22)
            z = z ^ (z >> 31)
            s.append(z if z else 1)
        self.s = s

    def next_float(self):
        s0, s1 = self.s
        result = (s0 + s1) & self.M
        s1 ^= s0
        self.s[0] = (((s0 << 55) | (s0 >> 9)) ^ s1 ^ (s1 << 14)) & self.M
        self.s[1] = ((s1 << 36) | (s1 >> 28)) & self.M
        return float(result >> 41) * (1.0 / float(1 << 23))


def argmax_lowest(logits):
    """Strict '>' scan: the lowest index wins ties (src/sampling.c:214-224)."""
    return int(np.argmax(logits))


def apply_repeat_penalty(logits, recent, penalty):
    """Divide positive, multiply negative logits of recent tokens, once per
    occurrence (src/sampling.c:59-74)."""
    if penalty <= 1.0:
        return logits
    logits = logits.copy()
    for t in recent:
        if 0 <= t < len(logits):
            logits[t] = logits[t] / penalty if logits[t] > 0 else logits[t] * penalty
    return logits


def top_k_filter(logits, k):
    """Everything below the k-th largest becomes -inf; ties at it stay
    (src/sampling.c:77-118)."""
    if k <= 0 or k >= len(logits):
        return logits
    thresh = np.sort(logits)[::-1][k - 1]
    return np.where(logits < thresh, -np.inf, logits)


def top_p_filter(logits, p):
    """Softmax, stable descending order, keep through the first index whose
    cumulative probability exceeds p (src/sampling.c:121-175)."""
    if p >= 1.0:
        return logits
    probs = softmax(logits)
    order = np.argsort(-probs, kind="stable")
    cum = np.cumsum(probs[order])
    over = np.nonzero(cum > p)[0]
    cutoff = int(over[0]) + 1 if len(over) else len(logits)
    out = logits.copy()
    out[order[cutoff:]] = -np.inf
    return out


def cdf_interval(probs, token):
    """[low, high] of the cumulative sums that make `token` the answer of the
    inverse-CDF draw (first i with cum >= r, src/sampling.c:199-211)."""
    cum = np.cumsum(probs)
    return (float(cum[token - 1]) if token > 0 else 0.0), float(cum[token])


def sample(logits, temperature, top_k, top_p, r):
    """The reference's pipeline (src/sampling.c:227-250) with the draw r given."""
    logits = np.asarray(logits, dtype=np.float64)
    if temperature < 0.01:
        return argmax_lowest(logits)
    if temperature != 1.0:
        logits = logits * (1.0 / temperature)
    if 0 < top_k < len(logits):
        logits = top_k_filter(logits, top_k)
    if 0.0 < top_p < 1.0:
        logits = top_p_filter(logits, top_p)
    probs = softmax(logits)
    cum = np.cumsum(probs)
    hit = np.nonzero(cum >= r)[0]
    if len(hit):
        return int(hit[0])
    nz = np.nonzero(probs > 0)[0]
    return int(nz[-1]) if len(nz) else 0


def generate_greedy(cfg, w, prompt, max_new_tokens, stop_tokens=()):
    """Greedy continuation by whole-sequence recomputation (the loop of
    src/engine.c:1315-1363 without its cache): a stop token ends the sequence
    and is not emitted (:1331)."""
    tokens = list(prompt)
    out = []
    for _ in range(max_new_tokens):
        nxt = argmax_lowest(logits_whole(cfg, w, tokens)[-1])
        if nxt in stop_tokens:
            break
        out.append(nxt)
        tokens.append(nxt)
    return out
