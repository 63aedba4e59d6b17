"""The engine at GPT-J-6B's layer sizes (2 of its 28 layers) against the plain model.

Width 4096, 16 heads of 256, rotary 64, inner 16384, vocabulary 50400, 2048 positions:
the sizes at which the benchmark runs, where the model takes kernels that the tiny
configurations never reach together (CTA-pair matrix products with K = 20480 for the
fused output projection, the head-size-256 prefill attention, split-K weight streaming,
decode attention over several splits of 256 keys, decode graphs of 8 and 16 rows with
padding rows, page tables of more than a dozen pages).  Compared in float32 and in
bfloat16, in the three cuttings: a request whole; its last 32 tokens one by one (at a
context beyond 1024); batches of unequal prompts decoded together, the shorter
requests ending earlier, one batch after another so that slots and pages are used again.

The weights are drawn once in bfloat16 (N(0, 0.02), norms 1 + U(-0.1, 0.1)) on the
device; the float32 engine gets the same values widened, so one pass of the plain
model (float64 throughout, numpy, on the host copy of those weights) serves both.
"""
import numpy as np
import pytest
import torch

import plain_gptj as P
import qstream_b200 as qs
from qstream_b200.csrc import ops
from qstream_b200.engine.model import declared_tensors
from qstream_b200.weights.random_init import random_tensors
from util import assert_logits_close, random_tokens

pytestmark = pytest.mark.gpu

N_LAYER, N_LAYER_FULL = 2, 28
SIZES = dict(n_layer=N_LAYER, n_embd=4096, n_head=16, n_positions=2048, vocab_size=50400, rotary_dim=64,
             n_inner=16384, activation_function="gelu_new", layer_norm_epsilon=1e-5,
             architectures=["GPTJForCausalLM"])
LONG = 1100                                 # tokens of the long request: 1068 in one step, 32 one by one
LONG_WANT = 8                               # places of its prompt whose logits are compared
# (prompt length, tokens decoded after it); six and nine live requests: graphs of 8 and 16 rows
BATCHES = [[(300, 4), (5, 10), (64, 2), (129, 6), (33, 8), (1, 12)],
           [(17, 3), (70, 5), (2, 9), (257, 3), (40, 1), (9, 7), (100, 2), (31, 4), (64, 6)]]


@pytest.fixture(scope="module")
def setup():
    cfg = qs.GptjConfig.from_dict(SIZES)
    spec = cfg.model_spec()
    dev = torch.device("cuda")
    bf16 = random_tensors(declared_tensors(spec), 3, torch.bfloat16, dev)
    rng = np.random.default_rng(66)
    long_req = random_tokens(rng, LONG, cfg.vocab_size)
    batches = [[random_tokens(rng, p + e, cfg.vocab_size) for p, e in b] for b in BATCHES]

    # the plain model, layer by layer; the head only where logits are compared
    w = {k: v.float().cpu().numpy().astype(np.float64) for k, v in bf16.items()}
    pcfg = P.normalise_config(cfg.to_dict())

    def plain(tokens, rows):
        x = P.embedding(w["transformer.wte.weight"], tokens)
        for i in range(N_LAYER):
            x = P.block(x, w, i, pcfg, np.arange(len(tokens)))
        return P.output_head(x[rows], w, pcfg)

    refs = {"long": plain(long_req, list(range(LONG - 32 - LONG_WANT, LONG)))}
    for bi, (shape, reqs) in enumerate(zip(BATCHES, batches)):
        for ri, ((p, e), toks) in enumerate(zip(shape, reqs)):
            refs[bi, ri] = plain(toks, list(range(p - 1, p + e)))
    del w
    return cfg, spec, bf16, long_req, batches, refs


def make_engine(setup, dtype):
    cfg, spec, bf16, *_ = setup
    if dtype == "bfloat16":
        tensors = bf16
    else:
        tensors = {k: ops.convert(v, torch.float32) for k, v in bf16.items()}
    model = qs.CausalLM(spec, tensors, dtype, "cuda", cfg)
    return qs.Engine(model, max_tokens=16 * 320 + 1152, max_batch=16)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_6b_layer_sizes_in_every_cutting(setup, dtype):
    cfg, spec, bf16, long_req, batches, refs = setup
    eng = make_engine(setup, dtype)
    what = f"6B sizes, {N_LAYER} of {N_LAYER_FULL} layers, {dtype}"

    # a request alone and whole
    slot = eng.acquire()
    rows = list(range(LONG - 32 - LONG_WANT, LONG))
    got = eng.step([slot], [long_req], [rows]).cpu().numpy()
    eng.check_status()
    eng.release(slot)
    assert_logits_close(got, refs["long"], dtype, f"{what}: whole")

    # the same request with its last 32 tokens one by one (decode at contexts 1068 .. 1099)
    slot = eng.acquire()
    head = LONG - 32
    parts = [eng.step([slot], [long_req[:head]], [list(range(head - LONG_WANT, head))]).cpu().numpy()]
    for t in range(head, LONG):
        parts.append(eng.step([slot], [[long_req[t]]]).cpu().numpy())
    eng.check_status()
    eng.release(slot)
    assert_logits_close(np.concatenate(parts), refs["long"], dtype, f"{what}: last 32 one by one")

    # batches of unequal prompts, one after another through the same slots and pages
    for bi, (shape, reqs) in enumerate(zip(BATCHES, batches)):
        slots = [eng.acquire() for _ in reqs]
        out = eng.step(slots, [r[:p] for r, (p, _) in zip(reqs, shape)]).cpu().numpy()
        got = [[out[i:i + 1]] for i in range(len(reqs))]
        pos = [p for p, _ in shape]
        live = list(range(len(reqs)))
        while live:
            out = eng.step([slots[i] for i in live], [[reqs[i][pos[i]]] for i in live]).cpu().numpy()
            nxt = []
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1])
                pos[i] += 1
                if pos[i] < len(reqs[i]):
                    nxt.append(i)
                else:
                    eng.release(slots[i])
            live = nxt
        eng.check_status()
        eng.cache.check()
        for ri in range(len(reqs)):
            assert_logits_close(np.concatenate(got[ri]), refs[bi, ri], dtype, f"{what}: batch {bi} request {ri}")
    assert eng.cache.slots.n_free == eng.cache.slots.n_slots


def test_bfloat16_engine_against_float32_engine(setup):
    """The two engines against each other (not only each against the plain model): same weights, the
    long request whole; the bfloat16 logits stay within the bfloat16 bound of the float32 logits."""
    cfg, spec, bf16, long_req, *_ = setup
    rows = list(range(LONG - 16, LONG))
    out = {}
    for dtype in ("float32", "bfloat16"):
        eng = make_engine(setup, dtype)
        slot = eng.acquire()
        out[dtype] = eng.step([slot], [long_req], [rows]).cpu().numpy()
        eng.check_status()
        eng.release(slot)
        del eng
    assert_logits_close(out["bfloat16"], out["float32"], "bfloat16", "bfloat16 engine against float32 engine")
