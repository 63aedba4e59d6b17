"""Generation through the Python entry point, against the plain model."""
import numpy as np
import pytest

import qstream_b200 as qs
import plain_gptj as P
from util import make_folder, random_tokens

pytestmark = pytest.mark.gpu


def plain_next(pcfg, w, toks):
    return P.logits_whole(pcfg, w, toks)[-1]


@pytest.mark.parametrize("which,dtype", [("A", "float32"), ("B", "float32"), ("A", "bfloat16"), ("B", "bfloat16")])
def test_greedy_generation(tmp_path, which, dtype):
    """Unequal prompts, more requests than slots (so batches follow one another and slots are used
    again).  Every generated token must be the plain model's argmax given the tokens before it; in
    bfloat16 a token may differ only where the plain model's two best logits are closer than rounding."""
    folder, cfg = make_folder(tmp_path, which, dtype)
    pcfg, w = P.load_model(folder)
    rng = np.random.default_rng(21)
    lens = [5, 9, 16, 1, 33, 2, 64]
    prompts = [random_tokens(rng, n, cfg.vocab_size) for n in lens]
    model = qs.load_model(folder, dtype=dtype, device="cuda")
    engine = qs.Engine(model, max_tokens=64 * 6, max_batch=3)
    res = qs.generate(engine, prompts, max_new_tokens=8, sampling=qs.SamplingConfig.greedy(), stop_tokens=())
    assert len(res.batches) >= 3 and all(len(t) == 8 for t in res.tokens)
    assert res.finish_reasons == ["length"] * len(prompts)
    for prompt, got in zip(prompts, res.tokens):
        toks = list(prompt)
        for g in got:
            logits = plain_next(pcfg, w, toks)
            best = int(np.argmax(logits))
            if g != best:
                gap = logits[best] - logits[g]
                assert dtype == "bfloat16" and gap < 0.03 * np.abs(logits).max(), (toks, g, best, gap)
            toks.append(g)
    engine.cache.check()
    assert engine.cache.slots.n_free == engine.cache.slots.n_slots


def test_temperature_sampling_follows_the_plain_distribution(tmp_path):
    """Tiny B at temperature 0.8 with seed 7: each token's interval of the plain model's CDF must
    contain the draw of the request's own random stream."""
    from qstream_b200.sampling import XorShift128Plus, request_seed
    folder, cfg = make_folder(tmp_path, "B", "float32")
    pcfg, w = P.load_model(folder)
    rng = np.random.default_rng(22)
    prompts = [random_tokens(rng, n, cfg.vocab_size) for n in (1, 7, 20, 33)]
    model = qs.load_model(folder, dtype="float32", device="cuda")
    engine = qs.Engine(model, max_tokens=64 * 8, max_batch=4)
    sampling = qs.SamplingConfig(temperature=0.8, top_k=0, top_p=1.0, repeat_penalty=1.0, seed=7)
    res = qs.generate(engine, prompts, max_new_tokens=12, sampling=sampling, stop_tokens=())
    again = qs.generate(engine, prompts[::-1], max_new_tokens=12, sampling=sampling, stop_tokens=())
    assert again.tokens[3] != res.tokens[0]             # request 3 of the second call has another stream
    for i, (prompt, got) in enumerate(zip(prompts, res.tokens)):
        stream = XorShift128Plus(request_seed(7, i))
        toks = list(prompt)
        for g in got:
            r = stream.next_float()
            y = plain_next(pcfg, w, toks) / 0.8
            lo, hi = P.cdf_interval(P.softmax(y), g)
            assert lo - 1e-4 <= r <= hi + 1e-4, (i, g, lo, hi, r)
            toks.append(g)


def test_stop_tokens_filters_and_penalty(tmp_path):
    folder, cfg = make_folder(tmp_path, "A", "float32")
    pcfg, w = P.load_model(folder)
    model = qs.load_model(folder, dtype="float32", device="cuda")
    engine = qs.Engine(model, max_tokens=256, max_batch=2)
    prompt = [5, 17, 3, 200, 9]
    free = qs.generate(engine, [prompt], max_new_tokens=6, sampling=qs.SamplingConfig.greedy(), stop_tokens=())
    toks = free.tokens[0]
    stopped = qs.generate(engine, [prompt], max_new_tokens=6, sampling=qs.SamplingConfig.greedy(),
                          stop_tokens=[toks[2]])
    cut = toks.index(toks[2])
    assert stopped.tokens[0] == toks[:cut] and stopped.finish_reasons == ["stop"]
    # top_k = 1 at any temperature is greedy
    k1 = qs.generate(engine, [prompt], max_new_tokens=6, stop_tokens=(),
                     sampling=qs.SamplingConfig(temperature=1.5, top_k=1, top_p=1.0, seed=3))
    assert k1.tokens[0] == toks
    # a huge repeat penalty on greedy decoding: no token of the window may come again
    pen = qs.generate(engine, [prompt], max_new_tokens=10, stop_tokens=(),
                      sampling=qs.SamplingConfig(temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1e6, seed=0))
    seq = prompt + pen.tokens[0]
    assert len(set(seq)) == len(seq)
    # and it follows the plain pipeline
    window = list(prompt)
    cur = list(prompt)
    for g in pen.tokens[0]:
        logits = P.apply_repeat_penalty(plain_next(pcfg, w, cur), window[-64:], 1e6)
        assert g == int(np.argmax(logits))
        cur.append(g); window.append(g)


def test_context_is_the_limit(tmp_path):
    folder, cfg = make_folder(tmp_path, "A", "bfloat16")
    model = qs.load_model(folder, dtype="bfloat16", device="cuda")
    engine = qs.Engine(model, max_tokens=256, max_batch=2)
    prompt = list(range(120))
    res = qs.generate(engine, [prompt, [1, 2]], max_new_tokens=50, sampling=qs.SamplingConfig.greedy(), stop_tokens=())
    assert res.finish_reasons == ["context", "length"]
    assert len(res.tokens[0]) == cfg.n_positions - 120 + 1 and len(res.tokens[1]) == 50
    with pytest.raises(qs.QStreamError) as e:
        qs.generate(engine, [[0] * 129], max_new_tokens=1)
    assert e.value.code == qs.QsError.SEQ_TOO_LONG
    with pytest.raises(qs.QStreamError) as e:
        qs.generate(engine, [[cfg.vocab_size]], max_new_tokens=1)
    assert e.value.code == qs.QsError.INVALID_INPUT
    engine.cache.check()
    assert engine.cache.slots.n_free == engine.cache.slots.n_slots


def plain_greedy(pcfg, w, prompt, n, stop=()):
    return P.generate_greedy(pcfg, w, prompt, n, stop)


def test_one_request_stops_while_the_others_go_on(tmp_path):
    """Three requests in one batch, greedy, float32.  The stop token is taken from a free run so that
    one request stops in mid-batch; a callback ends another a few tokens later; the third runs to its
    length.  Every request's tokens must be what the plain model generates for it alone: a row
    mix-up after a sequence leaves the batch would change the survivors' tokens."""
    folder, cfg = make_folder(tmp_path, "B", "float32")
    pcfg, w = P.load_model(folder)
    rng = np.random.default_rng(23)
    prompts = [random_tokens(rng, n, cfg.vocab_size) for n in (7, 20, 3)]
    model = qs.load_model(folder, dtype="float32", device="cuda")
    engine = qs.Engine(model, max_tokens=64 * 6, max_batch=3)
    greedy = qs.SamplingConfig.greedy()
    free = qs.generate(engine, prompts, max_new_tokens=14, sampling=greedy, stop_tokens=())
    for prompt, got in zip(prompts, free.tokens):
        assert got == plain_greedy(pcfg, w, prompt, 14)
    # a token that request 1 emits fourth and that the other two do not emit before their ends
    stop = free.tokens[1][3]
    assert stop not in free.tokens[1][:3]
    cut0 = free.tokens[0].index(stop) if stop in free.tokens[0] else 14
    cut2 = free.tokens[2].index(stop) if stop in free.tokens[2] else 14
    seen = []

    def callback(i, tok):
        seen.append((i, tok))
        return i == 0 and len([1 for j, _ in seen if j == 0]) == 8      # ends request 0 after its eighth token
    res = qs.generate(engine, prompts, max_new_tokens=14, sampling=greedy, stop_tokens=[stop], callback=callback)
    assert res.tokens[1] == free.tokens[1][:3] and res.finish_reasons[1] == "stop"
    want0 = free.tokens[0][:min(8, cut0)]
    assert res.tokens[0] == want0 and res.finish_reasons[0] == ("callback" if cut0 >= 8 else "stop")
    assert res.tokens[2] == free.tokens[2][:cut2] and res.finish_reasons[2] == ("length" if cut2 == 14 else "stop")
    assert [t for i, t in seen if i == 2] == res.tokens[2]
    engine.check_status()
    engine.cache.check()
    assert engine.cache.slots.n_free == engine.cache.slots.n_slots
    # the stop token emitted, as the last token of the request it ends
    res = qs.generate(engine, prompts, max_new_tokens=14, sampling=greedy, stop_tokens=[stop], emit_stop_token=True)
    assert res.tokens[1] == free.tokens[1][:4] and res.finish_reasons[1] == "stop"


def test_interrupt_from_a_callback(tmp_path):
    folder, cfg = make_folder(tmp_path, "A", "bfloat16")
    model = qs.load_model(folder, dtype="bfloat16", device="cuda")
    engine = qs.Engine(model, max_tokens=64 * 4, max_batch=2)
    gen = qs.Generator(engine)
    calls = []

    def callback(i, tok):
        calls.append(i)
        if len(calls) == 5:
            gen.interrupt()
    res = gen.generate([[1, 2, 3], [4, 5]], max_new_tokens=30, sampling=qs.SamplingConfig.greedy(), stop_tokens=(),
                       callback=callback)
    assert res.finish_reasons == ["interrupted", "interrupted"]
    assert [len(t) for t in res.tokens] == [3, 3]          # the step in which the fifth token came is finished
    engine.cache.check()
    assert engine.cache.slots.n_free == engine.cache.slots.n_slots
    # the engine serves the next call as if nothing had happened
    res = gen.generate([[1, 2, 3]], max_new_tokens=4, sampling=qs.SamplingConfig.greedy(), stop_tokens=())
    assert res.finish_reasons == ["length"] and len(res.tokens[0]) == 4


@pytest.mark.parametrize("which,dtype", [("A", "bfloat16"), ("B", "bfloat16"), ("B", "float32")])
def test_the_same_requests_give_the_same_tokens_again(tmp_path, which, dtype):
    """Sixty batches of random requests (unequal prompts, stop tokens, greedy and sampled, slots and pages
    used again and again) through two engines on the same model: the same tokens and the same reasons
    for stopping, request by request.  Nothing in a step may depend on timing."""
    folder, cfg = make_folder(tmp_path, which, dtype)
    model = qs.load_model(folder, dtype=dtype, device="cuda")
    runs = []
    for rep in range(2):
        eng = qs.Engine(model, max_tokens=64 * 60, max_batch=8)
        rng = np.random.default_rng(11)
        outs = []
        for _ in range(60):
            n = int(rng.integers(1, 9))
            prompts = [random_tokens(rng, int(rng.integers(1, cfg.n_positions - 45)), cfg.vocab_size) for _ in range(n)]
            stop = (int(rng.integers(0, cfg.vocab_size)),) if rng.random() < 0.5 else ()
            sampling = qs.SamplingConfig.greedy() if rng.random() < 0.6 else qs.SamplingConfig(
                temperature=0.8, top_k=20, top_p=0.9, repeat_penalty=1.1, seed=int(rng.integers(0, 1000)))
            res = qs.generate(eng, prompts, max_new_tokens=int(rng.integers(1, 40)), sampling=sampling, stop_tokens=stop)
            outs.append((res.tokens, res.finish_reasons))
        eng.cache.check()
        eng.check_status()
        runs.append(outs)
    for i, (a, b) in enumerate(zip(*runs)):
        assert a == b, f"batch {i}"
