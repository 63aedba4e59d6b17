"""The engine against the plain model: whole requests, the last tokens one by one,
batches of unequal lengths with slots used again, long decoding, first tokens."""
import numpy as np
import pytest
import torch

import qstream_b200 as qs
from util import TINY, assert_logits_close, make_folder, plain_logits, random_tokens

pytestmark = pytest.mark.gpu
CASES = [(w, d) for w in ("A", "B") for d in ("float32", "bfloat16")]


def engine_for(folder, dtype, max_tokens=1024, max_batch=8):
    model = qs.load_model(folder, dtype=dtype, device="cuda")
    return qs.Engine(model, max_tokens=max_tokens, max_batch=max_batch)


def all_places(n):
    return list(range(n))


@pytest.mark.parametrize("which,dtype", CASES)
def test_whole_request_alone(tmp_path, which, dtype):
    folder, cfg = make_folder(tmp_path, which, dtype)
    eng = engine_for(folder, dtype)
    rng = np.random.default_rng(10)
    for n in (1, 5, 33, 64, 65, cfg.n_positions):
        toks = random_tokens(rng, n, cfg.vocab_size)
        slot = eng.acquire()
        got = eng.step([slot], [toks], [all_places(n)]).cpu().numpy()
        eng.check_status()
        eng.release(slot)
        assert_logits_close(got, plain_logits(folder, toks), dtype, f"{which} {dtype} whole n={n}")
    eng.cache.check()


@pytest.mark.parametrize("which,dtype", CASES)
def test_last_32_tokens_one_by_one(tmp_path, which, dtype):
    folder, cfg = make_folder(tmp_path, which, dtype)
    eng = engine_for(folder, dtype)
    rng = np.random.default_rng(11)
    for n in (33, 70, 100):
        toks = random_tokens(rng, n, cfg.vocab_size)
        ref = plain_logits(folder, toks)
        slot = eng.acquire()
        head = n - 32
        rows = [eng.step([slot], [toks[:head]], [all_places(head)]).cpu().numpy()]
        for t in range(head, n):
            rows.append(eng.step([slot], [[toks[t]]], [[0]]).cpu().numpy())
        eng.check_status()
        eng.release(slot)
        assert_logits_close(np.concatenate(rows), ref, dtype, f"{which} {dtype} tail32 n={n}")


@pytest.mark.parametrize("which,dtype", CASES)
def test_unequal_batches_one_after_another(tmp_path, which, dtype):
    """Batches of unequal prompts, decoded token by token; shorter requests end earlier;
    the next batch takes the slots and pages the first gave back."""
    folder, cfg = make_folder(tmp_path, which, dtype)
    eng = engine_for(folder, dtype, max_tokens=512, max_batch=4)
    rng = np.random.default_rng(12)
    for round_no, (prompt_lens, extra) in enumerate([((5, 9, 16), (8, 3, 12)), ((1, 7, 20, 33), (12, 12, 2, 30)),
                                                      ((64, 3), (1, 70))]):
        reqs = [random_tokens(rng, p + e, cfg.vocab_size) for p, e in zip(prompt_lens, extra)]
        refs = [plain_logits(folder, r) for r in reqs]
        slots = [eng.acquire() for _ in reqs]
        got = [[] for _ in reqs]
        out = eng.step(slots, [r[:p] for r, p in zip(reqs, prompt_lens)],
                       [all_places(p) for p in prompt_lens]).cpu().numpy()
        row = 0
        for i, p in enumerate(prompt_lens):
            got[i].append(out[row:row + p])
            row += p
        live = list(range(len(reqs)))
        pos = list(prompt_lens)
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
        for i, ref in enumerate(refs):
            assert_logits_close(np.concatenate(got[i]), ref, dtype,
                                f"{which} {dtype} batch {round_no} request {i}")
    assert eng.cache.slots.n_free == eng.cache.slots.n_slots
    eng.cache.check_canaries()                          # nothing wrote behind the last cache page


@pytest.mark.parametrize("which,dtype", CASES)
def test_long_decoding(tmp_path, which, dtype):
    folder, cfg = make_folder(tmp_path, which, dtype)
    eng = engine_for(folder, dtype)
    rng = np.random.default_rng(13)
    n = cfg.n_positions
    toks = random_tokens(rng, n, cfg.vocab_size)
    ref = plain_logits(folder, toks)
    slot = eng.acquire()
    rows = [eng.step([slot], [toks[:3]], [all_places(3)]).cpu().numpy()]
    for t in range(3, n):
        rows.append(eng.step([slot], [[toks[t]]]).cpu().numpy())
    eng.check_status()
    assert_logits_close(np.concatenate(rows), ref, dtype, f"{which} {dtype} long decode")
    with pytest.raises(qs.QStreamError) as e:
        eng.step([slot], [[1]])
    assert e.value.code == qs.QsError.SEQ_TOO_LONG
    eng.release(slot)


@pytest.mark.parametrize("which,dtype", CASES)
def test_first_tokens(tmp_path, which, dtype):
    """Positions 0, 1, 2 of a sequence: single-token prompt, then one by one."""
    folder, cfg = make_folder(tmp_path, which, dtype)
    eng = engine_for(folder, dtype)
    toks = [3, 3, 7, 0, cfg.vocab_size - 1]
    ref = plain_logits(folder, toks)
    slot = eng.acquire()
    rows = [eng.step([slot], [[t]]).cpu().numpy() for t in toks]
    eng.release(slot)
    assert_logits_close(np.concatenate(rows), ref, dtype, f"{which} {dtype} first tokens")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_padding_changes_nothing(tmp_path, dtype):
    from qstream_b200.engine.step import StepContext
    folder, cfg = make_folder(tmp_path, "A", dtype)
    eng = engine_for(folder, dtype)
    toks = [[1, 2, 3, 4, 5], [9, 8]]
    slots = [eng.acquire(), eng.acquire()]
    plain = eng.step(slots, toks, [all_places(5), all_places(2)]).cpu()
    for s in slots:
        eng.release(s)
    slots = [eng.acquire(), eng.acquire()]
    batch = eng.build_batch(slots, toks, [all_places(5), all_places(2)], pad_to=16)
    padded = eng.model.forward(StepContext(batch, eng.cache, eng.status)).cpu()
    eng.cache.commit(batch.slots, batch.new_tokens)
    eng.check_status()
    assert torch.equal(plain, padded)


@pytest.mark.parametrize("which,dtype", CASES)
def test_mixed_steps_chunked_prompts_and_idle_sequences(tmp_path, which, dtype):
    """Steps that are neither a batch of whole prompts nor one token each: a prompt in two chunks of
    several tokens, a step in which one sequence brings a chunk and another a single token, a sequence
    that brings nothing in a step, and more than eight live sequences decoded together (a captured
    step of 16 rows with padding rows)."""
    folder, cfg = make_folder(tmp_path, which, dtype)
    eng = engine_for(folder, dtype, max_tokens=64 * 24, max_batch=12)
    rng = np.random.default_rng(14)
    lens = [70, 30, 9, 100, 5, 3, 2, 8, 1, 4]
    reqs = [random_tokens(rng, n, cfg.vocab_size) for n in lens]
    refs = [plain_logits(folder, r) for r in reqs]
    slots = [eng.acquire() for _ in reqs]
    got = [[] for _ in reqs]

    def step(parts):
        """parts: {request: (start, stop)}; logits at every place of every part."""
        idx = sorted(parts)
        out = eng.step([slots[i] for i in idx], [reqs[i][parts[i][0]:parts[i][1]] for i in idx],
                       [all_places(parts[i][1] - parts[i][0]) for i in idx])
        out = out.cpu().numpy() if out is not None else np.zeros((0, cfg.vocab_size))
        row = 0
        for i in idx:
            n = parts[i][1] - parts[i][0]
            got[i].append(out[row:row + n])
            row += n

    step({0: (0, 40), 1: (0, 29), 3: (0, 64)})                      # first chunks
    step({0: (40, 69), 1: (29, 30), 2: (0, 9), 3: (64, 64)})        # chunk + one token + whole prompt + idle
    step({0: (69, 70), 3: (64, 99), 4: (0, 5), 5: (0, 3), 6: (0, 1), 7: (0, 7), 8: (0, 1), 9: (0, 3)})
    step({3: (99, 100), 6: (1, 2), 7: (7, 8), 9: (3, 4)})           # decode, 4 rows
    eng.check_status()
    eng.cache.check()
    for i, ref in enumerate(refs):
        assert_logits_close(np.concatenate(got[i]), ref, dtype, f"{which} {dtype} request {i}")
    # ten sequences decode together: one more token each, fed as a decode step of ten rows
    more = [random_tokens(rng, 1, cfg.vocab_size)[0] for _ in reqs]
    keep = [i for i, n in enumerate(lens) if n < cfg.n_positions]
    out = eng.step([slots[i] for i in keep], [[more[i]] for i in keep]).cpu().numpy()
    eng.check_status()
    for j, i in enumerate(keep):
        ref = plain_logits(folder, reqs[i] + [more[i]])[-1:]
        assert_logits_close(out[j:j + 1], ref, dtype, f"{which} {dtype} ten rows, request {i}")
    for s in slots:
        eng.release(s)
    eng.cache.check()
    eng.cache.check_canaries()
    eng.cache.groups[0].v[1, -1, 0, 5, 3] = 0           # one element of a guard page
    with pytest.raises(qs.QStreamError, match="guard words"):
        eng.cache.check_canaries()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_page_that_held_inf_is_safe_for_its_next_owner(tmp_path, dtype):
    """A request leaves values that are not finite in its pages; the next request gets those pages and
    ends inside one of them: the rows past its end must not reach its result (0 * Inf would be NaN)."""
    folder, cfg = make_folder(tmp_path, "A", dtype)
    eng = engine_for(folder, dtype, max_tokens=128, max_batch=1)
    rng = np.random.default_rng(15)
    slot = eng.acquire()
    eng.step([slot], [random_tokens(rng, 128, cfg.vocab_size)])
    for g in eng.cache.groups:
        g.k.fill_(float("inf"))
        g.v.fill_(float("inf"))
    eng.release(slot)
    toks = random_tokens(rng, 70, cfg.vocab_size)
    slot = eng.acquire()
    got = eng.step([slot], [toks[:40]], [all_places(40)]).cpu().numpy()          # ends inside its first page
    got2 = eng.step([slot], [toks[40:]], [all_places(30)]).cpu().numpy()         # a chunk that ends inside the second
    eng.check_status()
    eng.release(slot)
    assert_logits_close(np.concatenate([got, got2]), plain_logits(folder, toks), dtype, f"{dtype} after Inf")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_check_nan_names_the_layer(tmp_path, dtype):
    """An Inf planted in one weight of layer 1: with `check_nan` the step raises NAN_DETECTED naming
    that layer (QStream src/engine.c:1176-1187); without it the step runs on."""
    folder, cfg = make_folder(tmp_path, "B", dtype)
    model = qs.load_model(folder, dtype=dtype, device="cuda")
    eng = qs.Engine(model, qs.EngineConfig(max_tokens=256, max_batch=2, check_nan=True))
    slot = eng.acquire()
    assert eng.step([slot], [[1, 2, 3]]) is not None            # clean weights: no report
    assert eng.step([slot], [[4]]) is not None                  # and none from a captured decode step
    model.blocks[1].ffn.up_bias[5] = float("inf")
    with pytest.raises(qs.QStreamError) as e:
        eng.step([slot], [[5, 6]])
    assert e.value.code == qs.QsError.NAN_DETECTED and "layer 1" in str(e.value)
    with pytest.raises(qs.QStreamError) as e:                   # the decode graph carries the check too
        eng.step([slot], [[7]])
    assert e.value.code == qs.QsError.NAN_DETECTED and "layer 1" in str(e.value)
    eng.release(slot)
    quiet = qs.Engine(model, max_tokens=256, max_batch=2)
    slot = quiet.acquire()
    quiet.step([slot], [[5, 6]])
    quiet.check_status()


def test_rotary_dim_zero_means_no_rotation(tmp_path):
    cfg = qs.GptjConfig.from_dict({**TINY["A"][0], "rotary_dim": 0, "architectures": ["GPTJForCausalLM"]})
    folder = qs.write_model_folder(tmp_path / "norot", cfg, 4, "float32", TINY["A"][1])
    eng = engine_for(folder, "float32")
    toks = random_tokens(np.random.default_rng(16), 40, cfg.vocab_size)
    slot = eng.acquire()
    rows = [eng.step([slot], [toks[:33]], [all_places(33)]).cpu().numpy()]
    rows += [eng.step([slot], [[t]]).cpu().numpy() for t in toks[33:]]
    eng.check_status()
    assert_logits_close(np.concatenate(rows), plain_logits(folder, toks), "float32", "rotary_dim 0")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_missing_page_is_reported_not_read(tmp_path, dtype):
    """The device's page table names no page where a key should lie: every kernel skips the access and
    sets a status code that `check_status` raises; nothing faults, and the engine works on afterwards."""
    folder, cfg = make_folder(tmp_path, "A", dtype)
    eng = engine_for(folder, dtype, max_tokens=256, max_batch=2)
    rng = np.random.default_rng(17)
    toks = random_tokens(rng, 80, cfg.vocab_size)
    for cut in (80, 79):                                # a whole prompt; a prompt and then a decode step
        slot = eng.acquire()
        group = eng.cache.groups[0]
        eng.step([slot], [toks[:cut - 10]])
        eng.check_status()
        group.table_dev[slot, 0] = -1                   # the first page's entry goes missing on the device
        eng.step([slot], [toks[cut - 10:cut]])
        if cut == 79:
            eng.step([slot], [[toks[79]]])
        with pytest.raises(qs.QStreamError) as e:
            eng.check_status()
        assert e.value.code == qs.QsError.INTERNAL and "page" in str(e.value)
        group.table_dev[slot, 0] = int(group.table_host[slot, 0])
        eng.release(slot)
    slot = eng.acquire()
    got = eng.step([slot], [toks], [all_places(80)]).cpu().numpy()
    eng.check_status()                                  # the report was cleared with the error
    assert_logits_close(got, plain_logits(folder, toks), dtype, f"{dtype} after the report")


@pytest.mark.parametrize("which,dtype", CASES)
def test_captured_steps_with_prompts(tmp_path, which, dtype):
    """Steps of up to 512 tokens for up to 8 sequences that want last logits only are captured once per
    padded size and replayed: the same graph serves other lengths, other slots and continuations of
    sequences that already hold tokens, and gives what the kernel-by-kernel step gives."""
    folder, cfg = make_folder(tmp_path, which, dtype)
    eng = engine_for(folder, dtype, max_tokens=64 * 40, max_batch=8)
    assert eng.captures_prefill
    rng = np.random.default_rng(18)
    limit = cfg.n_positions
    rounds = [[5], [64], [70, 3], [9, 100, 33], [2, 2, 2, 2, 2], [60, 1, 17, 40, 8, 8, 30, 12], [5], [120, 90]]
    for lens in rounds:
        lens = [min(n, limit - 20) for n in lens]
        reqs = [random_tokens(rng, n + 12, cfg.vocab_size) for n in lens]
        slots = [eng.acquire() for _ in reqs]
        got = [[] for _ in reqs]
        out = eng.step(slots, [r[:n] for r, n in zip(reqs, lens)]).cpu().numpy()        # captured: default want
        for i in range(len(reqs)):
            got[i].append(out[i:i + 1])
        # a second chunk of unequal sizes on top (positions do not start at 0), again captured
        more = [1 + (i * 5) % 11 for i in range(len(reqs))]
        out = eng.step(slots, [r[n:n + m] for r, n, m in zip(reqs, lens, more)]).cpu().numpy()
        for i in range(len(reqs)):
            got[i].append(out[i:i + 1])
        eng.check_status()
        for i, (r, n, m) in enumerate(zip(reqs, lens, more)):
            ref = plain_logits(folder, r[:n + m])
            assert_logits_close(np.concatenate(got[i]), ref[[n - 1, n + m - 1]], dtype, f"{which} {dtype} lens {lens} request {i}")
        for s in slots:
            eng.release(s)
    assert len(eng._prefill_graphs) >= 3
    eng.cache.check()
    # the same step kernel by kernel gives the same bits (same kernels, same order of sums)
    plain_eng = qs.Engine(eng.model, max_tokens=64 * 8, max_batch=4, use_graphs=False)
    toks = [random_tokens(rng, n, cfg.vocab_size) for n in (33, 7)]
    a = [eng.acquire(), eng.acquire()]
    b = [plain_eng.acquire(), plain_eng.acquire()]
    assert torch.equal(eng.step(a, toks), plain_eng.step(b, toks))


@pytest.mark.parametrize("which,dtype,seed", [("A", "float32", 0), ("B", "bfloat16", 1), ("A", "bfloat16", 2), ("B", "float32", 3)])
def test_random_walk_of_steps(tmp_path, which, dtype, seed):
    """Some three hundred steps drawn at random: sequences start and end at any time, a step brings any mix
    of prompt chunks, single tokens and idle sequences, wants the last place, every place or none, and slots
    and pages change hands all the while.  Every logits row that comes back is compared with the plain model
    on that sequence's tokens so far."""
    folder, cfg = make_folder(tmp_path, which, dtype)
    eng = engine_for(folder, dtype, max_tokens=64 * 14, max_batch=6)
    rng = np.random.default_rng(100 + seed)
    limit = cfg.n_positions
    live = {}                                           # slot -> (all tokens of the request, tokens fed so far)
    plain_cache = {}
    checked = 0

    def reference(tokens, upto):
        key = tuple(tokens)
        if key not in plain_cache:
            plain_cache[key] = plain_logits(folder, tokens)
        return plain_cache[key][:upto]

    for step_no in range(300):
        # sequences come ...
        while len(live) < 6 and (not live or rng.random() < 0.3):
            n = int(rng.integers(1, limit + 1)) if rng.random() < 0.2 else int(rng.integers(1, 70))
            try:
                live[eng.acquire()] = (random_tokens(rng, n, cfg.vocab_size), 0)
            except qs.QStreamError:
                break
        # ... a step for a random subset, each with a random number of its next tokens (0: idle)
        chosen = [s for s in live if rng.random() < 0.8] or list(live)
        kind = rng.random()
        tokens, want = [], []
        for s in chosen:
            toks, fed = live[s]
            left = len(toks) - fed
            n = min(left, 1 if kind < 0.45 else int(rng.integers(0, 40)))
            tokens.append(toks[fed:fed + n])
            w = rng.random()
            want.append(([n - 1] if n else []) if w < 0.5 else (list(range(n)) if w < 0.85 else []))
        try:
            out = eng.step(chosen, tokens, None if all(w == ([len(t) - 1] if t else []) for w, t in zip(want, tokens)) and all(tokens) else want)
        except qs.QStreamError as e:                    # the cache is full: end the longest sequence and go on
            assert e.code == qs.QsError.BUDGET_EXCEEDED, e
            victim = max(live, key=lambda s: live[s][1])
            eng.release(victim)
            del live[victim]
            continue
        rows = out.cpu().numpy() if out is not None else np.zeros((0, cfg.vocab_size))
        row = 0
        for s, t, w in zip(chosen, tokens, want):
            toks, fed = live[s]
            for place in w:
                ref = reference(toks, fed + place + 1)[-1]
                assert_logits_close(rows[row:row + 1], ref[None], dtype, f"step {step_no} slot {s} position {fed + place}")
                row += 1
                checked += 1
            live[s] = (toks, fed + len(t))
        assert row == rows.shape[0]
        # ... and go: when all their tokens are in, or at random
        for s in list(live):
            toks, fed = live[s]
            if fed == len(toks) or rng.random() < 0.03:
                eng.release(s)
                del live[s]
        if step_no % 50 == 49:
            eng.check_status()
            eng.cache.check()
    eng.check_status()
    eng.cache.check()
    eng.cache.check_canaries()
    assert checked > 300


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_odd_engine_sizes(tmp_path, dtype):
    """A context that is no multiple of a page or of a split, and more sequences than any usual batch: seventy
    sequences decode together (a captured step of 96 rows), each against the plain model."""
    folder, cfg = make_folder(tmp_path, "B", dtype)
    model = qs.load_model(folder, dtype=dtype, device="cuda")
    eng = qs.Engine(model, max_tokens=70 * 128, max_batch=70, max_context=100)
    rng = np.random.default_rng(19)
    lens = [int(rng.integers(1, 60)) for _ in range(70)]
    reqs = [random_tokens(rng, n + 3, cfg.vocab_size) for n in lens]
    slots = [eng.acquire() for _ in reqs]
    out = [eng.step(slots[a:a + 10], [r[:n] for r, n in zip(reqs[a:a + 10], lens[a:a + 10])]).cpu().numpy()
           for a in range(0, 70, 10)]
    got = [[row[None]] for chunk in out for row in chunk]
    for k in range(3):
        step = eng.step(slots, [[r[n + k]] for r, n in zip(reqs, lens)]).cpu().numpy()
        for i in range(70):
            got[i].append(step[i:i + 1])
    eng.check_status()
    for i in (0, 7, 33, 69):
        ref = plain_logits(folder, reqs[i])[lens[i] - 1:]
        assert_logits_close(np.concatenate(got[i]), ref, dtype, f"{dtype} request {i} of 70")
    # the context of 100 is the limit, whatever the pages could hold
    s = slots[0]
    eng.step([s], [random_tokens(rng, 100 - eng.length(s), cfg.vocab_size)])
    with pytest.raises(qs.QStreamError) as e:
        eng.step([s], [[1]])
    assert e.value.code == qs.QsError.SEQ_TOO_LONG
    for s in slots:
        eng.release(s)
    eng.cache.check()


@pytest.mark.parametrize("which", ["A", "B"])
def test_both_arrangements_of_the_parallel_block(tmp_path, which, monkeypatch):
    """Decode steps over few keys run the feed-forward beside the mixer and end in the mixer's output
    product; over many keys the two output projections are one product.  Both against the plain model,
    with the threshold moved so that the tiny models take each."""
    from qstream_b200.parts import block
    folder, cfg = make_folder(tmp_path, which, "bfloat16")
    rng = np.random.default_rng(77)
    prompts = [random_tokens(rng, n, cfg.vocab_size) for n in (70, 9, 41)]
    refs = [plain_logits(folder, p) for p in prompts]
    outs = {}
    for keys, graphs in ((0, True), (1 << 30, True), (1 << 30, False)):
        monkeypatch.setattr(block, "SIDE_BRANCH_SHARE", float(keys))
        monkeypatch.setattr(block, "SIDE_BRANCH_SHARE_MANY_ROWS", float(keys))
        eng = qs.Engine(qs.load_model(folder, dtype="bfloat16", device="cuda"), max_tokens=1024, max_batch=8, use_graphs=graphs)
        assert all(b.fused_weight is not None for b in eng.model.blocks)
        slots = [eng.acquire() for _ in prompts]
        heads = [len(p) - 8 for p in prompts]
        rows = [[eng.step([s], [p[:h]], [all_places(h)]).cpu().numpy()] for s, p, h in zip(slots, prompts, heads)]
        for t in range(8):
            got = eng.step(slots, [[p[h + t]] for p, h in zip(prompts, heads)], [[0]] * len(prompts)).cpu().numpy()
            for i in range(len(prompts)):
                rows[i].append(got[i:i + 1])
        eng.check_status()
        for i, ref in enumerate(refs):
            assert_logits_close(np.concatenate(rows[i]), ref, "bfloat16", f"{which} share<={keys} request {i}")
        if graphs:
            outs[keys] = [np.concatenate(r) for r in rows]
        else:       # launched kernel by kernel on the two streams: the same bits as the captured step
            for a, b in zip(outs[keys], rows):
                assert np.array_equal(a, np.concatenate(b))
        for s in slots:
            eng.release(s)
        eng.cache.check()
    # the two arrangements differ by the rounding of one intermediate, not more
    for a, b in zip(outs[0], outs[1 << 30]):
        assert np.abs(a - b).max() <= 0.03 * np.abs(a).max()
