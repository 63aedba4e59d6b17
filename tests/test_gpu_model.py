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
