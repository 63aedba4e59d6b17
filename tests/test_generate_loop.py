"""The generation loop's decisions, driven with stand-ins for the engine and the sampler (no GPU)."""
import pytest

import qstream_b200 as qs
from qstream_b200.engine import Generator, plan_batches
from qstream_b200.engine.step import TokenFeed
from qstream_b200.sampling import SamplingConfig, XorShift128Plus, request_seed
from qstream_b200.sampling.sampler import RequestSamplingState
import plain_gptj as P


class FakeCache:
    def __init__(self, max_tokens, max_context, page_tokens=64):
        self.max_tokens, self.max_context, self.page_tokens = max_tokens, max_context, page_tokens


class FakeSpec:
    stop_tokens = (99,)


class FakeModel:
    spec = FakeSpec()


class FakeEngine:
    """Remembers every step; its 'logits' are just the (slot, length) pairs of the rows.

    With `ahead` it offers what the real engine offers the loop: tokens fed from the sampler's
    buffer (`TokenFeed`), rows of a logits tensor, a status check; the loop then launches every step
    before it has read the step's tokens, as it does on the GPU."""

    def __init__(self, max_batch=3, max_tokens=64 * 6, max_context=20, ahead=False, status=None):
        self.max_batch, self.device, self.model = max_batch, "cpu", FakeModel()
        self.cache = FakeCache(max_tokens, max_context)
        self.free = list(range(max_batch))[::-1]
        self.lengths, self.steps, self.held_max = {}, [], 0
        self.accepts_device_tokens = self.use_graphs = ahead
        self.status, self.status_checks = status, 0

    def rows_of(self, logits, rows):
        return [logits[r] for r in rows]

    def check_status(self):
        self.status_checks += 1
        if self.status:
            raise qs.QStreamError(qs.QsError.INTERNAL, f"kernel status {self.status}")

    def acquire(self):
        s = self.free.pop()
        self.lengths[s] = 0
        self.held_max = max(self.held_max, len(self.lengths))
        return s

    def release(self, s):
        del self.lengths[s]
        self.free.append(s)

    def step(self, slots, tokens, want=None):
        assert len(set(slots)) == len(slots) and all(s in self.lengths for s in slots)
        if isinstance(tokens, TokenFeed):
            assert self.accepts_device_tokens and len(tokens.rows) == len(slots)
            tokens = [[tokens.buffer[r]] for r in tokens.rows]
        for s, t in zip(slots, tokens):
            self.lengths[s] += len(t)
            assert self.lengths[s] <= self.cache.max_context
        self.steps.append((list(slots), [list(t) for t in tokens]))
        return [(s, self.lengths[s]) for s in slots]


class ScriptedSampler:
    """Emits, for each request, the tokens of its script in turn."""

    def __init__(self, scripts):
        self.scripts = scripts
        self.calls = 0
        self.rows_seen = {}

    def __call__(self, sampling, device):
        return self

    def sample(self, logits, states):
        self.calls += 1
        assert len(logits) == len(states)
        for row, st in zip(logits, states):         # each request keeps its slot and grows by one token per call
            seen = self.rows_seen.setdefault(st.request, [])
            assert not seen or (row[0] == seen[-1][0] and row[1] == seen[-1][1] + 1), (st.request, seen, row)
            seen.append(row)
        return [self.scripts[st.request].pop(0) for st in states]


@pytest.fixture(autouse=True)
def tag_states(monkeypatch):
    orig = RequestSamplingState.__init__

    def init(self, config, request_index, prompt):
        orig(self, config, request_index, prompt)
        self.request = request_index
    monkeypatch.setattr(RequestSamplingState, "__init__", init)


def run(engine, prompts, scripts, **kw):
    gen = Generator(engine, sampler_factory=ScriptedSampler({i: list(s) for i, s in enumerate(scripts)}))
    return gen.generate(prompts, **kw)


AHEAD = pytest.mark.parametrize("ahead", [False, True], ids=["step-after-reading", "run-ahead"])


@AHEAD
def test_stop_length_and_early_finish(ahead):
    eng = FakeEngine(ahead=ahead)
    prompts = [[1, 2, 3], [4], [5, 6]]
    scripts = [[10, 11, 99, 12], [20, 21, 22, 23, 24], [99]]
    res = run(eng, prompts, scripts, max_new_tokens=4, sampling=SamplingConfig.greedy())
    assert res.tokens == [[10, 11], [20, 21, 22, 23], []]           # the stop token is not emitted
    assert res.finish_reasons == ["stop", "length", "stop"]
    # prompts in one step, then one token per live sequence; finished ones leave at once
    assert eng.steps[0][1] == prompts
    if ahead:       # launched before the tokens were read: a sequence that then stopped was stepped once more
        assert [s[1] for s in eng.steps[1:]] == [[[10], [20], [99]], [[11], [21]], [[99], [22]]]
    else:
        assert [s[1] for s in eng.steps[1:]] == [[[10], [20]], [[11], [21]], [[22]]]
    # no step after the last sampled token, and every slot is given back
    assert len(eng.steps) == 4 and eng.lengths == {} and sorted(eng.free) == [0, 1, 2]
    assert eng.status_checks == 1


@AHEAD
def test_a_stop_in_mid_batch_keeps_the_others_rows(ahead):
    """Three requests; the middle one stops first, then the first: the survivors' logits rows stay theirs
    (the scripted sampler checks slot and length of every row it is given)."""
    eng = FakeEngine(ahead=ahead)
    scripts = [[10, 11, 99], [99], [30, 31, 32, 33, 34]]
    res = run(eng, [[1, 1], [2], [3, 3, 3]], scripts, max_new_tokens=5)
    assert res.tokens == [[10, 11], [], [30, 31, 32, 33, 34]]
    assert res.finish_reasons == ["stop", "stop", "length"]
    assert eng.lengths == {} and sorted(eng.free) == [0, 1, 2]


@AHEAD
def test_emit_stop_token_and_custom_stop_set(ahead):
    eng = FakeEngine(ahead=ahead)
    res = run(eng, [[1]], [[7, 8, 9]], max_new_tokens=5, stop_tokens=[8], emit_stop_token=True)
    assert res.tokens == [[7, 8]] and res.finish_reasons == ["stop"]
    res = run(FakeEngine(ahead=ahead), [[1]], [[7, 99, 9]], max_new_tokens=3, stop_tokens=())
    assert res.tokens == [[7, 99, 9]] and res.finish_reasons == ["length"]


@AHEAD
def test_context_limit(ahead):
    eng = FakeEngine(max_context=6, ahead=ahead)
    res = run(eng, [[1, 2, 3, 4]], [[5, 6, 7, 8, 9]], max_new_tokens=10, stop_tokens=())
    # 4 prompt tokens + 2 fed tokens fill the context of 6; the third sampled token cannot be held
    assert res.tokens == [[5, 6, 7]] and res.finish_reasons == ["context"]
    assert eng.steps[-1][1] == [[6]]


def test_a_kernel_fault_report_ends_generation_with_an_error():
    with pytest.raises(qs.QStreamError) as e:
        run(FakeEngine(ahead=True, status=3), [[1]], [[7, 8]], max_new_tokens=2, stop_tokens=())
    assert e.value.code == qs.QsError.INTERNAL
    eng = FakeEngine(status=112)
    with pytest.raises(qs.QStreamError):
        run(eng, [[1]], [[7, 8]], max_new_tokens=2, stop_tokens=())
    assert eng.lengths == {}                            # the slots are given back all the same


@AHEAD
def test_callback_and_interrupt(ahead):
    eng = FakeEngine(ahead=ahead)
    seen = []

    def cb(i, tok):
        seen.append((i, tok))
        return tok == 21
    res = run(eng, [[1], [2]], [[10, 11, 12], [20, 21, 22]], max_new_tokens=3, stop_tokens=(), callback=cb)
    assert res.tokens == [[10, 11, 12], [20, 21]] and res.finish_reasons == ["length", "callback"]
    assert seen == [(0, 10), (1, 20), (0, 11), (1, 21), (0, 12)]

    eng = FakeEngine(ahead=ahead)
    gen = Generator(eng, sampler_factory=ScriptedSampler({0: [1, 2, 3, 4]}))
    res = gen.generate([[5]], max_new_tokens=4, stop_tokens=(), callback=lambda i, t: gen.interrupt())
    assert res.tokens == [[1]] and res.finish_reasons == ["interrupted"] and eng.lengths == {}


@AHEAD
def test_batches_one_after_another_reuse_slots(ahead):
    eng = FakeEngine(max_batch=2, ahead=ahead)
    prompts = [[1], [2, 2], [3], [4, 4, 4], [5]]
    res = run(eng, prompts, [[7, 7]] * 5, max_new_tokens=2, stop_tokens=())
    assert res.batches == [[0, 1], [2, 3], [4]] and eng.held_max == 2
    assert all(t == [7, 7] for t in res.tokens)
    assert [s[1] for s in eng.steps if len(s[1][0]) != 1 or s[1][0][0] not in (7,)] == \
        [[[1], [2, 2]], [[3], [4, 4, 4]], [[5]]]


def test_plan_batches_respects_the_cache():
    # 3 pages in total; each request may grow to 100 tokens = 2 pages: one request per batch
    assert plan_batches([60, 60, 60], 41, max_batch=8, max_tokens=192, max_context=512, page_tokens=64) == [[0], [1], [2]]
    assert plan_batches([10, 10, 10], 5, max_batch=8, max_tokens=192, max_context=512, page_tokens=64) == [[0, 1, 2]]
    assert plan_batches([10] * 5, 5, max_batch=2, max_tokens=6400, max_context=512, page_tokens=64) == [[0, 1], [2, 3], [4]]
    with pytest.raises(qs.QStreamError) as e:
        plan_batches([500], 100, max_batch=2, max_tokens=128, max_context=512, page_tokens=64)
    assert e.value.code == qs.QsError.BUDGET_EXCEEDED


def test_bad_requests():
    with pytest.raises(qs.QStreamError) as e:
        run(FakeEngine(), [[1], []], [[1], [1]], max_new_tokens=2)
    assert e.value.code == qs.QsError.INVALID_INPUT
    with pytest.raises(qs.QStreamError) as e:
        run(FakeEngine(max_context=4), [[1] * 5], [[1]], max_new_tokens=2)
    assert e.value.code == qs.QsError.SEQ_TOO_LONG
    res = run(FakeEngine(), [[1]], [[1]], max_new_tokens=0)
    assert res.tokens == [[]]


def test_random_streams():
    a, b = XorShift128Plus(7), P.XorShift128Plus(7)
    assert [a.next_float() for _ in range(50)] == [b.next_float() for _ in range(50)]
    first = XorShift128Plus(7).next_float()
    assert abs(first - 0.675828218460083) < 1e-12       # the reference's first draw for seed 7
    assert request_seed(42, 0) == 42                    # request 0 draws the reference's own sequence
    assert XorShift128Plus(request_seed(42, 1)).next_float() != XorShift128Plus(42).next_float()
    st = RequestSamplingState(SamplingConfig(), 0, list(range(100)))
    assert st.recent == list(range(36, 100))            # the window starts with the prompt's last 64
    st.push(7)
    assert len(st.recent) == 64 and st.recent[-1] == 7 and st.recent[0] == 37
