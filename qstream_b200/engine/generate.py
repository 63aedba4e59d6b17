"""The generation loop above the step function.

QStream's loop (`qsf_engine_generate`, src/engine.c:1250-1368) serves one prompt:
prefill token by token, then sample -> stop token? -> callback -> length? -> forward.
This one serves a list of requests: as many batches, one after another, as the requests
need; in a batch all prompts (of unequal lengths) run in one step, then one token per live
sequence; a sequence that ends leaves the batch at once and its slot and pages are free
for the next batch.  As in the reference a stop token ends the sequence before it is
emitted (:1331), the callback may end it (:1347), and so do the token limit and a full
context (:1351); unlike the reference no step is run for a token after which nothing is
sampled (:1358 runs one).

The loop needs of the engine only `acquire`, `release`, `step`, `max_batch`, `cache`
figures and of the sampler only `sample`; tests drive it with stand-ins.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Iterable, Optional, Sequence

from ..errors import QsError, QStreamError
from ..sampling import RequestSamplingState, Sampler, SamplingConfig


@dataclass
class GenerationResult:
    tokens: list                    # per request, the generated tokens
    finish_reasons: list            # "stop" | "length" | "context" | "callback" | "interrupted"
    prefill_tokens: int = 0
    prefill_seconds: float = 0.0
    decode_tokens: int = 0
    decode_seconds: float = 0.0
    batches: list = field(default_factory=list)     # request indices of each batch


def plan_batches(prompt_lengths: Sequence[int], max_new_tokens: int, max_batch: int,
                 max_tokens: int, max_context: int, page_tokens: int) -> list:
    """Cut the requests, in order, into batches that fit the slots and the cache's pages
    at their longest (prompt + new tokens, at most the context)."""
    total_pages = max_tokens // page_tokens
    batches, cur, cur_pages = [], [], 0
    for i, n in enumerate(prompt_lengths):
        longest = min(max_context, n + max(0, max_new_tokens - 1))
        pages = -(-longest // page_tokens)
        if pages > total_pages:
            raise QStreamError(QsError.BUDGET_EXCEEDED,
                               f"request {i} may hold {longest} tokens; the cache holds {max_tokens}")
        if cur and (len(cur) >= max_batch or cur_pages + pages > total_pages):
            batches.append(cur)
            cur, cur_pages = [], 0
        cur.append(i)
        cur_pages += pages
    if cur:
        batches.append(cur)
    return batches


class Generator:
    def __init__(self, engine, sampler_factory: Callable = Sampler):
        self.engine = engine
        self.sampler_factory = sampler_factory
        self.interrupted = False        # set from a signal handler to stop (src/engine.c:1371)

    def interrupt(self) -> None:
        self.interrupted = True

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 256,
                 sampling: Optional[SamplingConfig] = None,
                 stop_tokens: Optional[Iterable[int]] = None,
                 callback: Optional[Callable[[int, int], object]] = None,
                 emit_stop_token: bool = False) -> GenerationResult:
        """Generate up to `max_new_tokens` for every prompt (lists of token ids).

        stop_tokens: default the model's (its eos); pass () to run to the length.
        callback(request_index, token): called for each emitted token; a true return
        value ends that request.
        """
        eng = self.engine
        sampling = sampling or SamplingConfig()
        if stop_tokens is None:
            stop_tokens = getattr(eng.model.spec, "stop_tokens", ())
        stop = frozenset(int(t) for t in stop_tokens)
        cache = eng.cache
        for i, p in enumerate(prompts):
            if len(p) == 0:
                raise QStreamError(QsError.INVALID_INPUT, f"request {i}: empty prompt")
            if len(p) > cache.max_context:
                raise QStreamError(QsError.SEQ_TOO_LONG,
                                   f"request {i}: prompt of {len(p)} tokens, context {cache.max_context}")
        result = GenerationResult(tokens=[[] for _ in prompts], finish_reasons=[None] * len(prompts))
        if max_new_tokens <= 0 or not prompts:
            result.finish_reasons = ["length"] * len(prompts)
            return result
        sampler = self.sampler_factory(sampling, eng.device)
        self.interrupted = False
        result.batches = plan_batches([len(p) for p in prompts], max_new_tokens, eng.max_batch,
                                      cache.max_tokens, cache.max_context, cache.page_tokens)
        for batch in result.batches:
            self._run_batch(batch, prompts, max_new_tokens, sampler, sampling, stop, callback,
                            emit_stop_token, result)
        return result

    def _run_batch(self, batch, prompts, max_new_tokens, sampler, sampling, stop, callback,
                   emit_stop_token, result) -> None:
        """One batch from its prompts to its last token.

        The decisions (who stops, and why) are taken in one place, after the host has read the step's
        tokens.  What differs between engines is only *when* the next step is launched.  An engine
        that takes tokens from the device (`accepts_device_tokens` with graphs) is run ahead: the
        sampled tokens feed the next step on the device, and that step is launched before the host has
        read them, for every sequence that could go on whatever its token is (not at its token limit,
        room in the context); the host reads the tokens (a copy into pinned memory) while the step runs.
        A sequence that turns out to have stopped has then been stepped once too often, which only costs
        the work: its slot is given back all the same and nothing it wrote is read.  Any other engine is
        stepped after the decisions, with the tokens from the host."""
        eng = self.engine
        run_ahead = bool(getattr(eng, "accepts_device_tokens", False) and getattr(eng, "use_graphs", False))
        max_context = eng.cache.max_context
        slots = {i: eng.acquire() for i in batch}
        states = {i: RequestSamplingState(sampling, i, prompts[i]) for i in batch}
        live = list(batch)
        reader = _TokenReader(len(batch))
        try:
            t0 = time.perf_counter()
            logits = eng.step([slots[i] for i in live], [list(prompts[i]) for i in live])
            first = True
            while live:
                chosen_dev = sampler.sample(logits, [states[i] for i in live])
                n = len(live)
                reader.start(chosen_dev, n)
                ahead, may = None, []
                if run_ahead and not self.interrupted:
                    # who goes on whatever the token is: not at the token limit, room in the context
                    may = [k for k, i in enumerate(live)
                           if len(result.tokens[i]) + 1 < max_new_tokens
                           and len(prompts[i]) + len(result.tokens[i]) + 1 <= max_context]
                    if may:
                        from .step import TokenFeed
                        ahead = eng.step([slots[live[k]] for k in may], TokenFeed(chosen_dev, may))
                chosen = reader.finish()
                now = time.perf_counter()
                if first:
                    result.prefill_tokens += sum(len(prompts[i]) for i in live)
                    result.prefill_seconds += now - t0
                    first = False
                else:
                    result.decode_tokens += n
                    result.decode_seconds += now - t0
                t0 = now
                go_on, go_on_at, feed = [], [], []
                for k, (i, tok) in enumerate(zip(live, chosen)):
                    out = result.tokens[i]
                    reason = None
                    if tok in stop:
                        reason = "stop"
                        if emit_stop_token:
                            out.append(tok)
                    else:
                        out.append(tok)
                        states[i].push(tok)
                        if callback is not None and callback(i, tok):
                            reason = "callback"
                        elif len(out) >= max_new_tokens:
                            reason = "length"
                        elif len(prompts[i]) + len(out) > max_context:
                            reason = "context"      # the token just emitted cannot be held
                        elif self.interrupted:
                            reason = "interrupted"
                    if reason is None:
                        go_on.append(i)
                        go_on_at.append(k)
                        feed.append([tok])
                    else:
                        result.finish_reasons[i] = reason
                        eng.release(slots.pop(i))
                live = go_on
                if not live:
                    break
                if ahead is not None and all(k in may for k in go_on_at):
                    rows = [may.index(k) for k in go_on_at]
                    logits = ahead if len(rows) == len(may) else eng.rows_of(ahead, rows)
                else:                               # nothing was run ahead (or not for all of them): step now
                    logits = eng.step([slots[i] for i in live], feed)
            check = getattr(eng, "check_status", None)
            if check is not None:
                check()                             # a kernel's fault report ends the batch with an error, not with tokens
        finally:
            for i in list(slots):
                eng.release(slots.pop(i))
                if result.finish_reasons[i] is None:
                    result.finish_reasons[i] = "interrupted"


class _TokenReader:
    """Brings a step's sampled tokens to the host.  Tokens on a CUDA device are copied into pinned
    memory without waiting (`start`) and awaited later (`finish`), so that work launched in between
    overlaps the copy; anything else (a list, a host tensor) is read at once."""

    def __init__(self, n_max: int):
        self.n_max = n_max
        self.host = None
        self.event = None
        self.now = None

    def start(self, chosen, n: int) -> None:
        if getattr(chosen, "is_cuda", False):
            import torch
            if self.host is None:
                self.host = torch.empty(self.n_max, dtype=torch.int32).pin_memory()
            self.host[:n].copy_(chosen, non_blocking=True)
            self.event = torch.cuda.Event()
            self.event.record()
            self.now = n
        else:
            self.event = None
            self.now = [int(t) for t in (chosen.tolist() if hasattr(chosen, "tolist") else chosen)]

    def finish(self) -> list:
        if self.event is None:
            return self.now
        self.event.synchronize()
        return self.host[:self.now].tolist()
