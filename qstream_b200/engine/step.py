"""The step function: a batch of sequences, the tokens each brings, logits where wanted.

`Engine.step(slots, tokens, want)` runs only the tokens it is given, as one batch,
against the cache that earlier steps left: token t of a sequence that already holds
p0 tokens sits at position p0 + t and attends to positions 0..p0+t.  A batch whose
sequences start together gives its prompts (of unequal lengths) in one step and then one
token per live sequence; a prompt may also be cut into any pieces.  The reference's
counterpart handles one token of one sequence per call (`qsf_forward`,
QStream src/engine.c:694).

Per-token metadata (slot, position) drives every kernel, so the packed batch needs no
padding; rows added to reach a captured graph's size carry slot -1 and are skipped by
every kernel that touches the cache.
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Optional, Sequence

import numpy as np
import torch

from ..cache import SequenceCache
from ..errors import QsError, QStreamError
from .model import CausalLM


@dataclass
class StepBatch:
    """One step's tokens and where they belong, on the device and on the host."""
    n_seq: int
    n_tokens: int
    n_want: int
    tokens: torch.Tensor            # [T] int32
    tok_slot: torch.Tensor          # [T] int32, -1 = padding
    tok_pos: torch.Tensor           # [T] int32, position in the sequence
    want_rows: torch.Tensor         # [n_want] int32, rows of the packed batch
    seq_slot: torch.Tensor          # [n_seq] int32
    seq_start: torch.Tensor         # [n_seq + 1] int32, first row of each sequence
    seq_p0: torch.Tensor            # [n_seq] int32, tokens held before this step
    slots: list = field(default_factory=list)       # host copies
    new_tokens: list = field(default_factory=list)
    p0: list = field(default_factory=list)
    decode: bool = False            # every sequence brings exactly one token
    max_new: int = 0
    max_total: int = 0              # longest sequence after this step


@dataclass
class TokenFeed:
    """Tokens that are still on the device: sequence j of the step takes `buffer[rows[j]]`.
    `buffer` is the sampler's int32 output; the host need not have read it."""
    buffer: object
    rows: Sequence[int]


@dataclass
class EngineConfig:
    """How an engine is set up, in the manner of QStream's `QSFEngineConfig` with its
    `qsf_engine_config_default` (include/qsf/engine.h:25-32, src/engine.c:19-26).

    max_batch: the most sequences alive at once.  max_context: the longest sequence (0: the
    model's positions).  max_tokens: the tokens all live sequences may hold together, each
    rounded up to a whole page of 64; it sizes the cache (0: max_batch * max_context).
    mem_budget: bytes of device memory the cache may take (0: what is free).  check_nan: scan
    every layer's output for values that are not finite and raise NAN_DETECTED with the layer
    and the place (the reference's switch, src/engine.c:1176-1187); it makes every step wait
    for the device.  use_graphs: replay decode steps as CUDA graphs."""
    max_batch: int = 64
    max_context: int = 0
    max_tokens: int = 0
    mem_budget: int = 0
    verbose: int = 0
    check_nan: bool = False
    use_graphs: bool = True

    @classmethod
    def default(cls) -> "EngineConfig":
        return cls()


class StepContext:
    """What a part may touch during a step."""

    def __init__(self, batch: StepBatch, cache: SequenceCache, status: torch.Tensor, side_stream=None,
                 nan_record: Optional[torch.Tensor] = None):
        self.batch = batch
        self.cache = cache
        self.status = status
        # a second CUDA stream for work that does not depend on the mixer (None: everything in order)
        self.side_stream = side_stream
        # int32 [4] on the device when every layer's output is to be scanned for values that are not finite
        self.nan_record = nan_record

    def kv(self, cache_id: int):
        return self.cache.view(cache_id)

    def state(self, cache_id: int) -> Optional[torch.Tensor]:
        """The state tensor [slots, *shape] of a cache entry (None if it has none)."""
        return self.cache.state.get(cache_id)


STATUS_MESSAGES = {
    1: "a token's position lies outside the position table",
    2: "a token was to be written to a cache page its sequence does not hold",
    3: "attention met a cache page its sequence does not hold",
    199: "the self-test's wait ran out, as it must",
}


class Engine:
    """A model with its cache: sequences are acquired, stepped and released.

    Set up from an `EngineConfig` (default: `EngineConfig.default()`); keyword arguments
    with the names of its fields override single fields.
    """

    def __init__(self, model: CausalLM, config: Optional[EngineConfig] = None, **overrides):
        cfg = config or EngineConfig.default()
        unknown = [k for k in overrides if not hasattr(cfg, k)]
        if unknown:
            raise QStreamError(QsError.INVALID_INPUT, f"Engine: unknown option(s) {unknown}")
        cfg = replace(cfg, **{k: (v if v is not None else getattr(EngineConfig, k)) for k, v in overrides.items()})
        self.config = cfg
        self.model = model
        self.device = model.runtime.device
        self.dtype = model.runtime.dtype
        self.verbose = verbose = cfg.verbose
        ctx = model.spec.max_positions if not cfg.max_context else min(cfg.max_context, model.spec.max_positions)
        max_batch = cfg.max_batch
        max_tokens = cfg.max_tokens or max_batch * ctx
        self.max_batch = max_batch
        kv_needs, state_needs = model.kv_needs(), model.state_needs()
        self._check_budget(kv_needs, max_tokens, cfg.mem_budget)
        self.cache = SequenceCache(kv_needs, state_needs, max_tokens, max_batch, ctx, self.dtype, self.device)
        # words the kernels report through: [0] a fault code, [4:8] the finite check's record
        self._words = torch.zeros(8, dtype=torch.int32, device=self.device)
        self.status = self._words[0:1]
        self.check_nan = cfg.check_nan
        self.nan_record = self._words[4:8] if cfg.check_nan else None
        # decode steps run the feed-forward's first product beside the attention kernels
        self.side_stream = torch.cuda.Stream(device=self.device) if self.device.type == "cuda" else None
        self.use_graphs = cfg.use_graphs and self.device.type == "cuda"
        self._graphs = {}
        self._prefill_graphs = {}
        self.graph_pool = torch.cuda.graph_pool_handle() if self.use_graphs else None   # one pool: graphs never run at once
        # steps with prompts are captured too if every part goes by device metadata alone
        self.captures_prefill = self.use_graphs and all(getattr(b, "captures_any_step", False) for b in model.blocks) \
            and all(getattr(p, "captures_any_step", False) for p in (model.embedding, model.head)) \
            and (model.final_norm is None or getattr(model.final_norm, "captures_any_step", False))
        self._words_host = torch.zeros(9, dtype=torch.int32).pin_memory() if self.device.type == "cuda" else None
        if verbose:
            import sys
            print(f"[qstream] cache: {self.cache.bytes / 2**20:.1f} MB for {max_tokens} tokens, "
                  f"{self.cache.slots.n_slots} slots, context {ctx}; weights {model.weight_bytes / 2**20:.1f} MB",
                  file=sys.stderr)

    def _check_budget(self, kv_needs, max_tokens, mem_budget=0):
        elem = torch.empty((), dtype=self.dtype).element_size()
        want = sum(2 * max_tokens * n.n_kv_heads * n.head_dim * elem for n in kv_needs.values())
        if mem_budget and want > mem_budget:
            raise QStreamError(QsError.BUDGET_EXCEEDED,
                               f"a cache of {max_tokens} tokens needs {want / 2**20:.1f} MiB, "
                               f"the budget is {mem_budget / 2**20:.1f} MiB")
        if self.device.type != "cuda":
            return
        free, _ = torch.cuda.mem_get_info(self.device)
        if want > free:
            raise QStreamError(QsError.BUDGET_EXCEEDED,
                               f"a cache of {max_tokens} tokens needs {want / 2**30:.1f} GiB, "
                               f"{free / 2**30:.1f} GiB are free on the device")

    # ------------------------------------------------------------------ sequences
    def acquire(self) -> int:
        return self.cache.acquire()

    def release(self, slot: int) -> None:
        self.cache.release(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    # ------------------------------------------------------------------ one step
    def build_batch(self, slots: Sequence[int], tokens: Sequence[Sequence[int]],
                    want: Optional[Sequence[Sequence[int]]] = None, pad_to: int = 0) -> StepBatch:
        """Check the step, hand out its cache pages and upload its metadata."""
        if len(slots) != len(tokens) or (want is not None and len(want) != len(slots)):
            raise QStreamError(QsError.INVALID_INPUT, "step: slots, tokens and want differ in length")
        n_new = [len(t) for t in tokens]
        tokens = self._checked_tokens(slots, tokens)
        if want is None:
            want = [[n - 1] if n else [] for n in n_new]
        for w, n in zip(want, n_new):
            for p in w:
                if not 0 <= p < n:
                    raise QStreamError(QsError.INVALID_INPUT, f"wanted place {p} outside the {n} tokens given")
        self.cache.prepare(slots, n_new)                # raises before anything has changed

        T = sum(n_new)
        Tp = max(T, pad_to)
        n_seq = len(slots)
        n_want = sum(len(w) for w in want)
        p0 = [self.cache.length(s) for s in slots]
        sizes = [Tp, Tp, Tp, n_want, n_seq, n_seq + 1, n_seq]
        offs = np.concatenate([[0], np.cumsum(sizes)])
        host = np.zeros(int(offs[-1]), dtype=np.int32)
        tok, tslot, tpos, wrows, sslot, sstart, sp0 = (host[offs[i]:offs[i + 1]] for i in range(7))
        tslot[:] = -1
        row = 0
        wi = 0
        for i, (s, toks, w) in enumerate(zip(slots, tokens, want)):
            n = len(toks)
            tok[row:row + n] = toks
            tslot[row:row + n] = s
            tpos[row:row + n] = np.arange(p0[i], p0[i] + n)
            for p in w:
                wrows[wi] = row + p
                wi += 1
            sslot[i] = s
            sstart[i] = row
            sp0[i] = p0[i]
            row += n
        sstart[n_seq] = row
        dev = self._upload(host)
        views = [dev[offs[i]:offs[i + 1]] for i in range(7)]
        return StepBatch(
            n_seq=n_seq, n_tokens=Tp, n_want=n_want, tokens=views[0], tok_slot=views[1], tok_pos=views[2],
            want_rows=views[3], seq_slot=views[4], seq_start=views[5], seq_p0=views[6],
            slots=list(slots), new_tokens=n_new, p0=p0, decode=bool(n_new) and all(n == 1 for n in n_new),
            max_new=max(n_new, default=0), max_total=max((a + b for a, b in zip(p0, n_new)), default=0))

    def _checked_tokens(self, slots, tokens) -> list:
        """Each sequence's tokens as an int64 array, every id inside the vocabulary (checked in one pass each:
        a prompt of thousands of tokens is not walked in Python)."""
        V = self.model.vocab_size
        out = []
        for s, toks in zip(slots, tokens):
            try:
                a = np.asarray(toks, dtype=np.int64).reshape(-1)
            except (TypeError, ValueError, OverflowError):
                raise QStreamError(QsError.INVALID_INPUT, f"the tokens of slot {s} are not integers") from None
            if a.size and (int(a.min()) < 0 or int(a.max()) >= V):
                bad = int(a[(a < 0) | (a >= V)][0])
                raise QStreamError(QsError.INVALID_INPUT, f"token id {bad} (slot {s}) outside the vocabulary of {V}")
            out.append(a)
        return out

    def _upload(self, host: np.ndarray) -> torch.Tensor:
        t = torch.from_numpy(host)
        if self.device.type == "cuda":
            return t.pin_memory().to(self.device, non_blocking=True)
        return t

    accepts_device_tokens = True        # step() also takes a `TokenFeed`: one token per sequence, still on the device

    def step(self, slots: Sequence[int], tokens, want: Optional[Sequence[Sequence[int]]] = None) -> Optional[torch.Tensor]:
        """Run one step.  `tokens[i]` are sequence i's next tokens (any number, none for a
        sequence that idles in this step); a `TokenFeed` gives one token per sequence from a
        device buffer instead.  `want[i]` lists the places among sequence i's new tokens whose
        logits are asked for (default: the last).  Returns float32 logits [n_want, vocab] on
        the device, in the order of the sequences and of `want`; None if none is wanted.

        The logits of a captured step (one token per sequence; or at most 512 tokens for at most 8
        sequences with the default `want`) are a view of a buffer that the next captured step of the
        same size overwrites: copy what must outlive it."""
        if isinstance(tokens, TokenFeed):
            if not self.use_graphs:
                host = tokens.buffer.tolist()
                tokens = [[int(host[r])] for r in tokens.rows]
            else:
                return self._finish(self._decode_step(slots, tokens, want))
        if self.use_graphs and len(tokens) > 0 and all(len(t) == 1 for t in tokens):
            return self._finish(self._decode_step(slots, tokens, want))
        if self.captures_prefill:
            done = self._captured_step(slots, tokens, want)
            if done is not None:
                return self._finish(done)
        batch = self.build_batch(slots, tokens, want)
        if batch.n_tokens == 0:
            return None
        logits = self.model.forward(StepContext(batch, self.cache, self.status, self.side_stream, self.nan_record))
        self.cache.commit(batch.slots, batch.new_tokens)
        return self._finish(logits)

    def _finish(self, logits):
        if self.check_nan:
            self.check_status()
        return logits

    def _captured_step(self, slots, tokens, want):
        """A step with few tokens that wants each sequence's last logits only: replay the captured step of its
        padded size (None: the step is not of that kind and runs kernel by kernel)."""
        from .graphs import PrefillGraph, prefill_bucket
        n_new = [len(t) for t in tokens]
        if len(slots) != len(tokens) or not all(n_new):
            return None
        if want is not None and (len(want) != len(slots) or any(list(w) != [n - 1] for w, n in zip(want, n_new))):
            return None
        size = prefill_bucket(sum(n_new), len(slots))
        if size is None:
            return None
        tokens = self._checked_tokens(slots, tokens)
        self.cache.prepare(slots, n_new)
        p0 = [self.cache.length(s) for s in slots]
        graph = self._prefill_graphs.get(size)
        if graph is None:
            graph = self._prefill_graphs[size] = PrefillGraph(self, *size)
        logits = graph.run(slots, tokens, p0)
        self.cache.commit(slots, n_new)
        return logits[:len(slots)]

    def _decode_step(self, slots, tokens, want):
        """One token per sequence: replay the captured graph of the batch's size bucket."""
        from ..csrc import ops
        from .graphs import DecodeGraph, bucket_for, reach_for
        n = len(slots)
        fed = isinstance(tokens, TokenFeed)
        if (len(tokens.rows) if fed else len(tokens)) != n or (want is not None and len(want) != n):
            raise QStreamError(QsError.INVALID_INPUT, "step: slots, tokens and want differ in length")
        V = self.model.vocab_size
        if fed:
            buf = tokens.buffer
            if buf.dtype != torch.int32 or not buf.is_cuda or not buf.is_contiguous() or buf.dim() != 1:
                raise QStreamError(QsError.INVALID_INPUT, "step: fed tokens must be a contiguous int32 device vector")
            if any(not 0 <= int(r) < buf.numel() for r in tokens.rows):
                raise QStreamError(QsError.INVALID_INPUT, "step: a fed token's row lies outside the buffer")
            toks = tokens
        else:
            toks = [int(t[0]) for t in tokens]
            for s, tok in zip(slots, toks):
                if not 0 <= tok < V:
                    raise QStreamError(QsError.INVALID_INPUT, f"token id {tok} (slot {s}) outside the vocabulary of {V}")
        if want is not None:
            for w in want:
                if any(p != 0 for p in w):
                    raise QStreamError(QsError.INVALID_INPUT, f"wanted place {w} outside the 1 token given")
        ones = [1] * n
        self.cache.prepare(slots, ones)
        p0 = [self.cache.length(s) for s in slots]
        rows = bucket_for(n)
        reach = reach_for(max(p0) + 1, self.cache.max_context)
        graph = self._graphs.get((rows, reach))
        if graph is None:
            graph = self._graphs[rows, reach] = DecodeGraph(self, rows, reach)
        logits = graph.run(slots, toks, p0)
        self.cache.commit(slots, ones)
        if want is None or all(len(w) == 1 for w in want):
            return logits[:n]
        picked = [i for i, w in enumerate(want) for _ in w]
        if not picked:
            return None
        return self.rows_of(logits, picked)

    def capture_decode_graphs(self, batch_sizes: Sequence[int]) -> int:
        """Capture, ahead of their first use, the decode graphs of the given batch sizes for every length a
        sequence can reach (a graph is otherwise captured when a step first needs it, which costs that
        step some tens of milliseconds).  Returns how many graphs were captured."""
        from .graphs import DecodeGraph, REACH_STEP, bucket_for, reach_for
        if not self.use_graphs:
            return 0
        made = 0
        for n in sorted({bucket_for(int(b)) for b in batch_sizes}):
            for longest in range(REACH_STEP, self.cache.max_context + REACH_STEP, REACH_STEP):
                key = (n, reach_for(longest, self.cache.max_context))
                if key not in self._graphs:
                    self._graphs[key] = DecodeGraph(self, *key)
                    self._graphs[key].capture()
                    made += 1
        return made

    def rows_of(self, logits: torch.Tensor, rows: Sequence[int]) -> torch.Tensor:
        """The listed rows of a logits tensor, as a new tensor."""
        from ..csrc import ops
        idx = torch.tensor(list(rows), dtype=torch.int32)
        idx = idx.pin_memory().to(self.device, non_blocking=True) if self.device.type == "cuda" else idx
        return ops.gather_rows(logits, idx)

    def check_status(self) -> None:
        """Raise if a kernel reported a fault, a bounded wait ran out, or (with `check_nan`) a
        layer's output held a value that is not finite.  This waits for the device."""
        if self._words_host is None:
            words = self._words.tolist() + [0]
        else:
            from ..csrc import gemm_tc
            self._words_host[:8].copy_(self._words, non_blocking=True)
            self._words_host[8:9].copy_(gemm_tc.status_word(self.device), non_blocking=True)
            torch.cuda.current_stream(self.device).synchronize()
            words = self._words_host.tolist()
        code, nan, gemm = words[0], words[4:8], words[8]
        if not (code or nan[0] or gemm):
            return
        self._words.zero_()
        if gemm:
            from ..csrc import gemm_tc
            gemm_tc.status_word(self.device).zero_()
        if nan[0]:
            n_runs = len(self.model.spec.schedule)
            where = f"schedule entry {nan[1]}" if nan[1] < n_runs else ("the logits" if nan[1] == n_runs + 1 else "the embedding")
            raise QStreamError(QsError.NAN_DETECTED,
                               f"a value that is not finite in the output of {where} (layer "
                               f"{self.model.spec.schedule[nan[1]].layer if nan[1] < n_runs else '-'}), "
                               f"row {nan[2]} of the step, element {nan[3]}")
        if gemm:
            raise QStreamError(QsError.INTERNAL, f"tensor-core matrix product: a wait inside the kernel ran out (code {gemm})")
        if 100 <= code < 199:
            raise QStreamError(QsError.INTERNAL, f"attention: a wait inside the kernel ran out (code {code})")
        raise QStreamError(QsError.INTERNAL, STATUS_MESSAGES.get(code, f"kernel status {code}"))
