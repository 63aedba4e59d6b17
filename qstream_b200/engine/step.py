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

from dataclasses import dataclass, field
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


class StepContext:
    """What a part may touch during a step."""

    def __init__(self, batch: StepBatch, cache: SequenceCache, status: torch.Tensor, side_stream=None):
        self.batch = batch
        self.cache = cache
        self.status = status
        # a second CUDA stream for work that does not depend on the mixer (None: everything in order)
        self.side_stream = side_stream

    def kv(self, cache_id: int):
        return self.cache.view(cache_id)

    def state(self, cache_id: int) -> Optional[torch.Tensor]:
        """The state tensor [slots, *shape] of a cache entry (None if it has none)."""
        return self.cache.state.get(cache_id)


STATUS_MESSAGES = {
    1: "a token's position lies outside the position table",
    2: "a token was to be written to a cache page its sequence does not hold",
    3: "attention met a cache page its sequence does not hold",
}


class Engine:
    """A model with its cache: sequences are acquired, stepped and released.

    max_tokens: the tokens all live sequences may hold together, each rounded up to a
    whole page of 64; it sizes the cache.  max_batch: the most sequences alive at once.
    max_context: the longest sequence (default: the model's positions).
    """

    def __init__(self, model: CausalLM, max_tokens: Optional[int] = None, max_batch: int = 64,
                 max_context: Optional[int] = None, verbose: int = 0, use_graphs: bool = True):
        self.model = model
        self.device = model.runtime.device
        self.dtype = model.runtime.dtype
        self.verbose = verbose
        ctx = model.spec.max_positions if not max_context else min(max_context, model.spec.max_positions)
        if max_tokens is None:
            max_tokens = max_batch * ctx
        self.max_batch = max_batch
        kv_needs, state_needs = model.kv_needs(), model.state_needs()
        self._check_budget(kv_needs, max_tokens)
        self.cache = SequenceCache(kv_needs, state_needs, max_tokens, max_batch, ctx, self.dtype, self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        # decode steps run the feed-forward's first product beside the attention kernels
        self.side_stream = torch.cuda.Stream(device=self.device) if self.device.type == "cuda" else None
        self.use_graphs = use_graphs and self.device.type == "cuda"
        self._graphs = {}
        self._status_host = torch.zeros(1, dtype=torch.int32).pin_memory() if self.device.type == "cuda" else None
        if verbose:
            import sys
            print(f"[qstream] cache: {self.cache.bytes / 2**20:.1f} MB for {max_tokens} tokens, "
                  f"{self.cache.slots.n_slots} slots, context {ctx}; weights {model.weight_bytes / 2**20:.1f} MB",
                  file=sys.stderr)

    def _check_budget(self, kv_needs, max_tokens):
        if self.device.type != "cuda":
            return
        elem = torch.empty((), dtype=self.dtype).element_size()
        want = sum(2 * max_tokens * n.n_kv_heads * n.head_dim * elem for n in kv_needs.values())
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
        V = self.model.vocab_size
        n_new = [len(t) for t in tokens]
        for s, toks in zip(slots, tokens):
            for tok in toks:
                if not 0 <= int(tok) < V:
                    raise QStreamError(QsError.INVALID_INPUT,
                                       f"token id {tok} (slot {s}) outside the vocabulary of {V}")
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

    def _upload(self, host: np.ndarray) -> torch.Tensor:
        t = torch.from_numpy(host)
        if self.device.type == "cuda":
            return t.pin_memory().to(self.device, non_blocking=True)
        return t

    accepts_device_tokens = True        # step() also takes an int32 device tensor with one token per sequence

    def step(self, slots: Sequence[int], tokens: Sequence[Sequence[int]],
             want: Optional[Sequence[Sequence[int]]] = None) -> Optional[torch.Tensor]:
        """Run one step.  `want[i]` lists the places among sequence i's new tokens whose
        logits are asked for (default: the last).  Returns float32 logits [n_want, vocab]
        on the device, in the order of the sequences and of `want`; None if none is wanted."""
        if isinstance(tokens, torch.Tensor):
            if not self.use_graphs:
                tokens = [[int(t)] for t in tokens.tolist()]
            else:
                return self._decode_step(slots, tokens, want)
        if self.use_graphs and tokens and all(len(t) == 1 for t in tokens):
            return self._decode_step(slots, tokens, want)
        batch = self.build_batch(slots, tokens, want)
        if batch.n_tokens == 0:
            return None
        logits = self.model.forward(StepContext(batch, self.cache, self.status, self.side_stream))
        self.cache.commit(batch.slots, batch.new_tokens)
        return logits

    def _decode_step(self, slots, tokens, want):
        """One token per sequence: replay the captured graph of the batch's size bucket."""
        from ..csrc import ops
        from .graphs import DecodeGraph, bucket_for
        n = len(slots)
        if (not isinstance(tokens, torch.Tensor) and len(tokens) != n) or (want is not None and len(want) != n):
            raise QStreamError(QsError.INVALID_INPUT, "step: slots, tokens and want differ in length")
        V = self.model.vocab_size
        if isinstance(tokens, torch.Tensor):            # one token per sequence, already on the device (from the sampler)
            if tokens.dtype != torch.int32 or tokens.numel() != n or not tokens.is_cuda or not tokens.is_contiguous():
                raise QStreamError(QsError.INVALID_INPUT, "step: device tokens must be a contiguous int32 tensor, one per sequence")
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
        graph = self._graphs.get(rows)
        if graph is None:
            graph = self._graphs[rows] = DecodeGraph(self, rows)
        logits = graph.run(slots, toks, p0)
        self.cache.commit(slots, ones)
        if want is None or all(len(w) == 1 for w in want):
            return logits[:n]
        picked = [i for i, w in enumerate(want) for _ in w]
        if not picked:
            return None
        idx = torch.tensor(picked, dtype=torch.int32).pin_memory().to(self.device, non_blocking=True)
        return ops.gather_rows(logits, idx)

    def check_status(self) -> None:
        """Raise if a kernel reported a fault (this waits for the device)."""
        if self._status_host is None:
            code = int(self.status.item())
        else:
            self._status_host.copy_(self.status, non_blocking=False)
            code = int(self._status_host.item())
        if code:
            self.status.zero_()
            raise QStreamError(QsError.INTERNAL, STATUS_MESSAGES.get(code, f"kernel status {code}"))
