"""Decode steps, and steps with short prompts, as CUDA graphs.

A decode step (one token per sequence) launches a few hundred small kernels; captured
once per batch-size bucket and replayed, the launches cost the host almost nothing.  The
graph reads the step's metadata (tokens, slots, positions) from fixed device buffers that
are refreshed by one copy from pinned memory before each replay; rows beyond the live
sequences carry slot -1 and are skipped by every kernel that touches the cache.  Logits
of all rows land in a fixed buffer.
"""
from __future__ import annotations

import gc
import weakref

import numpy as np
import torch

from .step import StepBatch, StepContext, TokenFeed

BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)
_RING = 4


def bucket_for(n: int) -> int:
    for b in BUCKETS:
        if n <= b:
            return b
    return -(-n // 64) * 64


REACH_STEP = 256                # a decode graph serves sequences of up to a multiple of this many tokens


def reach_for(longest: int, max_context: int) -> int:
    """The bound on the longest sequence that a decode graph is captured for: the attention kernels' grids
    cover splits of 256 keys up to it, so a graph for short sequences launches no CTAs for keys nobody has."""
    return min(-(-max(longest, 1) // REACH_STEP) * REACH_STEP, -(-max_context // REACH_STEP) * REACH_STEP)


class DecodeGraph:
    """One captured decode step for `rows` packed rows whose sequences hold at most `reach` tokens."""

    def __init__(self, engine, rows: int, reach: int = 0):
        self._engine = weakref.ref(engine)          # the engine owns its graphs, not the other way round
        self.rows = rows
        self.reach = reach
        dev = engine.device
        sizes = [rows, rows, rows, rows, rows, rows + 1, rows, rows]        # the last: where a fed token comes from
        self.offs = np.concatenate([[0], np.cumsum(sizes)]).astype(int)
        n = int(self.offs[-1])
        self.meta = torch.zeros(n, dtype=torch.int32, device=dev)
        self.staging = [torch.zeros(n, dtype=torch.int32).pin_memory() for _ in range(_RING)]
        self.staging_np = [s.numpy() for s in self.staging]
        self.events = [None] * _RING
        self.turn = 0
        v = [self.meta[self.offs[i]:self.offs[i + 1]] for i in range(8)]
        self.tok_src = v[7]
        # fixed parts of the metadata: every row is wanted, row i is sequence i
        for s in self.staging_np:
            s[self.offs[1]:self.offs[2]] = -1
            s[self.offs[3]:self.offs[4]] = np.arange(rows)
            s[self.offs[5]:self.offs[6]] = np.arange(rows + 1)
            s[self.offs[7]:self.offs[8]] = -1
        self.meta.copy_(self.staging[0])
        self.batch = StepBatch(n_seq=rows, n_tokens=rows, n_want=rows, tokens=v[0], tok_slot=v[1], tok_pos=v[2],
                               want_rows=v[3], seq_slot=v[4], seq_start=v[5], seq_p0=v[6],
                               slots=[], new_tokens=[1] * rows, p0=[], decode=True, max_new=1, max_total=reach)
        self.graph = None
        self.logits = None
        self.launches = 0

    def capture(self) -> None:
        from ..csrc import ops
        eng = self._engine()
        ctx = StepContext(self.batch, eng.cache, eng.status, eng.side_stream, eng.nan_record)
        stream = torch.cuda.Stream(device=eng.device)
        stream.wait_stream(torch.cuda.current_stream(eng.device))
        with torch.cuda.stream(stream):
            eng.model.forward(ctx)                      # warm-up: first-call set-up happens outside the capture
        torch.cuda.current_stream(eng.device).wait_stream(stream)
        torch.cuda.synchronize(eng.device)
        self.graph = torch.cuda.CUDAGraph()
        before = ops.launch_count()
        # A dead graph freed by the garbage collector in mid-capture would invalidate the capture.
        gc.collect()
        gc_was_on = gc.isenabled()
        gc.disable()
        try:
            # the main chain of kernels is captured with a higher priority than the side stream's product,
            # which then only fills what the chain leaves idle
            with torch.cuda.graph(self.graph, pool=getattr(eng, "graph_pool", None),
                                  stream=torch.cuda.Stream(device=eng.device, priority=-1)):
                self.logits = eng.model.forward(ctx)
        finally:
            if gc_was_on:
                gc.enable()
        self.launches = ops.launch_count() - before

    def run(self, slots, tokens, p0) -> torch.Tensor:
        """Refresh the metadata and replay; returns the logits buffer [rows, vocab].
        `tokens`: a list of ints, or a `TokenFeed` (the tokens are on the device: no host round trip)."""
        if self.graph is None:
            self.capture()          # while the metadata still holds padding only: the warm-up run touches no sequence
        i = self.turn
        self.turn = (self.turn + 1) % _RING
        if self.events[i] is not None:
            self.events[i].synchronize()                # the copy that last read this buffer is done
        s, o, n = self.staging_np[i], self.offs, len(slots)
        on_device = isinstance(tokens, TokenFeed)
        s[o[0]:o[0] + n] = 0 if on_device else tokens
        s[o[7]:o[7] + n] = tokens.rows if on_device else -1
        s[o[7] + n:o[8]] = -1
        s[o[0] + n:o[1]] = 0
        s[o[1]:o[1] + n] = slots
        s[o[1] + n:o[2]] = -1
        s[o[2]:o[2] + n] = p0
        s[o[2] + n:o[3]] = 0
        s[o[4]:o[4] + n] = slots
        s[o[4] + n:o[5]] = -1
        s[o[6]:o[6] + n] = p0
        s[o[6] + n:o[7]] = 0
        self.meta.copy_(self.staging[i], non_blocking=True)
        from ..csrc import ops
        if on_device:                                   # the sampler's output goes straight into the graph's input
            ops.take_tokens(self.batch.tokens, tokens.buffer, self.tok_src, n)
        ev = torch.cuda.Event()
        ev.record()
        self.events[i] = ev
        self.graph.replay()
        ops.count_launches(self.launches)
        return self.logits


# Steps that bring prompts (or any mix of token counts) of up to 512 tokens in all, for up to 8 sequences, are
# bound by the host when launched kernel by kernel: some 170 launches cost more host time than the device
# needs for them.  They are captured once per (padded token count, padded sequence count) and replayed.
PREFILL_TOKENS = (64, 128, 256, 512)
PREFILL_SEQS = (1, 2, 4, 8)


def prefill_bucket(n_tokens: int, n_seq: int):
    """The (tokens, sequences) sizes of the captured step that serves this one, or None."""
    t = next((b for b in PREFILL_TOKENS if n_tokens <= b), None)
    s = next((b for b in PREFILL_SEQS if n_seq <= b), None)
    return None if t is None or s is None else (t, s)


class PrefillGraph:
    """One captured step of `t_pad` packed rows for up to `s_pad` sequences that bring any number of tokens
    each; the logits of every sequence's last token land in a fixed buffer.  Rows beyond the step's tokens
    carry slot -1, sequences beyond the step's point at row 0, unused entries of the query-tile list have no
    rows: every kernel skips them."""

    def __init__(self, engine, t_pad: int, s_pad: int):
        self._engine = weakref.ref(engine)
        self.t_pad, self.s_pad = t_pad, s_pad
        self.n_tiles = t_pad // 128 + s_pad               # pieces of at most 128 rows of one sequence
        dev = engine.device
        sizes = [t_pad, t_pad, t_pad, s_pad, s_pad, s_pad + 1, s_pad, 4 * self.n_tiles]
        self.offs = np.concatenate([[0], np.cumsum(sizes)]).astype(int)
        n = int(self.offs[-1])
        self.meta = torch.zeros(n, dtype=torch.int32, device=dev)
        self.staging = [torch.zeros(n, dtype=torch.int32).pin_memory() for _ in range(_RING)]
        self.staging_np = [s.numpy() for s in self.staging]
        self.events = [None] * _RING
        self.turn = 0
        v = [self.meta[self.offs[i]:self.offs[i + 1]] for i in range(8)]
        for s in self.staging_np:
            s[self.offs[1]:self.offs[2]] = -1
            s[self.offs[4]:self.offs[5]] = -1
        self.meta.copy_(self.staging[0])
        # new_tokens sums to less than the rows: the parts treat the step as padded; the host lists are not
        # the step's (they change from replay to replay), so parts must go by the device metadata
        self.batch = StepBatch(n_seq=s_pad, n_tokens=t_pad, n_want=s_pad, tokens=v[0], tok_slot=v[1], tok_pos=v[2],
                               want_rows=v[3], seq_slot=v[4], seq_start=v[5], seq_p0=v[6],
                               slots=[-1], new_tokens=[0], p0=[0], decode=False, max_new=t_pad, max_total=0)
        self.batch._prefill_tiles = v[7].view(self.n_tiles, 4)
        self.graph = None
        self.logits = None
        self.launches = 0

    capture = DecodeGraph.capture

    def run(self, slots, tokens, p0) -> torch.Tensor:
        if self.graph is None:
            self.capture()
        i = self.turn
        self.turn = (self.turn + 1) % _RING
        if self.events[i] is not None:
            self.events[i].synchronize()
        s, o = self.staging_np[i], self.offs
        tok, tslot, tpos, wrows, sslot, sstart, sp0, tiles = (s[o[j]:o[j + 1]] for j in range(8))
        tok[:] = 0
        tslot[:] = -1
        tpos[:] = 0
        wrows[:] = 0
        sslot[:] = -1
        sp0[:] = 0
        tiles[:] = 0
        row, pieces = 0, []
        for j, (slot, toks, base) in enumerate(zip(slots, tokens, p0)):
            n = len(toks)
            tok[row:row + n] = toks
            tslot[row:row + n] = slot
            tpos[row:row + n] = np.arange(base, base + n)
            wrows[j] = row + n - 1 if n else 0
            sslot[j], sstart[j], sp0[j] = slot, row, base
            for a in range(0, n, 128):
                pieces.append((row + a, min(128, n - a), base + a, slot))
            row += n
        sstart[len(slots):] = row
        pieces.sort(key=lambda t: -(t[2] + t[1]))           # longest context first, as the eager path orders them
        for j, piece in enumerate(pieces):
            tiles[4 * j:4 * j + 4] = piece
        self.meta.copy_(self.staging[i], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.events[i] = ev
        self.graph.replay()
        from ..csrc import ops
        ops.count_launches(self.launches)
        return self.logits
