"""The model: parts built from a `ModelSpec` and run in the order of its schedule.

Nothing here names an architecture.  The spec lists the layers (each a `BlockSpec`)
and the schedule (which layer runs when, against which cache entry); the part
registries turn specs into parts; the loader binds tensors by the names the specs
carry.  The forward pass is QStream's `qsf_forward` (src/engine.c:694-1247) for a
whole batch of tokens: embedding, the layers, then final norm and head for the rows
whose logits are wanted only (the reference runs the head for every prompt token,
src/engine.c:1289-1295).
"""
from __future__ import annotations

from pathlib import Path
from typing import Mapping

import torch

from ..cache import KvNeed, StateNeed
from ..config import ModelSpec, load_config
from ..csrc import ops
from ..errors import QsError, QStreamError
from ..parts import Runtime, build_block, part_class
from ..weights.loader import TensorDecl, bind_tensors, open_checkpoint
from ..weights.random_init import InitScales, random_tensors

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
          "fp32": torch.float32, torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def resolve_dtype(dtype) -> torch.dtype:
    try:
        return DTYPES[dtype]
    except KeyError:
        raise QStreamError(QsError.INVALID_INPUT, f"dtype {dtype!r}: want bfloat16 or float32") from None


def _part_declarations(spec: ModelSpec):
    """Yield (part spec, {own name: TensorDecl}) for every part that holds tensors."""
    yield spec.embedding, part_class("embedding", spec.embedding.kind).declare(spec.embedding)
    for block in spec.layers:
        for role, ps in part_class("arrangement", block.arrangement).part_specs(block):
            yield ps, part_class(role, ps.kind).declare(ps)
    if spec.final_norm is not None:
        yield spec.final_norm, part_class("norm", spec.final_norm.kind).declare(spec.final_norm)
    yield spec.head, part_class("head", spec.head.kind).declare(spec.head)


def declared_tensors(spec: ModelSpec) -> dict[str, TensorDecl]:
    """Checkpoint name -> declaration, for every tensor the model holds, in model order."""
    out: dict[str, TensorDecl] = {}
    for ps, decls in _part_declarations(spec):
        for own, decl in decls.items():
            try:
                name = ps.names[own]
            except KeyError:
                raise QStreamError(QsError.INVALID_MODEL,
                                   f"{type(ps).__name__} gives no checkpoint name for its tensor '{own}'") from None
            if name in out and out[name] != decl:
                raise QStreamError(QsError.INVALID_MODEL, f"tensor '{name}' is declared with two shapes")
            out[name] = decl
    return out


class CausalLM:
    """Parts, weights and the forward pass of one model."""

    def __init__(self, spec: ModelSpec, tensors: Mapping[str, torch.Tensor], dtype, device, config=None):
        self.spec = spec
        self.config = config
        self.runtime = Runtime(dtype=resolve_dtype(dtype), device=torch.device(device))
        self.vocab_size = spec.vocab_size

        def tensors_of(part_spec, decls):
            return {own: tensors[part_spec.names[own]] for own in decls}

        def make(role, part_spec):
            cls = part_class(role, part_spec.kind)
            return cls(part_spec, tensors_of(part_spec, cls.declare(part_spec)), self.runtime)

        self.embedding = make("embedding", spec.embedding)
        self.blocks = [build_block(b, tensors_of, self.runtime) for b in spec.layers]
        self.final_norm = make("norm", spec.final_norm) if spec.final_norm is not None else None
        self.head = make("head", spec.head)
        if getattr(spec.head, "tied", False):
            self.head.tie(self.embedding)
        self._check_schedule()
        self.n_parameters = sum(t.numel() for t in {id(t): t for t in tensors.values()}.values())
        self.weight_bytes = sum(t.numel() * t.element_size() for t in {id(t): t for t in tensors.values()}.values())

    @property
    def embedding_bytes(self) -> int:
        """Bytes of the embedding's tensors that the head does not share: a step gathers a few rows of them."""
        shared = {id(t) for t in vars(self.head).values() if isinstance(t, torch.Tensor)}
        return sum(t.numel() * t.element_size() for t in vars(self.embedding).values()
                   if isinstance(t, torch.Tensor) and id(t) not in shared)

    # ------------------------------------------------------------------ making a model
    @classmethod
    def from_folder(cls, folder, dtype="bfloat16", device="cuda", allow_mmap=True, verbose=0,
                    narrow_fp32_matrices=False):
        """config.json chooses the architecture; *.safetensors give the weights.
        narrow_fp32_matrices: round matrices that the files store in 32-bit to bfloat16 in a
        bfloat16 engine (default: a tensor stored in 32-bit stays in 32-bit)."""
        config = load_config(folder)
        spec = config.model_spec()
        files = open_checkpoint(folder, allow_mmap)
        try:
            tensors = bind_tensors(files, declared_tensors(spec), resolve_dtype(dtype), device,
                                   getattr(config, "ignored_tensor_suffixes", ()),
                                   narrow_fp32_matrices=narrow_fp32_matrices)
        finally:
            for f in files:
                f.close()
        return cls(spec, tensors, dtype, device, config)

    @classmethod
    def random(cls, config, seed=0, dtype="bfloat16", device="cuda", scales: InitScales = InitScales()):
        """Random weights made on the device, without a model folder."""
        spec = config.model_spec()
        tensors = random_tensors(declared_tensors(spec), seed, resolve_dtype(dtype), device, scales)
        return cls(spec, tensors, dtype, device, config)

    # ------------------------------------------------------------------ what the cache must hold
    def _cache_users(self):
        """Yield (schedule index, cache entry id, part) for every part of every run that uses the cache."""
        for i, run in enumerate(self.spec.schedule):
            if not 0 <= run.layer < len(self.blocks):
                raise QStreamError(QsError.INVALID_MODEL, f"schedule entry {i} names layer {run.layer}")
            parts = self.blocks[run.layer].cached_parts()
            ids = run.cache if isinstance(run.cache, (tuple, list)) else (run.cache,)
            if len(ids) != len(parts):
                raise QStreamError(QsError.INVALID_MODEL,
                                   f"schedule entry {i} names {len(ids)} cache entries, layer {run.layer} has "
                                   f"{len(parts)} parts that use the cache")
            yield from ((i, cid, part) for cid, part in zip(ids, parts))

    def _check_schedule(self):
        writers = {}
        for i, cid, part in self._cache_users():
            if part.kv_need() is not None or part.state_need() is not None:
                if cid in writers:
                    raise QStreamError(QsError.INVALID_MODEL,
                                       f"schedule entries {writers[cid]} and {i} both write cache entry {cid}")
                writers[cid] = i
        for i, cid, part in self._cache_users():
            if getattr(part.spec, "shares_cache", False):
                if cid not in writers or writers[cid] > i:
                    raise QStreamError(QsError.INVALID_MODEL,
                                       f"schedule entry {i} reads cache entry {cid} before any layer wrote it")

    def kv_needs(self) -> dict[int, KvNeed]:
        return {cid: part.kv_need() for _, cid, part in self._cache_users() if part.kv_need() is not None}

    def state_needs(self) -> dict[int, StateNeed]:
        return {cid: part.state_need() for _, cid, part in self._cache_users() if part.state_need() is not None}

    # ------------------------------------------------------------------ forward
    def forward(self, step) -> torch.Tensor | None:
        """Run the step's tokens through every scheduled layer; return float32 logits
        [n_want, vocab] of the wanted rows (None if none is wanted)."""
        b = step.batch
        record = getattr(step, "nan_record", None)      # the finite check (QStream's check_nan, src/engine.c:1176-1187)
        n_runs = len(self.spec.schedule)
        x = self.embedding.forward(step)
        if record is not None:
            ops.check_finite(x, n_runs, record, b.tok_slot)
        for i, run in enumerate(self.spec.schedule):
            x = self.blocks[run.layer].forward(x, step, run.cache)
            if record is not None:
                ops.check_finite(x, i, record, b.tok_slot)
        if b.n_want == 0:
            return None
        rows = ops.gather_rows(x, b.want_rows)
        z = self.final_norm.forward(rows) if self.final_norm is not None else rows
        logits = self.head.forward(z)
        if record is not None:
            # a captured decode step wants every row, padding included: row i of the logits is row i of the step
            every_row = b.decode and b.n_want == b.n_tokens
            ops.check_finite(logits, n_runs + 1, record, b.tok_slot if every_row else None)
        return logits


def load_model(folder, dtype="bfloat16", device="cuda", **kw) -> CausalLM:
    if not Path(folder).is_dir():
        raise QStreamError(QsError.FILE_NOT_FOUND, f"model folder {folder}")
    return CausalLM.from_folder(folder, dtype, device, **kw)
