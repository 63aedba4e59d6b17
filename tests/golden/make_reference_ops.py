#!/usr/bin/env python3
"""Run QStream's own scalar kernels and sampler on fixed inputs and store what they return.

    python tests/golden/make_reference_ops.py /path/to/Qstream tests/golden/reference_ops.json

Compiles src/kernels_scalar.c, src/quant.c and src/sampling.c of the reference (CPU, gcc, no
fast-math) into a shared object in a temporary folder, calls them through ctypes and writes
the inputs' seeds and the outputs as JSON.  The engine's rotary helper `apply_rope` is
`static` (src/engine.c:205-234), so a one-line translation unit that includes src/engine.c
and exports a wrapper is compiled beside them.  tests/test_plain.py compares the plain
implementation of the tests with this file, so the comparison needs neither the reference
nor a compiler at test time.  The reference's engine itself cannot serve as a model-level
oracle: it has no GPT-J forward pass (sequential residual, full-head rotary, no biases,
quantized weights only), so the whole-model results of the plain implementation rest on the
formulas.
"""
import ctypes
import json
import os
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np


def main(ref_root, out_path):
    ref = Path(ref_root)
    with tempfile.TemporaryDirectory() as tmp:
        so = Path(tmp) / "libqsf_ops.so"
        subprocess.check_call(["gcc", "-std=gnu11", "-O2", "-fPIC", "-shared", f"-I{ref / 'include'}",
                               str(ref / "src/kernels_scalar.c"), str(ref / "src/quant.c"),
                               str(ref / "src/sampling.c"), "-lm", "-o", str(so)])
        lib = ctypes.CDLL(str(so))
        fp = ctypes.POINTER(ctypes.c_float)
        shim_c = Path(tmp) / "rope_shim.c"
        shim_c.write_text('#include "src/engine.c"\n'
                          'void golden_apply_rope(float* q, float* k, int head_dim, int position, float theta,\n'
                          '                       int num_heads, int num_kv_heads) {\n'
                          '    apply_rope(q, k, head_dim, position, theta, num_heads, num_kv_heads);\n}\n')
        shim_so = Path(tmp) / "librope_shim.so"
        subprocess.check_call(["gcc", "-std=gnu11", "-O2", "-w", "-fPIC", "-shared", f"-I{ref / 'include'}", f"-I{ref}",
                               str(shim_c), "-lm", "-o", str(shim_so)])
        shim = ctypes.CDLL(str(shim_so), mode=os.RTLD_LAZY)      # the engine's other calls stay unresolved and unused

        def arr(a):
            a = np.array(a, dtype=np.float32, copy=True)      # the kernels work in place
            return a, a.ctypes.data_as(fp)

        rng = np.random.default_rng(2024)
        out = {}

        # LayerNorm with weight and bias: qsf_layer_norm_scalar(in, out, w, b, dim, eps)
        cases = []
        for dim, eps in ((17, 1e-5), (96, 1e-6), (256, 1e-3)):
            x, xp = arr(rng.normal(0.5, 2.0, dim))
            w, wp = arr(1 + rng.uniform(-0.2, 0.2, dim))
            b, bp = arr(rng.normal(0, 0.1, dim))
            y, yp = arr(np.zeros(dim))
            lib.qsf_layer_norm_scalar(xp, yp, wp, bp, ctypes.c_int(dim), ctypes.c_float(eps))
            cases.append(dict(x=x.tolist(), w=w.tolist(), b=b.tolist(), eps=eps, y=y.tolist()))
        out["layer_norm"] = cases

        # tanh GELU in place: qsf_gelu_scalar(x, n)
        x, xp = arr(np.linspace(-6, 6, 97))
        g = x.copy()
        lib.qsf_gelu_scalar(g.ctypes.data_as(fp), ctypes.c_int(len(g)))
        out["gelu_tanh"] = dict(x=x.tolist(), y=g.tolist())

        # softmax: qsf_softmax_scalar(in, out, n)
        x, xp = arr(rng.normal(0, 3, 50))
        y, yp = arr(np.zeros(50))
        lib.qsf_softmax_scalar(xp, yp, ctypes.c_int(50))
        out["softmax"] = dict(x=x.tolist(), y=y.tolist())

        # random numbers: qsf_rng_seed / qsf_rng_float
        class Rng(ctypes.Structure):
            _fields_ = [("s", ctypes.c_uint64 * 2)]
        lib.qsf_rng_float.restype = ctypes.c_float
        draws = {}
        for seed in (0, 7, 42, 2 ** 40 + 3):
            r = Rng()
            lib.qsf_rng_seed(ctypes.byref(r), ctypes.c_uint64(seed))
            draws[str(seed)] = [float(lib.qsf_rng_float(ctypes.byref(r))) for _ in range(8)]
        out["rng"] = draws

        # argmax with ties, repeat penalty
        x, xp = arr([1.0, 5.0, 5.0, -2.0, 5.0])
        out["argmax_tie"] = int(lib.qsf_argmax(xp, ctypes.c_int(5)))
        x, xp = arr([1.0, -2.0, 3.0, 0.5, -0.25])
        recent = (ctypes.c_uint32 * 4)(0, 1, 0, 4)
        lib.qsf_apply_repeat_penalty(xp, ctypes.c_int(5), recent, ctypes.c_int(4), ctypes.c_float(1.5))
        out["repeat_penalty"] = dict(x=[1.0, -2.0, 3.0, 0.5, -0.25], recent=[0, 1, 0, 4], penalty=1.5, y=x.tolist())

        # filters and the whole pipeline: qsf_top_k_filter, qsf_top_p_filter, qsf_sample
        class Cfg(ctypes.Structure):
            _fields_ = [("temperature", ctypes.c_float), ("top_k", ctypes.c_int), ("top_p", ctypes.c_float),
                        ("repeat_penalty", ctypes.c_float), ("seed", ctypes.c_uint64)]
        logits = rng.normal(0, 2.5, 64).astype(np.float32)
        x, xp = arr(logits)
        lib.qsf_top_k_filter(xp, ctypes.c_int(64), ctypes.c_int(10))
        out["top_k"] = dict(x=logits.tolist(), k=10, kept=[int(i) for i in np.nonzero(np.isfinite(x))[0]])
        x, xp = arr(logits)
        lib.qsf_top_p_filter(xp, ctypes.c_int(64), ctypes.c_float(0.8))
        out["top_p"] = dict(x=logits.tolist(), p=0.8, kept=[int(i) for i in np.nonzero(np.isfinite(x))[0]])
        pipeline = []
        for temperature, top_k, top_p, seed in ((0.0, 40, 0.9, 1), (0.8, 0, 1.0, 7), (0.7, 40, 0.9, 42),
                                                (1.0, 5, 1.0, 3), (1.3, 0, 0.5, 11)):
            cfg = Cfg(temperature, top_k, top_p, 1.0, seed)
            r = Rng()
            lib.qsf_rng_seed(ctypes.byref(r), ctypes.c_uint64(seed))
            toks = []
            for _ in range(12):
                x, xp = arr(logits)
                toks.append(int(lib.qsf_sample(xp, ctypes.c_int(64), ctypes.byref(cfg), ctypes.byref(r))))
            pipeline.append(dict(temperature=temperature, top_k=top_k, top_p=top_p, seed=seed, tokens=toks))
        out["sample"] = dict(logits=logits.tolist(), runs=pipeline)

        # rotary: apply_rope(q, k, head_dim, position, theta, heads, kv heads) rotates the whole head in place
        rope = []
        for head_dim in (8, 32, 64):
            for position in (0, 1, 63, 2047):
                q, qp = arr(rng.normal(0, 1, 2 * head_dim))
                k, kp = arr(rng.normal(0, 1, head_dim))
                q0, k0 = q.copy(), k.copy()
                shim.golden_apply_rope(qp, kp, ctypes.c_int(head_dim), ctypes.c_int(position), ctypes.c_float(10000.0),
                                       ctypes.c_int(2), ctypes.c_int(1))
                rope.append(dict(head_dim=head_dim, position=position, q=q0.tolist(), k=k0.tolist(),
                                 q_out=q.tolist(), k_out=k.tolist()))
        out["apply_rope"] = rope

    Path(out_path).write_text(json.dumps(out) + "\n")
    print(f"wrote {out_path} ({Path(out_path).stat().st_size} bytes)")


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2])
