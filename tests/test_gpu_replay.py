"""bin/trace_run as a user runs it: the same requests whole, with the last 32 tokens one by one,
and in batches of unequal lengths one after another, in float32 and bfloat16, against the plain model."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from util import assert_logits_close, make_folder, plain_logits, random_tokens

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def replay(folder, dtype, out, max_tokens, steps):
    text = "".join(json.dumps(s) + "\n" for s in steps)
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
                           "--out", str(out), "--max-tokens", str(max_tokens)], input=text, text=True,
                          capture_output=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == [w for s in steps for w in ("done", str(s["step"]))]
    return proc


def read(out, step, vocab):
    return np.fromfile(Path(out) / f"{step}.f32", dtype="<f4").reshape(-1, vocab)


@pytest.mark.parametrize("which,dtype", [("A", "float32"), ("B", "float32"), ("A", "bfloat16"), ("B", "bfloat16")])
def test_replay_in_every_cutting(tmp_path, which, dtype):
    folder, cfg = make_folder(tmp_path, which, dtype)
    V = cfg.vocab_size
    rng = np.random.default_rng(31)
    lens = [40, 33, 97, 64, 70]
    reqs = {f"r{i}": random_tokens(rng, n, V) for i, n in enumerate(lens)}
    refs = {k: plain_logits(folder, v) for k, v in reqs.items()}

    # 1. each request alone and whole; every position wanted; one slot's worth of cache, used again
    steps = [{"step": i, "entries": [{"id": k, "tokens": t, "want": list(range(len(t)))}], "end": [k]}
             for i, (k, t) in enumerate(reqs.items())]
    replay(folder, dtype, tmp_path / "whole", 128, steps)
    for i, k in enumerate(reqs):
        assert_logits_close(read(tmp_path / "whole", i, V), refs[k], dtype, f"whole {k}")

    # 2. each alone: all but the last 32 tokens in one step, then the last 32 one by one
    steps, where = [], {}
    for k, t in reqs.items():
        head = len(t) - 32
        steps.append({"step": len(steps), "entries": [{"id": k, "tokens": t[:head], "want": [head - 1]}], "end": []})
        where[(k, head - 1)] = steps[-1]["step"]
        for p in range(head, len(t)):
            steps.append({"step": len(steps), "entries": [{"id": k, "tokens": [t[p]], "want": [0]}],
                          "end": [k] if p == len(t) - 1 else []})
            where[(k, p)] = steps[-1]["step"]
    replay(folder, dtype, tmp_path / "tail", 128, steps)
    for (k, p), s in where.items():
        assert_logits_close(read(tmp_path / "tail", s, V), refs[k][p:p + 1], dtype, f"tail32 {k} at {p}")

    # 3. batches of unequal lengths, one after another; prompts in one step, then one token each;
    #    shorter requests end earlier; a step in which nothing is wanted writes no file
    steps, where = [], {}
    for batch in (["r0", "r1", "r2"], ["r3", "r4"]):
        prompt = {k: max(1, len(reqs[k]) - 36) for k in batch}
        prompt[batch[0]] = 1                                          # one request starts from a single token
        steps.append({"step": len(steps), "end": [],
                      "entries": [{"id": k, "tokens": reqs[k][:prompt[k]], "want": list(range(prompt[k]))} for k in batch]})
        where[len(steps) - 1] = [(k, p) for k in batch for p in range(prompt[k])]
        pos = dict(prompt)
        live = list(batch)
        while live:
            quiet = len(steps) % 5 == 0
            entries = [{"id": k, "tokens": [reqs[k][pos[k]]], "want": [] if quiet else [0]} for k in live]
            if not quiet:
                where[len(steps)] = [(k, pos[k]) for k in live]
            for k in live:
                pos[k] += 1
            ended = [k for k in live if pos[k] == len(reqs[k])]
            live = [k for k in live if k not in ended]
            steps.append({"step": len(steps), "entries": entries, "end": ended})
    max_tokens = 3 * 128                                              # three requests of at most 97 -> 2 pages each
    replay(folder, dtype, tmp_path / "batched", max_tokens, steps)
    for s, places in where.items():
        got = read(tmp_path / "batched", s, V)
        ref = np.stack([refs[k][p] for k, p in places])
        assert_logits_close(got, ref, dtype, f"batched step {s}")
    assert not (tmp_path / "batched" / "5.f32").exists()


def test_replay_reports_a_cache_that_is_too_small(tmp_path):
    folder, cfg = make_folder(tmp_path, "A", "float32")
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": list(range(70)), "want": [69]}], "end": []}]
    text = json.dumps(steps[0]) + "\n"
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32",
                           "--out", str(tmp_path / "o"), "--max-tokens", "64"], input=text, text=True,
                          capture_output=True, timeout=600)
    assert proc.returncode == 1 and "cache pages" in proc.stderr and "done" not in proc.stdout


def test_command_line(tmp_path):
    folder, cfg = make_folder(tmp_path, "A", "float32")
    run = lambda *a: subprocess.run([sys.executable, str(ROOT / "bin" / "qstream"), str(folder), *a], text=True,
                                    capture_output=True, timeout=600)
    greedy = run("-p", "5,17,3;1 2 3 4", "-n", "5", "-t", "0", "--repeat-penalty", "1.0", "--dtype", "float32",
                 "--stop-token", "none", "-v")
    assert greedy.returncode == 0, greedy.stderr[-2000:]
    lines = [[int(t) for t in l.split()] for l in greedy.stdout.strip().splitlines()]
    assert len(lines) == 2 and all(len(l) == 5 for l in lines)
    assert "Tokens generated: 10" in greedy.stderr and "tok/s" in greedy.stderr
    ref = plain_logits(folder, [5, 17, 3])
    assert lines[0][0] == int(np.argmax(ref[-1]))
    sampled = run("-p", "5,17,3", "-n", "6", "--seed", "7", "--dtype", "float32", "--stop-token", "none")
    again = run("-p", "5,17,3", "-n", "6", "--seed", "7", "--dtype", "float32", "--stop-token", "none")
    assert sampled.returncode == 0 and sampled.stdout == again.stdout
    bad = run("-p", "5,x")
    assert bad.returncode != 0
