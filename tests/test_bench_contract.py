"""What bench.py promises without a GPU: one line and exit code 2 for more than one GPU, and the
reference arm's `unavailable` line with exit code 0."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          timeout=120, cwd=ROOT)


def test_more_than_one_gpu_is_refused_with_one_line():
    for n in ("2", "8"):
        p = run("--gpus", n, "--steps", "4", "--warmup", "3")
        assert p.returncode == 2
        lines = [l for l in p.stdout.splitlines() if l.strip()]
        assert len(lines) == 1 and "one GPU" in lines[0]


def test_reference_arm_says_why_it_is_unavailable():
    p = run("--impl", "reference", "--gpus", "1", "--steps", "4", "--warmup", "3")
    assert p.returncode == 0
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference" and isinstance(rec["unavailable"], str) and "\n" not in rec["unavailable"]
