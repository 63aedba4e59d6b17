"""Compiling the CUDA sources into one shared library, in the tree, at first use.

`nvcc -gencode arch=compute_100a,code=sm_100a` for every `.cu` beside this file, linked
into `_build/libqstream_b200.so` (or under a temporary folder if the tree cannot be
written).  A stamp with the hash of sources and flags decides whether to rebuild.  The
library has no CPU twin: if it cannot be built or loaded, loading fails with the
compiler's output.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

from ..errors import QsError, QStreamError

SRC_DIR = Path(__file__).resolve().parent
LIB_NAME = "libqstream_b200.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def _say(msg: str) -> None:
    print(f"[qstream] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("QSTREAM_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise QStreamError(QsError.INTERNAL, "nvcc not found (set CUDA_HOME or QSTREAM_NVCC); "
                       "the kernel library cannot be built and there is no fallback")


def sources() -> list[Path]:
    return sorted(SRC_DIR.glob("*.cu"))


def _digest() -> str:
    h = hashlib.sha256()
    for p in sorted(list(SRC_DIR.glob("*.cu")) + list(SRC_DIR.glob("*.cuh")) + list(SRC_DIR.glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _build_dir() -> Path:
    """`_build` beside the sources if it can be written, else a per-user temporary folder."""
    d = SRC_DIR / "_build"
    try:
        d.mkdir(exist_ok=True)
        probe = d / f".probe{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return d
    except OSError:
        d = Path(tempfile.gettempdir()) / f"qstream_b200_build_{os.getuid()}_{_digest()[:12]}"
        d.mkdir(parents=True, exist_ok=True)
        return d


def _run(cmd: list[str], what: str) -> None:
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    if proc.returncode != 0:
        raise QStreamError(QsError.INTERNAL, f"{what} failed:\n{' '.join(cmd)}\n{proc.stdout}")


def build(force: bool = False, verbose: bool = True) -> Path:
    """Build the library if it is missing or stale; return its path."""
    out_dir = _build_dir()
    lib = out_dir / LIB_NAME
    stamp = out_dir / "stamp.txt"
    digest = _digest()
    if not force and lib.is_file() and stamp.is_file() and stamp.read_text().strip() == digest:
        return lib
    nvcc = find_nvcc()
    srcs = sources()
    if verbose:
        _say(f"building {LIB_NAME} for sm_100a from {len(srcs)} sources in {out_dir} ...")
    t0 = time.time()
    done = threading.Event()

    def ticker():
        while not done.wait(10.0):
            if verbose:
                _say(f"  still compiling ({time.time() - t0:.0f} s)")

    th = threading.Thread(target=ticker, daemon=True)
    th.start()
    try:
        objs = [out_dir / (s.stem + ".o") for s in srcs]

        def compile_one(pair):
            src, obj = pair
            _run([nvcc, *NVCC_FLAGS, "-I", str(SRC_DIR), "-c", str(src), "-o", str(obj)],
                 f"compiling {src.name}")
            if verbose:
                _say(f"  compiled {src.name} ({time.time() - t0:.0f} s)")

        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
            list(pool.map(compile_one, zip(srcs, objs)))
        tmp = out_dir / f".{LIB_NAME}.{os.getpid()}"
        _run([nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-gencode",
              "arch=compute_100a,code=sm_100a"], "linking")
        os.replace(tmp, lib)
        stamp.write_text(digest + "\n")
    finally:
        done.set()
    if verbose:
        _say(f"built {lib} in {time.time() - t0:.0f} s")
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
