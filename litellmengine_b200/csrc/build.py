"""Compiles the engine's CUDA sources for sm_100a, on demand, into shared libraries.

Each kernel family (`embedding`, `norm`, ...) is one `.cu` file and becomes one `.so`
under `csrc/_build/`, named by a hash of its source, the shared header and the flags, so
a stale library is never loaded.  A family is compiled the first time something asks
for it; `build_all()` compiles every family (in parallel).  While nvcc runs, a line is
printed to stderr every few seconds.  If the package folder cannot be written, the
libraries go to a per-user folder under the system's temporary directory.

There is no fallback: without nvcc and without a prebuilt library this raises.
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
from typing import Dict, List

CSRC = os.path.dirname(os.path.abspath(__file__))

FAMILIES: Dict[str, List[str]] = {
    "embedding": ["embedding.cu"],
    "norm": ["norm.cu"],
    "activation": ["activation.cu"],
    "rope_cache": ["rope_cache.cu"],
    "attention_generic": ["attention_generic.cu"],
    "attention_decode": ["attention_decode.cu"],
    "attention_prefill": ["attention_prefill.cu"],
    "attention_prefill_tcgen05": ["attention_prefill_tcgen05.cu"],
    "sampling": ["sampling.cu"],
    "gemm_skinny": ["gemm_skinny.cu"],
    "gemm_pair_tcgen05": ["gemm_pair_tcgen05.cu"],
    "host_core": ["host_core.cpp"],            # the host side's bookkeeping: plain C++, no device code
}
HOST_FAMILIES = {"host_core"}
HEADERS = ["common.cuh", "attention_decode_noalloc.h", "attention_decode_tma.cuh"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC",
]
HOST_FLAGS = ["-O2", "-std=c++17", "--shared", "-Xcompiler", "-fPIC"]
EXTRA_FLAGS: Dict[str, List[str]] = {}


def _flags(family: str) -> List[str]:
    return (HOST_FLAGS if family in HOST_FAMILIES else NVCC_FLAGS) + EXTRA_FLAGS.get(family, [])

_lock = threading.Lock()
_family_locks: Dict[str, threading.Lock] = {}


class BuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked at $NVCC, PATH and /usr/local/cuda/bin); "
                     "the engine's kernels cannot be compiled and there is no fallback")


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe{os.getpid()}")
        with open(probe, "w"):
            pass
        os.unlink(probe)
        return True
    except OSError:
        return False


_build_dir_cache = None


def build_dir() -> str:
    global _build_dir_cache
    if _build_dir_cache is None:
        env = os.environ.get("LITELLMENGINE_B200_BUILD_DIR")
        cands = [env] if env else []
        cands.append(os.path.join(CSRC, "_build"))
        cands.append(os.path.join(tempfile.gettempdir(), f"litellmengine_b200_build_{os.getuid()}"))
        for c in cands:
            if _writable_dir(c):
                _build_dir_cache = c
                break
        else:
            raise BuildError("no writable folder for compiled kernels among: " + ", ".join(cands))
    return _build_dir_cache


def _digest(family: str) -> str:
    h = hashlib.sha256()
    for fn in ([] if family in HOST_FAMILIES else HEADERS) + FAMILIES[family]:
        with open(os.path.join(CSRC, fn), "rb") as f:
            h.update(fn.encode())
            h.update(f.read())
    h.update(" ".join(_flags(family)).encode())
    return h.hexdigest()[:16]


def library_path(family: str) -> str:
    """Where the family's library is or will be; prefers an already built copy in the
    package folder even when that folder is read-only."""
    name = f"llmk_{family}-{_digest(family)}.so"
    in_tree = os.path.join(CSRC, "_build", name)
    if os.path.isfile(in_tree):
        return in_tree
    return os.path.join(build_dir(), name)


def ensure_built(family: str, verbose: bool = True) -> str:
    if family not in FAMILIES:
        raise BuildError(f"unknown kernel family {family!r}")
    with _lock:
        flock = _family_locks.setdefault(family, threading.Lock())
    with flock:
        out = library_path(family)
        if os.path.isfile(out):
            return out
        nvcc = _nvcc()
        srcs = [os.path.join(CSRC, fn) for fn in FAMILIES[family]]
        tmp = f"{out}.{os.getpid()}.{threading.get_ident()}.tmp"
        cmd = [nvcc] + _flags(family) + ["-I", CSRC, "-o", tmp] + srcs
        what = family if family in HOST_FAMILIES else f"{family} for sm_100a"
        t0 = time.time()
        if verbose:
            print(f"[litellmengine_b200] compiling {what} ...", file=sys.stderr, flush=True)
        proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                                cwd=build_dir())
        done = threading.Event()

        def heartbeat():
            while not done.wait(5.0):
                if verbose:
                    print(f"[litellmengine_b200] ... still compiling {family} ({time.time() - t0:.0f} s)",
                          file=sys.stderr, flush=True)

        hb = threading.Thread(target=heartbeat, daemon=True)
        hb.start()
        try:
            log, _ = proc.communicate()
        finally:
            done.set()
        if proc.returncode != 0:
            try:
                os.unlink(tmp)
            except OSError:
                pass
            raise BuildError(f"nvcc failed for {family} (exit {proc.returncode}):\n{log}")
        os.replace(tmp, out)
        for old in os.listdir(os.path.dirname(out)):         # drop builds of older sources
            if old.startswith(f"llmk_{family}-") and old.endswith(".so") and old != os.path.basename(out):
                try:
                    os.unlink(os.path.join(os.path.dirname(out), old))
                except OSError:
                    pass
        if verbose:
            print(f"[litellmengine_b200] compiled {family} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
        return out


def build_all(verbose: bool = True) -> Dict[str, str]:
    with ThreadPoolExecutor(max_workers=min(8, len(FAMILIES))) as pool:
        paths = list(pool.map(lambda f: ensure_built(f, verbose), FAMILIES))
    return dict(zip(FAMILIES, paths))


if __name__ == "__main__":
    for fam, p in build_all().items():
        print(fam, p)
