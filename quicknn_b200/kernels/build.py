"""Compile the CUDA sources in ``csrc/`` into one shared library, in-tree.

The library is named after a hash of the sources and flags, so a checkout whose
files were copied (new time stamps) reuses what was built and a changed source
builds anew.  Nothing is written to the user's home directory.  While nvcc runs,
a line is printed now and then so that a first call does not look hung.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import List, Optional, Sequence

CSRC = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "csrc"))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[quicknn_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for env in ("CUDA_HOME", "CUDA_PATH"):
        root = os.environ.get(env)
        if root and os.path.isfile(os.path.join(root, "bin", "nvcc")):
            return os.path.join(root, "bin", "nvcc")
    if os.path.isfile("/usr/local/cuda/bin/nvcc"):
        return "/usr/local/cuda/bin/nvcc"
    found = shutil.which("nvcc")
    if found:
        return found
    raise BuildError("nvcc was not found (looked at $CUDA_HOME, /usr/local/cuda and PATH); "
                     "the CUDA kernels of quicknn_b200 cannot be built")


def sources(names: Optional[Sequence[str]] = None) -> List[str]:
    all_cu = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    if names is None:
        return all_cu
    missing = [n for n in names if n not in all_cu]
    if missing:
        raise BuildError(f"no such kernel sources: {missing}")
    return list(names)


def _digest(files: Sequence[str], extra_flags: Sequence[str]) -> str:
    h = hashlib.sha256()
    for f in sorted(set(list(files) + [x for x in os.listdir(CSRC) if x.endswith((".cuh", ".h"))])):
        h.update(f.encode())
        with open(os.path.join(CSRC, f), "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + list(extra_flags)).encode())
    return h.hexdigest()[:16]


def _build_dir() -> str:
    d = os.path.join(CSRC, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"quicknn_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def library_path(name: str = "qnn_kernels", files: Optional[Sequence[str]] = None,
                 extra_flags: Sequence[str] = ()) -> str:
    files = sources(files)
    return os.path.join(_build_dir(), f"lib{name}_{_digest(files, extra_flags)}.so")


def build(name: str = "qnn_kernels", files: Optional[Sequence[str]] = None,
          extra_flags: Sequence[str] = (), verbose: bool = False) -> str:
    """Build (if needed) and return the path of the shared library."""
    files = sources(files)
    out = library_path(name, files, extra_flags)
    if os.path.isfile(out):
        return out
    nvcc = find_nvcc()
    bdir = os.path.dirname(out)
    tag = os.path.basename(out)[3:-3]
    _say(f"building {os.path.basename(out)} from {len(files)} CUDA sources with {nvcc} (first call only)")
    t0 = time.time()
    done = threading.Event()

    def heartbeat():
        while not done.wait(10.0):
            _say(f"  ... still compiling ({time.time() - t0:.0f} s)")

    hb = threading.Thread(target=heartbeat, daemon=True)
    hb.start()
    objs = []

    def compile_one(f: str) -> str:
        obj = os.path.join(bdir, f"{tag}_{f[:-3]}.o")
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, *extra_flags, "-I", CSRC, "-c", os.path.join(CSRC, f), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise BuildError(f"nvcc failed on {f}:\n{r.stdout}")
        if verbose and r.stdout:
            _say(r.stdout)
        _say(f"  compiled {f} ({time.time() - t0:.0f} s)")
        return obj

    try:
        workers = max(1, min(len(files), os.cpu_count() or 1, 8))
        with concurrent.futures.ThreadPoolExecutor(workers) as pool:
            objs = list(pool.map(compile_one, files))
        tmp = out + f".tmp{os.getpid()}"
        cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", tmp, *objs]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise BuildError(f"linking {out} failed:\n{r.stdout}")
        os.replace(tmp, out)
        for old in os.listdir(bdir):          # libraries of earlier sources
            if old.startswith(f"lib{name}_") and old.endswith(".so") and os.path.join(bdir, old) != out:
                try:
                    os.remove(os.path.join(bdir, old))
                except OSError:
                    pass
    finally:
        done.set()
        for o in objs:
            try:
                os.remove(o)
            except OSError:
                pass
    _say(f"built {os.path.basename(out)} in {time.time() - t0:.0f} s")
    return out


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv))
