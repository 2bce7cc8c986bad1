"""Compiles the CUDA sources beside this file into one shared library for sm_100a.

The library's file name carries a hash of the sources and flags, so a stale build is
never loaded. It is written to `_build/` beside the sources; when that folder cannot be
written (a read-only checkout) it goes to a per-user folder under the system's temporary
directory. Each source is compiled by its own nvcc process, a few at a time, and a
progress line goes to stderr every few seconds while they run. No header of PyTorch is
used: the exported functions take raw pointers, so a source compiles in seconds.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from typing import List, Optional

HERE = os.path.dirname(os.path.abspath(__file__))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
              "--expt-relaxed-constexpr"]
LIB_STEM = "libxs_b200"


class BuildError(RuntimeError):
    pass


def sources() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))


def find_nvcc() -> str:
    for cand in (os.environ.get("XS_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (PATH, CUDA_HOME, /usr/local/cuda); the CUDA kernels cannot be compiled")


def source_hash() -> str:
    h = hashlib.sha256()
    for name in sources() + _headers():
        h.update(name.encode())
        with open(os.path.join(HERE, name), "rb") as f:
            h.update(f.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _writable_dir() -> str:
    local = os.path.join(HERE, "_build")
    try:
        os.makedirs(local, exist_ok=True)
        probe = os.path.join(local, f".probe_{os.getpid()}")
        with open(probe, "w") as f:
            f.write("")
        os.remove(probe)
        return local
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"xpu_serve_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def library_path(create_dir: bool = True) -> str:
    name = f"{LIB_STEM}_{source_hash()}.so"
    local = os.path.join(HERE, "_build", name)
    if os.path.isfile(local):
        return local
    return os.path.join(_writable_dir() if create_dir else os.path.join(HERE, "_build"), name)


def _say(msg: str, verbose: bool) -> None:
    if verbose:
        print(f"[xpu_serve_b200 build] {msg}", file=sys.stderr, flush=True)


def build(verbose: bool = True, force: bool = False, jobs: Optional[int] = None) -> str:
    """Returns the path of the up-to-date library, compiling it first when needed."""
    out = library_path()
    if os.path.isfile(out) and not force:
        return out
    nvcc = find_nvcc()
    out_dir = os.path.dirname(out)
    obj_dir = os.path.join(out_dir, f"obj_{source_hash()}_{os.getpid()}")
    os.makedirs(obj_dir, exist_ok=True)
    srcs = sources()
    jobs = jobs or max(1, min(len(srcs), os.cpu_count() or 1, 8))
    _say(f"compiling {len(srcs)} CUDA sources for sm_100a with {os.path.basename(nvcc)} ({jobs} at a time)", verbose)
    t0 = time.time()
    pending = list(srcs)
    running = {}
    objects = []
    last_line = time.time()
    try:
        while pending or running:
            while pending and len(running) < jobs:
                src = pending.pop(0)
                obj = os.path.join(obj_dir, src[:-3] + ".o")
                cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", HERE, "-c", os.path.join(HERE, src), "-o", obj]
                running[src] = (subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True), obj)
            for src in list(running):
                proc, obj = running[src]
                if proc.poll() is None:
                    continue
                log = proc.stdout.read()
                del running[src]
                if proc.returncode != 0:
                    raise BuildError(f"nvcc failed on {src}:\n{log}")
                objects.append(obj)
                _say(f"compiled {src} ({time.time() - t0:.0f} s)", verbose)
                last_line = time.time()
            if running:
                time.sleep(0.2)
                if time.time() - last_line > 5:
                    _say(f"still compiling {', '.join(sorted(running))} ({time.time() - t0:.0f} s)", verbose)
                    last_line = time.time()
        tmp = out + f".tmp{os.getpid()}"
        link = [nvcc, *ARCH_FLAGS, "-shared", "-o", tmp, *sorted(objects), "-lcudart"]
        r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise BuildError(f"linking failed:\n{r.stdout}")
        os.replace(tmp, out)
        for old in os.listdir(out_dir):     # libraries of earlier source versions
            if old.startswith(LIB_STEM + "_") and old.endswith(".so") and os.path.join(out_dir, old) != out:
                try:
                    os.remove(os.path.join(out_dir, old))
                except OSError:
                    pass
    finally:
        for proc, _ in running.values():
            proc.kill()
        shutil.rmtree(obj_dir, ignore_errors=True)
    _say(f"built {out} in {time.time() - t0:.0f} s", verbose)
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
