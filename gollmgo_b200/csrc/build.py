"""Builds the CUDA library of this package for sm_100a with nvcc, in the tree.

Sources are the ``*.cu`` files beside this file.  The shared object is named after
a hash of the sources and flags, so a stale build is never loaded.  It is built
at first use (a fresh checkout has no built files) and progress is printed to
stderr now and then, since the first build takes a minute.
"""
from __future__ import annotations

import glob
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor

_HERE = os.path.dirname(os.path.abspath(__file__))
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]


class BuildError(RuntimeError):
    pass


def sources():
    return sorted(glob.glob(os.path.join(_HERE, "*.cu")))


def _digest() -> str:
    h = hashlib.sha256()
    for path in sources() + sorted(glob.glob(os.path.join(_HERE, "*.cuh"))) \
            + sorted(glob.glob(os.path.join(_HERE, "*.h"))):
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise BuildError("nvcc not found: this package compiles its CUDA kernels at first use "
                     "(set NVCC or put nvcc on PATH)")


def _build_dir() -> str:
    cands = [os.environ.get("GOLLMGO_B200_BUILD_DIR"), os.path.join(_HERE, "_build")]
    for d in cands:
        if not d:
            continue
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".w{os.getpid()}")
            open(probe, "w").close()
            os.remove(probe)
            return d
        except OSError:
            continue
    return tempfile.mkdtemp(prefix="gollmgo_b200_build_")


def _log(msg: str, verbose: bool) -> None:
    if verbose:
        print(f"[gollmgo_b200] {msg}", file=sys.stderr, flush=True)


def library_path() -> str:
    """Path the library has (or will have) for the current sources."""
    return os.path.join(_build_dir(), f"libgollmgo_b200_{_digest()}.so")


def ensure_built(verbose: bool = True) -> str:
    """Compile if needed; return the path of the shared object."""
    build_dir = _build_dir()
    so = os.path.join(build_dir, f"libgollmgo_b200_{_digest()}.so")
    if os.path.exists(so):
        return so
    nvcc = _nvcc()
    srcs = sources()
    obj_dir = os.path.join(build_dir, f"obj_{_digest()}_{os.getpid()}")
    os.makedirs(obj_dir, exist_ok=True)
    _log(f"compiling {len(srcs)} CUDA files for sm_100a into {build_dir} (first use only)", verbose)
    t0 = time.time()

    def compile_one(src):
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
        p = subprocess.run([nvcc, *NVCC_FLAGS, "-I", _HERE, "-c", src, "-o", obj],
                           capture_output=True, text=True)
        if p.returncode != 0:
            raise BuildError(f"nvcc failed on {os.path.basename(src)}:\n{p.stdout}\n{p.stderr}")
        return obj

    objs = []
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        futs = [pool.submit(compile_one, s) for s in srcs]
        pending = list(zip(srcs, futs))
        last = time.time()
        while pending:
            still = []
            for s, f in pending:
                if f.done():
                    objs.append(f.result())
                    _log(f"  compiled {os.path.basename(s)} ({len(objs)}/{len(srcs)}, "
                         f"{time.time() - t0:.0f} s)", verbose)
                else:
                    still.append((s, f))
            pending = still
            if pending:
                time.sleep(0.2)
                if time.time() - last > 10:
                    _log(f"  still compiling {len(pending)} files ({time.time() - t0:.0f} s)", verbose)
                    last = time.time()
    tmp_so = so + f".tmp{os.getpid()}"
    p = subprocess.run([nvcc, "-shared", "-o", tmp_so, *sorted(objs), "-lcuda"],
                       capture_output=True, text=True)
    if p.returncode != 0:
        raise BuildError(f"link failed:\n{p.stdout}\n{p.stderr}")
    os.replace(tmp_so, so)
    for old in glob.glob(os.path.join(build_dir, "libgollmgo_b200_*.so")):
        if old != so:                      # builds of older sources
            try:
                os.remove(old)
            except OSError:
                pass
    shutil.rmtree(obj_dir, ignore_errors=True)
    _log(f"built {os.path.basename(so)} in {time.time() - t0:.0f} s", verbose)
    return so


if __name__ == "__main__":
    print(ensure_built())
