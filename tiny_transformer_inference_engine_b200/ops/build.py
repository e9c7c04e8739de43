"""Builds the sm_100a kernel library in-tree with nvcc.

``csrc/*.cu`` are compiled one by one (in parallel) into ``csrc/_build/*.o`` and linked into
``ops/_ttie_b200.so``; a hash of the sources and flags beside the library tells whether it
is current.  The first use in a fresh checkout compiles what the model needs and prints a
line now and then meanwhile.  Nothing here needs a GPU: nvcc cross-compiles.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor, as_completed

PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(PKG, "csrc")
LIB_NAME = "_ttie_b200.so"

NVCC_FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v"] + os.environ.get("TTIE_NVCC_EXTRA", "").split()


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise RuntimeError("nvcc not found (looked at $NVCC, PATH and /usr/local/cuda/bin): the sm_100a kernel "
                       "library cannot be built, and this package has no other way to compute")


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers():
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def source_hash() -> str:
    h = hashlib.sha256()
    for name in sources() + _headers():
        h.update(name.encode())
        with open(os.path.join(CSRC, name), "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _writable_dir(preferred: str) -> str:
    try:
        os.makedirs(preferred, exist_ok=True)
        probe = os.path.join(preferred, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return preferred
    except OSError:
        d = os.environ.get("TTIE_BUILD_DIR") or os.path.join(tempfile.gettempdir(), f"ttie_b200_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def lib_path() -> str:
    """Where a current library is, or where it would be built."""
    here = os.path.join(PKG, "ops", LIB_NAME)
    if os.path.isfile(here):
        return here
    alt = os.path.join(os.environ.get("TTIE_BUILD_DIR") or os.path.join(tempfile.gettempdir(), f"ttie_b200_{os.getuid()}"), LIB_NAME)
    return alt if os.path.isfile(alt) else here


def is_current(path: str) -> bool:
    try:
        with open(path + ".hash") as f:
            return f.read().strip() == source_hash() and os.path.isfile(path)
    except OSError:
        return False


def build(verbose: bool = True, force: bool = False) -> str:
    """Compiles every kernel for sm_100a and returns the library's path."""
    path = lib_path()
    if not force and is_current(path):
        return path
    nvcc = _nvcc()
    out_dir = _writable_dir(os.path.join(PKG, "ops"))
    obj_dir = _writable_dir(os.path.join(CSRC, "_build"))
    path = os.path.join(out_dir, LIB_NAME)
    t0 = time.time()
    log = (lambda *a: print("[ttie_b200 build]", *a, file=sys.stderr, flush=True)) if verbose else (lambda *a: None)
    srcs = sources()
    log(f"compiling {len(srcs)} CUDA sources for sm_100a with {nvcc} (first use; takes a minute or two)")

    def compile_one(name):
        obj = os.path.join(obj_dir, name[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", CSRC, "-c", os.path.join(CSRC, name), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {name}:\n{r.stdout}\n{r.stderr}")
        with open(obj + ".ptxas.txt", "w") as f:
            f.write(r.stderr)
        return name, obj

    objs = []
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        futs = [pool.submit(compile_one, s) for s in srcs]
        for fut in as_completed(futs):
            name, obj = fut.result()
            objs.append(obj)
            log(f"  {name} done ({len(objs)}/{len(srcs)}, {time.time() - t0:.0f}s)")
    tmp = path + f".tmp{os.getpid()}"
    r = subprocess.run([nvcc, "-shared", "-o", tmp, *sorted(objs), "-gencode", "arch=compute_100a,code=sm_100a"],
                       capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, path)
    with open(path + ".hash", "w") as f:
        f.write(source_hash())
    log(f"built {path} in {time.time() - t0:.0f}s")
    return path


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
