#!/usr/bin/env python3
"""Puts an unmodified copy of the reference under ``baseline/_ref`` and builds its CUDA extensions.

    python baseline/build_reference.py --source DIR [--only NAME ...]

The reference is a flat script tree without a root ``setup.py`` or ``pyproject.toml``, so pip cannot
install it.  Each of its kernels has a ``setup.py`` of its own (kernels/pagedattn/setup.py,
kernels/rmsnorm_kernel/setup.py, kernels/rope_kernel/setup.py, kernels/flashattn/setup.py,
kernels/softmax_kernel/setup.py, kernels/cuda-kSAMPLING/setup.py); this script runs each of them
with ``build_ext --inplace`` in the copy, with ``TORCH_CUDA_ARCH_LIST=10.0`` in the environment so
that torch's extension builder targets sm_100.  ``kernels/pagedattn/setup.py`` names its own targets
(sm_80 and sm_90 machine code, no PTX), and torch adds none when a file does that, so for that one the
sm_100 target is handed to nvcc through its ``NVCC_APPEND_FLAGS`` environment variable.
No file of the reference is edited.  nvcc cross-compiles, so no GPU is needed.

``bench.py --impl reference`` imports the copy from ``baseline/_ref`` and reports ``unavailable``
if an extension is missing.
"""
import argparse
import glob
import os
import shutil
import subprocess
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
OWN_TARGETS = {"pagedattn"}      # folders whose setup.py fixes the nvcc targets itself
KERNELS = {                      # folder under kernels/ -> module it builds
    "rmsnorm_kernel": "rmsnorm_cuda",
    "rope_kernel": "rope_cuda",
    "softmax_kernel": "softmax_cuda",
    "cuda-kSAMPLING": "topk_cuda",
    "flashattn": "flash_acc_reg_ext",
    "pagedattn": "pagedattn",
}


def built(module: str, folder: str):
    tag = f"cpython-{sys.version_info.major}{sys.version_info.minor}"
    hits = glob.glob(os.path.join(DEST, "kernels", folder, f"{module}.{tag}-*.so"))
    return hits[0] if hits else None


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--source", default=os.environ.get("REFERENCE_DIR", ""), help="the reference's checkout (needed once, to make the copy)")
    ap.add_argument("--only", nargs="*", default=None)
    args = ap.parse_args()
    if not os.path.isdir(os.path.join(DEST, "kernels")):
        if not args.source or not os.path.isdir(args.source):
            print(f"no reference tree at {args.source!r}: give --source DIR", file=sys.stderr)
            return 1
        shutil.copytree(args.source, DEST, dirs_exist_ok=True)
    env = dict(os.environ, TORCH_CUDA_ARCH_LIST="10.0", MAX_JOBS=os.environ.get("MAX_JOBS", "4"))
    failed = []
    for folder, module in KERNELS.items():
        if args.only and folder not in args.only and module not in args.only:
            continue
        if built(module, folder):
            print(f"{module}: already built", flush=True)
            continue
        t0 = time.time()
        print(f"{module}: building in kernels/{folder} ...", flush=True)
        log = os.path.join(DEST, "kernels", folder, "build_sm100.log")
        with open(log, "w") as f:
            kenv = dict(env, NVCC_APPEND_FLAGS="-gencode=arch=compute_100,code=sm_100") if folder in OWN_TARGETS else env
            rc = subprocess.call([sys.executable, "setup.py", "build_ext", "--inplace"], cwd=os.path.join(DEST, "kernels", folder),
                                 env=kenv, stdout=f, stderr=subprocess.STDOUT)
        ok = rc == 0 and built(module, folder)
        print(f"{module}: {'ok' if ok else 'FAILED (see ' + log + ')'} after {time.time() - t0:.0f} s", flush=True)
        if not ok:
            failed.append(module)
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
