"""In-tree build of the sm_100a kernel library (``qkan_b200/lib/libqkan_b200.so``).

``python -m qkan_b200.build`` compiles every ``csrc/*.cu`` with nvcc for
``sm_100a`` only and links one shared library that exports the C ABI declared in
``include/qkan_b200.h``. nvcc cross-compiles, so no GPU is needed to build.
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "lib", "obj")
LIB = os.path.join(PKG, "lib", "libqkan_b200.so")
INCLUDE = os.path.join(os.path.dirname(PKG), "include")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC or put it on PATH)")


def _sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _deps():
    return _sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(INCLUDE, "*.h"))


def is_stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(p) > t for p in _deps())


# per-repetition template instantiations (csrc/*_inst.cu): 0 is the "real" ansatz, 12 and 16 serve 9..16 by padding
REPS_COMPILED = (0, 1, 2, 3, 4, 5, 6, 7, 8, 12, 16)


def _jobs():
    """(source, object stem, extra defines): *_inst.cu units are compiled once per repetition count."""
    jobs = []
    for src in _sources():
        stem = os.path.basename(src)[:-3]
        if stem.endswith("_inst"):
            jobs += [(src, f"{stem}_r{r}", [f"-DQK_INST_R={r}"]) for r in REPS_COMPILED]
        else:
            jobs.append((src, stem, []))
    return jobs


def _compile(job, extra, force: bool = False) -> str:
    src, stem, defs = job
    obj = os.path.join(OBJ, stem + ".o")
    if not force and not extra and os.path.exists(obj):  # object newer than its source and every header: keep it
        headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(INCLUDE, "*.h"))
        if os.path.getmtime(obj) > max(os.path.getmtime(p) for p in [src, __file__, *headers]):
            return obj
    cmd = [_nvcc(), *NVCC_FLAGS, *defs, *extra, "-c", src, "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    log = os.path.join(OBJ, stem + ".ptxas.log")
    with open(log, "w") as fh:
        fh.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stderr[-4000:]}")
    return obj


def build(force: bool = False, extra_flags=()) -> str:
    """Compile and link the library if it is missing or older than its sources; return its path."""
    if not force and not is_stale():
        return LIB
    os.makedirs(OBJ, exist_ok=True)
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(lambda j: _compile(j, list(extra_flags), force), _jobs()))
    res = subprocess.run([_nvcc(), "-shared", "-o", LIB, *objs, "-gencode",
                          "arch=compute_100a,code=sm_100a"], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stderr[-4000:]}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
