"""Build recipe for the CPU oracle (test infrastructure, never the product).

Compiles ``qkan_oracle.c`` twice (double and float symbol sets) into
``oracle/_build/libqkan_oracle.so``. The reference is a pure-Python package, so
there is nothing to compile into ``oracle/_ref``; the oracle's pin is the set of
reference outputs under ``tests/golden/``.

Run as ``python oracle/build_oracle.py``.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_build")
LIB = os.path.join(OUT, "libqkan_oracle.so")
SRC = os.path.join(HERE, "qkan_oracle.c")

# -ffp-contract=off: the oracle's rounding must not depend on FMA fusion.
CFLAGS = ["-O2", "-fPIC", "-fopenmp", "-fno-fast-math", "-ffp-contract=off", "-Wall", "-Wextra"]


def _compilers():
    seen = []
    for cand in ("/usr/bin/gcc", shutil.which("gcc"), os.environ.get("CC"), shutil.which("cc")):
        if cand and os.path.exists(cand) and cand not in seen:
            seen.append(cand)
    return seen


def build(force: bool = False) -> str:
    """Compile the oracle library if it is missing or older than its source; return its path."""
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    os.makedirs(OUT, exist_ok=True)
    errors = []
    for cc in _compilers():
        try:
            objs = []
            for tag, defs in (("f64", ["-DORACLE_F64"]), ("f32", [])):
                obj = os.path.join(OUT, f"qkan_oracle_{tag}.o")
                subprocess.run([cc, *CFLAGS, *defs, "-c", SRC, "-o", obj], check=True,
                               capture_output=True, text=True)
                objs.append(obj)
            subprocess.run([cc, "-shared", "-fopenmp", "-o", LIB, *objs, "-lm"], check=True,
                           capture_output=True, text=True)
            return LIB
        except subprocess.CalledProcessError as exc:  # try the next compiler
            errors.append(f"{cc}: {exc.stderr.strip()[-400:]}")
    raise RuntimeError("could not build the oracle library:\n" + "\n".join(errors))


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
