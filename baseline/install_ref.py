"""Install the UNMODIFIED reference package into ``baseline/_ref`` (untracked) for the baseline arms of bench.py.

    python baseline/install_ref.py [--src /path/to/reference/checkout] [--no-cuda]

What it does, and nothing else:

* copies the reference checkout to a scratch folder (its build writes into the source tree),
* runs ``pip install --no-index --no-build-isolation --no-deps --target baseline/_ref <copy>`` with the
  reference's own build switches (``setup.py``: ``QKAN_FORCE_BUILD``, ``QKAN_CUDA_ARCHS``, ``CUTLASS_PATH``)
  so that its CUDA extension ``qkan._C`` (``src/qkan/csrc/cute_kernels.cu`` and friends) is compiled HERE for
  sm_100 by nvcc's cross compilation, where no GPU time is metered. CUTLASS/CuTe headers come from the copy
  bundled with the ``flashinfer`` wheel of this image.

Nothing of the reference is copied into tracked files: ``baseline/_ref`` is git-ignored and travels with the
working tree like the repository's own built ``.so``. bench.py imports it only in its baseline legs
(``--impl reference`` and the ``baselines`` key), never on the product path.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
TARGET = os.path.join(HERE, "_ref")


def cutlass_root() -> str | None:
    """A CUTLASS tree (containing include/cute/tensor.hpp) bundled with a wheel of this image."""
    import importlib.util

    for pkg, rel in (("flashinfer", "data/cutlass"), ("tilelang", "3rdparty/cutlass")):
        spec = importlib.util.find_spec(pkg)
        if spec is None or not spec.submodule_search_locations:
            continue
        root = os.path.join(list(spec.submodule_search_locations)[0], rel)
        if os.path.isfile(os.path.join(root, "include", "cute", "tensor.hpp")):
            return root
    return None


def install(src: str, with_cuda: bool = True) -> int:
    if not os.path.isdir(os.path.join(src, "src", "qkan")):
        print(f"install_ref: {src} is not a reference checkout", file=sys.stderr)
        return 2
    work = tempfile.mkdtemp(prefix="qkan_ref_build_")
    copy = os.path.join(work, "reference")
    shutil.copytree(src, copy, ignore=shutil.ignore_patterns(".git", "docs", "datasets", "__pycache__"))
    env = dict(os.environ)
    env.update(QKAN_NO_GIT_VERSION="TRUE", QKAN_NO_CUTLASS_DOWNLOAD="1")
    cut = cutlass_root() if with_cuda else None
    if with_cuda and cut:
        env.update(QKAN_FORCE_BUILD="TRUE", QKAN_CUDA_ARCHS="100", CUTLASS_PATH=cut,
                   MAX_JOBS=str(os.cpu_count() or 4), NVCC_THREADS="4",
                   TORCH_CUDA_ARCH_LIST="10.0")
    else:
        env.update(QKAN_SKIP_CUDA_BUILD="TRUE")
    if os.path.isdir(TARGET):
        shutil.rmtree(TARGET)
    cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
           "--find-links", "/opt/wheelhouse", "--target", TARGET, copy]
    print("install_ref:", " ".join(cmd), flush=True)
    rc = subprocess.call(cmd, env=env)
    shutil.rmtree(work, ignore_errors=True)
    if rc == 0:
        built = [f for f in os.listdir(os.path.join(TARGET, "qkan")) if f.startswith("_C")]
        print(f"install_ref: installed into {TARGET}; CUDA extension: {built or 'not built'}")
    return rc


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--src", default=os.environ.get("QKAN_REFERENCE_ROOT", "/root/reference"))
    ap.add_argument("--no-cuda", action="store_true", help="pure-Python install (exact and flash arms only)")
    a = ap.parse_args()
    sys.exit(install(a.src, with_cuda=not a.no_cuda))
