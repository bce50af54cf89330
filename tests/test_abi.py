"""The C-ABI library loads and exports every symbol include/qkan_b200.h declares (no compute calls)."""
import ctypes
import os
import re

from qkan_b200 import _abi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "qkan_b200.h")


def _declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
    return sorted(set(re.findall(r"\b(qk_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_what_the_binding_binds():
    assert _declared_symbols() == sorted(_abi.SYMBOLS)


def test_library_exports_every_declared_symbol():
    from qkan_b200 import build

    lib = ctypes.CDLL(build.build())
    for name in _declared_symbols():
        assert hasattr(lib, name), name


def test_descriptor_layout_and_pure_host_queries():
    lib = _abi.load()
    assert ctypes.sizeof(_abi.QkDesc) == 36
    assert lib.qk_abi_version() == _abi.QK_ABI_VERSION
    d = _abi.QkDesc(65536, 256, 256, 3, _abi.QK_F32, _abi.QK_F32, 7, 0)
    fwd = lib.qk_forward_workspace_bytes(_abi.desc_pointer(d))
    bwd = lib.qk_backward_workspace_bytes(_abi.desc_pointer(d))
    assert fwd >= 256 * 19 * 256 * 4 and fwd % 256 == 0
    assert bwd > fwd
    bad = _abi.QkDesc(4, 4, 4, 0, 0, 0, 0, 0)  # reps = 0
    assert lib.qk_forward_workspace_bytes(_abi.desc_pointer(bad)) == 0
    assert b"reps" in lib.qk_last_error()
    assert lib.qk_noalloc_max_scratch_bytes() == 8 << 20
    # grouped parameters add the per-edge gradient scratch ahead of the group reduction
    g = _abi.QkDesc(65536, 256, 256, 3, _abi.QK_F32, _abi.QK_F32, 7, 0, 3)
    extra = lib.qk_backward_workspace_bytes(_abi.desc_pointer(g)) - bwd
    assert extra == 256 * 256 * (8 + 3 + 3) * 4
    assert lib.qk_forward_workspace_bytes(_abi.desc_pointer(g)) == fwd
    neg = _abi.QkDesc(4, 4, 4, 1, 0, 0, 0, 0, -1)
    assert lib.qk_backward_workspace_bytes(_abi.desc_pointer(neg)) == 0 and b"group" in lib.qk_last_error()
    # a small batch is cut into output slices: room for the slices' grad_x shares is part of the answer
    small = _abi.QkDesc(256, 256, 256, 3, _abi.QK_F32, _abi.QK_F32, 7, 0)
    assert lib.qk_backward_workspace_bytes(_abi.desc_pointer(small)) > 2 * 256 * 256 * 4


def test_source_tree_never_routes_the_product_through_the_oracle():
    pkg = os.path.join(ROOT, "qkan_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower() or f == "build.py", f
