"""The C-ABI library builds, loads on a CPU-only machine and exports every symbol the header declares."""
from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def declared_functions():
    text = (ROOT / "include" / "molt_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(molt_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for required in ("molt_nf4_dequant", "molt_nf4_lora_fwd", "molt_nf4_lora_bwd", "molt_nf4_lora_fwd_prepared",
                     "molt_nf4_lora_bwd_prepared", "molt_lora_shadow_refresh", "molt_nf4_dx", "molt_nf4_gemv",
                     "molt_swiglu_fwd", "molt_swiglu_bwd", "molt_mlp_fwd", "molt_mlp_bwd", "molt_workspace_bytes",
                     "molt_last_error", "molt_version"):
        assert required in names


def test_library_exports_every_declared_symbol(native_library):
    for name in declared_functions():
        assert hasattr(native_library, name), f"{name} is declared in the header but not exported"


def test_binding_covers_every_declared_symbol():
    from molt_b200 import _native

    assert sorted(_native.EXPORTS) == declared_functions()


def test_struct_layout_matches_header(native_library):
    from molt_b200 import _native

    # 4 pointers, 1 float, 5 int32, 2 int64, 16 floats
    assert ctypes.sizeof(_native.NF4Desc) == 4 * 8 + 4 + 5 * 4 + 2 * 8 + 16 * 4
    assert _native.NF4Desc.n.offset == 56 and _native.NF4Desc.codebook.offset == 72
    assert ctypes.sizeof(_native.LoraProj) == 40 and _native.LoraProj.shadow.offset == 32
    assert ctypes.sizeof(_native.LoraShadow) == 24
    # 2 pointers, float, int32, 2 int64, 3 pointers
    assert ctypes.sizeof(_native.LoraShadowItem) == 2 * 8 + 4 + 4 + 2 * 8 + 3 * 8 and _native.LoraShadowItem.a16.offset == 40


def test_version_and_workspace_queries_run_without_a_gpu(native_library):
    from molt_b200 import _native

    assert native_library.molt_version() >= 100
    fwd = native_library.molt_workspace_bytes(_native.OP_LORA_FWD, 512, 4864, 896, 16)
    bwd = native_library.molt_workspace_bytes(_native.OP_LORA_BWD, 512, 4864, 896, 16)
    assert fwd > 0 and bwd > fwd // 4
    assert native_library.molt_workspace_bytes(_native.OP_LORA_FWD, 512, 4864, 896, 65) == 0  # rank > 64 refused


def test_argument_errors_map_to_status_codes(native_library):
    from molt_b200 import _native

    desc = _native.NF4Desc()
    rc = native_library.molt_nf4_dequant(ctypes.byref(desc), None, 0, 0)
    assert rc == _native.E_VALUE
    assert b"NULL" in native_library.molt_last_error()
    with pytest.raises(ValueError):
        _native.check(rc)
