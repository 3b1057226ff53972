"""The C-ABI library loads on a machine without a GPU and exports every symbol the header declares."""

import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "ck_b200.h")).read()
    return sorted(set(re.findall(r"CK_API\s+[\w\s\*]+?\b(ck_\w+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    syms = _declared_symbols()
    for must in ("ck_continuous_count", "ck_route", "ck_swiglu_fwd", "ck_swiglu_bwd", "ck_moe_up_act_fwd",
                 "ck_moe_down_combine_fwd", "ck_moe_dgrad_down", "ck_moe_dgrad_up", "ck_moe_wgrad"):
        assert must in syms


def test_library_exports_every_declared_symbol():
    from cute_kernels import _lib

    lib = ctypes.CDLL(_lib.LIB_PATH)
    for s in _declared_symbols():
        assert hasattr(lib, s), f"{s} declared in include/ck_b200.h but not exported"
        assert s in _lib.PROTOTYPES, f"{s} has no ctypes prototype"
    assert set(_lib.PROTOTYPES) == set(_declared_symbols())


def test_host_only_entry_points():
    from cute_kernels import _lib

    assert _lib.lib.ck_abi_version() >= 1
    assert _lib.lib.ck_status_string(0) == b"CK_OK"
    assert _lib.lib.ck_status_string(-1) == b"CK_ERR_SHAPE"
    assert _lib.lib.ck_route_padded_capacity(1000, 8) == (1000 // 128 + 8) * 128
    assert _lib.lib.ck_route_workspace_bytes(1 << 20, 64) > 0
    assert _lib.lib.ck_route_workspace_bytes(10, 5000) < 0  # too many experts


def test_argument_validation_needs_no_gpu():
    """Shape errors are decided on the host before any CUDA call."""
    from cute_kernels import _lib

    assert _lib.lib.ck_continuous_count(None, 0, 10, CK := 20000, None, None) != 0  # noqa: F841
    assert _lib.lib.ck_swiglu_fwd(None, None, None, 1, 8, 4, 8, 2, None) == -1  # stride < cols
    assert _lib.lib.ck_moe_wgrad(None, None, None, None, 8, 1024, 64, 64, 2, None, None) == -1
