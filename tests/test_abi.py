"""CPU tests of the C-ABI boundary: the header parses into ctypes structs whose sizes match the
library, every declared symbol is exported, and host-side argument validation returns error
codes (never a launch) -- none of this needs a GPU."""
import ctypes

import pytest

from quamba_b200 import _lib


def test_header_declares_expected_entry_points():
    want = {"qb_last_error", "qb_abi_version", "qb_sizeof", "qb_read_device_status", "qb_causal_conv1d_fwd",
            "qb_causal_conv1d_update", "qb_quamba2_conv1d_fwd", "qb_quamba2_conv1d_update", "qb_hadamard_quant",
            "qb_sscan_fwd", "qb_sscan_update", "qb_ssd_workspace_bytes", "qb_ssd_chunk_scan_fwd", "qb_w4a8_unpack",
            "qb_w4a8_gemm", "qb_w8a8_gemm"}
    assert want <= set(_lib.FUNCTIONS)


def test_library_loads_and_exports_every_declared_symbol():
    lib = _lib.lib()
    for fn in _lib.FUNCTIONS:
        assert hasattr(lib, fn), fn
    assert lib.qb_abi_version() >= 1


def test_struct_sizes_match():
    lib = _lib.lib()
    for name, st in _lib.STRUCTS.items():
        assert lib.qb_sizeof(name.encode()) == ctypes.sizeof(st), name
    assert lib.qb_sizeof(b"nonsense") == -1


def test_workspace_size_formula():
    lib = _lib.lib()
    assert lib.qb_ssd_workspace_bytes(0, 1, 1, 1, 1, 1, 1) == -1
    small = lib.qb_ssd_workspace_bytes(1, 256, 8, 64, 1, 128, 256)
    big = lib.qb_ssd_workspace_bytes(4, 2048, 80, 64, 1, 128, 256)
    assert 0 < small < big and big % 256 == 0


@pytest.mark.parametrize("fn,struct", [
    ("qb_causal_conv1d_fwd", "qb_conv1d_fwd_args"), ("qb_causal_conv1d_update", "qb_conv1d_update_args"),
    ("qb_quamba2_conv1d_fwd", "qb_quamba2_conv1d_fwd_args"), ("qb_quamba2_conv1d_update", "qb_quamba2_conv1d_update_args"),
    ("qb_hadamard_quant", "qb_hadamard_quant_args"), ("qb_sscan_fwd", "qb_sscan_fwd_args"),
    ("qb_sscan_update", "qb_sscan_update_args"), ("qb_ssd_chunk_scan_fwd", "qb_ssd_args"),
    ("qb_w4a8_unpack", "qb_w4a8_unpack_args"), ("qb_w4a8_gemm", "qb_w4a8_gemm_args"), ("qb_w4a8_gemv_s4", "qb_w4a8_gemv_s4_args"), ("qb_w8a8_gemm", "qb_w8a8_gemm_args")])
def test_null_arguments_are_rejected_on_the_host(fn, struct):
    lib = _lib.lib()
    args = _lib.make(struct)  # all pointers null, all sizes zero
    rc = getattr(lib, fn)(ctypes.byref(args), None)
    assert rc == _lib.QB_ERR_INVALID_ARG
    assert len(lib.qb_last_error()) > 0
    with pytest.raises(RuntimeError):
        _lib.check(rc)


def test_reference_error_wording_for_conv_width():
    lib = _lib.lib()
    one = ctypes.c_char(0)
    p = ctypes.cast(ctypes.pointer(one), ctypes.c_void_p)
    args = _lib.make("qb_conv1d_fwd_args", x=p, out=p, weight=p, batch=1, dim=16, seqlen=4, width=5, x_sl=1, x_sd=4, out_sl=1)
    assert lib.qb_causal_conv1d_fwd(ctypes.byref(args), None) == _lib.QB_ERR_INVALID_ARG
    assert b"width between 2 and 4" in lib.qb_last_error()
    h = _lib.make("qb_hadamard_quant_args", x=p, out=p, rows=1, dim=5120, special=12, in_dtype=0, scale=1.0)
    assert lib.qb_hadamard_quant(ctypes.byref(h), None) == _lib.QB_ERR_INVALID_ARG
    h = _lib.make("qb_hadamard_quant_args", x=p, out=p, rows=1, dim=96, special=12, in_dtype=7, scale=1.0)
    assert lib.qb_hadamard_quant(ctypes.byref(h), None) == _lib.QB_ERR_INVALID_ARG
