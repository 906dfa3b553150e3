"""The C-ABI library loads and exports every entry point include/sfnx_b200.h declares (no compute without a GPU)."""
import os
import re


def test_library_exports_every_declared_symbol(fnx):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    header = open(os.path.join(root, "include", "sfnx_b200.h")).read()
    declared = set(re.findall(r"\b(fnx_[a-z0-9_]+)\s*\(", header))
    assert declared == set(fnx.declared_symbols())
    lib = fnx.load()
    for name in declared:
        assert getattr(lib, name) is not None
    assert lib.fnx_built_arch() == 100


def test_sizes_and_host_helpers(fnx):
    lib = fnx.load()
    assert lib.fnx_kv_rows_per_card(32768, 1) == 32768 and lib.fnx_kv_rows_per_card(32768, 8) == 4096
    assert lib.fnx_kv_rows_per_card(10, 4) == 4
    assert lib.fnx_gdn_scratch_floats(48) == 16 * 3 * 48 * 128 + 16 * 48 * 2
    assert lib.fnx_moe_h_bytes(160, 768) == 160 * 768 + 160 * 24 * 4


def test_refused_arguments_report_text(fnx):
    import pytest

    with pytest.raises(fnx.FnxError, match="multiple of 32"):
        fnx.call("fnx_quantize_q8_1", None, None, 100, 1, None)
    with pytest.raises(fnx.FnxError, match="outside 1..16"):
        fnx.call("fnx_gemv_f32", None, None, None, 4, 512, 17, None)
