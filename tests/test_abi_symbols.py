"""The C-ABI library loads without a GPU and exports every symbol include/px_b200.h declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "px_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    return sorted(set(re.findall(r"PX_API\s+[\w\s\*]+?\b(px_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    from protenix_b200 import build

    build.build()
    from protenix_b200 import _lib

    return _lib.load()


def test_header_declares_entry_points():
    syms = declared_symbols()
    assert len(syms) >= 15 and "px_layer_norm_fwd" in syms and "px_triangle_attention" in syms


def test_library_exports_every_declared_symbol(lib):
    for s in declared_symbols():
        assert hasattr(lib, s), f"{s} declared in px_b200.h but not exported"


def test_binding_table_matches_header(lib):
    from protenix_b200 import _lib

    assert sorted(_lib.SIGNATURES) == declared_symbols()
    # argument counts in the binding table equal those in the header
    text = open(HEADER).read()
    for name, (_res, args) in _lib.SIGNATURES.items():
        m = re.search(r"PX_API[^;]*?\b" + name + r"\s*\(([^;]*?)\)\s*;", text, flags=re.S)
        assert m, name
        params = m.group(1).strip()
        n = 0 if params in ("", "void") else len(params.split(","))
        assert n == len(args), (name, n, len(args))


def test_host_side_queries(lib):
    assert lib.px_version() >= 100
    assert lib.px_ld(1) == 8 and lib.px_ld(128) == 128 and lib.px_ld(129) == 136
    assert lib.px_trimul_workspace_bytes(128) == 4 * 128 * 128 * 128 * 2   # a, b, x and the standardised rows, fp16
    assert lib.px_triatt_workspace_bytes(64) > 4 * 64 * 64 * 128 * 2
    assert lib.px_status_string(0) == b"ok"
    assert b"workspace" in lib.px_status_string(-4)


def test_argument_errors_are_status_codes_not_crashes(lib):
    """Bad arguments are rejected on the host before any launch (no GPU needed)."""
    assert lib.px_layer_norm_fwd(None, None, None, None, None, None, 4, 128, 1e-5, 0, None) == -1
    assert lib.px_trimul_contract(None, None, None, 128, 16, 16, None) == -1
    assert lib.px_transition(None, None, 0, None, None, None, None, None, 10, 1, 1e-5, None) == -1
    buf = ctypes.create_string_buffer(64)
    p = ctypes.addressof(buf)
    # wrong leading dimension
    assert lib.px_trimul_contract(p, p, p, 128, 20, 20, None) == -1
    # unsupported dtype
    assert lib.px_layer_norm_fwd(p, None, None, p, None, None, 1, 8, 1e-5, 7, None) == -2
    # too many heads for the pair-bias projection
    assert lib.px_pair_bias_proj(p, 0, p, None, p, p, 4, 17, 1e-5, None) == -2
    # recycling update: null tensors, unknown dtype, misaligned pointer, empty input
    assert lib.px_recycle_update(None, p, p, 0, p, p, p, 4, 1e-5, None) == -1
    assert lib.px_recycle_update(p, p, p, 9, p, p, p, 4, 1e-5, None) == -2
    assert lib.px_recycle_update(p + 2, p, p, 0, p, p, p, 4, 1e-5, None) == -1
    assert lib.px_recycle_update(p, p, p, 0, p, None, p, 0, 1e-5, None) == 0
    # workspace too small
    assert lib.px_triangle_multiplication(p, p, 0, None, p, p, p, p, p, p, p, p, p, p, p, 64, 32, 0, 1, 1e-5, None) == -4
