"""The shared library loads on a machine without a GPU and exports every symbol the header declares."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    from torchgt_b200 import _cabi
    from torchgt_b200.build import build
    build()
    return _cabi.load()


def _declared_symbols():
    text = (ROOT / "include" / "torchgt_b200.h").read_text()
    return sorted(set(re.findall(r"TGT_API\s+[\w\s\*]+?\b(tgt_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(lib):
    from torchgt_b200 import _cabi
    declared = _declared_symbols()
    assert len(declared) >= 15
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert sorted(_cabi.SIGNATURES) == declared, "ctypes prototypes and header declarations differ"


def test_version_and_error_string(lib):
    assert lib.tgt_version() >= 100
    assert isinstance(lib.tgt_last_error(), bytes)


def test_argument_checks_run_before_any_cuda_call(lib):
    """These calls are rejected on their arguments alone, so they work without a device."""
    from torchgt_b200 import _cabi
    n = ctypes.c_size_t()
    assert lib.tgt_edge_layout_sizes(-1, 0, ctypes.byref(n)) == 1
    assert b"n_rows" in lib.tgt_last_error()
    assert lib.tgt_edge_layout_sizes(2**31, 0, ctypes.byref(n)) == 1
    assert lib.tgt_edge_layout_sizes(4, 4, None) == 1
    assert lib.tgt_edge_layout_build(None, 5, 0, 1, None, None, None, None, None, 0, None, None) == 1
    assert lib.tgt_edge_layout_build(None, 5, 10, 3, None, None, None, None, None, 0, None, None) == 1
    assert lib.tgt_debug_set_tile_edges(-1) == 1
    assert lib.tgt_debug_set_tile_edges(0) == 0
    layout = _cabi.TgtLayout(n_rows=4, n_edges=0, ptr=None, other=None, perm=None, seg=None)
    # dtype 9 is unknown; a layout with rows but no ptr is invalid; 3 heads of 12 are not supported
    assert lib.tgt_sparse_attn_fwd(None, None, None, None, 0, ctypes.byref(layout), None, None, 8, 8, 9, None, 0, None) == 1
    assert lib.tgt_sparse_attn_fwd(None, None, None, None, 0, ctypes.byref(layout), None, None, 8, 8, 0, None, 0, None) == 1
    assert b"ptr" in lib.tgt_last_error()
    layout.ptr = 256
    assert lib.tgt_sparse_attn_fwd(None, None, None, None, 0, ctypes.byref(layout), None, None, 3, 12, 0, None, 0, None) == 3
    assert lib.tgt_sparse_attn_fwd(None, None, None, None, 2, ctypes.byref(layout), None, None, 8, 8, 0, None, 0, None) == 1
    assert lib.tgt_sparse_attn_fwd(None, None, None, None, 0, None, None, None, 8, 8, 0, None, 0, None) == 1
    assert lib.tgt_sparse_attn_bwd_passes(None, None, None, None, None, 0, None, None, ctypes.byref(layout),
                                          ctypes.byref(layout), None, None, None, None, 8, 8, 0, None, 0, None, 0) == 1
    assert b"passes" in lib.tgt_last_error()
    assert lib.tgt_global_rows_broadcast(None, None, 2, 1, 8, 8, 5, None) == 1
    assert lib.tgt_a2a_pack_heads(None, None, None, 0, None, 1, 1, 1, 1, 0, None) == 1


def test_check_raises_with_the_library_message(lib):
    from torchgt_b200 import _cabi
    with pytest.raises(_cabi.TgtError, match="TGT_ERR_INVALID"):
        _cabi.check(lib.tgt_debug_set_tile_edges(-5))
