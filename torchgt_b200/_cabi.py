"""ctypes binding of ``libtorchgt_b200.so`` (the C ABI declared in ``include/torchgt_b200.h``).

There is no CPU fallback: if the library is missing or a call fails this module raises.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_float, c_int, c_int64, c_size_t, c_uint32, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libtorchgt_b200.so"

TGT_OK = 0
TGT_ERR_INDEX_RANGE = 5
TGT_F32 = 0
TGT_BF16 = 1
TGT_PUSH_FINAL, TGT_PUSH_STAGED, TGT_PUSH_WOVEN = 0, 1, 2

ERROR_NAMES = {
    1: "TGT_ERR_INVALID",
    2: "TGT_ERR_CUDA",
    3: "TGT_ERR_UNSUPPORTED",
    4: "TGT_ERR_WORKSPACE",
    5: "TGT_ERR_INDEX_RANGE",
}


class TgtError(RuntimeError):
    """A C-ABI call returned a non-zero code."""

    def __init__(self, code: int, message: str):
        super().__init__(f"{ERROR_NAMES.get(code, code)}: {message}")
        self.code = code


class TgtLayout(ctypes.Structure):
    """Mirror of ``struct tgt_layout``."""

    _fields_ = [
        ("n_rows", c_int64),
        ("n_edges", c_int64),
        ("ptr", c_void_p),
        ("other", c_void_p),
        ("perm", c_void_p),
        ("seg", c_void_p),
    ]


_PL = POINTER(TgtLayout)

# name -> (restype, argtypes); every symbol the header declares
SIGNATURES = {
    "tgt_version": (c_int, []),
    "tgt_last_error": (c_char_p, []),
    "tgt_debug_set_tile_edges": (c_int, [c_int]),
    "tgt_edge_layout_sizes": (c_int, [c_int64, c_int64, POINTER(c_size_t)]),
    "tgt_edge_layout_build": (c_int, [c_void_p, c_int64, c_int64, c_int, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]),
    "tgt_edge_layout_build_i32": (c_int, [c_void_p, c_int64, c_int64, c_int, c_void_p, c_void_p, c_void_p,
                                          c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]),
    "tgt_edge_prepare": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int, c_int64, c_int64,
                                 c_void_p, c_int64, c_void_p]),
    "tgt_sparse_attn_scratch_bytes": (c_int, [_PL, _PL, c_int, c_int, c_int, c_int, POINTER(c_size_t)]),
    "tgt_sparse_attn_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, _PL, c_void_p,
                                    c_void_p, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "tgt_sparse_attn_fwd_strided": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_int, _PL,
                                            c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "tgt_sparse_attn_bwd_strided": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int64,
                                            c_void_p, c_int, c_void_p, c_void_p, _PL, _PL, c_void_p, c_void_p,
                                            c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p,
                                            c_int]),
    "tgt_debug_set_lane_mode": (c_int, [c_int]),
    "tgt_debug_set_dependent_launch": (c_int, [c_int]),
    "tgt_sparse_attn_fwd_noalloc": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, _PL, c_void_p,
                                            c_void_p, c_int, c_int, c_int, c_void_p]),
    "tgt_sparse_attn_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                    c_void_p, _PL, _PL, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                    c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "tgt_sparse_attn_bwd_passes": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                           c_void_p, c_void_p, _PL, _PL, c_void_p, c_void_p, c_void_p,
                                           c_void_p, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p,
                                           c_int]),
    "tgt_a2a_pack_heads": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int64,
                                   c_int64, c_int, c_int, c_void_p]),
    "tgt_a2a_unpack_seq": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                   c_int64, c_int, c_int, c_void_p]),
    "tgt_a2a_pack_seq": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int64,
                                 c_int64, c_int, c_int, c_void_p]),
    "tgt_a2a_unpack_heads": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                     c_int64, c_int, c_int, c_void_p]),
    "tgt_global_rows_broadcast": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_int,
                                          c_void_p]),
    "tgt_global_rows_reduce": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_int,
                                       c_void_p]),
    "tgt_ln_qkv_push": (c_int, [c_void_p, c_void_p, c_void_p, ctypes.c_float, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_void_p, c_void_p, c_int, c_int, POINTER(c_void_p), c_size_t, c_int64, c_int64, c_int,
                                c_int, c_void_p]),
    "tgt_pull_out_proj": (c_int, [POINTER(c_void_p), c_size_t, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                  c_int64, c_int64, c_int, c_int, c_void_p, c_int, c_void_p]),
    "tgt_layer_norm_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_int64, c_int, c_void_p, c_void_p, c_void_p]),
    "tgt_layer_norm_bwd_scratch_bytes": (c_int, [c_int64, c_int, POINTER(c_size_t)]),
    "tgt_layer_norm_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_size_t, c_void_p]),
    "tgt_linear_wgrad_scratch_bytes": (c_int, [c_int64, c_int, c_int, POINTER(c_size_t)]),
    "tgt_linear_wgrad": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_size_t,
                                 c_void_p]),
    "tgt_p2p_control_bytes": (c_size_t, []),
    "tgt_p2p_push": (c_int, [c_void_p, c_void_p, c_void_p, c_int, POINTER(c_void_p), c_size_t, c_int64, c_int64,
                             c_int64, c_int, c_int, c_void_p, c_int, c_int64, c_int, c_void_p]),
    "tgt_p2p_pull": (c_int, [POINTER(c_void_p), c_size_t, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                             c_int64, c_int, c_int, c_void_p, c_int, c_void_p]),
    "tgt_p2p_barrier": (c_int, [POINTER(c_void_p), c_int, c_int, c_uint32, c_void_p, c_void_p]),
    "tgt_p2p_fetch": (c_int, [c_void_p, c_size_t, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int64,
                              c_void_p]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library (once) and attach prototypes.  Raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m torchgt_b200.build` "
            "(torchgt_b200 has no CPU or PyTorch fallback)")
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if a declared symbol is not exported
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def last_error() -> str:
    return load().tgt_last_error().decode("utf-8", "replace")


def check(code: int) -> None:
    if code != TGT_OK:
        raise TgtError(code, last_error())
