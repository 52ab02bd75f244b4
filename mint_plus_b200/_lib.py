"""ctypes binding of libmintb.so (the C ABI declared in include/mintb.h).

There is no fallback: if the library is missing, loading raises and every op that needs it fails.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_size_t, c_uint, c_ulonglong, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmintb.so")

OK, EINVAL, EUNSUPPORTED, EWORKSPACE, ECUDA = 0, -1, -2, -3, -4
F32, BF16, E4M3, E5M2 = 0, 1, 2, 3
FLAG_ROPE, FLAG_SQRT_SOFTMAX, FLAG_FORCE_SIMT, FLAG_OUT_SEQ_FIRST, FLAG_ROT_SAVED, FLAG_SKIP_PAD_QUERIES = 1, 2, 4, 8, 16, 32
FLAG_QK_PREROTATED, FLAG_GRAD_ROWMAJOR = 64, 128
STATIC_SCRATCH_BYTES = 32 << 20

_P = c_void_p
# name -> (restype, argtypes); mirrors include/mintb.h one to one
PROTOTYPES = {
    "mintb_version": (c_int, []),
    "mintb_last_error": (c_char_p, []),
    "mintb_kernel_launches": (c_ulonglong, []),
    "mintb_selftest_wait": (c_int, [c_ulonglong, _P, _P, _P]),
    "mintb_mask_meta_bytes": (c_size_t, [c_int, c_int]),
    "mintb_mask_meta_from_chain_ids": (c_int, [_P, _P, _P, c_int, c_int, _P]),
    "mintb_mask_meta_from_mask": (c_int, [_P, _P, _P, c_int, c_int, _P]),
    "mintb_rope_tables": (c_int, [_P, _P, _P, c_int, c_int, _P]),
    "mintb_reset_work_counters": (c_int, []),
    "mintb_attn_fwd_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int, c_uint]),
    "mintb_attn_fwd": (c_int, [_P] * 6 + [_P, _P, _P, _P, _P, _P, c_size_t, c_int, c_int, c_int, c_int, c_int, c_uint,
                               c_float, _P, _P]),
    "mintb_attn_fwd_static": (c_int, [_P] * 6 + [_P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_uint, c_float, _P,
                                      _P]),
    "mintb_attn_bwd_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int, c_uint]),
    "mintb_attn_bwd": (c_int, [_P] * 6 + [_P, _P, _P, _P, _P, _P] + [_P] * 6 + [_P, c_size_t, c_int, c_int, c_int, c_int,
                               c_int, c_uint, c_float, _P, _P]),
    "mintb_attn_bwd_rows": (c_int, [_P] * 6 + [_P, _P, _P, _P, _P, _P] + [_P] * 6 + [_P, c_size_t, c_int, c_int, c_int, c_int,
                                    c_int, c_uint, c_float, _P, _P, _P]),
    "mintb_linear_fwd": (c_int, [_P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, _P, _P]),
    "mintb_qkv_fwd": (c_int, [_P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, _P, _P, _P, c_int,
                              _P, _P]),
    "mintb_quantize_e4m3": (c_int, [_P, _P, c_size_t, c_float, _P]),
    "mintb_linear_res_fwd": (c_int, [_P, _P, _P, _P, c_float, c_float, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float,
                                     _P, _P]),
    "mintb_qkv2_fwd": (c_int, [_P] * 9 + [c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_float, _P, _P, _P, c_int, _P, _P]),
    "mintb_linear_dgrad": (c_int, [_P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_float, _P, _P]),
    "mintb_linear_wgrad_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "mintb_linear_wgrad": (c_int, [_P, _P, _P, _P, c_size_t, c_int, c_int, c_int, c_int, c_int, c_int, c_float, _P, _P]),
    "mintb_add_layernorm_fwd": (c_int, [_P, _P, c_float, c_float, _P, _P, c_int, _P, _P, _P, c_int, c_int, c_float, _P]),
    "mintb_add_layernorm_fwd_q": (c_int, [_P, _P, c_float, c_float, _P, _P, c_int, _P, _P, _P, c_int, c_int, c_float, _P, c_float, _P]),
    "mintb_add_layernorm_bwd_workspace_bytes": (c_size_t, [c_int, c_int]),
    "mintb_add_layernorm_bwd": (c_int, [_P, _P, _P, _P, c_float, c_float, _P, c_int, _P, _P, _P, _P, _P, _P, c_size_t, c_int,
                                        c_int, _P]),
    "mintb_gelu_bwd_colsum": (c_int, [_P, _P, _P, _P, c_int, c_int, _P]),
    "mintb_gelu_bwd_colsum_act": (c_int, [_P, _P, _P, _P, _P, c_int, c_int, _P]),
    "mintb_gelu_bwd_colsum_f8": (c_int, [_P, _P, _P, _P, _P, _P, c_float, c_int, c_int, _P]),
    "mintb_qkv_grad_pack": (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_float, _P]),
    "mintb_embed_fwd": (c_int, [_P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, _P]),
    "mintb_embed_bwd": (c_int, [_P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P]),
    "mintb_masked_ce_fwd": (c_int, [_P, _P, _P, _P, _P, c_int, c_int, c_int, _P]),
    "mintb_masked_ce_bwd": (c_int, [_P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, _P]),
    "mintb_combine_fwd": (c_int, [_P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P]),
    "mintb_combine_bwd_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "mintb_combine_bwd": (c_int, [_P] * 10 + [_P, c_size_t, c_int, c_int, c_int, c_int, c_int, _P]),
}

_lib = None


class MintbError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    """Load libmintb.so once and attach the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise MintbError(
            f"{LIB_PATH} is missing: build it with `python -m mint_plus_b200.build` "
            "(nvcc, sm_100a). There is no fallback path.")
    handle = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(handle, name)          # AttributeError if the library does not export it
        fn.restype = res
        fn.argtypes = args
    _lib = handle
    return _lib


def check(rc: int, what: str) -> None:
    """Map a MINTB_* return code to a Python exception (ValueError for rejected arguments)."""
    if rc == OK:
        return
    msg = lib().mintb_last_error().decode("utf-8", "replace")
    if rc in (EINVAL, EWORKSPACE):
        raise ValueError(f"{what}: {msg}")
    if rc == EUNSUPPORTED:
        raise NotImplementedError(f"{what}: {msg}")
    raise MintbError(f"{what}: {msg} (code {rc})")
