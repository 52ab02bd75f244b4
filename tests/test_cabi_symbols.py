"""The C-ABI library loads without a GPU and exports every symbol include/mintb.h declares; argument checks that
run on the host before any launch return the documented codes."""
import ctypes
import os
import re

import pytest

from mint_plus_b200 import _lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "mintb.h")).read()
    return sorted(set(re.findall(r"MINTB_API[^;(]*?\b(mintb_\w+)\s*\(", text)))


def test_header_declares_the_bound_prototypes():
    assert declared_symbols() == sorted(L.PROTOTYPES)


@pytest.mark.parametrize("name", declared_symbols())
def test_symbol_exported(name):
    handle = ctypes.CDLL(L.LIB_PATH)
    assert getattr(handle, name) is not None


def test_version_and_sizes():
    lib = L.lib()
    assert lib.mintb_version() >= 100
    assert lib.mintb_mask_meta_bytes(0, 16) == 0
    n = lib.mintb_mask_meta_bytes(2, 100)
    # two (B,T,TW) word arrays, the key-pad words and the class bytes, each rounded to 256 bytes
    tw, nt = 4, 2
    a = lambda x: (x + 255) // 256 * 256
    assert n == 2 * a(2 * 100 * tw * 4) + a(2 * tw * 4) + a(2 * nt * nt)
    assert lib.mintb_attn_bwd_workspace_bytes(2, 3, 50, 16, L.F32, 0) >= 2 * 3 * 50 * 4


def test_rejected_arguments_return_codes_without_touching_a_gpu():
    lib = L.lib()
    fake = ctypes.c_void_p(256 * 1024)       # aligned, never dereferenced: rejected before any launch
    args = [fake] * 6 + [fake, None, None, fake, fake, None, 0]
    assert lib.mintb_attn_fwd(*args, 1, 1, 16, 48, L.F32, 0, 1.0, None, None) == L.EUNSUPPORTED     # head_dim 48
    assert b"head_dim" in lib.mintb_last_error()
    assert lib.mintb_attn_fwd(*args, 0, 1, 16, 32, L.F32, 0, 1.0, None, None) == L.EINVAL           # B = 0
    assert lib.mintb_attn_fwd(*args, 1, 1, 16, 32, 7, 0, 1.0, None, None) == L.EINVAL               # dtype
    assert lib.mintb_attn_fwd(*args, 1, 1, 16, 32, L.F32, L.FLAG_ROPE, 1.0, None, None) == L.EINVAL  # rope w/o tables
    assert lib.mintb_attn_fwd(*args, 1, 1, 16, 32, L.F32, 0x100, 1.0, None, None) == L.EINVAL                # unknown flag bit
    assert lib.mintb_attn_fwd(*args, 1, 1, 16, 32, L.F32, 0, -1.0, None, None) == L.EINVAL          # scale
    bad = [ctypes.c_void_p(256 * 1024 + 2)] + [fake] * 5 + [fake, None, None, fake, fake, None, 0]
    assert lib.mintb_attn_fwd(*bad, 1, 1, 16, 32, L.F32, 0, 1.0, None, None) == L.EINVAL            # misaligned q
    assert lib.mintb_mask_meta_from_chain_ids(None, None, fake, 1, 16, None) == L.EINVAL
    with pytest.raises(ValueError):
        L.check(L.EINVAL, "x")
    with pytest.raises(NotImplementedError):
        L.check(L.EUNSUPPORTED, "x")
