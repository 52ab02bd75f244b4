"""The forward entry point that allocates nothing (mintb_attn_fwd_static), called through the C ABI.

Its scratch - the rotated copies of Q_self and K_self - lives in a fixed array inside the library instead of a
caller-provided workspace, for callers that may not allocate device memory when they call (stream capture in
progress, fixed memory budgets, bindings that only pass pre-made buffers).  The results must equal those of
mintb_attn_fwd, call after call: the array is shared and keeps the previous call's contents.
This file sorts last on purpose, so a run that stops at the first failure has already run every other test.
"""
import pytest
import torch

from oracle import multimer_attention as O

pytestmark = pytest.mark.gpu

import mint_plus_b200 as M  # noqa: E402
from mint_plus_b200 import _lib as L, ops  # noqa: E402

DEV = "cuda"
BF16_OUT_ATOL = 2e-2     # the tolerance the attention tests use for bf16 outputs


def _call_both(B, H, T, D, seed):
    ts, cid, pad, _ = O.make_op_inputs(B, H, T, D, seed=seed, max_pad=min(64, T // 4))
    dts = [t.to(DEV, torch.bfloat16).contiguous() for t in ts]
    meta = M.mask_meta_from_chain_ids(cid.to(DEV), pad.to(DEV))
    cos, sin, _ = ops.rope_tables(T, D, torch.device(DEV))
    lib = L.lib()
    flags, scale = L.FLAG_ROPE, D ** -0.5
    stream = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device=DEV)

    # existing entry point: caller-provided workspace
    out_a = torch.empty_like(dts[0])
    lse_a = torch.empty(B, H, T, dtype=torch.float32, device=DEV)
    ws_bytes = lib.mintb_attn_fwd_workspace_bytes(B, H, T, D, L.BF16, flags)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=DEV)
    rc = lib.mintb_attn_fwd(*[t.data_ptr() for t in dts], meta.buf.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                            out_a.data_ptr(), lse_a.data_ptr(), ws.data_ptr(), ws_bytes, B, H, T, D, L.BF16, flags, scale,
                            stream, status.data_ptr())
    L.check(rc, "mintb_attn_fwd")

    # new entry point: no workspace argument at all
    out_b = torch.full_like(dts[0], float("nan"))
    lse_b = torch.full((B, H, T), float("nan"), dtype=torch.float32, device=DEV)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    rc = lib.mintb_attn_fwd_static(*[t.data_ptr() for t in dts], meta.buf.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                   out_b.data_ptr(), lse_b.data_ptr(), B, H, T, D, L.BF16, flags, scale, stream,
                                   status.data_ptr())
    L.check(rc, "mintb_attn_fwd_static")
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before          # nothing went through torch's allocator either
    assert int(status.item()) == 0
    want = O.multimer_attention(*[t.bfloat16().float() for t in ts], O.chain_mask_from_ids(cid), pad)
    return out_a.float().cpu(), lse_a.cpu(), out_b.float().cpu(), lse_b.cpu(), want


def test_static_scratch_forward_matches_the_workspace_forward_twice_in_a_row():
    # two calls in a row with different shapes: the second finds the first call's rotated tensors in the array
    for (B, H, T, D, seed) in [(2, 4, 300, 32, 31), (1, 3, 200, 64, 32)]:
        out_a, lse_a, out_b, lse_b, want = _call_both(B, H, T, D, seed)
        assert torch.isfinite(out_b).all()
        assert (out_b - out_a).abs().max().item() <= BF16_OUT_ATOL
        assert torch.equal(out_b, out_a)                    # same kernels, same inputs: in fact bit-identical
        torch.testing.assert_close(lse_b, lse_a, rtol=1e-5, atol=1e-5)
        assert (out_b - want).abs().max().item() <= BF16_OUT_ATOL


def test_static_scratch_rejects_sizes_beyond_its_array():
    lib = L.lib()
    fake = 256 * 1024                                         # aligned, never dereferenced: rejected on the host
    B, H, T, D = 16, 20, 2048, 64                             # 2 * B*H*T*D * 2 bytes = 160 MiB > 32 MiB
    rc = lib.mintb_attn_fwd_static(*[fake] * 6, fake, fake, fake, fake, fake, B, H, T, D, L.BF16, L.FLAG_ROPE, 0.125,
                                   None, None)
    assert rc == L.EWORKSPACE
    assert b"built-in array" in lib.mintb_last_error()
    rc = lib.mintb_attn_fwd_static(*[fake] * 6, fake, fake, fake, fake, fake, 1, 1, 64, 32, L.F32, L.FLAG_ROPE, 0.125,
                                   None, None)
    assert rc == L.EUNSUPPORTED
