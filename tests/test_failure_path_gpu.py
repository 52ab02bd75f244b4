"""The bounded-wait error path, exercised without faulting or hanging the GPU: a self-test kernel waits (for a few
milliseconds at most) on a barrier that nothing completes; the wait gives up, the kernel records its code, releases TMEM
and returns, and `check_device_status()` turns the code into an exception and clears it.  Also: run-to-run spread of dQ,
the one result of the backward pass whose summation order is not fixed."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

import mint_plus_b200 as M  # noqa: E402
from mint_plus_b200 import _lib as L, ops  # noqa: E402
from oracle import multimer_attention as O  # noqa: E402


def test_wait_that_runs_out_sets_the_status_and_the_context_stays_usable():
    dev = torch.device("cuda", torch.cuda.current_device())
    ops.check_device_status(dev)                                   # clean on entry
    status = ops._dev_status(dev)
    trail = torch.zeros(2, dtype=torch.int32, device=dev)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    rc = L.lib().mintb_selftest_wait(2_000_000, status.data_ptr(), trail.data_ptr(), torch.cuda.current_stream().cuda_stream)
    t1.record()
    assert rc == L.OK
    torch.cuda.synchronize()                                       # returns: the kernel ended by itself
    assert 1.0 <= t0.elapsed_time(t1) < 500.0                      # it waited about the 2 ms it was given, not the 2 s default
    assert trail.tolist() == [2, 1]                                # the wait gave up; TMEM was released afterwards
    assert int(status.item()) == 0x901
    with pytest.raises(L.MintbError, match="0x901"):
        ops.check_device_status(dev)
    ops.check_device_status(dev)                                   # raising cleared it
    # the context is intact: a real kernel runs and is correct right after
    ts, cid, pad, _ = O.make_op_inputs(1, 2, 128, 32, seed=5)
    out = M.multimer_attention(*[t.to(dev, torch.bfloat16) for t in ts], chain_ids=cid.to(dev), key_padding_mask=pad.to(dev))
    want = O.multimer_attention(*[t.bfloat16().float() for t in ts], O.chain_mask_from_ids(cid), pad)
    assert (out.float().cpu() - want).abs().max().item() <= 2e-2
    ops.check_device_status(dev)


def test_selftest_rejects_bad_arguments_on_the_host():
    lib = L.lib()
    assert lib.mintb_selftest_wait(1000, None, None, None) == L.EINVAL
    fake = ctypes.c_void_p(4096)
    assert lib.mintb_selftest_wait(0, fake, None, None) == L.EINVAL
    assert lib.mintb_selftest_wait(2_000_000_000, fake, None, None) == L.EINVAL


def test_dq_run_to_run_spread_is_bounded_and_dk_dv_are_bit_reproducible():
    """dK and dV are reduced inside one CTA in a fixed order; dQ is accumulated across CTAs in arrival order (fp32
    additions into one accumulator, rounded to bf16 once at the end), so two runs may differ in the last bf16 bit."""
    B, H, T, D = 2, 4, 512, 32
    ts, cid, pad, grad = O.make_op_inputs(B, H, T, D, seed=77)
    kw = dict(chain_ids=cid.cuda(), key_padding_mask=pad.cuda())
    runs = []
    for _ in range(3):
        leaves = [t.cuda().bfloat16().requires_grad_(True) for t in ts]
        runs.append(torch.autograd.grad(M.multimer_attention(*leaves, **kw), leaves, grad.cuda().bfloat16()))
    ops.check_device_status()
    for other in runs[1:]:
        for i, (a, b) in enumerate(zip(runs[0], other)):
            if i in (0, 3):       # dq_self, dq_cross: within one bf16 step of the value (2^-8 relative) plus fp32 noise
                diff = (a.float() - b.float()).abs()
                assert (diff <= a.float().abs() * 2.0 ** -7 + 1e-6).all()
            else:
                assert torch.equal(a, b)
