"""The backward projection GEMMs (mintb_linear_dgrad / mintb_linear_wgrad, called through the C ABI) against fp32 torch:
dx = dz w (+ dz2 w2) and dw = dz^T x from the row-major matrices of the forward pass, bf16 operands; and the 8-bit variant
(e5m2 gradient against e4m3 operands, alt/munit_scaling.py:36-55 of the reference) against the same product formed in fp32
from the dequantised values."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from mint_plus_b200 import ops  # noqa: E402

DEV = "cuda"


def _rand(shape, g, scale=1.0):
    return (torch.randn(*shape, generator=g) * scale).bfloat16()


# (M, N, K): ragged in every dimension, a single tile, several tiles and splits
SHAPES = [(300, 384, 256), (128, 256, 256), (1000, 1280, 640), (77, 64, 8), (4096, 3840, 1280), (2500, 136, 520)]


@pytest.mark.parametrize("shape", SHAPES)
def test_dgrad_bf16(shape):
    M, N, K = shape
    g = torch.Generator().manual_seed(M + N + K)
    dz, w = _rand((M, N), g), _rand((N, K), g, N ** -0.5)
    got = ops.gemm_dgrad(dz.to(DEV), w.to(DEV), alpha=0.5)
    ops.check_device_status()
    want = 0.5 * (dz.float() @ w.float())
    assert tuple(got.shape) == (M, K)
    assert (got.float().cpu() - want).abs().max().item() <= 1e-2 * want.abs().max().item() + 1e-3


def test_dgrad_adds_a_second_operand_pair():
    M, N, K, N2 = 700, 384, 256, 192
    g = torch.Generator().manual_seed(5)
    dz, w, dz2, w2 = _rand((M, N), g), _rand((N, K), g, N ** -0.5), _rand((M, N2), g), _rand((N2, K), g, N2 ** -0.5)
    got = ops.gemm_dgrad(dz.to(DEV), w.to(DEV), dz2.to(DEV), w2.to(DEV))
    ops.check_device_status()
    want = dz.float() @ w.float() + dz2.float() @ w2.float()
    assert (got.float().cpu() - want).abs().max().item() <= 1e-2 * want.abs().max().item() + 1e-3


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", SHAPES)
def test_wgrad_bf16(shape, out_dtype):
    M, N, K = shape
    if K % 4:
        pytest.skip("K must be a multiple of 4")
    g = torch.Generator().manual_seed(M * 3 + N + K)
    dz, x = _rand((M, N), g), _rand((M, K), g)
    got = ops.gemm_wgrad(dz.to(DEV), x.to(DEV), alpha=2.0, out_dtype=out_dtype)
    ops.check_device_status()
    want = 2.0 * (dz.float().t() @ x.float())
    assert tuple(got.shape) == (N, K) and got.dtype == out_dtype
    tol = (1e-2 if out_dtype == torch.bfloat16 else 1e-4) * want.abs().max().item() + 1e-3
    assert (got.float().cpu() - want).abs().max().item() <= tol


def test_wgrad_over_many_tokens_uses_splits_and_stays_accurate():
    """The shape class of the training step: tens of thousands of token rows against a weight-sized result."""
    M, N, K = 32768, 1280, 1280
    g = torch.Generator().manual_seed(11)
    dz, x = _rand((M, N), g).to(DEV), _rand((M, K), g).to(DEV)
    got = ops.gemm_wgrad(dz, x, out_dtype=torch.float32)
    ops.check_device_status()
    want = dz.double().t() @ x.double()          # on the device, in fp64
    assert (got.double() - want).abs().max().item() <= 1e-4 * want.abs().max().item()
    again = ops.gemm_wgrad(dz, x, out_dtype=torch.float32)
    assert (again - got).abs().max().item() <= 1e-4 * want.abs().max().item()


@pytest.mark.parametrize("shape", [(300, 384, 256), (1024, 1280, 640), (4096, 256, 1280)])
def test_8bit_dgrad_and_wgrad_match_the_dequantised_products(shape):
    """e5m2 gradient x e4m3 weight / activation: exact products of the 8-bit values, fp32 accumulation."""
    M, N, K = shape
    g = torch.Generator().manual_seed(M + K)
    dz8 = (torch.randn(M, N, generator=g) * 4).to(torch.float8_e5m2)
    w8 = (torch.randn(N, K, generator=g) * 8).to(torch.float8_e4m3fn)
    x8 = (torch.randn(M, K, generator=g) * 8).to(torch.float8_e4m3fn)
    dx = ops.gemm_dgrad(dz8.to(DEV), w8.to(DEV), alpha=0.01)
    dw = ops.gemm_wgrad(dz8.to(DEV), x8.to(DEV), alpha=0.01, out_dtype=torch.float32)
    ops.check_device_status()
    want_dx = 0.01 * (dz8.float() @ w8.float())
    want_dw = 0.01 * (dz8.float().t() @ x8.float())
    assert (dx.float().cpu() - want_dx).abs().max().item() <= 1e-2 * want_dx.abs().max().item()     # bf16 result
    assert (dw.cpu() - want_dw).abs().max().item() <= 1e-4 * want_dw.abs().max().item()


def test_backward_gemms_reject_bad_arguments():
    a = torch.zeros(16, 24, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ValueError):
        ops.gemm_dgrad(a, torch.zeros(16, 24, dtype=torch.bfloat16, device=DEV))            # inner sizes disagree
    with pytest.raises(ValueError):
        ops.gemm_wgrad(a, torch.zeros(8, 24, dtype=torch.bfloat16, device=DEV))             # row counts disagree
    with pytest.raises(ValueError):
        ops.gemm_dgrad(a, torch.zeros(24, 12, dtype=torch.bfloat16, device=DEV))            # K * 2 not a 16-byte multiple
    with pytest.raises((TypeError, NotImplementedError)):
        ops.gemm_dgrad(a, torch.zeros(24, 16, dtype=torch.float8_e4m3fn, device=DEV))       # mixed bf16 / 8-bit
