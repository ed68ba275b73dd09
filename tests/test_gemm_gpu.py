"""tcgen05 GEMM against a PyTorch fp32 reference of the same (16-bit rounded) inputs."""
import pytest
import torch

from lbann_b200.ops import native
from lbann_b200.ops.gemm import gemm

pytestmark = pytest.mark.gpu


def _ref(a, b, ta, tb):
    A = a.float().transpose(-1, -2) if ta else a.float()
    B = b.float().transpose(-1, -2) if tb else b.float()
    return A @ B


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("ta,tb", [(False, True), (False, False), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 512, 256), (300, 200, 136), (77, 40, 24),
                                   (1024, 2048, 1024)])
def test_gemm_layouts(dtype, ta, tb, M, N, K):
    torch.manual_seed(0)
    a = torch.randn((K, M) if ta else (M, K), device="cuda").to(dtype)
    b = torch.randn((N, K) if tb else (K, N), device="cuda").to(dtype)
    out = gemm(a, b, trans_a=ta, trans_b=tb, out_dtype=torch.float32)
    assert native.consume_status() == 0
    ref = _ref(a, b, ta, tb)
    torch.testing.assert_close(out, ref, rtol=2e-3, atol=2e-2 * (K ** 0.5) / 8)


@pytest.mark.parametrize("bn", [64, 128, 256])
def test_gemm_tile_widths_and_epilogue(bn):
    torch.manual_seed(1)
    M, N, K = 384, 520, 192
    a = torch.randn(M, K, device="cuda").bfloat16()
    w = torch.randn(N, K, device="cuda").bfloat16()
    bias = torch.randn(N, device="cuda")
    prev = torch.randn(M, N, device="cuda").bfloat16()
    out = prev.clone()
    gemm(a, w, trans_b=True, out=out, alpha=0.5, beta=2.0, bias=bias, act=native.ACT_RELU,
         bn_hint=bn)
    assert native.consume_status() == 0
    ref = torch.relu(0.5 * (a.float() @ w.float().t()) + 2.0 * prev.float() + bias)
    torch.testing.assert_close(out.float(), ref, rtol=1.6e-2, atol=0.15)


def test_gemm_batched_and_row_bias():
    torch.manual_seed(2)
    B, M, N, K = 5, 200, 136, 72
    a = torch.randn(B, M, K, device="cuda").half()
    b = torch.randn(B, K, N, device="cuda").half()
    bias = torch.randn(M, device="cuda")
    out = gemm(a, b, out_dtype=torch.float32, bias=bias, bias_per_row=True)
    assert native.consume_status() == 0
    ref = a.float() @ b.float() + bias[None, :, None]
    torch.testing.assert_close(out, ref, rtol=2e-3, atol=3e-2)


def test_gemm_unaligned_operands_are_repacked():
    torch.manual_seed(3)
    a = torch.randn(50, 84, device="cuda").bfloat16()
    w = torch.randn(10, 84, device="cuda").bfloat16()
    out = gemm(a, w, trans_b=True, out_dtype=torch.float32)
    assert native.consume_status() == 0
    torch.testing.assert_close(out, a.float() @ w.float().t(), rtol=2e-3, atol=3e-2)
