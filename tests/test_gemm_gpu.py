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


@pytest.mark.parametrize("M,N,K,dtype", [(8, 2048, 16384, torch.float16), (130, 300, 4096, torch.bfloat16),
                                         (2, 256, 2048, torch.float16)])
def test_gemm_skinny_products_split_the_reduction(M, N, K, dtype, monkeypatch):
    """Few output tiles and a long K: the reduction is cut into ranges that run on different
    SMs and are summed by the warp that arrives last.  Twice in a row (the arrival counters
    must be back at zero), with bias, beta and activation applied once, against fp32 and
    against the same product without the split."""
    torch.manual_seed(5)
    a = (torch.randn(M, K, device="cuda") / K ** 0.25).to(dtype)
    w = (torch.randn(N, K, device="cuda") / K ** 0.25).to(dtype)
    bias = torch.randn(N, device="cuda")
    prev = torch.randn(M, N, device="cuda").to(dtype)
    ref = torch.relu(a.float() @ w.float().t() + bias + 0.5 * prev.float())
    before = native.splitk_offers
    outs = []
    for _ in range(2):
        out = prev.clone()
        gemm(a, w, trans_b=True, out=out, beta=0.5, bias=bias, act=native.ACT_RELU)
        assert native.consume_status() == 0
        outs.append(out)
    assert native.splitk_offers == before + 2
    assert torch.equal(outs[0], outs[1])          # summed in split order: bitwise repeatable
    torch.testing.assert_close(outs[0].float(), ref, rtol=1e-2, atol=3e-2)
    monkeypatch.setenv("LBANN_DISABLE_SPLITK", "1")
    plain = prev.clone()
    gemm(a, w, trans_b=True, out=plain, beta=0.5, bias=bias, act=native.ACT_RELU)
    assert native.splitk_offers == before + 2
    torch.testing.assert_close(outs[0].float(), plain.float(), rtol=1e-2, atol=2e-2)
