"""tcgen05 implicit-GEMM convolution against torch.nn.functional (fp32) on the same inputs."""
import pytest
import torch
import torch.nn.functional as F

from lbann_b200.ops import native
from lbann_b200.ops.conv import conv_fwd, pack_filter

pytestmark = pytest.mark.gpu

# the oracle (cuDNN / cuBLAS through torch) must not round its inputs to TF32
torch.backends.cudnn.allow_tf32 = False
torch.backends.cuda.matmul.allow_tf32 = False

CASES = [
    # N, C, D, H, W, K, k, pad, stride, dil
    (2, 16, 8, 8, 8, 32, 3, 1, 1, 1),
    (1, 32, 16, 16, 16, 64, 3, 1, 1, 1),
    (2, 64, 8, 8, 8, 128, 3, 1, 1, 1),
    (1, 128, 4, 8, 8, 256, 3, 1, 1, 1),
    (2, 16, 1, 28, 28, 48, 5, 2, 1, 1),
    (3, 64, 1, 14, 14, 64, 1, 0, 1, 1),
    (2, 32, 1, 30, 30, 40, 3, 1, 2, 1),
    (1, 24, 6, 10, 12, 16, 3, 2, 1, 2),
    (4, 8, 1, 7, 7, 24, 3, 1, 1, 1),
    # shapes the halo-slab kernel takes (stride 1, filter resident in shared memory)
    (1, 32, 6, 40, 64, 64, 3, 1, 1, 1),
    (2, 64, 4, 24, 32, 32, 3, 1, 1, 1),
    (1, 16, 1, 33, 50, 24, 3, 1, 1, 1),
    (1, 48, 3, 20, 28, 96, 3, 1, 1, 1),
    (1, 32, 3, 9, 130, 64, 3, 0, 1, 1),
]


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_conv_fwd(case, dtype):
    N, C, D, H, W, K, k, pad, stride, dil = case
    torch.manual_seed(0)
    ks = (1 if D == 1 else k, k, k)
    pd = (0 if D == 1 else pad, pad, pad)
    st = (1 if D == 1 else stride, stride, stride)
    dl = (1 if D == 1 else dil, dil, dil)
    x = torch.randn(N, C, D, H, W, device="cuda").to(dtype)
    w = (torch.randn(K, C, *ks, device="cuda") / (C * k * k) ** 0.5).to(dtype)
    bias = torch.randn(K, device="cuda")
    xl = x.permute(0, 2, 3, 4, 1).contiguous()
    y = conv_fwd(xl, pack_filter(w, dtype), ks, pad=pd, stride=st, dilation=dl, bias=bias,
                 out_dtype=torch.float32)
    assert native.consume_status() == 0
    ref = F.conv3d(x.float(), w.float(), bias, st, pd, dl).permute(0, 2, 3, 4, 1)
    torch.testing.assert_close(y, ref, rtol=2e-3, atol=2e-2)


def test_conv_dgrad_via_flipped_filter():
    torch.manual_seed(1)
    N, C, K, S = 2, 32, 64, 8
    x = torch.randn(N, C, S, S, S, device="cuda", requires_grad=True)
    w = (torch.randn(K, C, 3, 3, 3, device="cuda") / 30).bfloat16()
    y = F.conv3d(x, w.float(), None, 1, 1)
    dy = torch.randn_like(y).bfloat16()
    y.backward(dy.float())
    dyl = dy.permute(0, 2, 3, 4, 1).contiguous()
    dx = conv_fwd(dyl, pack_filter(w, torch.bfloat16, for_dgrad=True), 3, pad=1,
                  out_dtype=torch.float32)
    assert native.consume_status() == 0
    torch.testing.assert_close(dx, x.grad.permute(0, 2, 3, 4, 1), rtol=2e-3, atol=3e-2)


WGRAD_CASES = [
    # N, C, D, H, W, K, k, pad, stride
    (2, 16, 8, 8, 8, 32, 3, 1, 1),
    (2, 32, 8, 16, 16, 64, 3, 1, 1),
    (2, 64, 8, 8, 8, 128, 3, 1, 1),
    (1, 128, 4, 8, 8, 256, 3, 1, 1),
    (2, 16, 1, 28, 28, 48, 5, 2, 1),
    (3, 64, 1, 14, 14, 64, 1, 0, 1),
    (2, 32, 1, 30, 30, 40, 3, 1, 2),
    (4, 8, 1, 7, 7, 24, 3, 1, 1),
]


@pytest.mark.parametrize("case", WGRAD_CASES)
def test_conv_wgrad(case):
    from lbann_b200.ops.conv import conv_wgrad
    N, C, D, H, W, K, k, pad, stride = case
    torch.manual_seed(0)
    ks = (1 if D == 1 else k, k, k)
    pd = (0 if D == 1 else pad, pad, pad)
    st = (1 if D == 1 else stride, stride, stride)
    x = torch.randn(N, C, D, H, W, device="cuda").bfloat16()
    w = torch.zeros(K, C, *ks, device="cuda", requires_grad=True)
    y = F.conv3d(x.float(), w, None, st, pd)
    dy = torch.randn_like(y).bfloat16()
    y.backward(dy.float())
    xl = x.permute(0, 2, 3, 4, 1).contiguous()
    dyl = dy.permute(0, 2, 3, 4, 1).contiguous()
    prev = torch.ones(K, C, *ks, device="cuda")
    got = conv_wgrad(xl, dyl, ks, pad=pd, stride=st, out=prev.clone(), alpha=0.5)
    assert native.consume_status() == 0
    ref = prev + 0.5 * w.grad
    torch.testing.assert_close(got, ref, rtol=2e-3, atol=2e-2 * (N * D * H * W) ** 0.5 / 8)


@pytest.mark.parametrize("case", [(2, 256, 8, 8, 8, 256), (1, 128, 4, 16, 16, 200), (3, 64, 1, 12, 12, 96)])
def test_conv_deep_layers_split_the_reduction(case, monkeypatch):
    """The deep layers of a network on a small batch: a handful of output bricks, thousands of
    reduction steps.  The split result equals the unsplit one up to fp32 summation order."""
    N, C, D, H, W, K = case
    torch.manual_seed(4)
    ks = (1 if D == 1 else 3, 3, 3)
    pd = (0 if D == 1 else 1, 1, 1)
    x = torch.randn(N, C, D, H, W, device="cuda").half()
    w = (torch.randn(K, C, *ks, device="cuda") / (C * 27) ** 0.5).half()
    bias = torch.randn(K, device="cuda")
    xl = x.permute(0, 2, 3, 4, 1).contiguous()
    wp = pack_filter(w, torch.float16)
    before = native.splitk_offers
    ys = [conv_fwd(xl, wp, ks, pad=pd, bias=bias, act=native.ACT_LEAKY, act_param=0.01,
                   out_dtype=torch.float32) for _ in range(2)]
    assert native.consume_status() == 0
    assert native.splitk_offers == before + 2
    assert torch.equal(ys[0], ys[1])
    ref = F.leaky_relu(F.conv3d(x.float(), w.float(), bias, 1, pd), 0.01).permute(0, 2, 3, 4, 1)
    torch.testing.assert_close(ys[0], ref, rtol=2e-3, atol=2e-2)
    monkeypatch.setenv("LBANN_DISABLE_SPLITK", "1")
    plain = conv_fwd(xl, wp, ks, pad=pd, bias=bias, act=native.ACT_LEAKY, act_param=0.01,
                     out_dtype=torch.float32)
    torch.testing.assert_close(ys[0], plain, rtol=1e-4, atol=1e-4)
