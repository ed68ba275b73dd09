"""The smaller native kernels against PyTorch fp32 restatements of the same operation:
pooling (all modes, overlapping windows), standalone softmax (scale, causal mask), top-k
accuracy, per-sample losses, the element-wise tables, strided / dilated convolutions forward
and backward through autograd."""
import pytest
import torch
import torch.nn.functional as F

from lbann_b200.ops import elementwise as ew
from lbann_b200.ops import native, nn

pytestmark = pytest.mark.gpu

torch.backends.cudnn.allow_tf32 = False
torch.backends.cuda.matmul.allow_tf32 = False


def _handle(t):
    m = t.clone().float().requires_grad_(True)
    return nn.WeightHandle(m, torch.zeros_like(m), None)


# ------------------------------------------------------------------------------- pooling
@pytest.mark.parametrize("mode", ["max", "average", "average_no_pad"])
@pytest.mark.parametrize("shape,ks,pad,st", [
    ((2, 16, 8, 8, 8), (2, 2, 2), (0, 0, 0), (2, 2, 2)),
    ((2, 8, 6, 10, 12), (3, 3, 3), (1, 1, 1), (2, 2, 2)),       # overlapping windows, padding
    ((3, 24, 1, 15, 15), (1, 3, 3), (0, 1, 1), (1, 2, 2)),      # 2-D, odd extent
    ((1, 8, 1, 7, 7), (1, 7, 7), (0, 0, 0), (1, 1, 1)),         # global pooling
])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_pooling_modes_forward_and_backward(mode, shape, ks, pad, st, dtype):
    torch.manual_seed(0)
    x = torch.randn(*shape, device="cuda").to(dtype)
    xa = x.clone().requires_grad_(True)
    xr = x.float().requires_grad_(True)
    y = nn.pooling(xa, ks, pad, st, mode)
    if mode == "max":
        ref = F.max_pool3d(xr, ks, st, pad)
    else:
        ref = F.avg_pool3d(xr, ks, st, pad, count_include_pad=(mode == "average"))
    assert y.shape == ref.shape
    tol = 1e-2 if dtype == torch.bfloat16 else 2e-3
    torch.testing.assert_close(y.float(), ref, rtol=tol, atol=tol)
    dy = torch.randn_like(ref).to(dtype)
    y.backward(dy)
    ref.backward(dy.float())
    assert native.consume_status() == 0
    torch.testing.assert_close(xa.grad.float(), xr.grad, rtol=2 * tol, atol=4 * tol)


# ------------------------------------------------------------------------------- softmax
@pytest.mark.parametrize("log", [False, True])
@pytest.mark.parametrize("rows,cols,period,scale", [(64, 1000, 0, 1.0), (3 * 128, 128, 128, 0.125),
                                                    (48, 33, 0, 2.0), (2 * 64, 64, 64, 1.0), (5, 4096, 0, 1.0)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_softmax_standalone(log, rows, cols, period, scale, dtype):
    torch.manual_seed(1)
    x = torch.randn(rows, cols, device="cuda").to(dtype)
    xa = x.clone().requires_grad_(True)
    xr = x.float().requires_grad_(True)
    y = nn.softmax_lastdim(xa, log, scale, period)
    z = xr * scale
    if period:
        r = torch.arange(rows, device="cuda") % period
        z = z.masked_fill(torch.arange(cols, device="cuda")[None, :] > r[:, None], float("-inf"))
    ref = F.log_softmax(z, -1) if log else F.softmax(z, -1)
    keep = torch.isfinite(ref)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    torch.testing.assert_close(torch.where(keep, y.float(), 0), torch.where(keep, ref, 0), rtol=tol, atol=tol)
    dy = torch.where(keep, torch.randn_like(ref), 0).to(dtype)
    y.backward(dy)
    ref.backward(dy.float())
    assert native.consume_status() == 0
    torch.testing.assert_close(xa.grad.float(), xr.grad, rtol=2 * tol, atol=4 * tol)


# ------------------------------------------------------------------------ top-k, sample losses
@pytest.mark.parametrize("k", [1, 5])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_topk_accuracy(k, dtype):
    torch.manual_seed(2)
    s = torch.randn(200, 1000, device="cuda").to(dtype)
    s[7] = s[7, 0]                       # ties: the lower index wins
    lab = torch.randint(0, 1000, (200,), device="cuda")
    lab[11] = 1000                       # out of range never counts
    got = nn.topk_accuracy(s, lab, k)
    sf = s.float()
    v = sf.gather(1, lab.clamp(max=999)[:, None])
    idx = torch.arange(1000, device="cuda")[None, :]
    rank = ((sf > v) | ((sf == v) & (idx < lab[:, None]))).sum(1)
    ref = ((rank < k) & (lab < 1000)).float()
    assert native.consume_status() == 0
    assert torch.equal(got, ref)


@pytest.mark.parametrize("kind", ["mean_squared_error", "mean_absolute_error", "l1_norm", "l2_norm2",
                                  "cross_entropy"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_sample_losses(kind, dtype):
    torch.manual_seed(3)
    n, d = 12, 777
    if kind == "cross_entropy":
        a = torch.softmax(torch.randn(n, d, device="cuda"), 1).to(dtype)
        b = F.one_hot(torch.randint(0, d, (n,), device="cuda"), d).to(dtype)
    else:
        a = torch.randn(n, d, device="cuda").to(dtype)
        b = torch.randn(n, d, device="cuda").to(dtype)
    unary_kind = kind in ("l1_norm", "l2_norm2")
    aa = a.clone().requires_grad_(True)
    ar = a.float().requires_grad_(True)
    got = nn.sample_loss(kind, aa, None if unary_kind else b)
    bf = b.float()
    ref = {
        "mean_squared_error": lambda: ((ar - bf) ** 2).mean(1),
        "mean_absolute_error": lambda: (ar - bf).abs().mean(1),
        "l1_norm": lambda: ar.abs().sum(1),
        "l2_norm2": lambda: (ar * ar).sum(1),
        "cross_entropy": lambda: torch.where(bf > 0, -bf * torch.log(ar), torch.zeros_like(ar)).sum(1),
    }[kind]()
    tol = 1e-4 if dtype == torch.float32 else 3e-3
    torch.testing.assert_close(got, ref, rtol=tol, atol=tol)
    g = torch.randn(n, device="cuda")
    got.backward(g)
    ref.backward(g)
    assert native.consume_status() == 0
    torch.testing.assert_close(aa.grad.float(), ar.grad, rtol=10 * tol, atol=10 * tol)


# ----------------------------------------------------------------------- element-wise tables
_POSITIVE = {"sqrt", "rsqrt", "log", "log1p", "acosh"}
_UNIT = {"acos", "asin", "atanh", "erfinv"}
_PARAMS = {"leaky_relu": (0.1, 0), "elu": (0.7, 0), "add_constant": (1.5, 0), "scale": (-2.0, 0),
           "subtract_constant": (0.5, 0), "constant_subtract": (0.5, 0), "max_constant": (0.2, 0),
           "min_constant": (0.2, 0), "equal_constant": (0.0, 0), "not_equal_constant": (0.0, 0),
           "less_constant": (0.1, 0), "less_equal_constant": (0.1, 0), "greater_constant": (0.1, 0),
           "greater_equal_constant": (0.1, 0), "clamp": (-0.5, 0.5)}


@pytest.mark.parametrize("name", [n for n in ew.UNARY if n in ew._CPU_UNARY])
def test_unary_table_forward_and_gradient(name):
    torch.manual_seed(4)
    x = torch.randn(4099, device="cuda")
    if name in _POSITIVE:
        x = x.abs() + (1.1 if name == "acosh" else 0.1)
    elif name in _UNIT:
        x = torch.rand(4099, device="cuda") * 1.8 - 0.9
    elif name in ("reciprocal", "safe_reciprocal"):
        x = x + torch.sign(x) * 0.2
    elif name in ("round", "ceil", "floor", "sign", "relu", "leaky_relu", "abs"):
        x = x + torch.sign(x) * 0.05          # stay off the kinks
    p0, p1 = _PARAMS.get(name, (0.0, 0.0))
    xa = x.clone().requires_grad_(True)
    xr = x.clone().requires_grad_(True)
    y = ew.unary(name, xa, p0, p1)
    ref = ew._CPU_UNARY[name](xr, p0, p1)
    torch.testing.assert_close(y, ref.to(y.dtype), rtol=2e-5, atol=2e-5)
    if ref.requires_grad:
        g = torch.randn_like(x)
        y.backward(g)
        ref.backward(g)
        torch.testing.assert_close(xa.grad, xr.grad, rtol=1e-4, atol=1e-4)
    assert native.consume_status() == 0


@pytest.mark.parametrize("name", [n for n in ew.BINARY if n in ew._CPU_BINARY])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_binary_table_forward_and_gradient(name, dtype):
    torch.manual_seed(5)
    a = torch.randn(2051, device="cuda")
    b = torch.randn(2051, device="cuda")
    if name in ("divide", "safe_divide", "mod"):
        b = b + torch.sign(b) * 0.3
    if name == "pow":
        a = a.abs() + 0.2
    if "cross_entropy" in name:
        b = torch.rand(2051, device="cuda")
        if name == "binary_cross_entropy":
            a = torch.rand(2051, device="cuda") * 0.9 + 0.05
    if name in ("equal", "not_equal", "less_equal", "greater_equal"):
        b[::3] = a[::3]
    a, b = a.to(dtype), b.to(dtype)
    aa, ba = a.clone().requires_grad_(True), b.clone().requires_grad_(True)
    ar, br = a.float().requires_grad_(True), b.float().requires_grad_(True)
    y = ew.binary(name, aa, ba)
    ref = ew._CPU_BINARY[name](ar, br)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    torch.testing.assert_close(y.float(), ref.float(), rtol=tol, atol=tol)
    if ref.requires_grad and name not in ("mod", "max", "min"):
        g = torch.randn(2051, device="cuda").to(dtype)
        y.backward(g)
        ref.backward(g.float())
        torch.testing.assert_close(aa.grad.float(), ar.grad, rtol=5 * tol, atol=5 * tol)
        if br.grad is not None:
            torch.testing.assert_close(ba.grad.float(), br.grad, rtol=5 * tol, atol=5 * tol)
    assert native.consume_status() == 0


# ------------------------------------------------------ strided / dilated convolution layers
@pytest.mark.parametrize("case", [
    # N, C, D, H, W, K, kernel, pad, stride, dilation
    (2, 32, 1, 30, 30, 64, 3, 1, 2, 1),
    (2, 16, 1, 29, 31, 32, 3, 1, 2, 1),        # odd extents: the data gradient needs output padding
    (1, 16, 6, 12, 12, 32, 3, 2, 1, 2),        # dilated 3-D
    (2, 64, 1, 14, 14, 128, 1, 0, 2, 1),       # 1x1 stride 2 (ResNet shortcut)
    (1, 32, 1, 56, 56, 32, 7, 3, 2, 1),        # 7x7 stride 2 (ResNet stem shape class)
    (1, 16, 8, 8, 8, 16, 3, 1, 2, 1),          # 3-D stride 2
])
def test_strided_and_dilated_convolution_gradients(case):
    N, C, D, H, W, K, k, pad, stride, dil = case
    torch.manual_seed(6)
    ks = (1 if D == 1 else k, k, k)
    pd = (0 if D == 1 else pad, pad, pad)
    st = (1 if D == 1 else stride, stride, stride)
    dl = (1 if D == 1 else dil, dil, dil)
    x = torch.randn(N, C, D, H, W, device="cuda").half()
    w = (torch.randn(K, C, *ks, device="cuda") / (C * k * k) ** 0.5).half().float()
    b = torch.randn(K, device="cuda")
    wh, bh = _handle(w), _handle(b)
    xa = x.clone().requires_grad_(True)
    y = nn.convolution(xa, wh, bh, ks, pd, st, dl)
    xr = x.float().requires_grad_(True)
    wr, br = w.clone().requires_grad_(True), b.clone().requires_grad_(True)
    ref = F.conv3d(xr, wr, br, st, pd, dl)
    assert y.shape == ref.shape
    torch.testing.assert_close(y.float(), ref, rtol=1e-2, atol=2e-2)
    dy = torch.randn_like(ref).half()
    y.backward(dy)
    ref.backward(dy.float())
    assert native.consume_status() == 0
    torch.testing.assert_close(xa.grad.float(), xr.grad, rtol=2e-2, atol=3e-2)
    scale = (ref.numel() / K) ** 0.5
    torch.testing.assert_close(wh.grad, wr.grad, rtol=2e-2, atol=4e-3 * scale)
    torch.testing.assert_close(bh.grad, br.grad, rtol=2e-2, atol=4e-3 * scale)


# ------------------------------------------------------------- long rows, vector kernels
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,cols", [(37, 4096), (300, 50304 // 8), (5, 2048 + 8)])
def test_softmax_cross_entropy_long_rows(rows, cols, dtype):
    """Vocabulary-sized rows take the one-pass 16-byte-load kernels."""
    torch.manual_seed(7)
    logits = (torch.randn(rows, cols, device="cuda") * 3).to(dtype).requires_grad_(True)
    labels = torch.randint(0, cols, (rows,), device="cuda")
    labels[1] = cols + 5                       # out of range: contributes nothing
    loss = nn.softmax_cross_entropy(logits, labels)
    lr = logits.detach().float().requires_grad_(True)
    ok = labels < cols
    ref = F.cross_entropy(lr, labels.clamp(max=cols - 1), reduction="none") * ok
    torch.testing.assert_close(loss, ref, rtol=1e-3, atol=2e-3)
    w = torch.rand(rows, device="cuda") + 0.5
    (loss * w).sum().backward()
    (ref * w).sum().backward()
    assert native.consume_status() == 0
    torch.testing.assert_close(logits.grad.float(), lr.grad, rtol=2e-2, atol=2e-3)


@pytest.mark.parametrize("rows,cols", [(4096, 2048), (1000, 520), (33, 64), (7, 8)])
def test_layer_norm_parameter_gradients_vector_kernel(rows, cols):
    torch.manual_seed(8)
    z = torch.randn(rows, cols, device="cuda").bfloat16().requires_grad_(True)
    sh, bh = _handle(torch.rand(cols, device="cuda") + 0.5), _handle(torch.randn(cols, device="cuda"))
    out = nn.layer_norm(z, cols, sh, bh, 1e-5)
    zr = z.detach().float().requires_grad_(True)
    sr, br = sh.master.detach().clone().requires_grad_(True), bh.master.detach().clone().requires_grad_(True)
    ref = F.layer_norm(zr, (cols,), sr, br, 1e-5)
    g = torch.randn_like(ref).bfloat16()
    out.backward(g)
    ref.backward(g.float())
    assert native.consume_status() == 0
    scale = rows ** 0.5
    torch.testing.assert_close(sh.grad, sr.grad, rtol=3e-2, atol=2e-2 * scale)
    torch.testing.assert_close(bh.grad, br.grad, rtol=3e-2, atol=2e-2 * scale)
    torch.testing.assert_close(z.grad.float(), zr.grad, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("name", ["gelu", "gelu_tanh", "sigmoid", "tanh", "leaky_relu", "exp"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_unary_operators_on_16_bit_tensors(name, dtype):
    torch.manual_seed(9)
    x = (torch.randn(1 << 20, device="cuda")).to(dtype)
    p0 = 0.1 if name == "leaky_relu" else 0.0
    xa = x.clone().requires_grad_(True)
    xr = x.float().requires_grad_(True)
    y = ew.unary(name, xa, p0, 0.0)
    ref = ew._CPU_UNARY[name](xr, p0, 0.0)
    torch.testing.assert_close(y.float(), ref, rtol=1e-2, atol=1e-2)
    g = torch.randn_like(ref).to(dtype)
    y.backward(g)
    ref.backward(g.float())
    assert native.consume_status() == 0
    torch.testing.assert_close(xa.grad.float(), xr.grad, rtol=2e-2, atol=2e-2)
