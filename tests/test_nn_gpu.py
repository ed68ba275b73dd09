"""Native differentiable ops (ops/nn.py) against PyTorch fp32 autograd on the same inputs."""
import pytest
import torch
import torch.nn.functional as F

from lbann_b200.ops import native, nn

pytestmark = pytest.mark.gpu


def _handle(t):
    m = t.clone().float().requires_grad_(True)
    g = torch.zeros_like(m)
    return nn.WeightHandle(m, g, None)


@pytest.mark.parametrize("shape", [(2, 4, 8, 16, 64), (1, 3, 6, 10, 136), (2, 8, 4, 8, 128), (2, 4, 1, 12, 40),
                                   (2, 4, 4, 6, 160), (1, 2, 3, 5, 48), (1, 4, 3, 4, 256)])
@pytest.mark.parametrize("kout", [32, 16])
def test_conv_c8_first_layer(shape, kout):
    N, C, D, H, W = shape
    torch.manual_seed(0)
    ks = (1, 3, 3) if D == 1 else (3, 3, 3)
    pad = (0, 1, 1) if D == 1 else (1, 1, 1)
    x = torch.randn(N, C, D, H, W, device="cuda").half()
    w = (torch.randn(kout, C, *ks, device="cuda") / 6).half().float()
    wh = _handle(w)
    y = nn.convolution(x, wh, None, ks, pad, (1, 1, 1), (1, 1, 1), act=native.ACT_LEAKY, act_param=0.3)
    assert native.consume_status() == 0
    wr = w.clone().requires_grad_(True)
    ref = F.leaky_relu(F.conv3d(x.float(), wr, None, 1, pad), 0.3)
    torch.testing.assert_close(y.float(), ref, rtol=1e-2, atol=2e-2)
    dy = torch.randn_like(ref).half()
    y.backward(dy)
    ref.backward(dy.float())
    assert native.consume_status() == 0
    scale = (N * D * H * W) ** 0.5
    torch.testing.assert_close(wh.grad, wr.grad, rtol=2e-2, atol=3e-2 * scale / 8)


@pytest.mark.parametrize("shape,pad_d,bias,dtype", [
    ((2, 4, 8, 16, 64), 1, False, torch.float16),      # one row tile, padding along depth
    ((1, 3, 6, 10, 144), 1, True, torch.float16),      # three channels, two row tiles, ragged second tile
    ((2, 4, 6, 4, 128), 0, True, torch.bfloat16),      # halo planes come with the input (no depth padding)
    ((3, 4, 4, 6, 272), 1, False, torch.bfloat16),
])
@pytest.mark.parametrize("kout", [32, 16])
def test_conv_c8_with_pooling_inside_the_kernel(shape, pad_d, bias, dtype, kout):
    """First-layer convolution + leaky ReLU + 2x2x2 max pooling in one kernel: the pooled
    tensor equals that of the two separate kernels bit for bit, the gradients agree with
    them up to the choice between values that round to the same 16-bit number, and both
    agree with PyTorch fp32."""
    N, C, D, H, W = shape
    torch.manual_seed(3)
    pad = (pad_d, 1, 1)
    x = torch.randn(N, C, D, H, W, device="cuda").to(dtype)
    w = (torch.randn(kout, C, 3, 3, 3, device="cuda") / 6).to(dtype).float()
    b = torch.randn(kout, device="cuda") / 4 if bias else None
    outs = []
    for fused in (True, False):
        wh = _handle(w)
        bh = _handle(b) if bias else None
        fuse = nn.PoolFusion() if fused else None
        y = nn.convolution(x, wh, bh, (3, 3, 3), pad, (1, 1, 1), (1, 1, 1), act=native.ACT_LEAKY,
                           act_param=0.3, skip_act_grad=True, fuse_pool=fuse)
        if fused:
            assert fuse.done
        else:
            y = nn.pooling(y, (2, 2, 2), (0, 0, 0), (2, 2, 2), "max", native.ACT_LEAKY, 0.3)
        assert native.consume_status() == 0
        torch.manual_seed(4)
        dy = torch.randn(y.shape, device="cuda").to(dtype)
        y.backward(dy)
        assert native.consume_status() == 0
        outs.append((y.detach(), wh.grad.clone(), bh.grad.clone() if bias else None, dy))
    (yf, gwf, gbf, dy), (yu, gwu, gbu, _) = outs
    assert torch.equal(yf, yu)
    # the fused kernel picks the arg-max on the fp32 accumulators, the pooling kernel on the
    # rounded tensor: where two values of a window round to the same number the gradient may
    # go to the other one
    assert (gwf - gwu).norm() <= (0.1 if dtype == torch.float16 else 0.3) * gwu.norm() + 1e-3
    if bias:
        torch.testing.assert_close(gbf, gbu, rtol=1e-3, atol=1e-2)
    wr = w.clone().requires_grad_(True)
    br = b.clone().requires_grad_(True) if bias else None
    ref = F.max_pool3d(F.leaky_relu(F.conv3d(x.float(), wr, br, 1, pad), 0.3), 2, 2)
    tol = dict(rtol=1e-2, atol=2e-2) if dtype == torch.float16 else dict(rtol=3e-2, atol=6e-2)
    torch.testing.assert_close(yf.float(), ref, **tol)
    ref.backward(dy.float())
    # like PyTorch in fp32, the fused kernel takes the arg-max before rounding: it follows the
    # reference closely, the separate kernels only up to their near-ties
    scale = (N * D * H * W) ** 0.5
    assert (gwf - wr.grad).norm() <= 0.02 * wr.grad.norm() + 1e-3 * scale
    assert (gwu - wr.grad).norm() <= (0.1 if dtype == torch.float16 else 0.3) * wr.grad.norm() + 1e-3 * scale


def test_pool_bwd_tiled_with_fused_activation():
    torch.manual_seed(1)
    x = torch.randn(2, 16, 8, 8, 8, device="cuda").half()
    xr = x.float().requires_grad_(True)
    xa = x.clone().requires_grad_(True)
    # x plays the role of an already-activated tensor: derivative from its sign
    y = nn.pooling(xa, (2, 2, 2), (0, 0, 0), (2, 2, 2), "max", native.ACT_LEAKY, 0.3)
    ref = F.max_pool3d(xr, 2, 2)
    torch.testing.assert_close(y.float(), ref)
    dy = torch.randn_like(ref)
    y.backward(dy.half())
    ref.backward(dy.half().float())
    expect = xr.grad * torch.where(x.float() > 0, 1.0, 0.3)
    torch.testing.assert_close(xa.grad.float(), expect, rtol=2e-3, atol=2e-3)


def test_linear_and_layer_norm_softmax_ce():
    torch.manual_seed(2)
    x = torch.randn(64, 256, device="cuda").bfloat16().requires_grad_(True)
    w = torch.randn(128, 256, device="cuda") / 16
    b = torch.randn(128, device="cuda")
    wh, bh = _handle(w.bfloat16().float()), _handle(b)
    y = nn.linear(x, wh, bh, native.ACT_RELU)
    xr = x.detach().float().requires_grad_(True)
    wr = wh.master.detach().clone().requires_grad_(True)
    br = b.clone().requires_grad_(True)
    ref = torch.relu(F.linear(xr, wr, br))
    torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=3e-2)
    g = torch.randn_like(ref).bfloat16()
    y.backward(g)
    ref.backward(g.float())
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=3e-2, atol=5e-2)
    torch.testing.assert_close(wh.grad, wr.grad, rtol=3e-2, atol=1e-1)
    torch.testing.assert_close(bh.grad, br.grad, rtol=3e-2, atol=1e-1)

    z = torch.randn(32, 512, device="cuda").bfloat16().requires_grad_(True)
    sh, bh2 = _handle(torch.rand(512, device="cuda") + 0.5), _handle(torch.randn(512, device="cuda"))
    out = nn.layer_norm(z, 512, sh, bh2, 1e-5)
    zr = z.detach().float().requires_grad_(True)
    sr, b2r = sh.master.detach().clone().requires_grad_(True), bh2.master.detach().clone().requires_grad_(True)
    refn = F.layer_norm(zr, (512,), sr, b2r, 1e-5)
    torch.testing.assert_close(out.float(), refn, rtol=2e-2, atol=3e-2)
    gn = torch.randn_like(refn).bfloat16()
    out.backward(gn)
    refn.backward(gn.float())
    torch.testing.assert_close(z.grad.float(), zr.grad, rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(sh.grad, sr.grad, rtol=3e-2, atol=1e-1)
    torch.testing.assert_close(bh2.grad, b2r.grad, rtol=3e-2, atol=1e-1)

    logits = torch.randn(40, 1000, device="cuda").bfloat16().requires_grad_(True)
    labels = torch.randint(0, 1000, (40,), device="cuda")
    labels[3] = 5000
    loss = nn.softmax_cross_entropy(logits, labels)
    lr = logits.detach().float().requires_grad_(True)
    ok = labels < 1000
    refl = F.cross_entropy(lr, labels.clamp(max=999), reduction="none") * ok
    torch.testing.assert_close(loss, refl, rtol=1e-3, atol=1e-3)
    loss.sum().backward()
    refl.sum().backward()
    torch.testing.assert_close(logits.grad.float(), lr.grad, rtol=2e-2, atol=2e-3)


def test_batch_norm_matches_reference_formula():
    torch.manual_seed(3)
    x = torch.randn(4, 32, 6, 6, 6, device="cuda").half().requires_grad_(True)
    sh, bh = _handle(torch.rand(32, device="cuda") + 0.5), _handle(torch.randn(32, device="cuda"))
    rm, rv = torch.zeros(32, device="cuda"), torch.ones(32, device="cuda")
    y = nn.batch_norm(x, sh, bh, rm, rv, True, 1e-5, 0.9, True)
    xr = x.detach().float().requires_grad_(True)
    s2, b2 = _handle(sh.master.detach()), _handle(bh.master.detach())
    rm2, rv2 = torch.zeros(32, device="cuda"), torch.ones(32, device="cuda")
    ref = nn.batch_norm(xr, s2, b2, rm2, rv2, True, 1e-5, 0.9, True)   # PyTorch-composed path (fp32)
    torch.testing.assert_close(y.float(), ref, rtol=1e-2, atol=2e-2)
    torch.testing.assert_close(rm, rm2, rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(rv, rv2, rtol=1e-3, atol=1e-3)
    g = torch.randn_like(ref).half()
    y.backward(g)
    ref.backward(g.float())
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(sh.grad, s2.master.grad, rtol=3e-2, atol=2e-1)
    torch.testing.assert_close(bh.grad, b2.master.grad, rtol=3e-2, atol=2e-1)


@pytest.mark.parametrize("fused", [True, False])
@pytest.mark.parametrize("shape,act", [((4, 32, 6, 6, 6), 0), ((3, 64, 9, 7), 1), ((2, 8, 5, 5, 5), 2)])
def test_batch_norm_against_fp64_restatement(monkeypatch, fused, shape, act):
    """Both batch-norm implementations (one cooperative kernel per direction, and the
    three-kernel sequence) against src/layers/regularizers/batch_normalization.cu:139-196
    written out independently in fp64 on the CPU: mean, variance with Bessel correction
    clamped from below by eps, eps added again inside the square root, running statistics,
    optional fused (leaky) ReLU; gradients from autograd of that formula."""
    if not fused:
        monkeypatch.setenv("LBANN_BN_SEPARATE_KERNELS", "1")
    torch.manual_seed(11)
    C = shape[1]
    x = (torch.randn(*shape, device="cuda") * 1.5 + 0.3).half()
    if len(shape) == 4:
        x = x.contiguous(memory_format=torch.channels_last)
    x.requires_grad_(True)
    sh, bh = _handle(torch.rand(C, device="cuda") + 0.5), _handle(torch.randn(C, device="cuda"))
    rm, rv = torch.zeros(C, device="cuda"), torch.ones(C, device="cuda")
    eps, decay, slope = 1e-5, 0.9, 0.2
    y = nn.batch_norm(x, sh, bh, rm, rv, True, eps, decay, True, act=act, act_param=slope)
    g = torch.randn(*shape, device="cuda").half()
    y.backward(g)
    # ---- fp64 restatement
    xd = x.detach().double().cpu().requires_grad_(True)
    sd = sh.master.detach().double().cpu().requires_grad_(True)
    bd = bh.master.detach().double().cpu().requires_grad_(True)
    dims = [0] + list(range(2, len(shape)))
    bshape = [1, C] + [1] * (len(shape) - 2)
    n = xd.numel() / C
    mean = xd.mean(dims)
    sq = (xd * xd).mean(dims)
    var = (sq - mean * mean) * n / (n - 1.0)
    var = torch.clamp(var, min=eps)
    yd = (xd - mean.view(bshape)) * torch.rsqrt(var + eps).view(bshape) * sd.view(bshape) + bd.view(bshape)
    if act == 1:
        yd = torch.relu(yd)
    elif act == 2:
        yd = torch.nn.functional.leaky_relu(yd, slope)
    yd.backward(g.double().cpu())
    torch.testing.assert_close(y.float().cpu(), yd.detach().float(), rtol=1e-2, atol=2e-2)
    torch.testing.assert_close(rm.cpu(), ((1 - decay) * mean.detach()).float(), rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(rv.cpu(), (decay + (1 - decay) * var.detach()).float(), rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(x.grad.float().cpu(), xd.grad.float(), rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(sh.grad.cpu(), sd.grad.float(), rtol=3e-2, atol=2e-1)
    torch.testing.assert_close(bh.grad.cpu(), bd.grad.float(), rtol=3e-2, atol=2e-1)
    assert native.consume_status(False) == 0


def test_fused_batch_norm_twice_in_a_row_and_changing_batch():
    """The fused kernels keep their barrier counters and accumulators in a per-layer
    workspace: a second call, and a call with another number of rows, still agree with the
    three-kernel sequence."""
    import os
    torch.manual_seed(5)
    C = 64
    sh, bh = _handle(torch.rand(C, device="cuda") + 0.5), _handle(torch.randn(C, device="cuda"))
    for n in (8, 8, 5, 8):
        x = torch.randn(n, C, 14, 14, device="cuda").half().contiguous(memory_format=torch.channels_last)
        outs = []
        for sep in ("", "1"):
            if sep:
                os.environ["LBANN_BN_SEPARATE_KERNELS"] = "1"
            else:
                os.environ.pop("LBANN_BN_SEPARATE_KERNELS", None)
            rm, rv = torch.zeros(C, device="cuda"), torch.ones(C, device="cuda")
            xi = x.clone().requires_grad_(True)
            y = nn.batch_norm(xi, sh, bh, rm, rv, True, 1e-5, 0.9, True, act=1)
            y.backward(torch.ones_like(y))
            outs.append((y.detach().float(), xi.grad.float(), rm, rv))
        os.environ.pop("LBANN_BN_SEPARATE_KERNELS", None)
        for a, b in zip(*outs):
            torch.testing.assert_close(a, b, rtol=1e-2, atol=1e-2)
    assert native.consume_status(False) == 0


def test_fused_optimizer_matches_cpu_formulas():
    from lbann_b200.ops.optim import ParameterArena
    torch.manual_seed(4)
    arenas = []
    for dev in ("cuda", "cpu"):
        a = ParameterArena(dev)
        s1 = a.reserve("a", (300,)); s2 = a.reserve("b", (17, 9)); s3 = a.reserve("c", (5,))
        a.materialise()
        s1.kind, s1.hp = "adam", {"learn_rate": 1e-2, "beta1": 0.9, "beta2": 0.95, "eps": 1e-8, "adamw_weight_decay": 0.1}
        s2.kind, s2.hp = "sgd", {"learn_rate": 0.1, "momentum": 0.9, "nesterov": True}
        s3.kind, s3.hp = "rmsprop", {"learn_rate": 0.01, "decay_rate": 0.9, "eps": 1e-8}
        arenas.append(a)
    g = torch.Generator().manual_seed(0)
    init = torch.randn(arenas[0].master.numel(), generator=g)
    for a in arenas:
        a.master.copy_(init)
    for step in range(3):
        grad = torch.randn(arenas[0].master.numel(), generator=g)
        if step == 1:
            grad[7] = float("inf")
        for a in arenas:
            a.grad.copy_(grad)
            a.step()
    torch.cuda.synchronize()
    torch.testing.assert_close(arenas[0].master.cpu(), arenas[1].master, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("rows,out_f,in_f,dt", [(8, 256, 2048, torch.float16), (4, 100, 36, torch.bfloat16),
                                                (16, 64, 520, torch.float16), (3, 64, 128, torch.float16)])
def test_short_batch_weight_gradient(rows, out_f, in_f, dt):
    """grad += dy^T x for mini-batches of a few rows (rank-K update kernel; 3 rows falls back
    to the tensor-core GEMM) against fp32 matmul, accumulating onto a non-zero gradient."""
    torch.manual_seed(1)
    dy = torch.randn(rows, out_f, device="cuda").to(dt)
    x = torch.randn(rows, in_f, device="cuda").to(dt)
    grad = torch.randn(out_f, in_f, device="cuda")
    want = grad + dy.float().t() @ x.float()
    nn._weight_grad(dy, x, grad)
    assert native.consume_status() == 0
    torch.testing.assert_close(grad, want, rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("classes", [3, 7, 32])
def test_softmax_cross_entropy_with_few_classes(classes):
    """Per-voxel cross-entropy over a handful of classes (thread-per-row kernels) against
    PyTorch fp32, with an out-of-range label giving a zero loss and a zero gradient row."""
    torch.manual_seed(2)
    rows = 8200
    logits = torch.randn(rows, classes, device="cuda").bfloat16().requires_grad_(True)
    labels = torch.randint(0, classes, (rows,), device="cuda")
    labels[11] = classes + 4
    loss = nn.softmax_cross_entropy(logits, labels)
    assert native.consume_status() == 0
    lr = logits.detach().float().requires_grad_(True)
    ok = labels < classes
    ref = F.cross_entropy(lr, labels.clamp(max=classes - 1), reduction="none") * ok
    torch.testing.assert_close(loss, ref, rtol=1e-3, atol=1e-3)
    w = torch.rand(rows, device="cuda")
    (loss * w).sum().backward()
    (ref * w).sum().backward()
    torch.testing.assert_close(logits.grad.float(), lr.grad, rtol=2e-2, atol=2e-3)
    assert float(logits.grad[11].abs().max()) == 0.0


def test_add_relu_fused_kernel():
    """relu(a + b) in one kernel, gradient masked by the saved output and shared by both
    inputs; plain add passes its gradient through without a kernel."""
    from lbann_b200.ops import elementwise as ew
    torch.manual_seed(4)
    a = torch.randn(4, 16, 8, 8, device="cuda").bfloat16().requires_grad_(True)
    b = torch.randn(4, 16, 8, 8, device="cuda").bfloat16().requires_grad_(True)
    ar, br = a.detach().float().requires_grad_(True), b.detach().float().requires_grad_(True)
    y = ew.add_relu(a, b)
    ref = torch.relu((ar + br).bfloat16().float())
    torch.testing.assert_close(y.float(), ref, rtol=1e-2, atol=1e-2)
    g = torch.randn_like(y)
    y.backward(g)
    torch.relu(ar + br).backward(g.float())
    torch.testing.assert_close(a.grad.float(), ar.grad, rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(b.grad.float(), br.grad, rtol=1e-2, atol=1e-2)
    n0 = native.launches()
    c = torch.randn_like(a).requires_grad_(True)
    d = torch.randn_like(a).requires_grad_(True)
    s = ew.binary("add", c, d)
    n1 = native.launches()
    s.backward(g)
    assert native.launches() == n1 and n1 == n0 + 1
    torch.testing.assert_close(c.grad, g)
    assert native.consume_status() == 0


def test_sharded_update_with_state_for_owned_blocks_only():
    """Two ranks emulated on one GPU (each its own arena; the 'peer' master is the other
    arena's): every rank keeps Adam moments for its own blocks only (half the bytes), updates
    them and stores the new values into both masters.  Masters and the gathered moments equal
    an unsharded arena's after three steps."""
    from lbann_b200.ops.native import c_void_p
    from lbann_b200.ops.optim import ArenaShard, CHUNK, OWN_CHUNKS, ParameterArena
    torch.manual_seed(5)
    n1, n2 = 3 * OWN_CHUNKS * CHUNK + 777, 2 * OWN_CHUNKS * CHUNK - 55

    def make():
        a = ParameterArena("cuda", compute_dtype=torch.bfloat16)
        s1, s2 = a.reserve("a", (n1,)), a.reserve("b", (n2,))
        a.materialise()
        s1.kind, s1.hp = "adam", {"learn_rate": 1e-2, "beta1": 0.9, "beta2": 0.95, "eps": 1e-8}
        s2.kind, s2.hp = "sgd", {"learn_rate": 0.1, "momentum": 0.9}
        return a
    ref, ranks = make(), [make(), make()]
    init = torch.randn(ref.master.numel(), device="cuda")
    for a in [ref] + ranks:
        a.master.copy_(init)
        a.ensure_state1()
    peers = (c_void_p * 2)(ranks[0].master.data_ptr(), ranks[1].master.data_ptr())
    for r, a in enumerate(ranks):
        a.shard = ArenaShard(r, 2, peers)
        full_bytes = a.state_bytes()
        a.compact_state()
        assert a.state_bytes() <= 0.62 * full_bytes
    for step in range(3):
        grad = torch.randn(ref.master.numel(), device="cuda")
        for a in [ref] + ranks:
            a.grad.copy_(grad)
            a.step()
        torch.cuda.synchronize()
    assert native.consume_status(False) == 0
    for a in ranks:
        torch.testing.assert_close(a.master, ref.master, rtol=1e-6, atol=1e-7)
    for which, want in ((0, ref.state0), (1, ref.state1)):
        got = sum(a._unpack_state(a.state0 if which == 0 else a.state1) for a in ranks)
        if which == 1:      # the second moment exists for the Adam tensor only
            got, want = got[:n1], want[:n1]
        torch.testing.assert_close(got[:want.numel()], want, rtol=1e-6, atol=1e-7)
