"""Fused layer kernels (batch norm + residual + ReLU, max pooling, bias + ReLU + pooling) against
plain PyTorch fp32 restatements of the same ops."""
import pytest
import torch
import torch.nn.functional as F

from hipress_b200 import _C
from hipress_b200.models import resnet_tiny
from hipress_b200.models.layers import FusedBatchNormAct

pytestmark = pytest.mark.gpu


def reference(x, res, w, b, relu, eps=1e-5):
    """fp32 autograd restatement on the bf16-rounded inputs."""
    xf = x.float().detach().requires_grad_(True)
    rf = res.float().detach().requires_grad_(True) if res is not None else None
    wf, bf = w.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    y = F.batch_norm(xf, None, None, wf, bf, True, 0.1, eps)
    if rf is not None:
        y = y + rf
    if relu:
        y = F.relu(y)
    return xf, rf, wf, bf, y


@pytest.mark.parametrize("shape", [(4, 64, 56, 56), (3, 8, 7, 5), (2, 16, 9, 9), (5, 32, 6, 6),
                                    (2, 256, 14, 14), (2, 512, 7, 7), (1, 2048, 7, 7), (64, 128, 28, 28)])
@pytest.mark.parametrize("relu,residual", [(False, False), (True, False), (True, True), (False, True)])
def test_forward_backward_match_fp32_reference(shape, relu, residual):
    torch.manual_seed(0)
    n, c, h, w_ = shape
    x = (torch.randn(shape, device="cuda") * 1.7 + 0.4).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    res = torch.randn(shape, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last) if residual else None
    layer = FusedBatchNormAct(c, relu=relu).cuda().train()
    with torch.no_grad():
        layer.weight.uniform_(0.5, 1.5)
        layer.bias.uniform_(-0.5, 0.5)
    xg = x.clone().requires_grad_(True)
    rg = res.clone().requires_grad_(True) if residual else None
    y = layer(xg, rg)
    assert y.dtype == torch.bfloat16 and y.is_contiguous(memory_format=torch.channels_last)
    dy = torch.randn(shape, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    y.backward(dy)

    xf, rf, wf, bf, yr = reference(x, res, layer.weight, layer.bias, relu)
    # the fused kernel masks with the bf16-rounded output; do the same in the restatement
    yr.backward(dy.float())
    torch.testing.assert_close(y.float(), yr, atol=3e-2, rtol=2e-2)          # bf16 output rounding
    m = float(n * h * w_)
    torch.testing.assert_close(xg.grad.float(), xf.grad, atol=3e-2 * float(xf.grad.abs().max()) + 1e-3, rtol=3e-2)
    scale = (m ** 0.5)
    torch.testing.assert_close(layer.weight.grad, wf.grad, atol=2e-2 * scale, rtol=2e-2)
    torch.testing.assert_close(layer.bias.grad, bf.grad, atol=2e-2 * scale, rtol=2e-2)
    if residual:
        torch.testing.assert_close(rg.grad.float(), rf.grad, atol=1e-2, rtol=1e-2)
    # running statistics follow nn.BatchNorm2d (unbiased variance, momentum 0.1)
    xm = x.float().transpose(0, 1).reshape(c, -1)
    torch.testing.assert_close(layer.running_mean, 0.1 * xm.mean(1), atol=1e-4, rtol=1e-4)
    torch.testing.assert_close(layer.running_var, 0.9 + 0.1 * xm.var(1, unbiased=True), atol=1e-4, rtol=1e-4)
    assert int(layer.num_batches_tracked) == 1


def test_statistics_survive_a_large_mean():
    """Variance of data with |mean| >> std: the per-block + Chan combination must not cancel."""
    torch.manual_seed(1)
    shape = (8, 64, 28, 28)
    x = (torch.randn(shape, device="cuda") * 0.25 + 40.0).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    _, stats = _C.bn_forward(x, None, None, None, None, None, None, 0.1, 1e-5, False)
    xm = x.double().transpose(0, 1).reshape(64, -1)
    torch.testing.assert_close(stats[0].double(), xm.mean(1), atol=1e-4, rtol=1e-6)
    invstd = 1.0 / torch.sqrt(xm.var(1, unbiased=False) + 1e-5)
    torch.testing.assert_close(stats[1].double(), invstd, atol=0, rtol=2e-3)


def test_unsupported_inputs_take_the_stock_path():
    layer = FusedBatchNormAct(12, relu=True).cuda().train()     # 12 channels: not a multiple of 8
    x = torch.randn(2, 12, 5, 5, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    assert not _C.bn_supported(x)
    y = layer(x)
    assert y.shape == x.shape and float(y.min()) >= 0
    layer64 = FusedBatchNormAct(64, relu=False).cuda().train()
    xf = torch.randn(2, 64, 5, 5, device="cuda")                 # fp32 activations
    ref = F.batch_norm(xf, None, None, layer64.weight, layer64.bias, True, 0.1, 1e-5)
    torch.testing.assert_close(layer64(xf), ref)
    layer64.eval()
    xb = xf.to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    assert layer64(xb).shape == xb.shape


def test_resnet_with_fused_layers_matches_stock_layers():
    """Same tiny ResNet, once through the fused kernels (bf16 channels-last) and once with the
    layers forced onto the stock path: losses and input-layer gradients agree to bf16 accuracy."""
    torch.manual_seed(0)
    net = resnet_tiny(10).cuda().to(memory_format=torch.channels_last).train()
    x = torch.randn(16, 3, 64, 64, device="cuda").contiguous(memory_format=torch.channels_last)
    y = torch.randint(0, 10, (16,), device="cuda")

    def run(fused):
        net.zero_grad(set_to_none=True)
        saved = FusedBatchNormAct._fused_ok
        if not fused:
            FusedBatchNormAct._fused_ok = lambda self, a, b: False
        try:
            with torch.autocast("cuda", dtype=torch.bfloat16):
                loss = F.cross_entropy(net(x), y)
            loss.backward()
        finally:
            FusedBatchNormAct._fused_ok = saved
        return float(loss.detach()), net.conv1.weight.grad.clone(), net.fc.weight.grad.clone()

    l1, g1, f1 = run(True)
    l0, g0, f0 = run(False)
    assert abs(l1 - l0) < 3e-2, (l1, l0)
    cos = lambda a, b: float((a * b).sum() / (a.norm() * b.norm() + 1e-12))
    assert cos(f1, f0) > 0.99 and cos(g1, g0) > 0.95, (cos(f1, f0), cos(g1, g0))


@pytest.mark.parametrize("shape", [(2, 64, 112, 112), (3, 8, 7, 9), (1, 16, 1, 1), (2, 32, 10, 5)])
def test_maxpool_matches_torch(shape):
    from hipress_b200.models.layers import MaxPool3x3s2
    torch.manual_seed(0)
    x = torch.randn(shape, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    xg = x.clone().requires_grad_(True)
    y = MaxPool3x3s2()(xg)
    xr = x.float().requires_grad_(True)
    yr = F.max_pool2d(xr, 3, stride=2, padding=1)
    assert y.shape == yr.shape and y.is_contiguous(memory_format=torch.channels_last)
    assert torch.equal(y.float(), yr)                         # a maximum of bf16 values is exact
    dy = torch.randn(y.shape, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    y.backward(dy)
    yr.backward(dy.float())
    # up to four bf16 gradients summed in fp32, rounded once
    torch.testing.assert_close(xg.grad.float(), xr.grad, atol=2e-2, rtol=1e-2)


def test_maxpool_falls_back_for_other_inputs():
    from hipress_b200.models.layers import MaxPool3x3s2
    x = torch.randn(2, 6, 9, 9, device="cuda")
    assert torch.equal(MaxPool3x3s2()(x), F.max_pool2d(x, 3, stride=2, padding=1))


@pytest.mark.parametrize("shape", [(2, 64, 32, 32), (3, 8, 6, 10), (1, 512, 14, 14), (2, 256, 8, 8)])
@pytest.mark.parametrize("pool", [False, True])
def test_bias_relu_pool_matches_fp32_reference(shape, pool):
    from hipress_b200.models.layers import FusedBiasReLU
    torch.manual_seed(0)
    c = shape[1]
    x = torch.randn(shape, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    layer = FusedBiasReLU(c, pool=pool).cuda()
    with torch.no_grad():
        layer.bias.uniform_(-0.5, 0.5)
    xg = x.clone().requires_grad_(True)
    y = layer(xg)
    xr = x.float().requires_grad_(True)
    br = layer.bias.detach().clone().requires_grad_(True)
    yr = F.relu(xr + br.view(1, -1, 1, 1))
    if pool:
        yr = F.max_pool2d(yr, 2, 2)
    assert y.shape == yr.shape and y.dtype == torch.bfloat16
    torch.testing.assert_close(y.float(), yr, atol=2e-2, rtol=1e-2)       # one bf16 rounding
    dy = torch.randn(y.shape, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    y.backward(dy)
    yr.backward(dy.float())
    # gradients are dy or 0: exact wherever the bf16-rounded output and the fp32 output agree on
    # y > 0 (an output that rounds to exactly 0 cannot: relu(x + b) > 0 never rounds to 0 in bf16)
    assert torch.equal(xg.grad.float(), xr.grad)
    torch.testing.assert_close(layer.bias.grad, br.grad, atol=1e-3, rtol=1e-4)


def test_vgg_with_fused_epilogues_trains():
    from hipress_b200.models import vgg_tiny
    torch.manual_seed(0)
    net = vgg_tiny(10).cuda().to(memory_format=torch.channels_last).train()
    opt = torch.optim.SGD(net.parameters(), lr=0.05, momentum=0.9)
    x = torch.randn(32, 3, 32, 32, device="cuda").contiguous(memory_format=torch.channels_last)
    y = torch.randint(0, 10, (32,), device="cuda")
    losses = []
    for _ in range(30):
        opt.zero_grad()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = F.cross_entropy(net(x), y)
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    assert losses[-1] < losses[0] - 0.05, losses        # a tiny VGG without normalisation learns slowly
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in net.parameters())


@pytest.mark.parametrize("shape", [(4, 128, 1024), (3, 7, 64), (5, 256), (2, 33, 1536), (1, 9, 2048), (6, 40)])
@pytest.mark.parametrize("with_delta", [True, False])
def test_add_layer_norm_matches_fp32_reference(shape, with_delta):
    from hipress_b200.models.layers import FusedAddLayerNorm
    torch.manual_seed(0)
    h = shape[-1]
    x = (torch.randn(shape, device="cuda") * 1.3 + 0.2).to(torch.bfloat16)
    d = torch.randn(shape, device="cuda").to(torch.bfloat16) if with_delta else None
    layer = FusedAddLayerNorm(h, eps=1e-12).cuda()
    with torch.no_grad():
        layer.weight.uniform_(0.5, 1.5)
        layer.bias.uniform_(-0.5, 0.5)
    xg = x.clone().requires_grad_(True)
    dg = d.clone().requires_grad_(True) if with_delta else None
    y = layer(xg, dg)
    assert y.dtype == torch.bfloat16 and y.shape == x.shape
    dy = torch.randn(shape, device="cuda").to(torch.bfloat16)
    y.backward(dy)

    # restatement: the sum rounded to bf16 (what the kernel normalises), everything else fp32
    z = (x.float() + d.float()).to(torch.bfloat16).float() if with_delta else x.float()
    zr = z.detach().requires_grad_(True)
    wr, br = layer.weight.detach().clone().requires_grad_(True), layer.bias.detach().clone().requires_grad_(True)
    yr = F.layer_norm(zr, (h,), wr, br, 1e-12)
    yr.backward(dy.float())
    torch.testing.assert_close(y.float(), yr, atol=3e-2, rtol=2e-2)
    torch.testing.assert_close(xg.grad.float(), zr.grad, atol=3e-2, rtol=3e-2)
    if with_delta:
        assert torch.equal(dg.grad, xg.grad)
    rows = x.numel() // h
    torch.testing.assert_close(layer.weight.grad, wr.grad, atol=2e-3 * rows ** 0.5 + 1e-3, rtol=1e-3)
    torch.testing.assert_close(layer.bias.grad, br.grad, atol=2e-3 * rows ** 0.5 + 1e-3, rtol=1e-3)


def test_add_layer_norm_stock_path_for_fp32():
    from hipress_b200.models.layers import FusedAddLayerNorm
    layer = FusedAddLayerNorm(48).cuda()
    x, d = torch.randn(4, 48, device="cuda"), torch.randn(4, 48, device="cuda")
    torch.testing.assert_close(layer(x, d), F.layer_norm(x + d, (48,), layer.weight, layer.bias, layer.eps))


def test_bert_tiny_trains_on_bf16_residual_stream():
    from hipress_b200.models import bert_tiny
    torch.manual_seed(0)
    net = bert_tiny().cuda().train()
    opt = torch.optim.AdamW(net.parameters(), lr=1e-3)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 1000, (8, 32), generator=g).cuda()
    labels = torch.where(torch.rand(8, 32, generator=g) < 0.15, ids.cpu(), torch.full((8, 32), -100)).cuda()
    losses = []
    for _ in range(30):
        opt.zero_grad()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = net(ids, labels)
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    assert losses[-1] < losses[0] - 0.5, losses
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in net.parameters())


@pytest.mark.parametrize("shape,out", [((4, 128, 1024), 1024), ((3, 7, 64), 256), ((40, 64), 8), ((2, 5, 96), 100)])
def test_fused_linear_matches_autocast_linear(shape, out):
    from hipress_b200.models.layers import FusedLinear
    torch.manual_seed(0)
    fused = FusedLinear(shape[-1], out).cuda()
    stock = torch.nn.Linear(shape[-1], out).cuda()
    stock.load_state_dict(fused.state_dict())
    x = torch.randn(shape, device="cuda").to(torch.bfloat16)
    dy = torch.randn(*shape[:-1], out, device="cuda").to(torch.bfloat16)
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        ya, yb = fused(xa), stock(xb)
    assert ya.dtype == torch.bfloat16
    torch.testing.assert_close(ya, yb, atol=2e-2, rtol=2e-2)
    ya.backward(dy)
    yb.backward(dy)
    assert fused.weight.grad.dtype == torch.float32 and fused.bias.grad.dtype == torch.float32
    torch.testing.assert_close(xa.grad, xb.grad, atol=5e-2, rtol=2e-2)
    # fp32 accumulation and output here, bf16-rounded output in the stock path
    ref_w = dy.reshape(-1, out).float().t() @ x.reshape(-1, shape[-1]).float()
    torch.testing.assert_close(fused.weight.grad, ref_w, atol=2e-2 * ref_w.abs().max().item(), rtol=2e-2)
    torch.testing.assert_close(fused.bias.grad, dy.reshape(-1, out).float().sum(0), atol=1e-2, rtol=1e-3)


@pytest.mark.parametrize("tokens,in_f,out_f", [(4096, 1024, 1024), (4096, 1024, 4096), (4096, 4096, 1024), (21, 64, 256)])
def test_linear_wgrad_bgrad_matches_fp32(tokens, in_f, out_f):
    """Weight gradient and bias gradient from one GEMM (bias-gradient epilogue) against fp32 products of the
    same bf16 operands; shapes of BERT-large's attention and feed-forward layers plus a small ragged one."""
    import hipress_b200 as hp
    torch.manual_seed(tokens + in_f + out_f)
    dy = torch.randn(tokens, out_f, device="cuda").to(torch.bfloat16)
    x = torch.randn(tokens, in_f, device="cuda").to(torch.bfloat16)
    both = hp._C.linear_wgrad_bgrad(dy, x)
    if not both:
        pytest.skip("the GEMM library offers no bias-gradient epilogue for this shape; the two-kernel path runs")
    dw, db = both
    assert dw.dtype == torch.float32 and db.dtype == torch.float32 and dw.shape == (out_f, in_f) and db.shape == (out_f,)
    ref_w = dy.float().t() @ x.float()
    torch.testing.assert_close(dw, ref_w, atol=1e-3 * ref_w.abs().max().item(), rtol=1e-3)
    torch.testing.assert_close(db, dy.float().sum(0), atol=1e-3 * (tokens ** 0.5), rtol=1e-3)
    # a second call of the same shape reuses the cached plan and gives the same bits
    dw2, db2 = hp._C.linear_wgrad_bgrad(dy, x)
    assert torch.equal(dw, dw2) and torch.equal(db, db2)
