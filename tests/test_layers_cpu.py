"""The model-zoo layers away from their CUDA kernels: CPU tensors (and anything else the kernels do
not cover) must take the stock PyTorch path with identical semantics and state-dict layout."""
import torch
import torch.nn as nn
import torch.nn.functional as F

from hipress_b200.models import bert_tiny, resnet_tiny, vgg_tiny
from hipress_b200.models.layers import (FusedAddLayerNorm, FusedBatchNormAct, FusedBiasReLU, FusedLinear,
                                        MaxPool3x3s2)


def test_fused_batch_norm_is_batch_norm_on_cpu():
    torch.manual_seed(0)
    fused, stock = FusedBatchNormAct(16, relu=True), nn.BatchNorm2d(16)
    assert set(fused.state_dict()) == set(stock.state_dict())       # drop-in for checkpoints
    stock.load_state_dict(fused.state_dict())
    x, res = torch.randn(4, 16, 5, 5), torch.randn(4, 16, 5, 5)
    torch.testing.assert_close(fused(x, res), F.relu(stock(x) + res))
    torch.testing.assert_close(fused.running_mean, stock.running_mean)
    torch.testing.assert_close(fused.running_var, stock.running_var)
    assert int(fused.num_batches_tracked) == 1
    fused.eval(), stock.eval()
    torch.testing.assert_close(fused(x), F.relu(stock(x)))


def test_bias_relu_pool_on_cpu():
    torch.manual_seed(0)
    layer = FusedBiasReLU(6, pool=True)
    with torch.no_grad():
        layer.bias.uniform_(-1, 1)
    x = torch.randn(2, 6, 8, 8, requires_grad=True)
    y = layer(x)
    torch.testing.assert_close(y, F.max_pool2d(F.relu(x + layer.bias.view(1, -1, 1, 1)), 2, 2))
    y.sum().backward()
    assert layer.bias.grad is not None and x.grad is not None
    assert FusedBiasReLU(6)(x).shape == x.shape


def test_add_layer_norm_and_linear_on_cpu():
    torch.manual_seed(0)
    ln = FusedAddLayerNorm(24, eps=1e-12)
    x, d = torch.randn(3, 5, 24), torch.randn(3, 5, 24)
    torch.testing.assert_close(ln(x, d), F.layer_norm(x + d, (24,), ln.weight, ln.bias, 1e-12))
    torch.testing.assert_close(ln(x), F.layer_norm(x, (24,), ln.weight, ln.bias, 1e-12))
    assert set(ln.state_dict()) == set(nn.LayerNorm(24).state_dict())
    lin = FusedLinear(24, 10)
    torch.testing.assert_close(lin(x), F.linear(x, lin.weight, lin.bias))
    assert set(lin.state_dict()) == set(nn.Linear(24, 10).state_dict())


def test_max_pool_on_cpu():
    x = torch.randn(2, 8, 9, 11)
    assert torch.equal(MaxPool3x3s2()(x), F.max_pool2d(x, 3, stride=2, padding=1))


def test_models_keep_their_parameter_counts():
    from hipress_b200.models import resnet50, vgg19
    assert sum(p.numel() for p in resnet50().parameters()) == 25_557_032
    assert sum(p.numel() for p in vgg19().parameters()) == 143_667_240


def test_tiny_models_train_on_cpu():
    torch.manual_seed(0)
    for net, batch in ((resnet_tiny(10), (torch.randn(4, 3, 32, 32), torch.randint(0, 10, (4,)))),
                       (vgg_tiny(10), (torch.randn(4, 3, 32, 32), torch.randint(0, 10, (4,))))):
        opt = torch.optim.SGD(net.parameters(), lr=0.05)
        first = last = None
        for _ in range(8):
            opt.zero_grad()
            loss = F.cross_entropy(net(batch[0]), batch[1])
            loss.backward()
            opt.step()
            first = float(loss.detach()) if first is None else first
            last = float(loss.detach())
        assert last < first
    bert = bert_tiny()
    ids = torch.randint(0, 1000, (2, 16))
    labels = torch.where(torch.rand(2, 16) < 0.3, ids, torch.full((2, 16), -100))
    labels[0, 0] = ids[0, 0]
    plain = float(bert(ids, labels).detach())
    bert.masked_capacity = 32                       # fixed-shape selection used under CUDA graphs
    assert abs(float(bert(ids, labels).detach()) - plain) < 1e-5
