"""Forward + backward replayed from one CUDA graph must train exactly like the eager step."""
import copy

import pytest
import torch

from hipress_b200.models import bert_tiny, resnet_tiny, vgg_tiny
from hipress_b200.parallel import CompressedDataParallel, CompressionConfig, GraphedTrainStep
from hipress_b200.parallel.baseline import NcclDataParallel
from hipress_b200.parallel.powersgd import PowerSGDDataParallel

pytestmark = pytest.mark.gpu


def image_loss(module, x, y):
    with torch.autocast("cuda", dtype=torch.bfloat16):
        return torch.nn.functional.cross_entropy(module(x), y)


def batches(count, n=16, classes=10, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [(torch.randn(n, 3, 32, 32, generator=g).cuda(), torch.randint(0, classes, (n,), generator=g).cuda())
            for _ in range(count)]


@pytest.mark.parametrize("algorithm", ["dense", "tbq", "terngrad"])
def test_graphed_step_matches_eager(algorithm):
    torch.manual_seed(0)
    base = resnet_tiny(10).cuda().train()
    data = batches(6)

    def make():
        cfg = CompressionConfig(algorithm, bitwidth=2, enable_random=False, threshold=1e-3)
        return CompressedDataParallel(copy.deepcopy(base), cfg, lr=0.05, momentum=0.9, fused_sgd=True)

    eager, graphed = make(), make()
    eager_losses = []
    for x, y in data:
        loss = image_loss(eager, x, y)
        loss.backward()
        eager.step()
        eager_losses.append(float(loss.detach()))
    step = GraphedTrainStep(graphed, image_loss, data[0])
    graph_losses = [float(step(x, y).detach()) for x, y in data]
    eager.check()
    graphed.check()
    # same kernels in the same order on the same data; batch-norm statistics seen during the
    # capture warm-up only touch running averages, which training-mode forward does not read
    torch.testing.assert_close(torch.tensor(graph_losses), torch.tensor(eager_losses), atol=2e-2, rtol=0)
    if algorithm == "dense":
        torch.testing.assert_close(graphed.flat_param, eager.flat_param, atol=5e-3, rtol=0)


def test_graphed_powersgd_keeps_error_feedback_and_trains():
    torch.manual_seed(1)
    net = vgg_tiny(10).cuda().train()
    model = PowerSGDDataParallel(net, rank_r=4, lr=0.05, momentum=0.9)
    x, y = batches(1, n=32)[0]
    step = GraphedTrainStep(model, image_loss, (x, y))
    assert model.flat_M.abs().sum().item() == 0       # capture and its warm-up left no gradient behind
    losses = [float(step(x, y).detach()) for _ in range(30)]
    model.check()
    assert min(losses[-5:]) < losses[0] - 0.05, losses
    assert model.flat_M.abs().sum().item() > 0


def test_graphed_nccl_wrapper_and_bert():
    torch.manual_seed(2)
    net = bert_tiny().cuda().train()
    net.masked_capacity = 64          # >= the masked positions of any batch below (8 x 32 x ~0.15)
    model = NcclDataParallel(net, lr=1e-3, optimizer="adamw", weight_decay=0.01)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 1000, (8, 32), generator=g).cuda()
    labels = torch.where(torch.rand(8, 32, generator=g) < 0.15, ids.cpu(), torch.full((8, 32), -100)).cuda()
    assert int((labels >= 0).sum()) <= 64

    def loss_fn(module, a, b):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            return module(a, b)

    step = GraphedTrainStep(model, loss_fn, (ids, labels))
    losses = [float(step(ids, labels).detach()) for _ in range(20)]
    assert losses[-1] < losses[0], losses


def test_whole_step_capture_powersgd_matches_eager():
    """PowerSGD with the exchange inside the graph: one captured graph per accumulator parity,
    replayed in turn, flag values read from the device epoch."""
    torch.manual_seed(1)
    base = vgg_tiny(10).cuda().train()
    data = batches(7, n=32)

    def make(capturable):
        return PowerSGDDataParallel(copy.deepcopy(base), rank_r=4, lr=0.05, momentum=0.9, graph_capturable=capturable)

    eager, graphed = make(False), make(True)
    for x, y in data:
        image_loss(eager, x, y).backward()
        eager.step()
    step = GraphedTrainStep(graphed, image_loss, data[0])
    assert step.whole_step and step.variants == 2
    losses = [float(step(x, y).detach()) for x, y in data]
    eager.check()
    graphed.check()
    assert graphed.steps == eager.steps == len(data) and graphed.epoch == eager.epoch
    assert all(l == l for l in losses)
    torch.testing.assert_close(graphed.flat_param, eager.flat_param, atol=2e-2, rtol=0)
    torch.testing.assert_close(graphed.vec_param, eager.vec_param, atol=2e-2, rtol=0)
    assert (graphed.flat_param - eager.flat_param).abs().mean().item() < 1e-3
    # the error-feedback memory is carried across replays
    assert graphed.flat_M.abs().sum().item() > 0


@pytest.mark.parametrize("algorithm", ["tbq", "terngrad", "ecq", "dense"])
def test_whole_step_capture_matches_eager(algorithm):
    """Exchange captured inside the graph (epoch kept on the device): same parameters as the
    eager engine after every step, stochastic rounding included (same seed schedule)."""
    torch.manual_seed(0)
    base = resnet_tiny(10).cuda().train()
    data = batches(7)

    def make(capturable):
        cfg = CompressionConfig(algorithm, bitwidth=2, enable_random=True, threshold=1e-3, seed=5,
                                graph_capturable=capturable)
        return CompressedDataParallel(copy.deepcopy(base), cfg, lr=0.05, momentum=0.9, fused_sgd=True)

    eager, graphed = make(False), make(True)
    for x, y in data:
        image_loss(eager, x, y).backward()
        eager.step()
    step = GraphedTrainStep(graphed, image_loss, data[0])
    assert step.whole_step and step.launches_per_step > 0
    losses = [float(step(x, y).detach()) for x, y in data]
    eager.check()
    graphed.check()
    assert graphed.engine.steps == eager.engine.steps == len(data)
    if algorithm in ("tbq", "terngrad"):
        assert graphed.metrics()["kernel_launches"] == len(data) * step.launches_per_step
    # identical kernels on identical data; cuDNN may pick different algorithms for the two module
    # copies, and a last-bit difference can flip a stochastic rounding (one quantisation step of
    # one element): parameters agree to a few such steps.  (Bit-exactness of the device-epoch
    # protocol itself is covered by the engine tests against the CPU codec.)
    torch.testing.assert_close(graphed.flat_param, eager.flat_param, atol=5e-2, rtol=0)
    assert (graphed.flat_param - eager.flat_param).abs().mean().item() < 2e-3
    assert int(graphed.flat_grad.abs().sum()) == 0           # left cleared by the fused update
    assert all(l == l for l in losses)


def test_whole_step_capture_dgc_adamw():
    """DGC (momentum correction, clipping) with the fused AdamW: exchange and optimizer captured
    with the step; the step count of the bias correction comes from the device epoch."""
    from hipress_b200.parallel.dgc import DGCDataParallel
    torch.manual_seed(0)
    base = resnet_tiny(10).cuda().train()
    data = batches(6)

    def make(capturable):
        return DGCDataParallel(copy.deepcopy(base), keep_fraction=0.05, sample_rate=0.1, warmup_steps=0, lr=1e-3,
                               bucket_mb=0.05, graph_capturable=capturable)

    eager, graphed = make(False), make(True)
    for x, y in data:
        image_loss(eager, x, y).backward()
        eager.step()
    step = GraphedTrainStep(graphed, image_loss, data[0])
    assert step.whole_step
    losses = [float(step(x, y).detach()) for x, y in data]
    eager.check()
    graphed.check()
    assert graphed.engine.steps == eager.engine.steps == len(data)
    assert all(l == l for l in losses)
    # same selection rule, seeds and optimizer maths; cuDNN algorithm choice is the only freedom
    torch.testing.assert_close(graphed.flat_param, eager.flat_param, atol=2e-2, rtol=0)
    assert (graphed.flat_param - eager.flat_param).abs().mean().item() < 1e-3
