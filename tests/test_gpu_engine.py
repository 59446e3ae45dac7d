"""The DDP engine on one GPU: world 1 end to end, and several ranks emulated in one process.

Emulated ranks share one device, so no kernel may wait for a kernel that is not yet running.
The engines are built with ``defer_recv``: ``bucket_ready`` only issues the compress-and-push
half; the test synchronises the device once every rank has pushed, and only then lets
``finish_step`` issue the flag waits (which find their flags already published) and unpacks.
"""
import pytest
import torch

import hipress_b200 as hp
from hipress_b200 import ops
from hipress_b200.models import resnet_tiny
from hipress_b200.parallel import CompressedDataParallel, CompressionConfig, SymmetricMemory, plan_buckets

pytestmark = pytest.mark.gpu


def gauss(n, std=0.01, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(n, generator=g) * std


def make_engines(codec, world, n, **kw):
    cfgs = [dict(rank=r, world=world, device=0, codec=codec, seed=3, flag_timeout_s=2.0, defer_recv=1, **kw)
            for r in range(world)]
    engines = [hp._C.DdpEngine(c, [(0, n, 1)], [0]) for c in cfgs]
    mems = SymmetricMemory.emulate(engines[0].symmetric_bytes, world)
    return engines, mems


@pytest.mark.parametrize("codec,kw", [
    ("terngrad", dict(bitwidth=2, enable_random=1, error_feedback=1)),
    ("terngrad", dict(bitwidth=4, enable_random=0, error_feedback=0)),
    ("tbq", dict(threshold=0.01)),
    # epoch, slot parity and rounding seed resolved on the device (CUDA-graph capturable steps)
    ("terngrad", dict(bitwidth=2, enable_random=1, error_feedback=1, device_epoch=1, num_workers=0)),
    ("tbq", dict(threshold=0.01, device_epoch=1, num_workers=0)),
    ("graddrop", dict(keep_fraction=0.01, sample_rate=0.05, device_epoch=1, num_workers=0)),
    ("graddrop", dict(keep_fraction=0.01, sample_rate=0.05)),
    ("ecq", dict(bitwidth=4, alpha=1.0, beta=0.9)),
    ("ecq", dict(bitwidth=2, alpha=1.0, beta=0.9, device_epoch=1, num_workers=0)),
    ("dense", dict()),
])
@pytest.mark.parametrize("world,n", [(1, 100000 + 12), (2, 100000 + 12), (4, 100000 + 12), (3, 4099), (8, 50000 + 7),
                                     # large enough for the chunked compress path (16-byte peer stores)
                                     (2, 700000 + 12), (8, 620000 + 5)])
def test_engine_matches_cpu_codec(codec, kw, world, n):
    if n > 200000 and codec not in ("terngrad", "tbq"):
        pytest.skip("the chunked path exists for tbq and terngrad")
    engines, mems = make_engines(codec, world, n, **kw)
    grads = [gauss(n, seed=10 + r).cuda() for r in range(world)]
    resid = [torch.zeros(n, device="cuda") for _ in range(world)]
    for e, m, g, r in zip(engines, mems, grads, resid):
        e.set_buffers(g, r, None, None)
        e.set_symmetric(m.buf)
        e.set_sgd(0.0, 0.0, 0.0, False)
    cpu_grads = [g.cpu().clone() for g in grads]
    cpu_resid = [torch.zeros(n) for _ in range(world)]
    for step in range(2):
        for e in engines:
            e.begin_step()
        # every rank pushes before any rank's step is finished
        for e in engines:
            e.bucket_ready(0, 0)
        for e in engines:
            e.drain()
        torch.cuda.synchronize()   # all payloads delivered, all flags published
        for e in engines:
            e.finish_step(0)
        torch.cuda.synchronize()
        for e in engines:
            assert e.check_status() == 0
        # CPU restatement with the engine's seed schedule
        epoch = step + 1
        seed = (3 + epoch * 0x9E3779B97F4A7C15) % (1 << 64)
        seed_signed = seed - (1 << 64) if seed >= (1 << 63) else seed
        payloads = []
        for r in range(world):
            g, res = cpu_grads[r], cpu_resid[r]
            if codec == "terngrad":
                payloads.append(ops.terngrad_compress(g, kw["bitwidth"], bool(kw["enable_random"]), seed_signed,
                                                      residual=res if kw["error_feedback"] else None))
            elif codec == "tbq":
                payloads.append(ops.tbq_compress(g, res, kw["threshold"]))
            elif codec == "graddrop":
                payloads.append(ops.graddrop_compress(g, res, kw["sample_rate"], 1 - kw["keep_fraction"], seed_signed))
            elif codec == "ecq":
                payloads.append(ops.ecq_compress(g, res, kw["alpha"], kw["beta"], kw["bitwidth"], seed_signed))
        expect = torch.empty(n)
        if codec == "terngrad":
            ops.terngrad_decompress(payloads, expect, post_scale=1.0 / world)
        elif codec == "tbq":
            ops.tbq_decompress(payloads, expect, kw["threshold"], post_scale=1.0 / world)
        elif codec == "graddrop":
            ops.sparse_decompress(payloads, expect, post_scale=1.0 / world)
        elif codec == "ecq":
            ops.ecq_decompress(payloads, expect, post_scale=1.0 / world)
        else:
            acc = cpu_grads[0].clone()
            for r in range(1, world):
                acc += cpu_grads[r]
            expect = acc * (1.0 / world)
        for r in range(world):
            assert torch.equal(grads[r].cpu(), expect), f"rank {r} step {step}"
            if codec != "dense":
                assert torch.equal(resid[r].cpu(), cpu_resid[r])
        # next step: fresh gradients
        for r in range(world):
            fresh = gauss(n, seed=100 * (step + 1) + r)
            grads[r].copy_(fresh)
            cpu_grads[r] = fresh.clone()


@pytest.mark.parametrize("codec,kw,opt", [
    ("tbq", dict(threshold=0.01), "sgd"),
    ("terngrad", dict(bitwidth=2), "sgd"),
    ("terngrad", dict(bitwidth=2, sharded=1, num_workers=0), "sgd"),
    ("graddrop", dict(keep_fraction=0.01, sample_rate=0.05), "adamw"),
    ("ecq", dict(bitwidth=4), "sgd"),
])
def test_flag_wait_times_out_with_status(codec, kw, opt):
    """A flag that nobody publishes: the bounded wait gives up and records it, the kernels queued
    behind it leave parameters and optimizer state untouched, and the context lives on."""
    n = 8192 + 4
    cfg = dict(rank=0, world=2, device=0, codec=codec, flag_timeout_s=0.2, **kw)
    e = hp._C.DdpEngine(cfg, [(0, n, 1)], [0])
    mems = SymmetricMemory.emulate(e.symmetric_bytes, 2)
    g, r = gauss(n).cuda(), torch.zeros(n, device="cuda")
    param, mom, second = gauss(n, 1.0, seed=5).cuda(), gauss(n, 1.0, seed=6).cuda(), gauss(n, 1.0, seed=7).cuda().abs()
    e.set_buffers(g, r, param, mom, None, second)
    e.set_symmetric(mems[0].buf)
    if opt == "adamw":
        e.set_adamw(0.1, 0.9, 0.999, 1e-8, 0.01)
    else:
        e.set_sgd(0.1, 0.9, 0.0, True)
    before = [t.clone() for t in (param, mom, second)]
    e.begin_step()
    e.bucket_ready(0, 0)   # rank 1 never pushes
    e.finish_step(0)
    assert e.check_status() == 1
    for t, b in zip((param, mom, second), before):
        assert torch.equal(t, b)
    assert e.check_status() == 0
    total_ns, max_ns, waits = e.wait_stats()
    assert waits >= 1 and max_ns >= 0.15e9
    # the device is still usable
    assert torch.equal(torch.ones(4, device="cuda") * 2, torch.full((4,), 2.0, device="cuda"))


def test_plan_buckets_reverse_order_and_alignment():
    plan = plan_buckets([10, 7, 100, 3], bucket_elems=64)
    assert all(o % 4 == 0 for o in plan.offsets)
    assert plan.offsets[3] == 0 and plan.offsets[2] == 4       # last parameter first
    assert sum(b[2] for b in plan.buckets) == 4
    for off, numel, _ in plan.buckets:
        assert off % 4 == 0 and numel % 4 == 0
    assert plan.total == sum(b[1] for b in plan.buckets)


@pytest.mark.parametrize("algorithm", ["terngrad", "tbq", "graddrop", "ecq", "dense", "terngrad_sharded", "tbq_sharded"])
def test_ddp_wrapper_world1_trains(algorithm):
    torch.manual_seed(0)
    net = resnet_tiny(10).cuda().to(memory_format=torch.channels_last)
    sharded = algorithm.endswith("_sharded")       # owner reduce + re-compress + fused SGD in the last phase
    algorithm = algorithm[:-8] if sharded else algorithm
    cfg = CompressionConfig(algorithm, bucket_mb=0.05, threshold=1e-3, keep_fraction=0.05, sample_rate=0.05,
                            bitwidth=4 if algorithm == "ecq" else 2, sharded=sharded)
    model = CompressedDataParallel(net, cfg, lr=0.05, momentum=0.9)
    assert len(model.plan.buckets) > 1
    x = torch.randn(16, 3, 32, 32, device="cuda")
    y = torch.randint(0, 10, (16,), device="cuda")
    losses = []
    for _ in range(12):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = torch.nn.functional.cross_entropy(model(x), y)
        loss.backward()
        model.step()
        losses.append(float(loss.detach()))
    model.check()
    assert all(l == l for l in losses)
    assert min(losses[-4:]) < losses[0], losses
    m = model.metrics()
    assert m["kernel_launches"] > 0 and m["steps"] == 12
    if cfg.needs_residual:
        assert m["residual_norm"] >= 0 and m["residual_norm"] == m["residual_norm"]


def test_ddp_dense_world1_equals_torch_sgd():
    torch.manual_seed(0)
    net_a = resnet_tiny(10).cuda()
    net_b = resnet_tiny(10).cuda()
    net_b.load_state_dict(net_a.state_dict())
    model = CompressedDataParallel(net_a, CompressionConfig("dense", bucket_mb=0.05), lr=0.1, momentum=0.9,
                                   weight_decay=1e-4)
    opt = torch.optim.SGD(net_b.parameters(), lr=0.1, momentum=0.9, weight_decay=1e-4)
    x = torch.randn(8, 3, 32, 32, device="cuda")
    y = torch.randint(0, 10, (8,), device="cuda")
    for _ in range(3):
        torch.nn.functional.cross_entropy(model(x), y).backward()
        model.step()
        opt.zero_grad()
        torch.nn.functional.cross_entropy(net_b(x), y).backward()
        opt.step()
    for pa, pb in zip(net_a.parameters(), net_b.parameters()):
        torch.testing.assert_close(pa, pb, atol=2e-5, rtol=1e-4)


@pytest.mark.parametrize("codec,kw", [
    ("tbq", dict(threshold=0.01)),
    ("terngrad", dict(bitwidth=2, enable_random=1, error_feedback=1)),
    ("terngrad", dict(bitwidth=4, enable_random=0, error_feedback=0)),
])
@pytest.mark.parametrize("device_epoch", [0, 1])
@pytest.mark.parametrize("world,n", [(1, 100000 + 12), (2, 100000 + 12), (4, 100000 + 12), (4, 100), (8, 70001),
                                     (3, 5 * 4096), (8, 300000 + 3)])
def test_sharded_exchange_matches_cpu_restatement(codec, kw, world, n, device_epoch):
    """Compressed reduce-scatter + compressed all-gather, ranks emulated on one device phase by
    phase (a device synchronise between phases, so no wait ever spins on an unlaunched kernel)."""
    from sharded_ref import expected, shard_elems
    engines, mems = make_engines(codec, world, n, sharded=1, num_workers=0, device_epoch=device_epoch, **kw)
    grads = [gauss(n, seed=10 + r).cuda() for r in range(world)]
    resid = [torch.zeros(n, device="cuda") for _ in range(world)]
    for e, m, g, r in zip(engines, mems, grads, resid):
        e.set_buffers(g, r, None, None)
        e.set_symmetric(m.buf)
        e.set_sgd(0.0, 0.0, 0.0, False)
    cpu_grads = [g.cpu().clone() for g in grads]
    cpu_resid = [torch.zeros(n) for _ in range(world)]
    cpu_resid2 = [torch.zeros(shard_elems(n, world)) for _ in range(world)]
    for step in range(3):
        for e in engines:
            e.begin_step()
        for e in engines:
            e.bucket_ready(0, 0)
        torch.cuda.synchronize()        # every shard payload delivered, phase-1 flags published
        for e in engines:
            e.reduce_step()
        torch.cuda.synchronize()        # every owner's re-compressed shard delivered
        for e in engines:
            e.finish_step(0)
        torch.cuda.synchronize()
        for e in engines:
            assert e.check_status() == 0
        want = expected(codec, kw, 3, step + 1, cpu_grads, cpu_resid, cpu_resid2, world)
        for r in range(world):
            assert torch.equal(grads[r].cpu(), want), f"rank {r} step {step}"
            assert torch.equal(resid[r].cpu(), cpu_resid[r]), f"residual rank {r} step {step}"
        for r in range(world):
            fresh = gauss(n, seed=100 * (step + 1) + r)
            grads[r].copy_(fresh)
            cpu_grads[r] = fresh.clone()
