"""Worker of the multi-GPU tests: one process per GPU, launched by torch.distributed.run.

Checks, on real peer memory over NVLink:
  1. every codec through the engine gives, on every rank and bit for bit, the result the CPU
     codec predicts from all ranks' (seeded) gradients;
  2. the DDP wrapper keeps the replicas' parameters bit-identical while training;
  3. PowerSGD data parallel keeps replicas identical.
Prints one line ``MP_OK <name>`` per passed check on rank 0.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import hipress_b200 as hp  # noqa: E402
from hipress_b200 import ops  # noqa: E402
from hipress_b200.models import resnet_tiny, vgg_tiny  # noqa: E402
from hipress_b200.parallel import CompressedDataParallel, CompressionConfig, SymmetricMemory  # noqa: E402
from hipress_b200.parallel.powersgd import PowerSGDDataParallel  # noqa: E402


def gauss(n, std, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(n, generator=g) * std


def same_on_all_ranks(t: torch.Tensor) -> bool:
    world = dist.get_world_size()
    mine = t.detach().flatten().view(torch.int32).to(torch.int64).sum().view(1)
    # exact integer checksum of the bit patterns
    allv = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(allv, mine)
    return all(int(v) == int(allv[0]) for v in allv)


def check_codec(codec, kw, rank, world, local, n=300000 + 8, nvls=False):
    """Returns False when ``nvls`` was asked for and the host exposes no multicast mapping."""
    cfg = dict(rank=rank, world=world, device=local, codec=codec, seed=5, flag_timeout_s=10.0, nvls=int(nvls), **kw)
    eng = hp._C.DdpEngine(cfg, [(0, n, 1)], [0])
    sym = SymmetricMemory(eng.symmetric_bytes, torch.device("cuda", local), multicast=nvls)
    if nvls and not sym.multicast:
        if rank == 0:
            print("NVLS unavailable:", getattr(sym, "multicast_note", ""), flush=True)
        dist.barrier()
        del eng, sym
        return False
    grad = torch.zeros(n, device="cuda")
    resid = torch.zeros(n, device="cuda")
    eng.set_buffers(grad, resid, None, None)
    eng.set_symmetric(sym.buf)
    eng.set_sgd(0.0, 0.0, 0.0, False)
    cpu_resid = [torch.zeros(n) for _ in range(world)]
    for step in range(3):
        cpu_grads = [gauss(n, 0.01, 1000 * step + r) for r in range(world)]
        grad.copy_(cpu_grads[rank])
        eng.begin_step(local)
        eng.bucket_ready(0, local)
        eng.finish_step(local)
        torch.cuda.synchronize()
        assert eng.check_status() == 0
        seed = (5 + (step + 1) * 0x9E3779B97F4A7C15) % (1 << 64)
        seed = seed - (1 << 64) if seed >= (1 << 63) else seed
        payloads = []
        for r in range(world):
            g, res = cpu_grads[r], cpu_resid[r]
            if codec == "terngrad":
                payloads.append(ops.terngrad_compress(g, 2, True, seed, residual=res))
            elif codec == "tbq":
                payloads.append(ops.tbq_compress(g, res, kw["threshold"]))
            elif codec == "graddrop":
                payloads.append(ops.graddrop_compress(g, res, kw["sample_rate"], 1 - kw["keep_fraction"], seed))
            elif codec == "ecq":
                payloads.append(ops.ecq_compress(g, res, 1.0, 0.9, kw["bitwidth"], seed))
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
        assert torch.equal(grad.cpu(), expect), f"{codec} rank {rank} step {step}"
        if codec != "dense":
            assert torch.equal(resid.cpu(), cpu_resid[rank]), f"{codec} residual rank {rank} step {step}"
    dist.barrier()
    del eng, sym
    return True


def check_sharded(codec, kw, rank, world, local, device_epoch=0):
    """Compressed reduce-scatter + compressed all-gather across real GPUs against the CPU restatement."""
    from sharded_ref import expected, shard_elems
    n = 300000 + 8
    cfg = dict(rank=rank, world=world, device=local, codec=codec, seed=5, flag_timeout_s=10.0, sharded=1,
               num_workers=0, device_epoch=device_epoch, **kw)
    eng = hp._C.DdpEngine(cfg, [(0, n, 1)], [0])
    sym = SymmetricMemory(eng.symmetric_bytes, torch.device("cuda", local))
    grad = torch.zeros(n, device="cuda")
    resid = torch.zeros(n, device="cuda")
    eng.set_buffers(grad, resid, None, None)
    eng.set_symmetric(sym.buf)
    eng.set_sgd(0.0, 0.0, 0.0, False)
    cpu_resid = [torch.zeros(n) for _ in range(world)]
    cpu_resid2 = [torch.zeros(shard_elems(n, world)) for _ in range(world)]
    for step in range(3):
        cpu_grads = [gauss(n, 0.01, 1000 * step + r) for r in range(world)]
        grad.copy_(cpu_grads[rank])
        eng.begin_step(local)
        eng.bucket_ready(0, local)
        eng.finish_step(local)
        torch.cuda.synchronize()
        assert eng.check_status() == 0
        want = expected(codec, kw, 5, step + 1, cpu_grads, cpu_resid, cpu_resid2, world)
        assert torch.equal(grad.cpu(), want), f"sharded {codec} rank {rank} step {step}"
        assert torch.equal(resid.cpu(), cpu_resid[rank]), f"sharded {codec} residual rank {rank} step {step}"
    dist.barrier()
    del eng, sym


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    for codec, kw in [("terngrad", dict(bitwidth=2, enable_random=1, error_feedback=1)),
                      ("tbq", dict(threshold=0.01)),
                      ("graddrop", dict(keep_fraction=0.01, sample_rate=0.05)),
                      ("ecq", dict(bitwidth=4, alpha=1.0, beta=0.9)),
                      ("dense", dict())]:
        check_codec(codec, kw, rank, world, local)
        if rank == 0:
            print(f"MP_OK codec_{codec}", flush=True)
    # the same protocol with the epoch, slot parity and seed resolved on the device
    for codec, kw in [("terngrad", dict(bitwidth=2, enable_random=1, error_feedback=1)), ("tbq", dict(threshold=0.01))]:
        check_codec(codec, dict(kw, device_epoch=1, num_workers=0), rank, world, local)
        if rank == 0:
            print(f"MP_OK codec_{codec}_device_epoch", flush=True)

    # large enough for the chunked compress path: 16-byte stores into the peers' slots
    for codec, kw in [("terngrad", dict(bitwidth=2, enable_random=1, error_feedback=1)), ("tbq", dict(threshold=0.01))]:
        check_codec(codec, kw, rank, world, local, n=1400000 + 8)
        if rank == 0:
            print(f"MP_OK codec_{codec}_wide", flush=True)
    check_codec("ecq", dict(bitwidth=2, alpha=1.0, beta=0.9, device_epoch=1, num_workers=0), rank, world, local)
    if rank == 0:
        print("MP_OK codec_ecq_device_epoch", flush=True)
    # payloads delivered with NVLS multicast stores: bit-identical to the peer-store path
    # (no rank leaves during this check; the rank-exit tests keep multicast off)
    if os.environ.get("HIPRESS_TEST_NVLS", "1") != "0":
        ran = True
        for codec, kw, size in [("terngrad", dict(bitwidth=2, enable_random=1, error_feedback=1), 1400000 + 8),
                                ("tbq", dict(threshold=0.01), 300000 + 8),
                                ("graddrop", dict(keep_fraction=0.01, sample_rate=0.05), 300000 + 8)]:
            ran = check_codec(codec, kw, rank, world, local, n=size, nvls=True) and ran
        if rank == 0:
            print("MP_OK codec_nvls" if ran else "MP_SKIP codec_nvls (no multicast on this host)", flush=True)

    for codec, kw in [("terngrad", dict(bitwidth=2, enable_random=1, error_feedback=1)), ("tbq", dict(threshold=0.01))]:
        check_sharded(codec, kw, rank, world, local)
        if rank == 0:
            print(f"MP_OK sharded_{codec}", flush=True)
        check_sharded(codec, kw, rank, world, local, device_epoch=1)
        if rank == 0:
            print(f"MP_OK sharded_{codec}_device_epoch", flush=True)

    # DDP wrapper: replicas stay bit-identical, loss goes down
    torch.manual_seed(0)
    net = resnet_tiny(10).cuda().to(memory_format=torch.channels_last)
    model = CompressedDataParallel(net, CompressionConfig("terngrad", bucket_mb=0.05), lr=0.05, momentum=0.9)
    g = torch.Generator().manual_seed(77 + rank)
    x = torch.randn(16, 3, 32, 32, generator=g).cuda()
    y = torch.randint(0, 10, (16,), generator=g).cuda()
    losses = []
    for _ in range(10):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = torch.nn.functional.cross_entropy(model(x), y)
        loss.backward()
        model.step()
        losses.append(float(loss))
    model.check()
    assert same_on_all_ranks(model.flat_param), "replicas diverged"
    assert min(losses[-3:]) < losses[0]
    if rank == 0:
        print("MP_OK ddp_terngrad", flush=True)

    # whole training step (hooks + exchange) replayed from one CUDA graph on every rank
    from hipress_b200.parallel import GraphedTrainStep

    def loss_fn(module, a, b):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            return torch.nn.functional.cross_entropy(module(a), b)

    torch.manual_seed(0)
    net = resnet_tiny(10).cuda().to(memory_format=torch.channels_last)
    gm = CompressedDataParallel(net, CompressionConfig("terngrad", bucket_mb=0.05, graph_capturable=True),
                                lr=0.05, momentum=0.9)
    xc = x.contiguous(memory_format=torch.channels_last)
    step = GraphedTrainStep(gm, loss_fn, (xc, y))
    assert step.whole_step
    losses = [float(step(xc, y).detach()) for _ in range(10)]
    gm.check()
    assert same_on_all_ranks(gm.flat_param), "graphed replicas diverged"
    assert min(losses[-3:]) < losses[0]
    if rank == 0:
        print("MP_OK ddp_graphed", flush=True)

    # the sharded exchange inside the captured step
    torch.manual_seed(0)
    net = resnet_tiny(10).cuda().to(memory_format=torch.channels_last)
    sm = CompressedDataParallel(net, CompressionConfig("terngrad", bucket_mb=0.05, graph_capturable=True, sharded=True),
                                lr=0.05, momentum=0.9)
    sstep = GraphedTrainStep(sm, loss_fn, (xc, y))
    assert sstep.whole_step
    slosses = [float(sstep(xc, y).detach()) for _ in range(10)]
    sm.check()
    assert same_on_all_ranks(sm.flat_param), "graphed sharded replicas diverged"
    assert min(slosses[-3:]) < slosses[0]
    if rank == 0:
        print("MP_OK ddp_graphed_sharded", flush=True)

    # DGC (momentum correction, clipping, fused AdamW) with the exchange captured in the graph
    from hipress_b200.parallel.dgc import DGCDataParallel
    torch.manual_seed(0)
    net = resnet_tiny(10).cuda().to(memory_format=torch.channels_last)
    dm = DGCDataParallel(net, keep_fraction=0.05, sample_rate=0.1, warmup_steps=0, lr=1e-3, bucket_mb=0.05,
                         graph_capturable=True)
    dstep = GraphedTrainStep(dm, loss_fn, (xc, y))
    assert dstep.whole_step
    dlosses = [float(dstep(xc, y).detach()) for _ in range(10)]
    dm.check()
    assert same_on_all_ranks(dm.flat_param), "graphed DGC replicas diverged"
    assert all(v == v for v in dlosses)
    if rank == 0:
        print("MP_OK ddp_graphed_dgc", flush=True)

    torch.manual_seed(0)
    net = vgg_tiny(10).cuda()
    pm = PowerSGDDataParallel(net, rank_r=2, lr=0.05, momentum=0.9)
    for _ in range(5):
        torch.nn.functional.cross_entropy(pm(x), y).backward()
        pm.step()
    pm.check()
    assert same_on_all_ranks(pm.flat_param) and same_on_all_ranks(pm.vec_param), "PowerSGD replicas diverged"
    if rank == 0:
        print("MP_OK ddp_powersgd", flush=True)

    # PowerSGD with the exchange inside the captured step: two graphs (one per accumulator parity)
    torch.manual_seed(0)
    net = vgg_tiny(10).cuda()
    gp = PowerSGDDataParallel(net, rank_r=2, lr=0.05, momentum=0.9, graph_capturable=True)

    def plain_loss(module, a, b):
        return torch.nn.functional.cross_entropy(module(a), b)

    pstep = GraphedTrainStep(gp, plain_loss, (x, y))
    assert pstep.whole_step and pstep.variants == 2
    plosses = [float(pstep(x, y).detach()) for _ in range(8)]
    gp.check()
    assert same_on_all_ranks(gp.flat_param) and same_on_all_ranks(gp.vec_param), "graphed PowerSGD replicas diverged"
    assert all(v == v for v in plosses)
    if rank == 0:
        print("MP_OK ddp_graphed_powersgd", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
