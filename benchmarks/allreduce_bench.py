"""Compressed all-reduce microbenchmark.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node W --master-addr 127.0.0.1 \
        --master-port 29511 benchmarks/allreduce_bench.py [--sizes-mb 0.25 4 64 512] [--iters 20]

Per-rank fp32 buffers of 256 KB / 4 MB / 64 MB / 512 MB with values N(0, 1e-3^2) seeded by
rank are synchronised (sum / W on every rank) by

* ``nccl``      torch.distributed all_reduce (the uncompressed baseline),
* ``dense``     this framework's peer-to-peer dense path,
* ``tbq``       threshold 2e-3,
* ``terngrad``  2-bit, stochastic, error feedback,
* ``dgc``       top-k 0.1 % with 1 % sample threshold estimation,
* ``tbq_sharded`` / ``terngrad_sharded``  the same codecs as a compressed reduce-scatter to shard
  owners followed by a compressed all-gather of the re-quantised averages (``--codecs ... tbq_sharded``),
* ``tbq_auto`` / ``terngrad_auto``  whichever of the two forms the library's size rule picks
  (``hipress_b200.parallel.prefer_sharded``),
* any of these with ``_nvls`` appended (``terngrad_nvls``, ``tbq_sharded_nvls``): payloads delivered
  with one NVLS multicast store per packed word instead of one store per destination, where the
  host exposes multicast (the row says so when it does not),

each as ONE fused pipeline per step: compress kernels that store the packed payload straight
into every peer's receive slot over NVLink, a bounded flag wait, and a one-pass unpack +
accumulate of all W payloads.  Every number is device-timed with CUDA events (one pair per
iteration, L2 flushed before each, ranks aligned by a barrier) and reported as the max over
ranks of the median.  Effective GB/s = dense bytes (4 N) / time.  The roofline is the slower
of the kernels' HBM traffic at the measured copy bandwidth and the bytes a rank must send
over NVLink at 770 GB/s.

``--graph 1`` replays every arm from a CUDA graph (NCCL's all-reduce included; this framework's
engine then keeps the step's epoch on the device, as a captured training step does), which takes
the host's launch calls out of the measurement: small buffers are otherwise bound by them.
The reference extension's composition (its compress task, NCCL all-gather, its decompress tasks)
is measured by ``benchmarks/reference_codec_bench.py`` under the same launcher.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import hipress_b200 as hp  # noqa: E402
from hipress_b200.parallel import SymmetricMemory, prefer_sharded  # noqa: E402
from hipress_b200.utils.timing import flush_l2, max_over_ranks  # noqa: E402

NVLINK_GBS = 770.0


def measured_hbm_gbs() -> float:
    try:
        return float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"])
    except Exception:
        return 6650.0


def hbm_bytes_per_elem(codec: str, world: int) -> float:
    """Algorithmic HBM traffic of the fused pipeline per fp32 element."""
    if codec.endswith("_sharded"):
        # phase 1 compresses everything once (payload written once); the owner decodes `world`
        # payloads of 1/world of the elements and re-compresses them; phase 3 decodes one payload
        first = {"tbq": 4 + 8 + 0.25, "terngrad": 8 + 8 + 4 + 0.25}[codec[:-8]]
        return first + (0.25 * world + 4 + first) / world + 0.25 + 4
    if codec == "tbq":       # compress: R grad + RW residual + W payload ; unpack: R payloads + W dense
        return 4 + 8 + 0.25 * world + 0.25 * world + 4
    if codec == "terngrad":  # min/max pass (grad + residual) then quantise pass
        return 8 + (8 + 4 + 0.25 * world) + 0.25 * world + 4
    if codec == "dgc":       # count pass RW, write pass R(+sparse W), zero-fill + scatter
        return 12 + 4 + 4
    if codec == "dense":
        return 4 + 4 + 4 * world + 4
    return 0.0


def wire_bytes(codec: str, n: int, world: int) -> float:
    if codec.endswith("_sharded"):  # one payload's worth out to the owners, one shard payload to everyone
        return 2.0 * wire_bytes(codec[:-8], n, 2) * (world - 1) / world
    per = {"tbq": n / 4, "terngrad": 10 + n / 4, "dgc": 4 + 8 * max(1, int(n * 0.001 + 0.999)),
           "dense": 0.0}[codec]
    if codec == "dense":
        return 4.0 * n * (world - 1)  # pulled: every rank reads every peer's buffer
    return per * (world - 1)


def maybe_graphed(step, graph: int):
    """(callable, keep-alive): `step` itself, or a replay of `step` captured in a CUDA graph."""
    if not graph:
        return step, None
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()                                   # NCCL sets its communicator up on first use
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        step()
    return g.replay, g


def time_iters(fn, iters: int, warmup: int):
    times = []
    for i in range(warmup + iters):
        flush_l2()
        if dist.is_initialized():
            dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(a.elapsed_time(b))
    return max_over_ranks(statistics.median(times))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes-mb", type=float, nargs="+", default=[0.25, 4, 64, 512])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--codecs", nargs="+", default=["nccl", "dense", "tbq", "terngrad", "dgc"])
    ap.add_argument("--graph", type=int, default=0, help="1 = replay each arm from a CUDA graph")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    hbm = measured_hbm_gbs()
    results = []
    for mb in args.sizes_mb:
        n = int(mb * (1 << 20) / 4)
        gen = torch.Generator(device="cuda").manual_seed(1234 + rank)
        grad0 = torch.randn(n, device=dev, generator=gen) * 1e-3
        nccl_ms = None
        for codec in args.codecs:
            grad = grad0.clone()
            if codec == "nccl":
                if world == 1:
                    continue

                def step():
                    dist.all_reduce(grad)
                    grad.mul_(1.0 / world)
                fn, keep = maybe_graphed(step, args.graph)
                ms = time_iters(fn, args.iters, args.warmup)
                nccl_ms = ms
                launches = None
            else:
                base, *flags = codec.split("_")       # e.g. terngrad_sharded_nvls
                sharded = "sharded" in flags or ("auto" in flags and prefer_sharded(n * 4, world))
                nvls = "nvls" in flags
                graphable = bool(args.graph)
                cfg = dict(rank=rank, world=world, device=local, codec=base,
                           threshold=2e-3, bitwidth=2, enable_random=1, error_feedback=1, keep_fraction=0.001,
                           sample_rate=0.01, seed=1, sharded=1 if sharded else 0,
                           device_epoch=1 if graphable else 0, num_workers=0 if (graphable or sharded) else 1,
                           nvls=1 if nvls else 0)
                eng = hp._C.DdpEngine(cfg, [(0, n, 1)], [0])
                sym = SymmetricMemory(eng.symmetric_bytes, dev, multicast=nvls)
                if nvls and not sym.multicast:
                    if rank == 0:
                        print(json.dumps({"codec": codec, "world": world, "buffer_mb": mb,
                                          "unavailable": "no NVLS multicast mapping: " + getattr(sym, "multicast_note", "")}),
                              flush=True)
                    del eng, sym
                    continue
                resid = torch.zeros(n, device=dev)
                eng.set_buffers(grad, resid, None, None)
                eng.set_symmetric(sym.buf)
                eng.set_sgd(0.0, 0.0, 0.0, False)

                def step():
                    eng.begin_step(local)
                    eng.bucket_ready(0, local)
                    eng.finish_step(local)
                if graphable:
                    step()                       # first-use set-up outside the capture
                    torch.cuda.synchronize()
                    if dist.is_initialized():
                        dist.barrier()
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g):
                        step()
                    per_step = eng.end_capture()

                    def fn():
                        g.replay()
                        eng.note_replay(1, per_step)
                else:
                    fn = step
                l0 = eng.launches
                ms = time_iters(fn, args.iters, args.warmup)
                status = eng.check_status()
                assert status == 0, f"engine status {status}"
                launches = (eng.launches - l0) // (args.iters + args.warmup)
                if dist.is_initialized():
                    dist.barrier()           # nobody frees its buffer while a peer may still read it
                del eng, sym
            dense_bytes = 4.0 * n
            row = {"codec": codec, "world": world, "buffer_mb": mb, "n": n, "graph": int(args.graph), "ms": round(ms, 4),
                   "effective_gbs": round(dense_bytes / (ms * 1e-3) / 1e9, 2), "launches_per_step": launches}
            if codec != "nccl":
                model = (base + "_sharded") if sharded else base
                row["form"] = "sharded" if sharded else "all-gather"
                row["transport"] = "nvls" if nvls else "p2p"
                t_hbm = hbm_bytes_per_elem(model, world) * n / (hbm * 1e9)
                t_link = wire_bytes(model, n, world) / (NVLINK_GBS * 1e9)
                roof = max(t_hbm, t_link)
                row.update({"roofline_ms": round(roof * 1e3, 4), "roofline_bound": "hbm" if t_hbm >= t_link else "nvlink",
                            "fraction_of_roofline": round(roof * 1e3 / ms, 3),
                            "hbm_gbs_measured_peak": hbm})
                if nccl_ms:
                    row["speedup_vs_nccl"] = round(nccl_ms / ms, 2)
            results.append(row)
            if rank == 0:
                print(json.dumps(row), flush=True)
    # captured graphs hold on to the communicator: drop them before it is torn down
    fn = keep = step = None  # noqa: F841
    import gc
    gc.collect()
    torch.cuda.synchronize()
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps({"done": True, "rows": len(results)}), flush=True)
    sys.stdout.flush()
    os._exit(0)   # leave without waiting on library teardown (an NCCL graph capture can stall it)


if __name__ == "__main__":
    main()
