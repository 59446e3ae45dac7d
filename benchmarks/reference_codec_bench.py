"""Per-buffer cost of the unmodified reference extension through its own public API
(``submit_task`` + ``getResults`` polling, CPU staging buffer), next to this framework's engine
on the same buffers.  One GPU; TernGrad 2-bit and TBQ (threshold 2e-3); buffers of 256 KB /
4 MB / 64 MB / 512 MB of fp32 ~ N(0, 1e-3^2).

    python benchmarks/reference_codec_bench.py [--sizes-mb 0.25 4 64 512] [--iters 5]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node W --master-addr 127.0.0.1 --master-port P \
        benchmarks/reference_codec_bench.py --arm reference-terngrad     # or -tbq, -graddrop

Under a multi-rank launcher the reference arms measure the composition the reference leaves to its
caller: its compress task, an NCCL all-gather of the payloads, a copy of the W payloads into the
host buffers its decompress task reads, and W decompress tasks (overwrite, then accumulate) --
"compress -> all-gather -> decompress -> sum" with the unmodified extension.

The reference's API is host driven (the caller learns of completion by polling), so its
numbers are wall-clock from submit to the name appearing in ``getResults``, compress task plus
decompress task; ours are CUDA-event times of the engine's whole pipeline (compress, flag,
unpack) on one rank.  Prints one JSON line per (codec, size).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_reference(alg, sizes, iters):
    # the reference keeps one algorithm per process: init() after end() never restarts its
    # threads (ref hp_cuda.cpp:814), so each algorithm gets a process of its own
    import math
    import torch
    import torch.distributed as dist
    sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
    import hp_cuda
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    out = []
    params = {"terngrad": {"enable_random": 1.0, "bitwidth": 2.0}, "tbq": {"threshold": 2e-3},
              "graddrop": {"drop_ratio": 0.999, "sample_rate": 0.01}}[alg]
    assert hp_cuda.init(alg, params, local, rank, world)
    for mb in sizes:
        n = int(mb * (1 << 20) / 4)
        gen = torch.Generator(device="cuda").manual_seed(1234 + rank)
        g = torch.randn(n, device=dev, generator=gen) * 1e-3
        r = torch.zeros(n, device=dev)
        alloc = None
        if alg == "terngrad":
            size = 10 + (n + 3) // 4
        elif alg == "tbq":
            size = (n + 3) // 4
        else:
            # staging size of the reference's GradDrop loop (ref hp_cuda.cpp:230); B must also hold
            # the compressor's sample scratch and its untrimmed index list (ref gd_body.h:117, 165-187),
            # which the module does not check
            expected = math.ceil(n * 0.001)
            size = 4 + int(2 * expected) * 4
            alloc = max(size, 4 * math.ceil(n * 0.01) + 64, 4 + 8 * 4 * expected)
        B = torch.zeros(alloc or size, dtype=torch.uint8, device=dev)
        C = torch.zeros(size, dtype=torch.uint8).pin_memory()
        G = [torch.zeros(size, dtype=torch.uint8, device=dev) for _ in range(world)]
        peerB = [torch.zeros(size, dtype=torch.uint8, device=dev) for _ in range(world)]
        peerC = [torch.zeros(size, dtype=torch.uint8).pin_memory() for _ in range(world)]

        def submit(Bt, Ct, is_root, task):
            if alg == "terngrad":
                hp_cuda.submit_task("x", g, Bt, Ct, is_root, task)
            else:
                hp_cuda.submit_task("x", g, r, Bt, Ct, is_root, task)
            while "x" not in hp_cuda.getResults(task):
                pass

        times = []
        for it in range(iters + 2):
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
                torch.cuda.synchronize()
            t0 = time.perf_counter()
            submit(B, C, 0, 10)
            if world == 1:
                submit(B, C, 0, 20)
            else:
                dist.all_gather(G, B[:size])
                for q in range(world):
                    peerC[q].copy_(G[q], non_blocking=True)
                torch.cuda.current_stream().synchronize()
                for q in range(world):
                    submit(peerB[q], peerC[q], 0 if q == 0 else 1, 20)
                g.div_(world)
            torch.cuda.synchronize()
            if it >= 2:
                times.append((time.perf_counter() - t0) * 1e3)
            g.copy_(torch.randn(n, device=dev, generator=gen) * 1e-3)
        ms = statistics.median(times)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t)
        out.append({"impl": "reference", "codec": alg, "world": world, "buffer_mb": mb, "ms": round(ms, 3),
                    "effective_gbs": round(4.0 * n / (ms * 1e-3) / 1e9, 2)})
        if rank == 0:
            print(json.dumps(out[-1]), flush=True)
    if world > 1:
        dist.barrier()
    return out


def run_ours(sizes, iters):
    import torch
    sys.path.insert(0, ROOT)
    import hipress_b200 as hp
    from hipress_b200.parallel import SymmetricMemory
    from hipress_b200.utils.timing import flush_l2
    for codec in ("terngrad", "tbq"):
        for mb in sizes:
            n = int(mb * (1 << 20) / 4)
            g = torch.randn(n, device="cuda") * 1e-3
            r = torch.zeros(n, device="cuda")
            eng = hp._C.DdpEngine(dict(rank=0, world=1, device=0, codec=codec, threshold=2e-3, bitwidth=2,
                                       error_feedback=0 if codec == "terngrad" else 1, num_workers=0), [(0, n, 1)], [0])
            sym = SymmetricMemory(eng.symmetric_bytes)
            eng.set_buffers(g, r, None, None)
            eng.set_symmetric(sym.buf)
            eng.set_sgd(0.0, 0.0, 0.0, False)
            times = []
            for it in range(iters + 2):
                flush_l2()
                torch.cuda.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                eng.begin_step()
                eng.bucket_ready(0, 0)
                eng.finish_step(0)
                b.record()
                torch.cuda.synchronize()
                if it >= 2:
                    times.append(a.elapsed_time(b))
            ms = statistics.median(times)
            print(json.dumps({"impl": "ours", "codec": codec, "buffer_mb": mb, "ms": round(ms, 4),
                              "effective_gbs": round(4.0 * n / (ms * 1e-3) / 1e9, 2)}), flush=True)
            del eng, sym


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes-mb", type=float, nargs="+", default=[0.25, 4, 64, 512])
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--arm", default="both", choices=["both", "ours", "reference-terngrad", "reference-tbq", "reference-graddrop"])
    args = ap.parse_args()
    if args.arm == "both":
        for arm in ("reference-terngrad", "reference-tbq", "reference-graddrop", "ours"):
            subprocess.run([sys.executable, __file__, "--arm", arm, "--iters", str(args.iters), "--sizes-mb",
                            *map(str, args.sizes_mb)], check=False)
        return
    if args.arm == "ours":
        run_ours(args.sizes_mb, args.iters)
    else:
        run_reference(args.arm.split("-")[1], args.sizes_mb, args.iters)
        os._exit(0)  # leave without running the reference's static destructors


if __name__ == "__main__":
    main()
