"""Per-buffer cost of the unmodified reference extension through its own public API
(``submit_task`` + ``getResults`` polling, CPU staging buffer), next to this framework's engine
on the same buffers.  One GPU; TernGrad 2-bit and TBQ (threshold 2e-3); buffers of 256 KB /
4 MB / 64 MB / 512 MB of fp32 ~ N(0, 1e-3^2).

    python benchmarks/reference_codec_bench.py [--sizes-mb 0.25 4 64 512] [--iters 5]

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
    import torch
    sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
    import hp_cuda
    out = []
    params = {"terngrad": {"enable_random": 1.0, "bitwidth": 2.0}, "tbq": {"threshold": 2e-3}}[alg]
    if True:
        assert hp_cuda.init(alg, params, 0, 0, 1)
        for mb in sizes:
            n = int(mb * (1 << 20) / 4)
            g = torch.randn(n, device="cuda") * 1e-3
            r = torch.zeros(n, device="cuda")
            size = 10 + (n + 3) // 4 if alg == "terngrad" else (n + 3) // 4
            B = torch.zeros(size, dtype=torch.uint8, device="cuda")
            C = torch.zeros(size, dtype=torch.uint8).pin_memory()
            times = []
            for it in range(iters + 2):
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                for task in (10, 20):
                    if alg == "terngrad":
                        hp_cuda.submit_task("x", g, B, C, 0, task)
                    else:
                        hp_cuda.submit_task("x", g, r, B, C, 0, task)
                    while "x" not in hp_cuda.getResults(task):
                        pass
                torch.cuda.synchronize()
                if it >= 2:
                    times.append((time.perf_counter() - t0) * 1e3)
            out.append({"impl": "reference", "codec": alg, "buffer_mb": mb, "ms": round(statistics.median(times), 3),
                        "effective_gbs": round(4.0 * n / (statistics.median(times) * 1e-3) / 1e9, 2)})
            print(json.dumps(out[-1]), flush=True)
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
    ap.add_argument("--arm", default="both", choices=["both", "ours", "reference-terngrad", "reference-tbq"])
    args = ap.parse_args()
    if args.arm == "both":
        for arm in ("reference-terngrad", "reference-tbq", "ours"):
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
