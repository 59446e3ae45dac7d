"""CPU codec round-trip benchmark: one fp32 gradient of 2^22 elements ~ N(0, 0.01^2) (torch seed 0),
10 iterations of compress + decompress for TBQ (threshold 0.01, residual carried) and TernGrad
(2-bit, stochastic, seed 1).  Times this library's CPU codec and, when a checkout of the reference
and nvcc are present, the reference's own host path (thrust::host) through ``oracle/ref_oracle.cu``.

    python benchmarks/cpu_codec_bench.py [--reference-dir /path/to/reference]
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from hipress_b200 import ops  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference-dir", default=os.environ.get("HIPRESS_REFERENCE_DIR", os.path.join(os.path.dirname(ROOT), "reference")))
    ap.add_argument("--n", type=int, default=1 << 22)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--threads", type=int, default=1,
                    help="threads this framework's CPU codec may use (the reference's host path has one)")
    args = ap.parse_args()
    torch.manual_seed(0)
    torch.set_num_threads(1)
    ops.set_cpu_threads(args.threads)
    n = args.n
    g = torch.randn(n) * 0.01
    resid, dense = torch.zeros(n), torch.empty(n)
    p1 = torch.empty(ops.tbq_payload_bytes(n), dtype=torch.uint8)
    p2 = torch.empty(ops.terngrad_payload_bytes(n, 2), dtype=torch.uint8)
    t0 = time.perf_counter()
    for _ in range(args.iters):
        ops.tbq_compress(g, resid, 0.01, out=p1)
        ops.tbq_decompress(p1, dense, 0.01)
    t1 = time.perf_counter()
    for _ in range(args.iters):
        ops.terngrad_compress(g, 2, True, 1, out=p2)
        ops.terngrad_decompress(p2, dense)
    t2 = time.perf_counter()
    out = {"n": n, "iters": args.iters, "threads": ops.get_cpu_threads(),
           "ours": {"tbq_ms_per_iter": round((t1 - t0) * 1e3 / args.iters, 3),
                    "terngrad_ms_per_iter": round((t2 - t1) * 1e3 / args.iters, 3)}}
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if os.path.isdir(os.path.join(args.reference_dir, "ZQ_CPP_LIB")) and os.path.exists(nvcc):
        exe = os.path.join(tempfile.gettempdir(), "hipress_ref_oracle")
        src = os.path.join(ROOT, "oracle", "ref_oracle.cu")
        if not os.path.exists(exe) or os.path.getmtime(exe) < os.path.getmtime(src):
            subprocess.run([nvcc, "-std=c++17", "-O2", "-Xcompiler", "-ffp-contract=off", "-w",
                            f"-I{args.reference_dir}", "-o", exe, src], check=True)
        with tempfile.NamedTemporaryFile(suffix=".bin") as f:
            g.numpy().tofile(f.name)
            res = subprocess.run([exe, "bench", f.name, str(n), str(args.iters)], capture_output=True, text=True, check=True)
        out["reference_host_path"] = json.loads(res.stdout.strip().splitlines()[-1])
    else:
        out["reference_host_path"] = "unavailable (no reference checkout / nvcc)"
    print(json.dumps(out))


if __name__ == "__main__":
    main()
