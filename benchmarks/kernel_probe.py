"""Run one kernel family on a small, fixed case (for ncu captures and quick event timings).

    python benchmarks/kernel_probe.py --kernel terngrad --mb 64 --iters 3

Inputs are larger than the 126 MB L2 by default (64 MB gradient + 64 MB residual + outputs) but
hold well under 1 GB on the device, so a ``ncu --set full`` capture of one launch ends quickly.
Prints device-timed ms per call (CUDA events, L2 flushed between calls) and achieved GB/s of
algorithmic traffic against the measured copy bandwidth.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from hipress_b200 import ops  # noqa: E402
from hipress_b200.utils.timing import flush_l2  # noqa: E402


def peak_hbm():
    try:
        return float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"])
    except Exception:
        return 6650.0


def timed(fn, iters):
    out = []
    for _ in range(iters):
        flush_l2()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        out.append(a.elapsed_time(b))
    return min(out)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default="terngrad",
                    choices=["terngrad", "terngrad_words", "terngrad_unpack", "tbq", "tbq_unpack", "sparse", "ecq", "psgd_p", "psgd_q", "psgd_group_p", "psgd_group_q", "psgd_loop_p", "psgd_loop_q", "psgd_group_expand", "psgd_loop_expand",
                             "psgd_expand", "sgd", "adamw", "terngrad_unpack_apply", "bn_fwd", "bn_bwd",
                             "bias_relu_pool_fwd", "bias_relu_pool_bwd", "add_ln_fwd", "add_ln_bwd", "maxpool_fwd",
                             "maxpool_bwd"])
    ap.add_argument("--mb", type=float, default=64.0)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--world", type=int, default=8, help="payload count for the unpack kernels")
    ap.add_argument("--graph", type=int, default=0,
                    help="1: time the op as a CUDA-graph replay (no host work between its launches, as a captured "
                         "training step runs it)")
    ap.add_argument("--rows", type=int, default=4096, help="matrix rows for the psgd kernels (columns follow from --mb)")
    ap.add_argument("--cols", type=int, default=0, help="matrix columns for the psgd kernels (0: from --mb and --rows)")
    args = ap.parse_args()
    n = int(args.mb * (1 << 20) / 4)
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    g = torch.randn(n, device=dev) * 1e-3
    r = torch.zeros(n, device=dev)
    hbm = peak_hbm()
    k = args.kernel
    if k in ("terngrad", "terngrad_words"):
        # the engine places a payload 6 bytes into its slot so that the packed data behind the
        # 10-byte header is 16-byte aligned (chunked path, 16-byte stores); "terngrad_words" keeps
        # the payload at the start of a tensor, which takes the 4-byte-store path
        shift = 6 if k == "terngrad" else 0
        nbytes = ops.terngrad_payload_bytes(n, 2)
        out = torch.empty(nbytes + 16, dtype=torch.uint8, device=dev)[shift:shift + nbytes]
        fn = lambda: ops.terngrad_compress(g, 2, True, 1, residual=r, out=out)
        traffic = n * (8 + 8 + 4 + 0.25)
    elif k == "terngrad_unpack":
        # payloads sit 6 bytes into their buffers, as in the engine's receive slots: the packed
        # data behind the 10-byte header is then 16-byte aligned and is read with 32-bit loads
        nbytes = ops.terngrad_payload_bytes(n, 2)
        pl = []
        for s in range(args.world):
            buf = torch.empty(nbytes + 16, dtype=torch.uint8, device=dev)[6:6 + nbytes]
            ops.terngrad_compress(torch.randn(n, device=dev) * 1e-3, 2, True, s, out=buf)
            pl.append(buf)
        fn = lambda: ops.terngrad_decompress(pl, g, post_scale=1.0 / args.world, bitwidth=2)
        traffic = n * (0.25 * args.world + 4)
    elif k == "tbq":
        out = torch.empty(ops.tbq_payload_bytes(n), dtype=torch.uint8, device=dev)
        fn = lambda: ops.tbq_compress(g, r, 2e-3, out=out)
        traffic = n * (4 + 8 + 0.25)
    elif k == "tbq_unpack":
        pl = [ops.tbq_compress(torch.randn(n, device=dev) * 1e-3, torch.zeros(n, device=dev), 2e-3) for _ in range(args.world)]
        fn = lambda: ops.tbq_decompress(pl, g, 2e-3, post_scale=1.0 / args.world)
        traffic = n * (0.25 * args.world + 4)
    elif k == "sparse":
        out = torch.empty(ops.sparse_payload_bytes(n, 0.001), dtype=torch.uint8, device=dev)
        seed = [0]

        def fn():
            seed[0] += 1
            ops.graddrop_compress(g, r, 0.01, 0.999, seed[0], out=out)
        traffic = n * (12 + 4)
    elif k == "ecq":
        out = torch.empty(ops.ecq_payload_bytes(n, 2), dtype=torch.uint8, device=dev)
        fn = lambda: ops.ecq_compress(g, r, 1.0, 0.9, 2, 1, out=out)
        traffic = n * (8 + 8 + 4 + 0.25)
    elif k in ("psgd_p", "psgd_q", "psgd_expand"):
        rows = args.rows
        cols = args.cols if args.cols > 0 else n // rows
        n = rows * cols
        M = torch.randn(rows, cols, device=dev)
        Q = torch.randn(cols, 4, device=dev)
        P = torch.randn(rows, 4, device=dev)
        if k == "psgd_p":
            acc = torch.zeros(rows, 4, device=dev)
            fn = lambda: ops.psgd_project(0, M, Q, [acc])
            traffic = rows * cols * 4
        elif k == "psgd_q":
            acc = torch.zeros(cols, 4, device=dev)
            fn = lambda: ops.psgd_project(1, M, P, [acc])
            traffic = rows * cols * 4
        else:
            out = torch.zeros(rows * cols, device=dev)
            fn = lambda: ops.psgd_expand_feedback(P, Q, M, out)
            traffic = rows * cols * 12
    elif k in ("psgd_group_p", "psgd_group_q", "psgd_loop_p", "psgd_loop_q"):
        # the 19 weight matrices of VGG-19 (16 convolutions as [out, in*9], 3 classifier layers): one grouped
        # launch ("group") against one launch per matrix ("loop"); --mb is ignored
        mode = 0 if k.endswith("_p") else 1
        chans = [(64, 3), (64, 64), (128, 64), (128, 128), (256, 128), (256, 256), (256, 256), (256, 256),
                 (512, 256), (512, 512), (512, 512), (512, 512), (512, 512), (512, 512), (512, 512), (512, 512)]
        shapes = [(o, i * 9) for o, i in chans] + [(4096, 25088), (4096, 4096), (1000, 4096)]
        Ms = [torch.randn(a, b, device=dev) for a, b in shapes]
        Xs = [torch.randn(b if mode == 0 else a, 4, device=dev) for a, b in shapes]
        outs = [torch.zeros(a if mode == 0 else b, 4, device=dev) for a, b in shapes]
        if k.startswith("psgd_group"):
            fn = lambda: ops.psgd_project_grouped(mode, Ms, Xs, outs)
        else:
            def fn():
                for M, X, o in zip(Ms, Xs, outs):
                    ops.psgd_project(mode, M, X, [o])
        traffic = sum(a * b for a, b in shapes) * 4
        n = traffic // 4
    elif k in ("psgd_group_expand", "psgd_loop_expand"):
        # M -= P Q^T and the SGD-momentum step from P Q^T for the 19 weight matrices of VGG-19: one grid over all
        # of them against one launch per matrix; --mb is ignored
        import hipress_b200 as hp
        chans = [(64, 3), (64, 64), (128, 64), (128, 128), (256, 128), (256, 256), (256, 256), (256, 256),
                 (512, 256), (512, 512), (512, 512), (512, 512), (512, 512), (512, 512), (512, 512), (512, 512)]
        shapes = [(o, i * 9) for o, i in chans] + [(4096, 25088), (4096, 4096), (1000, 4096)]
        Ms = [torch.randn(a, b, device=dev) for a, b in shapes]
        Ps = [torch.randn(a, 4, device=dev) * 0.01 for a, b in shapes]
        Qs = [torch.randn(b, 4, device=dev) * 0.01 for a, b in shapes]
        params = [torch.randn(a * b, device=dev) for a, b in shapes]
        moms = [torch.zeros(a * b, device=dev) for a, b in shapes]
        if k == "psgd_group_expand":
            fn = lambda: hp._C.psgd_expand_sgd_grouped(Ps, Qs, Ms, params, moms, 1.0, 0.01, 0.9, 0.0, False)
        else:
            def fn():
                for P_, Q_, M_, p_, m_ in zip(Ps, Qs, Ms, params, moms):
                    hp._C.psgd_expand_sgd(P_, Q_, M_, p_, m_, 1.0, 0.01, 0.9, 0.0, False)
        n = sum(a * b for a, b in shapes)
        traffic = n * 24          # read and write the matrix, the parameters and the momentum
    elif k == "terngrad_unpack_apply":
        # what a training step runs per bucket: decode `world` payloads, average, fused SGD step,
        # zeros left in the gradient bucket
        import hipress_b200 as hp
        from hipress_b200.parallel import SymmetricMemory
        cfg = dict(rank=0, world=1, device=0, codec="terngrad", bitwidth=2, enable_random=1, error_feedback=1,
                   clear_grad=1, num_workers=0)
        eng = hp._C.DdpEngine(cfg, [(0, n, 1)], [0])
        sym = SymmetricMemory(eng.symmetric_bytes, dev, None)
        p, m = torch.randn(n, device=dev), torch.zeros(n, device=dev)
        eng.set_buffers(g, r, p, m, None, None)
        eng.set_symmetric(sym.buf)
        eng.set_sgd(0.1, 0.9, 0.0, True)

        def fn():
            eng.begin_step()
            eng.bucket_ready(0, 0)
            eng.finish_step(0)
        traffic = n * (8 + 8 + 4 + 0.25) + n * (0.25 + 4 + 16)   # compress (with min/max pass) + unpack/apply
    elif k in ("bn_fwd", "bn_bwd"):
        # one ResNet-50 stage-1 activation: [N, 256, 56, 56] bf16 channels-last, --mb = its size
        import hipress_b200 as hp
        c = 256
        imgs = max(1, int(args.mb * (1 << 20) / 2 / (c * 56 * 56)))
        shape = (imgs, c, 56, 56)
        x = torch.randn(shape, device=dev).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        res = torch.randn(shape, device=dev).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        w, b = torch.ones(c, device=dev), torch.zeros(c, device=dev)
        y, stats = hp._C.bn_forward(x, res, w, b, None, None, None, 0.1, 1e-5, True)
        nbytes = x.numel() * 2
        if k == "bn_fwd":
            fn = lambda: hp._C.bn_forward(x, res, w, b, None, None, None, 0.1, 1e-5, True)
            traffic = nbytes * 4          # stats: read x; apply: read x, residual, write y
        else:
            dy = torch.randn(shape, device=dev).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
            fn = lambda: hp._C.bn_backward(dy, x, y, w, stats, True, True)
            traffic = nbytes * 8          # reduce: dy, x, y; elemt: dy, x, y -> dx, dres
        n = x.numel()
    elif k in ("bias_relu_pool_fwd", "bias_relu_pool_bwd", "maxpool_fwd", "maxpool_bwd"):
        # a VGG-19 block-1 / ResNet stem activation: [N, 64, 224, 224] (or 112) bf16 channels-last, --mb = its size
        import hipress_b200 as hp
        c, hw = 64, (224 if k.startswith("bias") else 112)
        imgs = max(1, int(args.mb * (1 << 20) / 2 / (c * hw * hw)))
        x = torch.randn(imgs, c, hw, hw, device=dev).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        nbytes = x.numel() * 2
        if k.startswith("bias"):
            b = torch.randn(c, device=dev)
            y, idx = hp._C.bias_relu_forward(x, b, True)
            dy = torch.randn_like(y)
            if k.endswith("fwd"):
                fn = lambda: hp._C.bias_relu_forward(x, b, True)
                traffic = nbytes * (1 + 0.25 + 0.125)          # read x, write y (1/4) and one index byte per output
            else:
                fn = lambda: hp._C.bias_relu_backward(dy, y, idx, True)
                traffic = nbytes * (0.25 + 0.25 + 0.125 + 1)   # read dy, y, idx; write dz
        else:
            y, idx = hp._C.maxpool3x3s2_forward(x)
            dy = torch.randn_like(y)
            if k.endswith("fwd"):
                fn = lambda: hp._C.maxpool3x3s2_forward(x)
                traffic = nbytes * (1 + 0.25 + 0.125)
            else:
                fn = lambda: hp._C.maxpool3x3s2_backward(dy, idx, hw, hw)
                traffic = nbytes * (0.25 + 0.125 + 1)
        n = x.numel()
    elif k in ("add_ln_fwd", "add_ln_bwd"):
        # BERT-large residual stream: [tokens, 1024] bf16, --mb = its size (8 MB = the benchmark's 4096 tokens)
        import hipress_b200 as hp
        hsz = 1024
        rows = max(1, int(args.mb * (1 << 20) / 2 / hsz))
        x = torch.randn(rows, hsz, device=dev).to(torch.bfloat16)
        d = torch.randn(rows, hsz, device=dev).to(torch.bfloat16)
        w, b = torch.ones(hsz, device=dev), torch.zeros(hsz, device=dev)
        y, z, stats = hp._C.add_ln_forward(x, d, w, b, 1e-12)
        dy = torch.randn_like(y)
        nbytes = x.numel() * 2
        if k.endswith("fwd"):
            fn = lambda: hp._C.add_ln_forward(x, d, w, b, 1e-12)
            traffic = nbytes * 4          # read x, delta; write z, y
        else:
            fn = lambda: hp._C.add_ln_backward(dy, z, stats, w)
            traffic = nbytes * 3          # read dy, z; write dz
        n = x.numel()
    elif k == "adamw":
        import hipress_b200 as hp
        p, m, v = torch.randn(n, device=dev), torch.zeros(n, device=dev), torch.zeros(n, device=dev)
        fn = lambda: hp._C.adamw_apply(g, p, m, v, 0.5, 1e-4, 0.9, 0.999, 1e-8, 0.01, 3, True)
        traffic = n * 32
    else:
        import hipress_b200 as hp
        p, m = torch.randn(n, device=dev), torch.zeros(n, device=dev)
        fn = lambda: hp._C.sgd_apply(g, p, m, 0.5, 0.1, 0.9, 0.0, False)
        traffic = n * 24
    fn()
    torch.cuda.synchronize()
    if args.graph:
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            fn()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                fn()
        torch.cuda.synchronize()
        fn = graph.replay
    ms = timed(fn, args.iters)
    gbs = traffic / (ms * 1e-3) / 1e9
    print(json.dumps({"kernel": k, "mb": round(n * 4 / (1 << 20), 1) if k.startswith("psgd") else args.mb, "n": n,
                      "graph": args.graph, "ms": round(ms, 4), "algorithmic_gbs": round(gbs, 1),
                      "fraction_of_measured_hbm": round(gbs / hbm, 3), "hbm_gbs_measured_peak": hbm}))


if __name__ == "__main__":
    main()
