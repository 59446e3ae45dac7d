"""sm_100a kernels against the CPU codec (byte-exact) and fp64 restatements (PowerSGD)."""
import struct

import pytest
import torch

from hipress_b200 import ops
import hipress_b200 as hp

pytestmark = pytest.mark.gpu

SIZES = [1, 3, 4, 5, 31, 127, 128, 129, 1000, 4099, 65536, 1 << 20, (1 << 20) + 7]


def gauss(n, std=0.01, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(n, generator=g) * std


def dev(t):
    return t.cuda()


def check_status(like):
    assert ops.read_status(like) == 0


# ----------------------------------------------------------------------------- TBQ
@pytest.mark.parametrize("n", SIZES)
def test_tbq_compress_matches_cpu(n):
    t = 0.01
    g, r = gauss(n, seed=n), gauss(n, 0.004, seed=n + 1)
    rc = r.clone()
    ref = ops.tbq_compress(g, rc, t)
    rg = dev(r)
    out = ops.tbq_compress(dev(g), rg, t)
    assert torch.equal(out.cpu(), ref)
    assert torch.equal(rg.cpu(), rc)


def test_tbq_unaligned_views():
    n, t = 10001, 0.01
    base_g, base_r = gauss(n + 3, seed=1), gauss(n + 3, 0.004, seed=2)
    g, r = base_g[1:n + 1], base_r[3:n + 3].clone()
    ref_r = r.clone()
    ref = ops.tbq_compress(g.contiguous(), ref_r, t)
    dg, dr = dev(base_g)[1:n + 1], dev(base_r)[3:n + 3]
    out = torch.empty(ops.tbq_payload_bytes(n) + 1, dtype=torch.uint8, device="cuda")[1:]
    ops.tbq_compress(dg, dr, t, out=out)
    assert torch.equal(out.cpu(), ref)
    assert torch.equal(dr.cpu(), ref_r)


@pytest.mark.parametrize("n", [5, 1000, 65537])
@pytest.mark.parametrize("world", [1, 3, 8])
def test_tbq_unpack_all_ranks_one_pass(n, world):
    t = 0.02
    payloads = [ops.tbq_compress(gauss(n, 0.03, seed=s), torch.zeros(n), t) for s in range(world)]
    for add in (False, True):
        base = gauss(n, 1.0, seed=77)
        ref = base.clone()
        ops.tbq_decompress(payloads, ref, t, add=add, post_scale=1.0 / world)
        out = dev(base)
        ops.tbq_decompress([dev(p) for p in payloads], out, t, add=add, post_scale=1.0 / world)
        assert torch.equal(out.cpu(), ref)


# ----------------------------------------------------------------------------- TernGrad
@pytest.mark.parametrize("bw", [1, 2, 4, 8])
@pytest.mark.parametrize("random", [False, True])
@pytest.mark.parametrize("n", SIZES)
def test_terngrad_compress_matches_cpu(bw, random, n):
    g = gauss(n, seed=n + bw)
    ref = ops.terngrad_compress(g, bw, random, seed=1)
    out = ops.terngrad_compress(dev(g), bw, random, seed=1)
    assert torch.equal(out.cpu(), ref)


@pytest.mark.parametrize("n", [7, 4099, 1 << 18])
def test_terngrad_error_feedback_matches_cpu(n):
    g, r = gauss(n, seed=1), gauss(n, 0.003, seed=2)
    rc = r.clone()
    ref = ops.terngrad_compress(g, 2, True, seed=5, residual=rc)
    rg = dev(r)
    out = ops.terngrad_compress(dev(g), 2, True, seed=5, residual=rg)
    assert torch.equal(out.cpu(), ref)
    assert torch.equal(rg.cpu(), rc)


def test_terngrad_back_to_back_calls_reuse_scratch():
    outs = []
    for s in range(4):
        g = gauss(50000 + s, seed=s)
        outs.append((ops.terngrad_compress(dev(g), 2, True, seed=s), ops.terngrad_compress(g, 2, True, seed=s)))
    for a, b in outs:
        assert torch.equal(a.cpu(), b)


@pytest.mark.parametrize("bw", [1, 2, 4, 8])
@pytest.mark.parametrize("n", [3, 1000, 65541])
@pytest.mark.parametrize("world", [1, 4, 8])
def test_terngrad_unpack_all_ranks_one_pass(bw, n, world):
    payloads = [ops.terngrad_compress(gauss(n, 0.01 * (s + 1), seed=s), bw, True, seed=s) for s in range(world)]
    for add in (False, True):
        base = gauss(n, 1.0, seed=9)
        ref = base.clone()
        ops.terngrad_decompress(payloads, ref, add=add, post_scale=1.0 / world)
        out = dev(base)
        ops.terngrad_decompress([dev(p) for p in payloads], out, add=add, post_scale=1.0 / world)
        assert torch.equal(out.cpu(), ref)
        check_status(out)


def test_terngrad_unpack_reports_bad_header():
    n = 1000
    p = dev(ops.terngrad_compress(gauss(n), 2, False))
    p[0] = 3  # invalid bitwidth
    out = torch.zeros(n, device="cuda")
    ops.terngrad_decompress(p, out)
    assert ops.read_status(out) == 3
    assert ops.read_status(out) == 0  # reading resets


# ----------------------------------------------------------------------------- sparse
def _parse(payload):
    raw = bytes(payload.cpu().tolist())
    total = struct.unpack("<i", raw[:4])[0]
    k = (total - 4) // 8
    return total, k


@pytest.mark.parametrize("n,keep,rate", [(1000, 0.01, 0.05), (100000, 0.001, 0.01), (4097, 0.05, 0.1),
                                         (1 << 20, 0.001, 0.01), ((1 << 21) + 5, 0.001, 0.01),
                                         (50000, 0.01, 0.0)])
@pytest.mark.parametrize("accumulate", [True, False])
def test_sparse_compress_matches_cpu(n, keep, rate, accumulate):
    g, r = gauss(n, seed=n), gauss(n, 0.003, seed=n + 1)
    for seed in (1, 2, 3):  # different seeds land on both sides of the over-selection branch
        rc, rg = r.clone(), dev(r)
        if accumulate:
            ref = ops.graddrop_compress(g, rc, rate, 1 - keep, seed)
            out = ops.graddrop_compress(dev(g), rg, rate, 1 - keep, seed)
        else:
            ref = ops.dgc_compress(rc, rate, keep, seed)
            out = ops.dgc_compress(rg, rate, keep, seed)
        total, k = _parse(ref)
        assert torch.equal(out[:total].cpu(), ref[:total]), f"seed {seed} k {k}"
        assert torch.equal(rg.cpu(), rc)


@pytest.mark.parametrize("keep,rate", [(0.001, 0.01), (0.01, 0.02)])
def test_sparse_clustered_values_match_cpu(keep, rate):
    """All the large values sit in a few short index ranges (one layer with large gradients):
    the lists of the warps that own those ranges grow over many pool blocks."""
    n = (1 << 21) + 77
    r = gauss(n, 1e-4, seed=3)
    big = gauss(n, 1.0, seed=4)
    for lo in (1000, 700000, n - 6000):
        r[lo:lo + 5000] = big[lo:lo + 5000]
    for seed in (1, 2):
        rc, rg = r.clone(), dev(r)
        ref = ops.dgc_compress(rc, rate, keep, seed)
        out = ops.dgc_compress(rg, rate, keep, seed)
        total, k = _parse(ref)
        assert k > 0
        assert torch.equal(out[:total].cpu(), ref[:total]), f"seed {seed} k {k}"
        assert torch.equal(rg.cpu(), rc)


@pytest.mark.parametrize("n,keep,rate", [(300000 + 3, 0.001, 0.01), (1 << 20, 0.01, 0.01), (70000, 0.05, 0.1)])
def test_dgc_momentum_fused_matches_restatement(n, keep, rate):
    """u = m*u + g, v += u, select from v, mask u and v: the fused pipeline against the same steps
    spelled out with tensor ops and the CPU selector (momentum 0.5 keeps the products exact, so the
    restatement rounds like the kernel's fused multiply-add)."""
    g, u, v = gauss(n, seed=1), gauss(n, 0.02, seed=2), gauss(n, 0.03, seed=3)
    for seed in (5, 6):
        cu = 0.5 * u + g
        cv = v + cu
        ref = ops.dgc_compress(cv, rate, keep, seed)        # zeroes the selected entries of cv
        total, k = _parse(ref)
        idx = ref[4:4 + 4 * k].view(torch.int32).long()
        cu[idx] = 0.0
        dg, du, dv = dev(g), dev(u), dev(v)
        out = ops.dgc_momentum_compress(dg, du, dv, rate, keep, seed, momentum=0.5, zero_grad=True)
        assert torch.equal(out[:total].cpu(), ref[:total]), f"seed {seed} k {k}"
        assert torch.equal(dv.cpu(), cv) and torch.equal(du.cpu(), cu)
        assert float(dg.abs().max()) == 0.0
        u, v = cu, cv
        g = gauss(n, seed=10 + seed)


def test_sparse_ties_and_trim_on_gpu():
    v = torch.tensor([1.0, -1.0, 1.0, 0.5, 1.0, -1.0, 0.25, 1.0] * 300)
    ref_v, dev_v = v.clone(), dev(v)
    ref = ops.dgc_compress(ref_v, 0.0, 0.1, 0)
    out = ops.dgc_compress(dev_v, 0.0, 0.1, 0)
    total, _ = _parse(ref)
    assert torch.equal(out[:total].cpu(), ref[:total])
    assert torch.equal(dev_v.cpu(), ref_v)


@pytest.mark.parametrize("world", [1, 4, 8])
def test_sparse_unpack_matches_cpu(world):
    n = 200000
    payloads = [ops.dgc_compress(gauss(n, seed=s), 0.01, 0.002, seed=s) for s in range(world)]
    for add in (False, True):
        base = gauss(n, 1.0, seed=5)
        ref = base.clone()
        ops.sparse_decompress(payloads, ref, add=add, post_scale=1.0 / world)
        out = dev(base)
        ops.sparse_decompress([dev(p) for p in payloads], out, add=add, post_scale=1.0 / world)
        assert torch.equal(out.cpu(), ref)
        check_status(out)


def test_sparse_unpack_bounds_checked():
    n = 1000
    p = dev(ops.dgc_compress(gauss(n), 0.0, 0.01, 0))
    p[0:4] = torch.tensor(list(struct.pack("<i", 4 + 8 * 5000)), dtype=torch.uint8, device="cuda")
    out = torch.zeros(n, device="cuda")
    ops.sparse_decompress(p, out)
    assert ops.read_status(out) == 2


# ----------------------------------------------------------------------------- ECQ
@pytest.mark.parametrize("bw", [2, 4, 8])
@pytest.mark.parametrize("n", [5, 1000, 65541])
def test_ecq_matches_cpu(bw, n):
    g, h = gauss(n, seed=n), gauss(n, 0.002, seed=n + 1)
    hc, hg = h.clone(), dev(h)
    ref = ops.ecq_compress(g, hc, 1.0, 0.9, bw, seed=4)
    out = ops.ecq_compress(dev(g), hg, 1.0, 0.9, bw, seed=4)
    assert torch.equal(out.cpu(), ref)
    assert torch.equal(hg.cpu(), hc)
    d_ref = torch.empty(n)
    ops.ecq_decompress([ref, ref], d_ref)
    d_out = torch.empty(n, device="cuda")
    ops.ecq_decompress([out, out], d_out)
    assert torch.equal(d_out.cpu(), d_ref)


# ----------------------------------------------------------------------------- PowerSGD
PSGD_SHAPES = [(128, 128, 4), (256, 512, 4), (300, 1000, 4), (64, 4608, 4), (512, 4608, 2),
               (1000, 4096, 4), (4096, 2048, 1), (130, 36, 4), (77, 60, 3), (200, 1024, 16)]


@pytest.mark.parametrize("n,m,r", PSGD_SHAPES)
@pytest.mark.parametrize("simt", [False, True])
def test_psgd_project_matches_fp64(n, m, r, simt):
    torch.manual_seed(n + m + r)
    M = torch.randn(n, m, device="cuda")
    Q = torch.randn(m, r, device="cuda")
    P = torch.zeros(n, r, device="cuda")
    ops.psgd_project(0, M, Q, [P], simt=simt)
    ref = (M.double() @ Q.double())
    # TF32 inputs (10-bit mantissa), fp32 accumulation
    tol = 5e-3 * (m ** 0.5) if not simt else 1e-4 * (m ** 0.5)
    assert (P.double() - ref).abs().max().item() <= tol
    Pn = torch.randn(n, r, device="cuda")
    Qo = torch.zeros(m, r, device="cuda")
    ops.psgd_project(1, M, Pn, [Qo], simt=simt)
    ref = (M.double().T @ Pn.double())
    tol = 5e-3 * (n ** 0.5) if not simt else 1e-4 * (n ** 0.5)
    assert (Qo.double() - ref).abs().max().item() <= tol
    assert ops.read_status(M) == 0


@pytest.mark.parametrize("bk,stages", [(32, 4), (64, 3), (64, 4)])
@pytest.mark.parametrize("n,m,r", [(128, 128, 4), (300, 1000, 4), (1000, 4096, 4), (130, 36, 4), (512, 4608, 2)])
def test_psgd_project_variants_match_fp64(monkeypatch, bk, stages, n, m, r):
    """Every pipeline shape of the tensor-core projection (one or two 128-byte boxes per row and stage, ring
    depth) gives the same TF32-level result."""
    monkeypatch.setenv("HIPRESS_PSGD_BK", str(bk))
    monkeypatch.setenv("HIPRESS_PSGD_STAGES", str(stages))
    torch.manual_seed(n + m + r)
    M = torch.randn(n, m, device="cuda")
    Q = torch.randn(m, r, device="cuda")
    P = torch.zeros(n, r, device="cuda")
    ops.psgd_project(0, M, Q, [P])
    ref = M.double() @ Q.double()
    assert (P.double() - ref).abs().max().item() <= 5e-3 * (m ** 0.5)
    Pn = torch.randn(n, r, device="cuda")
    Qo = torch.zeros(m, r, device="cuda")
    ops.psgd_project(1, M, Pn, [Qo])
    ref = M.double().T @ Pn.double()
    assert (Qo.double() - ref).abs().max().item() <= 5e-3 * (n ** 0.5)
    assert ops.read_status(M) == 0


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("count", [1, 5, 30])
def test_psgd_project_grouped_matches_fp64(mode, count):
    """One grid over a list of matrices (mixed sizes, ragged tiles, one SIMT-only shape, more matrices than a
    launch holds) equals the per-matrix products."""
    torch.manual_seed(count + mode)
    shapes = [(64, 576), (512, 4608), (300, 1000), (128, 1152), (77, 61), (1000, 4096), (256, 2304), (130, 36)]
    Ms, Xs, outs, refs = [], [], [], []
    for i in range(count):
        n, m = shapes[i % len(shapes)]
        M = torch.randn(n, m, device="cuda")
        X = torch.randn(m if mode == 0 else n, 4, device="cuda")
        Ms.append(M)
        Xs.append(X)
        outs.append(torch.zeros(n if mode == 0 else m, 4, device="cuda"))
        refs.append(M.double() @ X.double() if mode == 0 else M.double().T @ X.double())
    ops.psgd_project_grouped(mode, Ms, Xs, outs)
    for M, o, ref in zip(Ms, outs, refs):
        k = M.shape[1] if mode == 0 else M.shape[0]
        assert (o.double() - ref).abs().max().item() <= 5e-3 * (k ** 0.5), tuple(M.shape)
    assert ops.read_status(Ms[0]) == 0


def test_psgd_expand_sgd_grouped_matches_per_matrix():
    """One grid over a list of matrices (vectorised and ragged shapes mixed) leaves the same bits in the error
    feedback, the parameters and the momentum as one launch per matrix."""
    torch.manual_seed(5)
    shapes = [(64, 576), (512, 4608), (300, 1000), (77, 61), (1000, 4096), (130, 36)] * 7   # more than one launch holds
    def make():
        torch.manual_seed(6)
        return ([torch.randn(a, b, device="cuda") for a, b in shapes],
                [torch.randn(a, 4, device="cuda") * 0.1 for a, b in shapes],
                [torch.randn(b, 4, device="cuda") * 0.1 for a, b in shapes],
                [torch.randn(a * b, device="cuda") for a, b in shapes],
                [torch.randn(a * b, device="cuda") * 0.01 for a, b in shapes])
    Ms, Ps, Qs, params, moms = make()
    hp._C.psgd_expand_sgd_grouped(Ps, Qs, Ms, params, moms, 0.5, 0.01, 0.9, 1e-4, False)
    Mr, Pr, Qr, pr, mr = make()
    for P_, Q_, M_, p_, m_ in zip(Pr, Qr, Mr, pr, mr):
        hp._C.psgd_expand_sgd(P_, Q_, M_, p_, m_, 0.5, 0.01, 0.9, 1e-4, False)
    for a, b in zip(Ms + params + moms, Mr + pr + mr):
        assert torch.equal(a, b)


def test_psgd_project_relative_error_tf32():
    torch.manual_seed(0)
    n, m, r = 1024, 4096, 4
    M = torch.randn(n, m, device="cuda")
    Q = torch.randn(m, r, device="cuda")
    P = torch.zeros(n, r, device="cuda")
    assert hp._C.psgd_tensor_core_eligible(M)
    ops.psgd_project(0, M, Q, [P])
    ref = M.double() @ Q.double()
    rel = ((P.double() - ref).norm() / ref.norm()).item()
    assert rel < 2e-3, rel


def test_psgd_owner_split_accumulates_into_owners():
    torch.manual_seed(3)
    n, m, r, world = 512, 1024, 4, 4
    M = torch.randn(n, m, device="cuda")
    Q = torch.randn(m, r, device="cuda")
    owners = [torch.zeros(n, r, device="cuda") for _ in range(world)]
    ops.psgd_project(0, M, Q, owners)
    ref = (M.double() @ Q.double()).float()
    rows = (n + world - 1) // world
    for w, o in enumerate(owners):
        lo, hi = w * rows, min(n, (w + 1) * rows)
        torch.testing.assert_close(o[lo:hi], ref[lo:hi], atol=0.3, rtol=1e-2)
        rest = o.clone()
        rest[lo:hi] = 0
        assert rest.abs().max().item() == 0


@pytest.mark.parametrize("n,r", [(64, 1), (1000, 4), (25088, 4), (4096, 16)])
def test_gram_schmidt(n, r):
    torch.manual_seed(n)
    P = torch.randn(n, r, device="cuda")
    ref = P.cpu().clone()
    ops.gram_schmidt(ref)
    ops.gram_schmidt(P)
    eye = (P.double().T @ P.double()).cpu()
    torch.testing.assert_close(eye, torch.eye(r, dtype=torch.float64), atol=1e-4, rtol=0)
    torch.testing.assert_close(P.cpu(), ref, atol=1e-4, rtol=1e-3)


def test_powersgd_stages_match_cpu():
    torch.manual_seed(0)
    n, m, r = 256, 1152, 4
    N = n * m - 5
    grad, resid = torch.randn(N), torch.randn(N) * 0.1
    Q0 = torch.randn(m, r)
    cpu = dict(grad=grad.clone(), resid=resid.clone(), Q=Q0.clone(), M=torch.zeros(n, m), P=torch.zeros(n, r))
    gpu = {k: v.cuda() for k, v in cpu.items()}
    for d in (cpu, gpu):
        ops.powersgd_encode1(d["grad"], d["resid"], d["Q"], d["M"], d["P"])
    torch.testing.assert_close(gpu["M"].cpu(), cpu["M"], atol=0, rtol=0)
    torch.testing.assert_close(gpu["P"].cpu(), cpu["P"], atol=0.2, rtol=1e-2)
    for d in (cpu, gpu):
        ops.powersgd_encode2(d["P"], d["M"], d["Q"])
    eye = gpu["P"].double().T @ gpu["P"].double()
    torch.testing.assert_close(eye.cpu(), torch.eye(r, dtype=torch.float64), atol=1e-4, rtol=0)
    # decode from identical factors
    gpu["P"].copy_(cpu["P"])
    gpu["Q"].copy_(cpu["Q"])
    for d in (cpu, gpu):
        ops.powersgd_decode(d["P"], d["Q"], d["M"], d["resid"], d["grad"])
    torch.testing.assert_close(gpu["grad"].cpu(), cpu["grad"], atol=1e-4, rtol=1e-4)
    torch.testing.assert_close(gpu["resid"].cpu(), cpu["resid"], atol=1e-4, rtol=1e-4)


def test_psgd_expand_feedback():
    torch.manual_seed(1)
    n, m, r = 100, 333, 4
    P, Q = torch.randn(n, r, device="cuda"), torch.randn(m, r, device="cuda")
    M = torch.randn(n, m, device="cuda")
    M0 = M.clone()
    out = torch.zeros(n * m - 3, device="cuda")
    ops.psgd_expand_feedback(P, Q, M, out, post_scale=0.5)
    approx = P @ Q.T
    torch.testing.assert_close(M, M0 - approx, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(out, approx.view(-1)[: out.numel()] * 0.5, atol=1e-5, rtol=1e-5)


# ----------------------------------------------------------------------------- fused SGD
def test_sgd_apply_matches_torch():
    torch.manual_seed(0)
    n = 100003
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda")
    ref_p = torch.nn.Parameter(p.clone())
    opt = torch.optim.SGD([ref_p], lr=0.1, momentum=0.9, weight_decay=1e-4)
    mom = torch.zeros(n, device="cuda")
    for step in range(3):
        ref_p.grad = (g * 0.5).clone()
        opt.step()
        hp._C.sgd_apply(g.clone(), p, mom, 0.5, 0.1, 0.9, 1e-4, step == 0)
        torch.testing.assert_close(p, ref_p.data, atol=1e-6, rtol=1e-6)


@pytest.mark.parametrize("n,m,r", [(128, 512, 4), (300, 1024, 2), (64, 4608, 8), (100, 333, 4)])
def test_psgd_expand_paths_match_torch(n, m, r):
    """Vectorised (m % 4 == 0) and generic expand kernels: feedback form and fused-SGD form."""
    torch.manual_seed(n + m)
    P, Q = torch.randn(n, r, device="cuda"), torch.randn(m, r, device="cuda")
    M0 = torch.randn(n, m, device="cuda")
    approx = P @ Q.T
    M = M0.clone()
    out = torch.zeros(n * m, device="cuda")
    ops.psgd_expand_feedback(P, Q, M, out, post_scale=0.25)
    torch.testing.assert_close(M, M0 - approx, atol=1e-4, rtol=1e-5)
    torch.testing.assert_close(out.view(n, m), approx * 0.25, atol=1e-4, rtol=1e-5)
    # fused SGD: two steps against torch.optim.SGD fed with the same approximations
    M = M0.clone()
    param = torch.randn(n * m, device="cuda")
    ref = torch.nn.Parameter(param.clone())
    opt = torch.optim.SGD([ref], lr=0.1, momentum=0.9, weight_decay=1e-4)
    mom = torch.zeros(n * m, device="cuda")
    for step in range(2):
        ref.grad = approx.reshape(-1).clone()
        opt.step()
        hp._C.psgd_expand_sgd(P, Q, M, param, mom, 1.0, 0.1, 0.9, 1e-4, step == 0)
        torch.testing.assert_close(param, ref.data, atol=1e-4, rtol=1e-5)
    torch.testing.assert_close(M, M0 - 2 * approx, atol=2e-4, rtol=1e-5)


def test_adamw_apply_matches_torch():
    torch.manual_seed(0)
    n = 50001
    p = torch.randn(n, device="cuda")
    ref = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    for step in range(1, 4):
        g = torch.randn(n, device="cuda")
        ref.grad = (g * 0.5).clone()
        opt.step()
        hp._C.adamw_apply(g, p, m, v, 0.5, 1e-2, 0.9, 0.999, 1e-8, 0.01, step)
        torch.testing.assert_close(p, ref.data, atol=1e-5, rtol=1e-5)
