"""PowerSGD and DGC data-parallel wrappers on one GPU (world 1, and two ranks emulated in one
process phase by phase, with a device synchronise between phases so that no kernel waits for
one that has not been launched)."""
import copy

import pytest
import torch

from hipress_b200.models import bert_tiny, vgg_tiny
from hipress_b200.parallel import SymmetricMemory
from hipress_b200.parallel.dgc import DGCDataParallel, warmup_schedule
from hipress_b200.parallel.powersgd import PowerSGDDataParallel

pytestmark = pytest.mark.gpu


def test_powersgd_world1_trains_and_keeps_error_feedback():
    torch.manual_seed(0)
    net = vgg_tiny(10).cuda()
    model = PowerSGDDataParallel(net, rank_r=4, lr=0.05, momentum=0.9)
    x = torch.randn(32, 3, 32, 32, device="cuda")
    y = torch.randint(0, 10, (32,), device="cuda")
    losses = []
    for _ in range(30):
        loss = torch.nn.functional.cross_entropy(model(x), y)
        loss.backward()
        model.step()
        losses.append(float(loss))
    model.check()
    assert min(losses[-5:]) < losses[0] - 0.05, losses   # rank-4 updates of a tiny VGG learn slowly
    assert model.flat_M.abs().sum().item() > 0          # residual is carried
    # columns are unit length unless the gradient has lost rank (then norm + eps shrinks them)
    for P in model.P:
        gram = P.double().T @ P.double()
        assert gram.diagonal().max().item() <= 1.0 + 1e-3


def test_powersgd_two_emulated_ranks_stay_identical_and_match_restatement():
    torch.manual_seed(0)
    base = vgg_tiny(10).cuda()
    nets = [copy.deepcopy(base), copy.deepcopy(base)]
    world = 2
    models = []
    probe = PowerSGDDataParallel(copy.deepcopy(base), rank_r=2, world=1, rank=0)
    need = probe.symmetric.nbytes
    mems = SymmetricMemory.emulate(need, world)
    for r in range(world):
        models.append(PowerSGDDataParallel(nets[r], rank_r=2, lr=0.05, momentum=0.0, rank=r, world=world,
                                           symmetric=mems[r], emulated=True, flag_timeout_s=2.0))
    vmems = SymmetricMemory.emulate(models[0].vec_engine.symmetric_bytes, world)
    for m, vm in zip(models, vmems):
        m._attach_vec(vm)
    xs = [torch.randn(16, 3, 32, 32, device="cuda") for _ in range(world)]
    ys = [torch.randint(0, 10, (16,), device="cuda") for _ in range(world)]
    # restatement in plain torch (fp64 factors) for the first step of the largest matrix
    i_big = max(range(len(models[0].mats)), key=lambda i: models[0].mats[i].numel())
    for step in range(3):
        for m, x, y in zip(models, xs, ys):
            torch.nn.functional.cross_entropy(m(x), y).backward()
        if step == 0:
            n, mm = models[0].shapes[i_big]
            Ms = [m._mat(i_big).double().clone() for m in models]
            Q0 = models[0].Q[i_big].double().clone()
            P = sum(M @ Q0 for M in Ms) / world
            Pq, _ = torch.linalg.qr(P)
            Qn = sum(M.T @ Pq for M in Ms) / world
            approx_ref = Pq @ Qn.T
            before = models[0].flat_param[models[0].offsets[i_big]:models[0].offsets[i_big] + n * mm].double().clone()
        for phase in ("phase_project_p", "phase_project_q", "phase_apply"):
            for m in models:
                getattr(m, phase)()
            for m in models:
                if m.vec_engine is not None:
                    m.vec_engine.drain()
            torch.cuda.synchronize()
        if step == 0:
            after = models[0].flat_param[models[0].offsets[i_big]:models[0].offsets[i_big] + n * mm].double()
            applied = (before - after).view(n, mm) / 0.05     # = approximation used as the gradient
            rel = ((applied - approx_ref).norm() / approx_ref.norm()).item()
            assert rel < 2e-2, rel
        for m in models:
            m.check()
        assert torch.equal(models[0].flat_param, models[1].flat_param)
        assert torch.equal(models[0].vec_param, models[1].vec_param)


def test_dgc_schedule():
    s = warmup_schedule(0.001, 400)
    assert s[0] == (0, 0.25) and s[-1] == (400, 0.001)
    assert [k for _, k in s] == sorted([k for _, k in s], reverse=True)


def test_dgc_world1_trains_with_warmup_and_adamw():
    torch.manual_seed(0)
    net = bert_tiny().cuda()
    model = DGCDataParallel(net, keep_fraction=0.01, warmup_steps=8, lr=2e-3, weight_decay=0.0, bucket_mb=0.05,
                            clip_norm=1.0)
    ids = torch.randint(0, 1000, (8, 32), device="cuda")
    labels = torch.full_like(ids, -100)
    labels[:, ::5] = ids[:, ::5]
    losses = []
    keeps = []
    for step in range(30):
        keeps.append(model.keep_fraction_at(model.engine.steps))
        loss = model(ids, labels)
        loss.backward()
        model.step()
        losses.append(float(loss))
    model.check()
    assert keeps[0] == 0.25 and keeps[-1] == 0.01
    assert min(losses[-5:]) < losses[0], losses
    st = model.compression_state()
    assert {"residual", "momentum", "second_moment", "velocity"} <= set(st)


def test_psgd_engine_batched_step_matches_per_matrix_ops():
    """40 matrices (two parameter-space batches of the small kernels) through the native step
    driver against the same step issued one op at a time."""
    from hipress_b200 import _C
    torch.manual_seed(3)
    r, dev = 4, "cuda"
    shapes = [(64 + 8 * i, 96 + 4 * i) for i in range(38)] + [(30, 27), (513, 1000)]
    eng = _C.PsgdEngine(1, r, torch.zeros(1, device=dev))
    state = []
    for n, m in shapes:
        M = torch.randn(n, m, device=dev)
        param, mom = torch.randn(n * m, device=dev), torch.zeros(n * m, device=dev)
        P, Q = torch.zeros(n, r, device=dev), torch.randn(m, r, device=dev)
        Pt = torch.zeros(16 * _C.psgd_kpad(n), device=dev)
        Qt = torch.zeros(16 * _C.psgd_kpad(m), device=dev)
        accP = [[torch.zeros(n, r, device=dev)] for _ in range(2)]
        accQ = [[torch.zeros(m, r, device=dev)] for _ in range(2)]
        state.append(dict(M=M, param=param, mom=mom, P=P, Q=Q, Pt=Pt, Qt=Qt, accP=accP, accQ=accQ,
                          M0=M.clone(), p0=param.clone(), Q0=Q.clone()))
        eng.add_matrix(M, param, mom, P, Q, Pt, Qt, accP, accQ)
    assert eng.matrices == 40
    eng.project_p(1, 0)
    eng.project_q(1, 0)
    eng.apply(1, 0.1, 0.9, 0.0, True, 0)
    torch.cuda.synchronize()
    assert _C.read_status(state[0]["M"], True) == 0
    for s in state:
        n, m = s["M0"].shape
        P = torch.zeros(n, r, device=dev)
        _C.psgd_project(0, s["M0"], s["Q0"], [P], False)
        _C.gram_schmidt(P, 1e-8)
        Q = torch.zeros(m, r, device=dev)
        _C.psgd_project(1, s["M0"], P, [Q], False)
        M, param, mom = s["M0"].clone(), s["p0"].clone(), torch.zeros(n * m, device=dev)
        _C.psgd_expand_sgd(P, Q, M, param, mom, 1.0, 0.1, 0.9, 0.0, True)
        # split-K partial sums are combined with atomics: equal up to summation order
        torch.testing.assert_close(s["P"], P, atol=2e-5, rtol=1e-4)
        torch.testing.assert_close(s["Q"], Q, atol=2e-3, rtol=1e-4)
        torch.testing.assert_close(s["M"], M, atol=2e-3, rtol=1e-4)
        torch.testing.assert_close(s["param"], param, atol=2e-3, rtol=1e-4)
