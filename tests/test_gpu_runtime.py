"""The reference's module API (init / submit_task / getResults / end) on CUDA tensors with the
CPU staging buffer ``C`` of the original contract."""
import struct

import pytest
import torch

from hipress_b200 import hp_cuda, ops

pytestmark = pytest.mark.gpu


@pytest.fixture()
def runtime():
    yield hp_cuda
    hp_cuda.end()


def gauss(n, std=0.01, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(n, generator=g) * std


def test_terngrad_tasks_on_gpu_match_cpu_codec(runtime):
    runtime.init("terngrad", {"enable_random": 0, "bitwidth": 2}, 0, 0, 1)
    names = [f"t{i}" for i in range(16)]
    grads = {k: gauss(20000 + 37 * i, seed=i) for i, k in enumerate(names)}
    dev = {k: g.cuda() for k, g in grads.items()}
    Bs = {k: torch.zeros(ops.terngrad_payload_bytes(g.numel(), 2), dtype=torch.uint8, device="cuda") for k, g in grads.items()}
    Cs = {k: torch.zeros(b.numel(), dtype=torch.uint8).pin_memory() for k, b in Bs.items()}
    for k in names:
        assert runtime.submit_task(k, dev[k], Bs[k], Cs[k], 0, runtime.COMP_TASK)
    assert sorted(runtime.wait_for(runtime.COMP_TASK, names)) == sorted(names)
    for k in names:
        assert torch.equal(Cs[k], ops.terngrad_compress(grads[k], 2, False)), k
    outs = {k: torch.zeros_like(v) for k, v in dev.items()}
    for k in names:
        Bs[k].zero_()
        runtime.submit_task(k, outs[k], Bs[k], Cs[k], 0, runtime.DECOMP_TASK)
    runtime.wait_for(runtime.DECOMP_TASK, names)
    for k in names:
        ref = torch.empty_like(grads[k])
        ops.terngrad_decompress(Cs[k], ref)
        assert torch.equal(outs[k].cpu(), ref), k
    assert runtime.getErrors() == []


def test_tbq_root_task_on_gpu(runtime):
    world, rank, n, t = 4, 2, 30001, 0.01
    runtime.init("tbq", {"threshold": t}, 0, rank, world)
    size = ops.tbq_payload_bytes(n)
    payloads = [ops.tbq_compress(gauss(n, 0.02, seed=r), torch.zeros(n), t) for r in range(world)]
    C = torch.cat(payloads).pin_memory()
    own = gauss(n, 0.02, seed=50)
    tensor, resid = own.cuda(), torch.zeros(n, device="cuda")
    B = torch.zeros(size, dtype=torch.uint8, device="cuda")
    assert runtime.submit_task("w", tensor, resid, B, C, 1, runtime.ROOT_DECOMP_COMP_TASK)
    runtime.wait_for(runtime.ROOT_DECOMP_COMP_TASK, ["w"])
    acc = own.clone()
    for r in range(world):
        if r != rank:
            ops.tbq_decompress(payloads[r], acc, t, add=True)
    assert torch.equal(tensor.cpu(), acc)
    r2 = torch.zeros(n)
    expect = ops.tbq_compress(acc, r2, t)
    assert torch.equal(B.cpu(), expect) and torch.equal(C[:size], expect)
    assert torch.equal(resid.cpu(), r2)


def test_graddrop_tasks_on_gpu(runtime):
    n, drop = 200000, 0.999
    runtime.init("graddrop", {"drop_ratio": drop, "sample_rate": 0.01, "seed": 3}, 0, 0, 1)
    g = gauss(n, seed=1)
    gd, resid = g.cuda(), torch.zeros(n, device="cuda")
    cap = ops.sparse_payload_bytes(n, 1 - drop)
    B = torch.zeros(cap, dtype=torch.uint8, device="cuda")
    C = torch.zeros(cap, dtype=torch.uint8).pin_memory()
    runtime.submit_task("g", gd, resid, B, C, 0, runtime.COMP_TASK)
    runtime.wait_for(runtime.COMP_TASK, ["g"])
    total = struct.unpack("<i", bytes(C[:4].tolist()))[0]
    assert 4 < total <= cap
    out = torch.zeros(n, device="cuda")
    runtime.submit_task("g", out, resid, torch.zeros_like(B), C, 0, runtime.DECOMP_TASK)
    runtime.wait_for(runtime.DECOMP_TASK, ["g"])
    torch.testing.assert_close(out.cpu() + resid.cpu(), g, atol=0, rtol=0)


def test_powersgd_tasks_on_gpu(runtime):
    runtime.init("powersgd", {"matrix_approximation_rank": 4}, 0, 0, 1)
    n, m, r = 256, 1024, 4
    torch.manual_seed(1)
    grad = torch.randn(n * m, device="cuda")
    g0 = grad.clone()
    resid = torch.zeros(n * m, device="cuda")
    M, P = torch.zeros(n, m, device="cuda"), torch.zeros(n, r, device="cuda")
    Q = torch.randn(m, r, device="cuda")
    Q0 = Q.clone()
    runtime.submit_task("p", grad, resid, M, P, Q, runtime.POWERSGD_ENCODE1)
    runtime.wait_for(runtime.POWERSGD_ENCODE1, ["p"])
    ref = g0.view(n, m).double() @ Q0.double()
    assert ((P.double() - ref).norm() / ref.norm()).item() < 5e-3
    runtime.submit_task("p", grad, resid, M, P, Q, runtime.POWERSGD_ENCODE2)
    runtime.wait_for(runtime.ROOT_DECOMP_COMP_TASK, ["p"])
    eye = P.double().T @ P.double()
    torch.testing.assert_close(eye, torch.eye(r, dtype=torch.float64, device="cuda"), atol=1e-4, rtol=0)
    runtime.submit_task("p", grad, resid, M, P, Q, runtime.POWERSGD_DECODE)
    runtime.wait_for(runtime.DECOMP_TASK, ["p"])
    approx = (P @ Q.T).view(-1)
    torch.testing.assert_close(grad, approx, atol=1e-3, rtol=1e-3)
    torch.testing.assert_close(resid, g0 - approx, atol=1e-3, rtol=1e-3)
    assert runtime.getErrors() == []
