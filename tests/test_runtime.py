"""Task runtime with the reference's module API, exercised on CPU tensors."""
import struct

import pytest
import torch

from hipress_b200 import hp_cuda, ops


@pytest.fixture()
def runtime():
    yield hp_cuda
    hp_cuda.end()


def gauss(n, std=0.01, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(n, generator=g) * std


def test_init_rejects_unknown_algorithm(runtime):
    assert runtime.init("nope", {}, 0, 0, 1) is False


def test_thread_counts(runtime):
    assert runtime.init("tbq", {"threshold": 0.01}, 0, 0, 1)
    assert runtime.numThreads() == 1  # tbq is single-threaded in the reference too
    runtime.end()
    assert runtime.init("terngrad", {"enable_random": 0, "bitwidth": 2}, 0, 0, 1)
    assert runtime.numThreads() == 5


def test_submit_validation(runtime):
    runtime.init("terngrad", {"enable_random": 0, "bitwidth": 2}, 0, 0, 1)
    g = gauss(16)
    B = torch.zeros(14, dtype=torch.uint8)
    C = torch.zeros(14, dtype=torch.uint8)
    assert runtime.submit_task("x", g, B, C, 2, runtime.COMP_TASK) is False      # is_root not 0/1
    assert runtime.submit_task("x", g, B, C, 0, 40) is False                    # wrong id for overload
    assert runtime.getResults(999) == []


def test_submit_before_init_raises():
    hp_cuda.end()
    with pytest.raises(RuntimeError):
        hp_cuda.submit_task("x", gauss(4), torch.zeros(11, dtype=torch.uint8),
                            torch.zeros(11, dtype=torch.uint8), 0, hp_cuda.COMP_TASK)


def test_terngrad_comp_then_decomp(runtime):
    runtime.init("terngrad", {"enable_random": 0, "bitwidth": 2}, 0, 0, 1)
    names = [f"t{i}" for i in range(12)]
    grads = {k: gauss(1000 + i, seed=i) for i, k in enumerate(names)}
    Bs = {k: torch.zeros(ops.terngrad_payload_bytes(g.numel(), 2), dtype=torch.uint8) for k, g in grads.items()}
    Cs = {k: torch.zeros_like(b) for k, b in Bs.items()}
    for k in names:
        assert runtime.submit_task(k, grads[k], Bs[k], Cs[k], 0, runtime.COMP_TASK)
    done = runtime.wait_for(runtime.COMP_TASK, names)
    assert sorted(done) == sorted(names)
    for k in names:
        assert torch.equal(Cs[k], ops.terngrad_compress(grads[k], 2, False))
    outs = {k: torch.zeros_like(g) for k, g in grads.items()}
    for k in names:
        Bs[k].zero_()
        runtime.submit_task(k, outs[k], Bs[k], Cs[k], 0, runtime.DECOMP_TASK)
    runtime.wait_for(runtime.DECOMP_TASK, names)
    for k in names:
        ref = torch.empty_like(grads[k])
        ops.terngrad_decompress(Cs[k], ref)
        assert torch.equal(outs[k], ref)
    # results are drained by the poll
    assert runtime.getResults(runtime.COMP_TASK) == []


def test_tbq_root_task_gathers_and_recompresses(runtime):
    world, rank, n, t = 4, 1, 999, 0.01
    runtime.init("tbq", {"threshold": t}, 0, rank, world)
    size = ops.tbq_payload_bytes(n)
    payloads = [ops.tbq_compress(gauss(n, 0.02, seed=r), torch.zeros(n), t) for r in range(world)]
    C = torch.cat(payloads)
    own = gauss(n, 0.02, seed=50)
    tensor = own.clone()
    resid = torch.zeros(n)
    B = torch.zeros(size, dtype=torch.uint8)
    assert runtime.submit_task("w", tensor, resid, B, C, 1, runtime.ROOT_DECOMP_COMP_TASK)
    runtime.wait_for(runtime.ROOT_DECOMP_COMP_TASK, ["w"])
    # expected: own + decode of every peer but self in ascending rank order, then recompress
    acc = own.clone()
    for r in range(world):
        if r != rank:
            ops.tbq_decompress(payloads[r], acc, t, add=True)
    assert torch.equal(tensor, acc)
    r2 = torch.zeros(n)
    expect = ops.tbq_compress(acc, r2, t)
    assert torch.equal(B, expect)
    assert torch.equal(C[:size], expect)
    assert torch.equal(resid, r2)


def test_graddrop_tasks(runtime):
    n, drop = 20000, 0.99
    runtime.init("graddrop", {"drop_ratio": drop, "sample_rate": 0.05, "seed": 3}, 0, 0, 1)
    g = gauss(n, seed=1)
    resid = torch.zeros(n)
    cap = ops.sparse_payload_bytes(n, 1 - drop)
    B = torch.zeros(cap, dtype=torch.uint8)
    C = torch.zeros(cap, dtype=torch.uint8)
    runtime.submit_task("g", g, resid, B, C, 0, runtime.COMP_TASK)
    runtime.wait_for(runtime.COMP_TASK, ["g"])
    total = struct.unpack("<i", bytes(C[:4].tolist()))[0]
    assert 4 < total <= cap
    out = torch.zeros(n)
    runtime.submit_task("g", out, resid, torch.zeros_like(B), C, 0, runtime.DECOMP_TASK)
    runtime.wait_for(runtime.DECOMP_TASK, ["g"])
    torch.testing.assert_close(out + resid, g, atol=0, rtol=0)


def test_powersgd_tasks_and_queue_mapping(runtime):
    runtime.init("powersgd", {"matrix_approximation_rank": 2}, 0, 0, 1)
    n, m, r = 32, 48, 2
    torch.manual_seed(1)
    grad = torch.randn(n * m)
    resid = torch.zeros(n * m)
    M = torch.zeros(n, m)
    P = torch.zeros(n, r)
    Q = torch.randn(m, r)
    runtime.submit_task("p", grad, resid, M, P, Q, runtime.POWERSGD_ENCODE1)
    runtime.wait_for(runtime.POWERSGD_ENCODE1, ["p"])        # 40 shares the COMP queue
    torch.testing.assert_close(P, grad.view(n, m) @ Q, atol=1e-4, rtol=1e-4)
    runtime.submit_task("p", grad, resid, M, P, Q, runtime.POWERSGD_ENCODE2)
    runtime.wait_for(runtime.ROOT_DECOMP_COMP_TASK, ["p"])   # 50 shares the ROOT queue
    runtime.submit_task("p", grad, resid, M, P, Q, runtime.POWERSGD_DECODE)
    runtime.wait_for(runtime.DECOMP_TASK, ["p"])             # 60 shares the DECOMP queue
    approx = (P @ Q.T).view(-1)
    torch.testing.assert_close(grad, approx, atol=1e-4, rtol=1e-4)


def test_failed_task_is_reported_and_runtime_keeps_serving(runtime):
    runtime.init("terngrad", {"enable_random": 0, "bitwidth": 2}, 0, 0, 1)
    g = gauss(100)
    badB = torch.zeros(5, dtype=torch.uint8)  # wrong payload size -> the op raises in the worker
    runtime.submit_task("bad", g, badB, torch.zeros(5, dtype=torch.uint8), 0, runtime.COMP_TASK)
    with pytest.raises(RuntimeError):
        runtime.wait_for(runtime.COMP_TASK, ["bad"], timeout_s=10)
    B = torch.zeros(ops.terngrad_payload_bytes(100, 2), dtype=torch.uint8)
    runtime.submit_task("good", g, B, torch.zeros_like(B), 0, runtime.COMP_TASK)
    assert runtime.wait_for(runtime.COMP_TASK, ["good"]) == ["good"]


def test_reinit_after_end(runtime):
    for _ in range(3):
        assert runtime.init("tbq", {"threshold": 0.5}, 0, 0, 1)
        g = gauss(64, 1.0)
        r = torch.zeros(64)
        B = torch.zeros(16, dtype=torch.uint8)
        runtime.submit_task("a", g, r, B, torch.zeros_like(B), 0, runtime.COMP_TASK)
        runtime.wait_for(runtime.COMP_TASK, ["a"])
        assert runtime.end()
