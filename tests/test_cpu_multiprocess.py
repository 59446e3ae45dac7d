"""Multi-process host-side logic on CPU ranks (gloo, world size 3, rendezvous on 127.0.0.1).

* the reference's parameter-server pattern through the module API: every rank compresses
  (task 10), payloads are gathered, the root decodes all peers and recompresses (task 30),
  the result is broadcast and decoded (task 20);
* failure detection without any GPU: a rank leaves between steps; the others learn it from
  the heartbeat store before they would launch the next step.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _gauss(n, seed):
    return torch.randn(n, generator=torch.Generator().manual_seed(seed)) * 0.02


def _ps_worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from hipress_b200 import hp_cuda, ops
    n, t, root = 5003, 0.01, 0
    hp_cuda.init("tbq", {"threshold": t}, 0, rank, world)
    size = ops.tbq_payload_bytes(n)
    grad = _gauss(n, 100 + rank)
    resid = torch.zeros(n)
    B, C = torch.zeros(size, dtype=torch.uint8), torch.zeros(size, dtype=torch.uint8)
    expect_payload = ops.tbq_compress(grad, torch.zeros(n), t)
    if rank != root:
        hp_cuda.submit_task("w", grad, resid, B, C, 0, hp_cuda.COMP_TASK)
        hp_cuda.wait_for(hp_cuda.COMP_TASK, ["w"])
        assert torch.equal(C, expect_payload)
    gathered = [torch.zeros(size, dtype=torch.uint8) for _ in range(world)]
    dist.all_gather(gathered, C)
    out = torch.zeros(size, dtype=torch.uint8)
    if rank == root:
        Call = torch.cat(gathered)
        hp_cuda.submit_task("w", grad, resid, B, Call, 1, hp_cuda.ROOT_DECOMP_COMP_TASK)
        hp_cuda.wait_for(hp_cuda.ROOT_DECOMP_COMP_TASK, ["w"])
        out.copy_(Call[:size])
    dist.broadcast(out, src=root)
    final = torch.zeros(n)
    hp_cuda.submit_task("w", final, torch.zeros(n), torch.zeros(size, dtype=torch.uint8), out, 0, hp_cuda.DECOMP_TASK)
    hp_cuda.wait_for(hp_cuda.DECOMP_TASK, ["w"])
    hp_cuda.end()
    # independent restatement
    acc = _gauss(n, 100 + root)
    for r in range(world):
        if r != root:
            ops.tbq_decompress(ops.tbq_compress(_gauss(n, 100 + r), torch.zeros(n), t), acc, t, add=True)
    ref = torch.zeros(n)
    ops.tbq_decompress(ops.tbq_compress(acc, torch.zeros(n), t), ref, t)
    results[rank] = bool(torch.equal(final, ref))
    dist.barrier()
    dist.destroy_process_group()


def _heartbeat_worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import time
    from hipress_b200.utils.health import Heartbeat
    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world)
    t = torch.ones(4)
    # step 0: everyone participates
    dist.all_reduce(t)
    hb.beat(0)
    assert hb.missing(0, timeout_s=10.0) == []
    store.set(f"checked0/{rank}", "1")
    if rank == world - 1:
        # leave only after everyone has seen step 0 complete
        store.wait([f"checked0/{r}" for r in range(world)])
        hb.leave()                      # orderly exit between steps; no collective in flight
        results[rank] = "left"
    else:
        # before launching step 1 the survivors check that everyone finished step 0 and is still there
        deadline = time.monotonic() + 10.0
        gone = []
        while not gone and time.monotonic() < deadline:
            gone = hb.missing(0, timeout_s=0.2)
        results[rank] = gone            # they must NOT call the collective now
        hb.beat(1)
    # rank 0 hosts the store: it stays until everybody else is done with it; nobody touches the
    # store after announcing "done", and processes leave without tearing the group down
    store.set(f"done/{rank}", "1")
    if rank == 0:
        store.wait([f"done/{r}" for r in range(world)])
        time.sleep(0.2)
    os._exit(0)


@pytest.mark.parametrize("worker", ["ps", "heartbeat"])
def test_cpu_ranks(worker):
    world = 3
    port = _free_port()
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        results = mgr.dict()
        fn = _ps_worker if worker == "ps" else _heartbeat_worker
        procs = [ctx.Process(target=fn, args=(r, world, port, results)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=120)
        for p in procs:
            if p.is_alive():           # never leave a stuck rank behind
                p.kill()
                p.join()
        assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
        res = dict(results)
    if worker == "ps":
        assert res == {0: True, 1: True, 2: True}
    else:
        assert res[2] == "left" and res[0] == [2] and res[1] == [2]
