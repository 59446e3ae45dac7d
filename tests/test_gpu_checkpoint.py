"""Checkpoint / resume of the synchronisers: train k steps, save, rebuild the wrapper from
scratch, load, and require the following steps to match an uninterrupted run bit for bit.

What has to survive: residuals, momentum / moments, DGC's velocity and its position in the
sparsity warm-up, PowerSGD's warm-start factors, and the step / epoch counters that seed the
stochastic rounding and drive AdamW's bias correction.  (The reference keeps all of this state
in caller-owned tensors, ref hp_cuda.h:28-50, and has no counters to restore.)
"""
import copy

import pytest
import torch
import torch.nn as nn

from hipress_b200.parallel import CompressedDataParallel, CompressionConfig
from hipress_b200.parallel.dgc import DGCDataParallel
from hipress_b200.parallel.powersgd import PowerSGDDataParallel

pytestmark = pytest.mark.gpu


def make_net(seed=0):
    torch.manual_seed(seed)
    return nn.Sequential(nn.Linear(96, 256), nn.ReLU(), nn.Linear(256, 128), nn.ReLU(), nn.Linear(128, 10)).cuda()


def batches(count, seed=1):
    g = torch.Generator().manual_seed(seed)
    return [(torch.randn(32, 96, generator=g).cuda(), torch.randint(0, 10, (32,), generator=g).cuda())
            for _ in range(count)]


def run_steps(model, data):
    for x, y in data:
        loss = nn.functional.cross_entropy(model(x), y)
        loss.backward()
        model.step()
    torch.cuda.synchronize()


def params_of(model):
    return [p.detach().clone() for p in model.module.parameters()]


BUILDERS = {
    "terngrad_stochastic": lambda net: CompressedDataParallel(
        net, CompressionConfig("terngrad", bitwidth=2, enable_random=True, error_feedback=True, bucket_mb=0.05, seed=7),
        lr=0.05, momentum=0.9),
    "terngrad_device_epoch": lambda net: CompressedDataParallel(
        net, CompressionConfig("terngrad", bitwidth=2, enable_random=True, bucket_mb=0.05, seed=7, graph_capturable=True),
        lr=0.05, momentum=0.9),
    "tbq_sharded": lambda net: CompressedDataParallel(
        net, CompressionConfig("tbq", threshold=1e-3, bucket_mb=0.05, sharded=True, num_workers=0), lr=0.05, momentum=0.9),
    "dgc_mid_warmup_adamw": lambda net: DGCDataParallel(
        net, keep_fraction=0.01, sample_rate=0.1, warmup_steps=8, lr=1e-3, bucket_mb=0.05),
    "powersgd_warm_start": lambda net: PowerSGDDataParallel(net, rank_r=2, lr=0.05, momentum=0.9),
}


@pytest.mark.parametrize("name", list(BUILDERS))
def test_resume_matches_uninterrupted_run(name):
    data = batches(6)
    build = BUILDERS[name]
    # uninterrupted: 6 steps
    ref = build(make_net())
    run_steps(ref, data[:3])
    saved_params = copy.deepcopy(params_of(ref))
    saved_state = {k: (v.clone() if torch.is_tensor(v) else copy.deepcopy(v)) for k, v in ref.compression_state().items()}
    run_steps(ref, data[3:])
    want = params_of(ref)
    ref.check()
    # resumed: a fresh wrapper around a fresh network, parameters and state loaded, 3 more steps
    net = make_net(seed=123)           # different weights: they must come from the checkpoint
    resumed = build(net)
    with torch.no_grad():
        for p, s in zip(resumed.module.parameters(), saved_params):
            p.copy_(s)
    resumed.load_compression_state(saved_state)
    run_steps(resumed, data[3:])
    resumed.check()
    got = params_of(resumed)
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    # and the carried state agrees too
    s1, s2 = ref.compression_state(), resumed.compression_state()
    assert set(s1) == set(s2)
    for k in s1:
        if torch.is_tensor(s1[k]):
            assert torch.equal(s1[k], s2[k]), k
        else:
            for a, b in zip(s1[k], s2[k]):
                assert torch.equal(a, b), k
    ref.close()
    resumed.close()
