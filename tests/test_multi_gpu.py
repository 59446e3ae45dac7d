"""Multi-GPU tests: launched as one process per GPU with torch.distributed.run on 127.0.0.1."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run_workers(nproc: int, port: int):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "mp_worker.py")]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT)


@pytest.mark.parametrize("nproc", [2, 4, 8])
def test_engine_and_wrappers_across_gpus(nproc):
    if torch.cuda.device_count() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    res = _run_workers(nproc, 29540 + nproc)
    print("\n".join(l for l in res.stdout.splitlines() if l.startswith(("MP_", "NVLS"))))   # shown with -s / -rP
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    for name in ("codec_terngrad", "codec_tbq", "codec_graddrop", "codec_ecq", "codec_dense",
                 "codec_terngrad_device_epoch", "codec_tbq_device_epoch", "codec_terngrad_wide", "codec_tbq_wide",
                 "codec_ecq_device_epoch", "sharded_terngrad", "sharded_tbq", "sharded_terngrad_device_epoch",
                 "sharded_tbq_device_epoch", "ddp_terngrad", "ddp_graphed", "ddp_graphed_sharded", "ddp_graphed_dgc",
                 "ddp_powersgd", "ddp_graphed_powersgd"):
        assert f"MP_OK {name}" in res.stdout, res.stdout[-2000:]
