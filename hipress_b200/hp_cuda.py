"""Drop-in module with the reference extension's Python API.

The reference builds a pybind module ``hp_cuda`` with six definitions
(ref hp_cuda.cpp:1073-1080)::

    init(alg_name, alg_paras, device_id, rank_id, size) -> bool
    end() -> bool
    getResults(task_id) -> list[str]
    submit_task(name, tensor, B, C, is_root, task_id)                 # terngrad
    submit_task(name, tensor, residual, B, C, is_root, task_id)      # tbq, graddrop
    submit_task(name, tensor, residual, M, P, Q, task_id)            # powersgd

``import hipress_b200.hp_cuda as hp_cuda`` gives the same names with the same
semantics, served by this framework's runtime and kernels.  Differences a
caller can observe: ``alg_paras`` may carry ``seed`` (base seed of stochastic
rounding / sampling; the reference seeds from the clock) and ``num_threads``;
``getErrors()`` returns the messages of failed tasks; ``C`` may be a CUDA tensor
as well as a CPU tensor; all tensors may be CPU tensors, in which case the CPU
codec runs.
"""
from __future__ import annotations

import time
from typing import Dict, List

from . import _C

COMP_TASK = _C.COMP_TASK                          # 10
DECOMP_TASK = _C.DECOMP_TASK                      # 20
ROOT_DECOMP_COMP_TASK = _C.ROOT_DECOMP_COMP_TASK  # 30
POWERSGD_ENCODE1 = _C.POWERSGD_ENCODE1            # 40
POWERSGD_ENCODE2 = _C.POWERSGD_ENCODE2            # 50
POWERSGD_DECODE = _C.POWERSGD_DECODE              # 60

init = _C.init
end = _C.end
getResults = _C.getResults
getErrors = _C.getErrors
submit_task = _C.submit_task
numThreads = _C.numThreads


def wait_for(task_id: int, names, timeout_s: float = 60.0) -> List[str]:
    """Poll ``getResults(task_id)`` until every name in ``names`` has been reported.

    Convenience for callers of the polling API; raises on timeout or on a failed task.
    """
    pending = set(names)
    done: List[str] = []
    deadline = time.monotonic() + timeout_s
    while pending:
        for key in getResults(task_id):
            done.append(key)
            pending.discard(key)
        if not pending:
            break
        errors = getErrors()
        if errors:
            raise RuntimeError("hipress task failed: " + "; ".join(errors))
        if time.monotonic() > deadline:
            raise TimeoutError(f"tasks not finished after {timeout_s}s: {sorted(pending)}")
        time.sleep(0.0002)
    return done


def algorithm_parameters(alg_name: str) -> Dict[str, float]:
    """Parameter keys each algorithm reads (ref hp_cuda.cpp:836-850), with neutral defaults."""
    return {
        "terngrad": {"enable_random": 0.0, "bitwidth": 2.0},
        "tbq": {"threshold": 0.0},
        "graddrop": {"drop_ratio": 0.999, "sample_rate": 0.01},
        "powersgd": {"matrix_approximation_rank": 4.0},
    }[alg_name]
