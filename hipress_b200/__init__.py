"""hipress_b200: compressed gradient synchronisation for data-parallel PyTorch on B200.

Layers (top to bottom):

* ``hipress_b200.parallel``  data-parallel wrapper, bucketing, symmetric memory, compressors
* ``hipress_b200.hp_cuda``   the reference extension's module API (init / submit_task / getResults / end)
* ``hipress_b200.ops``       per-algorithm compress / decompress ops on tensors
* ``hipress_b200._C``        native extension: sm_100a kernels, CPU codecs, C++ runtime
* ``hipress_b200.models``    ResNet-50, VGG-19, BERT-large used by the benchmarks
* ``hipress_b200.utils``     synthetic data, timing, clocks sampling, metrics

The native extension is built in-tree by ``python -m hipress_b200.build`` and is
required: nothing here falls back to eager PyTorch when it is missing.
"""
from __future__ import annotations

import importlib
import os

__version__ = "0.1.0"


def _load_native():
    try:
        return importlib.import_module("hipress_b200._C")
    except ImportError as first:
        if os.environ.get("HIPRESS_NO_AUTOBUILD"):
            raise ImportError(
                "hipress_b200._C is not built; run `python -m hipress_b200.build`") from first
        from . import build as _build
        _build.build()
        return importlib.import_module("hipress_b200._C")


import torch  # noqa: E402  (must be imported before the extension: it links against libtorch)

if os.environ.get("HIPRESS_SKIP_NATIVE"):
    # only the pure-Python helpers (hipress_b200.utils) are wanted, e.g. by the benchmark's
    # reference arm, which must not load this framework's kernels
    _C = None
else:
    _C = _load_native()
    from . import ops  # noqa: E402,F401
    from . import hp_cuda  # noqa: E402,F401

__all__ = ["_C", "ops", "hp_cuda", "__version__"]
