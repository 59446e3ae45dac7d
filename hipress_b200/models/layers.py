"""Layers of the model zoo that run on this framework's own kernels.

``MaxPool3x3s2`` is the ResNet stem's pooling layer on a gather-style kernel pair.
``FusedBiasReLU`` is the epilogue of VGG's convolutions: bias + ReLU (+ 2x2 max pooling).
``FusedAddLayerNorm`` is BERT's residual add + LayerNorm on a bf16 residual stream.
``FusedLinear`` is ``nn.Linear`` whose backward yields fp32 weight gradients from the GEMM and the
bias gradient from a two-stage column sum.

``FusedBatchNormAct`` is ``nn.BatchNorm2d`` (same parameters, buffers and state-dict keys)
whose training-mode forward and backward on channels-last bf16 CUDA activations run on the
hand-written streaming kernels of ``csrc/kernels/bn.cu``, with the ReLU and the residual add
of a ResNet block folded in:

    y = relu(batch_norm(x) [+ residual])

Profiling the ResNet-50 benchmark step showed the stock channels-last batch-norm kernels at
54 % of the device time; these kernels do the same maths in two passes forward and two
backward, each close to one read/write of the activations at HBM speed.  Anything the kernels
do not cover (CPU tensors, fp32 activations, NCHW layout, eval mode, odd channel counts) takes
the stock PyTorch path with identical semantics.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import _C


class _FusedBnFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, weight, bias, running_mean, running_var, num_batches,
                momentum: float, eps: float, relu: bool):
        y, stats = _C.bn_forward(x, residual, weight, bias, running_mean, running_var, num_batches,
                                 momentum, eps, relu)
        ctx.save_for_backward(x, y if relu else None, weight, stats)
        ctx.relu = relu
        ctx.has_residual = residual is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, y, weight, stats = ctx.saved_tensors
        dy = dy.contiguous(memory_format=torch.channels_last)
        out = _C.bn_backward(dy, x, y, weight, stats, ctx.relu, ctx.has_residual)
        dres = out[3] if ctx.has_residual else None
        return out[0], dres, out[1], out[2], None, None, None, None, None, None


class FusedBatchNormAct(nn.BatchNorm2d):
    """Batch norm, optional residual add, optional ReLU: ``forward(x, residual=None)``."""

    def __init__(self, num_features: int, relu: bool = False, eps: float = 1e-5, momentum: float = 0.1):
        super().__init__(num_features, eps=eps, momentum=momentum, affine=True, track_running_stats=True)
        self.relu = relu

    def _fused_ok(self, x: torch.Tensor, residual: Optional[torch.Tensor]) -> bool:
        if _C is None or not (self.training and x.is_cuda and x.dtype == torch.bfloat16 and self.momentum is not None):
            return False
        if residual is not None and (residual.dtype != x.dtype or residual.shape != x.shape or
                                     not residual.is_contiguous(memory_format=torch.channels_last)):
            return False
        return _C.bn_supported(x)

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self._fused_ok(x, residual):
            return _FusedBnFunction.apply(x, residual, self.weight, self.bias, self.running_mean,
                                          self.running_var, self.num_batches_tracked,
                                          float(self.momentum), float(self.eps), self.relu)
        y = super().forward(x)
        if residual is not None:
            y = y + residual
        return F.relu(y) if self.relu else y

    def extra_repr(self) -> str:
        return super().extra_repr() + f", relu={self.relu}"


class _MaxPoolFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        y, idx = _C.maxpool3x3s2_forward(x)
        ctx.save_for_backward(idx)
        ctx.hw = (x.shape[2], x.shape[3])
        return y

    @staticmethod
    def backward(ctx, dy):
        (idx,) = ctx.saved_tensors
        return _C.maxpool3x3s2_backward(dy.contiguous(memory_format=torch.channels_last), idx, *ctx.hw)


class MaxPool3x3s2(nn.Module):
    """``nn.MaxPool2d(3, stride=2, padding=1)``; channels-last bf16 CUDA activations run on
    ``csrc/kernels/pool.cu`` (one index byte per output, gather backward without atomics)."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if _C is not None and x.is_cuda and _C.maxpool_supported(x):
            return _MaxPoolFunction.apply(x)
        return F.max_pool2d(x, 3, stride=2, padding=1)


class _BiasReluFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias, pool: bool):
        out = _C.bias_relu_forward(x, bias, pool)
        ctx.save_for_backward(out[0], out[1] if pool else None)
        ctx.pool = pool
        return out[0]

    @staticmethod
    def backward(ctx, dy):
        y, idx = ctx.saved_tensors
        dz, db = _C.bias_relu_backward(dy.contiguous(memory_format=torch.channels_last), y, idx, ctx.pool)
        return dz, db, None


class FusedBiasReLU(nn.Module):
    """Epilogue of a bias-free convolution: ``relu(x + bias)`` and, with ``pool=True``, the
    2x2 / stride 2 max pooling that follows it, in one pass on ``csrc/kernels/bias_act.cu``
    (pooling commutes with the monotonic bias + ReLU, so the full-size activation is never
    written).  Owns the bias the convolution would have had."""

    def __init__(self, num_features: int, pool: bool = False):
        super().__init__()
        self.bias = nn.Parameter(torch.zeros(num_features))
        self.pool = pool

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if _C is not None and x.is_cuda and _C.bias_relu_supported(x, self.pool):
            return _BiasReluFunction.apply(x, self.bias, self.pool)
        y = F.relu(x + self.bias.view(1, -1, 1, 1).to(x.dtype))
        return F.max_pool2d(y, 2, 2) if self.pool else y

    def extra_repr(self) -> str:
        return f"{self.bias.numel()}, pool={self.pool}"


class _AddLayerNormFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, delta, weight, bias, eps: float):
        y, z, stats = _C.add_ln_forward(x, delta, weight, bias, eps)
        ctx.save_for_backward(z, stats, weight)
        ctx.has_delta = delta is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        z, stats, weight = ctx.saved_tensors
        dz, dw, db = _C.add_ln_backward(dy.contiguous(), z, stats, weight)
        return dz, (dz if ctx.has_delta else None), dw, db, None


class FusedAddLayerNorm(nn.LayerNorm):
    """``LayerNorm(x + delta)`` (``delta`` optional) with ``nn.LayerNorm``'s parameters.  bf16 CUDA
    inputs run on ``csrc/kernels/layernorm.cu`` and keep the residual stream in bf16 (autocast
    would run the stock LayerNorm, the add before it and everything between them in fp32);
    anything else takes the stock path."""

    def forward(self, x: torch.Tensor, delta: Optional[torch.Tensor] = None) -> torch.Tensor:
        if (_C is not None and x.is_cuda and x.dtype == torch.bfloat16 and self.elementwise_affine
                and (delta is None or (delta.dtype == x.dtype and delta.shape == x.shape))):
            xc = x.contiguous()
            if _C.add_ln_supported(xc):
                return _AddLayerNormFunction.apply(xc, None if delta is None else delta.contiguous(),
                                                   self.weight, self.bias, float(self.eps))
        return super().forward(x if delta is None else x + delta)


_MM_FP32_OUT = None   # whether torch.mm(bf16, bf16, out_dtype=float32) works here; probed on first use


def _mm_fp32(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a @ b with bf16 operands and an fp32 result written by the GEMM itself when the installed
    PyTorch exposes that (no separate conversion pass); otherwise bf16 GEMM + conversion."""
    global _MM_FP32_OUT
    if _MM_FP32_OUT is None:
        try:
            torch.mm(a[:1], b[:, :1], out_dtype=torch.float32)
            _MM_FP32_OUT = True
        except (TypeError, RuntimeError):
            _MM_FP32_OUT = False
    return torch.mm(a, b, out_dtype=torch.float32) if _MM_FP32_OUT else torch.mm(a, b).float()


class _LinearFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        w16 = weight.to(x.dtype)
        ctx.save_for_backward(x, w16)
        ctx.has_bias = bias is not None
        return F.linear(x, w16, None if bias is None else bias.to(x.dtype))

    @staticmethod
    def backward(ctx, dy):
        x, w16 = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        x2 = x.reshape(-1, x.shape[-1])
        dx = torch.mm(dy2, w16).view(x.shape) if ctx.needs_input_grad[0] else None
        if (ctx.has_bias and dy2.is_cuda and dy2.dtype == torch.bfloat16 and x2.dtype == torch.bfloat16
                and hasattr(_C, "linear_wgrad_bgrad")):
            # weight gradient (fp32) and bias gradient from ONE GEMM: the library's bias-gradient epilogue
            # reduces dy over the tokens while the GEMM reads it; an empty answer = no such algorithm here
            both = _C.linear_wgrad_bgrad(dy2.contiguous(), x2.contiguous())
            if both:
                return dx, both[0], both[1]
        dw = _mm_fp32(dy2.t(), x2)                      # fp32 straight from the GEMM: no bf16 -> fp32 pass
        db = None
        if ctx.has_bias:
            dyc = dy2.contiguous()
            db = _C.colsum(dyc) if _C.colsum_supported(dyc) else dyc.float().sum(0)
        return dx, dw, db


class FusedLinear(nn.Linear):
    """``nn.Linear`` for bf16 activations under autocast with fp32 master weights.  Same forward
    GEMM; in backward the weight gradient comes out of its GEMM in fp32 (autocast produces it in
    bf16 and converts it in a separate pass) and the bias gradient out of the same GEMM's epilogue
    (cuBLASLt BGRADB) where the library has one for the shape, else from a two-stage column sum on
    this framework's kernels instead of a generic strided reduction -- together a fifth of the
    device time of the BERT-large benchmark step before."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if (_C is not None and x.is_cuda and torch.is_autocast_enabled()
                and torch.get_autocast_dtype("cuda") == torch.bfloat16 and self.weight.dtype == torch.float32):
            with torch.autocast("cuda", enabled=False):
                return _LinearFunction.apply(x.to(torch.bfloat16), self.weight, self.bias)
        return super().forward(x)
