"""Per-algorithm compress / decompress ops on tensors.

Every function accepts CUDA tensors (sm_100a kernels on the current stream, no
host synchronisation) or CPU tensors (the bit-exact CPU codec).  The packed
payload layouts are the reference's (ZQ_CPP_LIB/gradient_compression_body/*.h):

=========  ============================================================
TBQ        ``ceil(N/4)`` bytes, 2-bit fields {0: -t, 1: 0, 2: +t}
TernGrad   10-byte header {u8 bits, u8 tail, f32 min, f32 max} + packed k-bit levels
GradDrop   {i32 total = 4 + 8k}{k x i32 index}{k x f32 value}
DGC        same layout, no residual accumulation inside the codec
ECQ        {i32 total, f32 max, u8 bits, u8 unused} + packed levels
PowerSGD   dense fp32 factors P (n x r) and Q (m x r)
=========  ============================================================

The batched ``hp_cuda_*`` functions at the bottom mirror the reference's nine
C++ entrypoints (ref hp_cuda.cpp:18-102): they take lists, like the originals
take vectors.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .. import _C

__all__ = [
    "tbq_payload_bytes", "terngrad_payload_bytes", "sparse_payload_bytes", "ecq_payload_bytes",
    "tbq_compress", "tbq_decompress", "terngrad_compress", "terngrad_decompress",
    "graddrop_compress", "dgc_compress", "sparse_decompress", "sparse_payload_k",
    "ecq_compress", "ecq_decompress",
    "powersgd_encode1", "powersgd_encode2", "powersgd_decode",
    "psgd_project", "psgd_project_grouped", "gram_schmidt", "psgd_expand_feedback", "read_status",
    "hp_cuda_tbq", "hp_cuda_tbqr", "hp_cuda_terngrad", "hp_cuda_terngradr", "hp_cuda_gd",
    "hp_cuda_gdr", "hp_cuda_powersgd_encode1", "hp_cuda_powersgd_encode2", "hp_cuda_powersgd_decode",
    "set_cpu_threads", "get_cpu_threads",
]

tbq_payload_bytes = _C.tbq_payload_bytes


def set_cpu_threads(threads: int) -> None:
    """Threads the TBQ / TernGrad codecs may use on CPU tensors (default 1).  Payloads, residuals and decodes
    are bit-identical for every setting: each payload byte depends on its own elements only and stochastic
    rounding is seeded per byte.  (The reference's host path is single-threaded.)"""
    _C.set_cpu_threads(int(threads))


def get_cpu_threads() -> int:
    return int(_C.get_cpu_threads())


terngrad_payload_bytes = _C.terngrad_payload_bytes
sparse_payload_bytes = _C.sparse_payload_bytes
ecq_payload_bytes = _C.ecq_payload_bytes
read_status = _C.read_status


def _as_list(payloads) -> list:
    return [payloads] if isinstance(payloads, torch.Tensor) else list(payloads)


def _u8(n: int, like: torch.Tensor) -> torch.Tensor:
    return torch.empty(int(n), dtype=torch.uint8, device=like.device)


# ----------------------------------------------------------------------------- TBQ
def tbq_compress(grad: torch.Tensor, residual: torch.Tensor, threshold: float,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Threshold quantisation with residual feedback (ref tbq_body.h:90-158).

    ``residual += grad``; elements at or beyond ``+-threshold`` emit ``+-threshold`` and keep
    the remainder.  ``grad`` is not modified.  Returns the ``ceil(N/4)``-byte payload.
    """
    g = grad.reshape(-1)
    if out is None:
        out = _u8(tbq_payload_bytes(g.numel()), g)
    _C.tbq_compress(g, residual.reshape(-1), out, float(threshold))
    return out


def tbq_decompress(payloads, out: torch.Tensor, threshold: float, add: bool = False,
                   post_scale: float = 1.0) -> torch.Tensor:
    """Decode one payload, or the payloads of all ranks in one pass (ascending list order).

    ``add=False`` overwrites ``out`` with the sum of the decoded payloads, ``add=True``
    accumulates onto it (ref tbq_body.h:160-200, one launch per payload there).
    """
    _C.tbq_decompress(_as_list(payloads), out.view(-1), float(threshold), bool(add), float(post_scale))
    return out


# ----------------------------------------------------------------------------- TernGrad
def terngrad_compress(grad: torch.Tensor, bitwidth: int = 2, enable_random: bool = True,
                      seed: int = 0, residual: Optional[torch.Tensor] = None,
                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Min-max linear ``bitwidth``-bit quantiser (ref terngrad_body.h:162-307).

    ``seed`` replaces the reference's wall-clock seed: data byte ``i`` is rounded by an LCG
    seeded with ``uint32(seed + i)``.  With ``residual`` the quantised tensor is
    ``grad + residual`` and the quantisation error is written back (error feedback).
    """
    g = grad.reshape(-1)
    if out is None:
        out = _u8(terngrad_payload_bytes(g.numel(), bitwidth), g)
    _C.terngrad_compress(g, out, int(bitwidth), bool(enable_random), int(seed),
                         None if residual is None else residual.reshape(-1))
    return out


def terngrad_decompress(payloads, out: torch.Tensor, add: bool = False,
                        post_scale: float = 1.0, bitwidth: int = 0) -> torch.Tensor:
    """Decode payload(s); each carries its own header (ref terngrad_body.h:309-409).

    ``bitwidth`` (optional) names the bitwidth all payloads are known to have, which selects a
    kernel compiled for it; 0 reads it from the headers on the device."""
    _C.terngrad_decompress(_as_list(payloads), out.view(-1), bool(add), float(post_scale), int(bitwidth))
    return out


# ----------------------------------------------------------------------------- sparse
def graddrop_compress(grad: torch.Tensor, residual: torch.Tensor, sample_rate: float,
                      drop_ratio: float, seed: int = 0,
                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """GradDrop (ref gd_body.h:102-232): ``residual += grad``; keep the entries whose magnitude
    exceeds a threshold estimated from a random sample; selected residual entries are zeroed.
    The returned buffer has the worst-case size; the first int32 holds the bytes in use."""
    g = grad.reshape(-1)
    keep = 1.0 - float(drop_ratio)
    if out is None:
        out = _u8(sparse_payload_bytes(g.numel(), keep), g)
    _C.sparse_compress(g, residual.reshape(-1), out, float(sample_rate), keep, int(seed), True)
    return out


def dgc_compress(values: torch.Tensor, sample_rate: float, keep_fraction: float, seed: int = 0,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """DGC selector (ref dgc_body.h:154-229): like GradDrop but selects from ``values`` itself
    (the caller owns momentum / accumulation); selected entries of ``values`` are zeroed."""
    v = values.reshape(-1)
    if out is None:
        out = _u8(sparse_payload_bytes(v.numel(), keep_fraction), v)
    _C.sparse_compress(None, v, out, float(sample_rate), float(keep_fraction), int(seed), False)
    return out


def dgc_momentum_compress(grad: torch.Tensor, u: torch.Tensor, v: torch.Tensor, sample_rate: float,
                          keep_fraction: float, seed: int = 0, momentum: float = 0.9, clip: float = 0.0,
                          zero_grad: bool = False, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """DGC with momentum correction as one fused pipeline (CUDA tensors): ``u = momentum*u + s*grad``,
    ``v += u``, sampled-threshold top-k of ``v`` into the payload, ``u`` and ``v`` cleared at the
    sent positions (momentum factor masking).  ``s = min(1, clip / |grad|)`` when ``clip > 0``.
    For keep fractions up to 1 % the three tensors are read once.  (Momentum correction, clipping
    and masking are not in the reference, whose dgc_body.h is the selector alone.)"""
    if out is None:
        out = _u8(sparse_payload_bytes(v.numel(), keep_fraction), v)
    _C.dgc_momentum_compress(grad.reshape(-1), u.reshape(-1), v.reshape(-1), out, float(sample_rate),
                             float(keep_fraction), int(seed), float(momentum), float(clip), bool(zero_grad))
    return out


def sparse_decompress(payloads, out: torch.Tensor, add: bool = False,
                      post_scale: float = 1.0) -> torch.Tensor:
    """Scatter payload(s) into ``out`` (ref gd_body.h:283-353); ``add=False`` zero-fills first."""
    _C.sparse_decompress(_as_list(payloads), out.view(-1), bool(add), float(post_scale))
    return out


def sparse_payload_k(payload: torch.Tensor) -> int:
    """Number of (index, value) pairs in a sparse payload (reads the header; synchronises)."""
    total = int(payload[:4].cpu().view(torch.int32).item())
    return (total - 4) // 8


# ----------------------------------------------------------------------------- ECQ
def ecq_compress(grad: torch.Tensor, history: torch.Tensor, alpha: float, beta: float,
                 bitwidth: int = 2, seed: int = 0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Error-compensated quantisation (layout of ref ecq_body.h:266-276, corrected semantics):
    ``v = grad + alpha*history`` is stochastically rounded on a symmetric grid of step
    ``max|v| / (2^(bits-1) - 1)``; ``history = beta*history + (v - decoded)``."""
    g = grad.reshape(-1)
    if out is None:
        out = _u8(ecq_payload_bytes(g.numel(), bitwidth), g)
    _C.ecq_compress(g, history.reshape(-1), out, float(alpha), float(beta), int(bitwidth), int(seed))
    return out


def ecq_decompress(payloads, out: torch.Tensor, add: bool = False, post_scale: float = 1.0) -> torch.Tensor:
    _C.ecq_decompress(_as_list(payloads), out.view(-1), bool(add), float(post_scale))
    return out


# ----------------------------------------------------------------------------- PowerSGD
def powersgd_encode1(grad, residual, Q, M, P):
    """``M[:N] = grad + residual; P = M Q`` (ref powersgd_body.h:10-31, intended maths)."""
    _C.powersgd_encode1(grad.reshape(-1), residual.reshape(-1), Q, M, P)


def powersgd_encode2(P, M, Q):
    """``P = orthonormalise(P); Q = M^T P`` (ref powersgd_body.h:33-52)."""
    _C.powersgd_encode2(P, M, Q)


def powersgd_decode(P, Q, M, residual, grad):
    """``M = P Q^T; residual = grad - M[:N]; grad = M[:N]`` (ref powersgd_body.h:54-78)."""
    _C.powersgd_decode(P, Q, M, residual.view(-1), grad.view(-1))


def psgd_project_grouped(mode: int, Ms: Sequence[torch.Tensor], Xs: Sequence[torch.Tensor],
                         outs: Sequence[torch.Tensor]) -> None:
    """outs[i] += Ms[i] @ Xs[i] (mode 0) or Ms[i].T @ Xs[i] (mode 1) for a list of CUDA matrices of one rank:
    every tensor-core-eligible matrix of the list is projected by the same grid (what the PowerSGD step
    driver launches per phase).  Reference: one `mm` per matrix, powersgd_body.h:28, 49."""
    _C.psgd_project_grouped(int(mode), list(Ms), list(Xs), list(outs))


def psgd_project(mode: int, M: torch.Tensor, X: torch.Tensor, owners: Sequence[torch.Tensor],
                 simt: bool = False) -> None:
    """Accumulate ``M @ X`` (mode 0) or ``M.T @ X`` (mode 1) into the owners' buffers."""
    _C.psgd_project(int(mode), M, X, list(owners), bool(simt))


def gram_schmidt(P: torch.Tensor, eps: float = 1e-8) -> torch.Tensor:
    _C.gram_schmidt(P, float(eps))
    return P


def psgd_expand_feedback(P, Q, M, grad_out, post_scale: float = 1.0) -> None:
    _C.psgd_expand_feedback(P, Q, M, grad_out.view(-1), float(post_scale))


# ----------------------------------------------------------------------------- batched entrypoints
def hp_cuda_tbq(to_compress, residuals, outs, thresholds) -> None:
    """ref hp_cuda_kernel.cu:120-158"""
    for g, r, o, t in zip(to_compress, residuals, outs, thresholds):
        tbq_compress(g, r, t, out=o)


def hp_cuda_tbqr(outs, ins, thresholds, is_add_tos) -> None:
    """ref hp_cuda_kernel.cu:161-198"""
    for o, p, t, a in zip(outs, ins, thresholds, is_add_tos):
        tbq_decompress(p, o, t, add=bool(a))


def hp_cuda_terngrad(ins, outs, bitwidths, enable_randoms, seeds=None) -> None:
    """ref hp_cuda_kernel.cu:30-65"""
    seeds = seeds if seeds is not None else range(len(ins))
    for g, o, b, r, s in zip(ins, outs, bitwidths, enable_randoms, seeds):
        terngrad_compress(g, b, bool(r), s, out=o)


def hp_cuda_terngradr(outs, ins, is_add_tos) -> None:
    """ref hp_cuda_kernel.cu:200-230"""
    for o, p, a in zip(outs, ins, is_add_tos):
        terngrad_decompress(p, o, add=bool(a))


def hp_cuda_gd(ins, residuals, outs, sample_rates, drop_ratios, seeds=None) -> None:
    """ref hp_cuda_kernel.cu:67-94"""
    seeds = seeds if seeds is not None else range(len(ins))
    for g, r, o, sr, dr, s in zip(ins, residuals, outs, sample_rates, drop_ratios, seeds):
        graddrop_compress(g, r, sr, dr, s, out=o)


def hp_cuda_gdr(ins, outs, is_add_tos) -> None:
    """ref hp_cuda_kernel.cu:96-118"""
    for p, o, a in zip(ins, outs, is_add_tos):
        sparse_decompress(p, o, add=bool(a))


def hp_cuda_powersgd_encode1(grads, residuals, Qs, Ms, Ps) -> None:
    """ref hp_cuda_kernel.cu:232-255"""
    for g, r, q, m, p in zip(grads, residuals, Qs, Ms, Ps):
        powersgd_encode1(g, r, q, m, p)


def hp_cuda_powersgd_encode2(Ps, Ms, Qs) -> None:
    """ref hp_cuda_kernel.cu:257-276"""
    for p, m, q in zip(Ps, Ms, Qs):
        powersgd_encode2(p, m, q)


def hp_cuda_powersgd_decode(Ps, Qs, Ms, residuals, grads) -> None:
    """ref hp_cuda_kernel.cu:278-301"""
    for p, q, m, r, g in zip(Ps, Qs, Ms, residuals, grads):
        powersgd_decode(p, q, m, r, g)
