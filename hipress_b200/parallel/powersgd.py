"""Data-parallel training with PowerSGD rank-r gradient compression.

Every parameter with two or more dimensions is treated as a matrix ``n x m``
(``n`` = first dimension).  Per step and matrix (Vogels et al., with warm start and
error feedback):

    M  = grad + residual            (free: ``p.grad`` *is* a view of M, so autograd
                                     accumulates the new gradient onto the residual)
    P  = mean_ranks(M Q)            tcgen05 GEMM whose epilogue adds each row block into the
                                     owning rank's buffer over NVLink (reduce-scatter), then a
                                     peer gather (all-gather)
    P  = orthonormalise(P)          hand-written Gram-Schmidt
    Q  = mean_ranks(M^T P)          same fused GEMM + reduce-scatter, MN-major operand
    M -= P Q^T ; param -= lr * (mu * buf + P Q^T)      one fused expand / feedback / SGD pass

1-D parameters (biases, norms) are averaged uncompressed through the engine's dense
peer-to-peer path.  The reference ships three PowerSGD stages whose results are
discarded and leaves warm start, the 1-D bypass and both all-reduces to its caller
(ref powersgd_body.h:10-78, hp_cuda.cpp:640-772).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import _C
from .ddp import ALIGN, _view_like
from .symmetric import SymmetricMemory


def _round_up(v: int, a: int) -> int:
    return (v + a - 1) // a * a


class PowerSGDDataParallel(nn.Module):
    def __init__(self, module: nn.Module, rank_r: int = 4, *, lr: float = 0.1, momentum: float = 0.9,
                 weight_decay: float = 0.0, seed: int = 0, process_group: Optional[dist.ProcessGroup] = None,
                 symmetric: Optional[SymmetricMemory] = None, rank: Optional[int] = None,
                 world: Optional[int] = None, flag_timeout_s: float = 20.0, emulated: bool = False,
                 graph_capturable: bool = False):
        super().__init__()
        if not 1 <= rank_r <= 16:
            raise ValueError("rank must be between 1 and 16")
        self.module = module
        self.r = rank_r
        self.group = process_group
        self.rank = rank if rank is not None else (dist.get_rank(process_group) if dist.is_initialized() else 0)
        self.world = world if world is not None else (dist.get_world_size(process_group) if dist.is_initialized() else 1)
        self.lr, self.momentum, self.weight_decay = lr, momentum, weight_decay
        self.timeout = flag_timeout_s
        # Whole-step CUDA graph capture (GraphedTrainStep): the flag value of a step lives in device
        # memory (advanced by a one-thread kernel), and because which of the two accumulator sets a
        # step uses depends on the epoch's parity, the step is captured twice, once per parity, and
        # the two graphs are replayed in turn (capture_variants).
        self.graph_capturable = bool(graph_capturable)
        self.capture_variants = 2 if self.graph_capturable else 1
        self._forced_parity: Optional[int] = None
        params = [p for p in module.parameters() if p.requires_grad]
        self.device = params[0].device
        self.mats = [p for p in params if p.dim() >= 2]
        self.vecs = [p for p in params if p.dim() < 2]
        dev = self.device

        # ---- matrices: flat M (gradient accumulator + error feedback), params, momentum
        self.shapes, self.offsets = [], []
        cursor = 0
        for p in self.mats:
            n = p.shape[0]
            m = p.numel() // n
            self.shapes.append((n, m))
            self.offsets.append(cursor)
            cursor += _round_up(p.numel(), ALIGN)
        self.flat_M = torch.zeros(max(cursor, ALIGN), device=dev)
        self.flat_param = torch.zeros_like(self.flat_M)
        self.flat_momentum = torch.zeros_like(self.flat_M)
        gen = torch.Generator(device="cpu").manual_seed(seed)
        self.P: List[torch.Tensor] = []
        self.Q: List[torch.Tensor] = []
        with torch.no_grad():
            for p, off, (n, m) in zip(self.mats, self.offsets, self.shapes):
                view = _view_like(self.flat_param[off:off + p.numel()], p)
                view.copy_(p.data)
                p.data = view
                p.grad = _view_like(self.flat_M[off:off + p.numel()], p)
                self.P.append(torch.zeros(n, self.r, device=dev))
                self.Q.append(torch.randn(m, self.r, generator=gen).to(dev))   # identical on every rank

        # ---- symmetric layout: flags, then per parity the P and Q accumulators of every matrix
        fl = _round_up(2 * self.world * 4, 256)           # P-phase flags, Q-phase flags
        self.flag_off = {"P": 0, "Q": self.world * 4}
        acc = 0
        self.acc_off = []
        for (n, m) in self.shapes:
            self.acc_off.append((acc, acc + _round_up(n * self.r * 4, 256)))
            acc += _round_up(n * self.r * 4, 256) + _round_up(m * self.r * 4, 256)
        self.acc_bytes = acc
        self.sym_base = fl
        need = fl + 2 * acc
        self.symmetric = symmetric or SymmetricMemory(max(need, 1024), dev, process_group)
        if self.symmetric.nbytes < need:
            raise ValueError("symmetric buffer too small")
        self.emulated = emulated
        self.epoch_dev = torch.zeros(16, dtype=torch.int32, device=dev) if self.graph_capturable else None

        # ---- native step driver: batched small kernels + one grouped GEMM / expand grid per phase
        self.engine = _C.PsgdEngine(self.world, self.r, self.flat_M)
        tsize = sum(16 * (_C.psgd_kpad(n) + _C.psgd_kpad(m)) for n, m in self.shapes)
        self.operand_scratch = torch.zeros(max(tsize, 16), device=dev)
        cur = 0
        for i, p in enumerate(self.mats):
            n, m = self.shapes[i]
            off = self.offsets[i]
            pt = self.operand_scratch[cur:cur + 16 * _C.psgd_kpad(n)]
            cur += pt.numel()
            qt = self.operand_scratch[cur:cur + 16 * _C.psgd_kpad(m)]
            cur += qt.numel()
            self.engine.add_matrix(
                self._mat(i), self.flat_param[off:off + p.numel()], self.flat_momentum[off:off + p.numel()],
                self.P[i], self.Q[i], pt, qt,
                [[self._acc(r, i, 0, par) for r in range(self.world)] for par in (0, 1)],
                [[self._acc(r, i, 1, par) for r in range(self.world)] for par in (0, 1)])

        # ---- vectors: dense P2P average + fused SGD through the engine (one bucket)
        self.vec_engine = None
        if self.vecs:
            voffs, cur = [], 0
            for p in self.vecs:
                voffs.append(cur)
                cur += _round_up(p.numel(), ALIGN)
            self.vec_param = torch.zeros(cur, device=dev)
            self.vec_grad = torch.zeros(cur, device=dev)
            self.vec_momentum = torch.zeros(cur, device=dev)
            with torch.no_grad():
                for p, off in zip(self.vecs, voffs):
                    v = self.vec_param[off:off + p.numel()].view_as(p)
                    v.copy_(p.data)
                    p.data = v
                    p.grad = self.vec_grad[off:off + p.numel()].view_as(p)
            cfg = dict(rank=self.rank, world=self.world, device=dev.index, codec="dense",
                       flag_timeout_s=flag_timeout_s, defer_recv=1 if emulated else 0,
                       device_epoch=1 if self.graph_capturable else 0,
                       num_workers=0 if self.graph_capturable else 1)
            self.vec_engine = _C.DdpEngine(cfg, [(0, cur, 1)], [0])
            self.vec_symmetric = SymmetricMemory(self.vec_engine.symmetric_bytes, dev, process_group) \
                if not emulated else None
            if self.vec_symmetric is not None:
                self._attach_vec(self.vec_symmetric)
        if self.world > 1 and dist.is_initialized() and not emulated:
            dist.broadcast(self.flat_param, src=0, group=process_group)
            if self.vecs:
                dist.broadcast(self.vec_param, src=0, group=process_group)
        self.epoch = 0
        self.steps = 0
        self.launches = 0
        self.hooks_enabled = True      # no hooks here; kept for the common wrapper interface

    def _attach_vec(self, sym: SymmetricMemory) -> None:
        self.vec_symmetric = sym
        self.vec_engine.set_buffers(self.vec_grad, None, self.vec_param, self.vec_momentum)
        self.vec_engine.set_symmetric(sym.buf)
        self.vec_engine.set_sgd(self.lr, self.momentum, self.weight_decay, True)

    # ------------------------------------------------------------------ helpers
    def _acc(self, rank: int, i: int, which: int, parity: int) -> torch.Tensor:
        n, m = self.shapes[i]
        rows = n if which == 0 else m
        off = self.sym_base + parity * self.acc_bytes + self.acc_off[i][which]
        return self.symmetric.tensor(rank, off, rows * self.r, "float32").view(rows, self.r)

    def _mat(self, i: int) -> torch.Tensor:
        n, m = self.shapes[i]
        off = self.offsets[i]
        return self.flat_M[off:off + n * m].view(n, m)

    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    # The step is split into phases so that a single-process emulation of several ranks can
    # run every rank's phase k before any rank's phase k+1 (no kernel then waits for a kernel
    # that has not been launched).  ``step()`` simply runs them back to back.
    def _parity(self) -> int:
        return self.epoch & 1 if self._forced_parity is None else self._forced_parity

    def phase_project_p(self) -> None:
        self.epoch += 1
        if self.epoch_dev is not None:
            _C.bump_epoch(self.epoch_dev)
        par = self._parity()
        self.engine.project_p(par, self.device.index)
        _C.signal_flags(self.symmetric.buf, self.flag_off["P"], self.epoch, self.device.index, self.epoch_dev)
        if self.vec_engine is not None:
            self.vec_engine.begin_step(self.device.index)
            self.vec_engine.bucket_ready(0, self.device.index)
        self.launches += 1

    def phase_project_q(self) -> None:
        par = self._parity()
        _C.wait_flags(self.symmetric.buf, self.flag_off["P"], self.epoch, self.timeout, self.flat_M, self.epoch_dev)
        # every rank has finished reading the other parity's accumulators: clear them for the next step
        other = self.sym_base + (1 - par) * self.acc_bytes
        self.symmetric.tensor(self.rank, other, self.acc_bytes, "uint8").zero_()
        self.engine.project_q(par, self.device.index)
        _C.signal_flags(self.symmetric.buf, self.flag_off["Q"], self.epoch, self.device.index, self.epoch_dev)
        self.launches += 3

    def phase_apply(self) -> None:
        par = self._parity()
        _C.wait_flags(self.symmetric.buf, self.flag_off["Q"], self.epoch, self.timeout, self.flat_M, self.epoch_dev)
        # momentum starts at zero, so mu * buf + g equals the first step's buf = g: a captured step
        # must not bake the first-step flag in
        first = self.steps == 0 and not self.graph_capturable
        self.engine.apply(par, self.lr, self.momentum, self.weight_decay, first, self.device.index)
        if self.vec_engine is not None:
            self.vec_engine.finish_step(self.device.index)
            self.vec_grad.zero_()
        self.launches += 1
        self.steps += 1

    # ---- whole-step CUDA graph capture (GraphedTrainStep)
    def begin_capture_variant(self, variant: int) -> None:
        """The next step is being captured for epochs of parity ``variant``."""
        self._forced_parity = int(variant)

    def next_variant(self) -> int:
        """Which captured graph the next step must replay: the parity of its epoch."""
        return (self.epoch + 1) & 1

    def end_capture(self) -> int:
        """The step issued during a capture did not run: take it back out of the host counters."""
        self._forced_parity = None
        self.epoch -= 1
        self.steps -= 1
        per_step = self.launches - self._launches_mark + (self.engine.launches - self._engine_mark)
        self.launches = self._launches_mark
        self._vec_per_step = int(self.vec_engine.end_capture()) if self.vec_engine is not None else 0
        return per_step + self._vec_per_step

    def note_replay(self, launches_per_step: int, count: int = 1) -> None:
        self.epoch += count
        self.steps += count
        self.launches += count * (launches_per_step - self._vec_per_step)
        if self.vec_engine is not None:
            self.vec_engine.note_replay(count, self._vec_per_step)

    def begin_step(self) -> None:
        """Nothing to arm: the whole exchange runs in ``step``."""
        self._launches_mark = self.launches
        self._engine_mark = self.engine.launches

    def grad_buffers(self):
        return [self.flat_M] + ([self.vec_grad] if self.vecs else [])

    def step(self) -> None:
        self.phase_project_p()
        self.phase_project_q()
        self.phase_apply()

    def zero_grad(self, set_to_none: bool = False) -> None:
        """Matrix gradients live in the error-feedback memory and must not be cleared."""
        if self.vecs:
            self.vec_grad.zero_()

    def check(self) -> None:
        torch.cuda.synchronize(self.device)
        status = _C.read_status(self.flat_M, True)
        if self.vec_engine is not None:
            status = status or self.vec_engine.check_status()
        if status:
            raise RuntimeError(f"hipress PowerSGD: device status {status}")

    def compression_state(self) -> Dict[str, torch.Tensor]:
        """Error-feedback memory, warm-start factors, momentum and the step / epoch counters (flag
        values and accumulator parity derive from the epoch), for checkpoints."""
        torch.cuda.synchronize(self.device)
        out = {"residual": self.flat_M.clone(), "momentum": self.flat_momentum.clone(),
               "Q": [q.clone() for q in self.Q], "steps": torch.tensor(self.steps),
               "epoch": torch.tensor(self.epoch)}
        if self.vecs:
            out["vec_momentum"] = self.vec_momentum.clone()
        return out

    def load_compression_state(self, state: Dict) -> None:
        """Continue from ``compression_state()``; call it on every rank, parameters restored,
        before the next step."""
        torch.cuda.synchronize(self.device)
        self.flat_M.copy_(state["residual"])
        self.flat_momentum.copy_(state["momentum"])
        for q, s in zip(self.Q, state["Q"]):
            q.copy_(s)
        self.steps = int(state.get("steps", 0))
        self.epoch = int(state.get("epoch", self.steps))
        if self.vecs:
            if "vec_momentum" in state:
                self.vec_momentum.copy_(state["vec_momentum"])
            self.vec_engine.set_progress(self.steps, self.epoch)
        torch.cuda.synchronize(self.device)

    def close(self) -> None:
        """Synchronise, wait for every rank, then release the engines and the symmetric memory
        (peers read this rank's accumulators; see ``CompressedDataParallel.close``)."""
        if getattr(self, "engine", None) is None:
            return
        torch.cuda.synchronize(self.device)
        if self.world > 1 and dist.is_initialized() and not self.emulated:
            dist.barrier(group=self.group)
        self.engine = None
        self.vec_engine = None
        self.symmetric = None
        self.vec_symmetric = None

    def metrics(self) -> Dict[str, float]:
        dense = sum(n * m for n, m in self.shapes) * 4
        wire = sum((n + m) * self.r for n, m in self.shapes) * 4
        return {"kernel_launches": self.launches + self.engine.launches
                + (self.vec_engine.launches if self.vec_engine else 0),
                "steps": self.steps, "matrices": len(self.mats), "dense_bytes_per_step": dense,
                "factor_bytes_per_step": wire, "compression_ratio": dense / wire if wire else float("inf")}
