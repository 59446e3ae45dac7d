"""Data-parallel training with compressed gradient synchronisation.

``CompressedDataParallel`` wraps a module the way ``DistributedDataParallel``
does, but gradients are synchronised by this framework's engine: parameters and
gradients are re-homed into flat fp32 buffers cut into buckets (25 MB by
default), backward hooks tell the C++ engine which parameters are ready, and for
every full bucket the engine launches, on its own streams and overlapped with
the rest of backward,

    compress -> packed bytes stored into every rank's receive slot over NVLink
    -> bounded flag wait -> one-pass unpack + average of all ranks' payloads
    (-> fused SGD-momentum update of the flat parameters).

Nothing of this exists in the reference, whose caller has to submit per-tensor
tasks, poll ``getResults`` and move CPU buffers itself (ref hp_cuda.cpp:904-1060).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import _C
from .symmetric import SymmetricMemory

ALIGN = 4  # elements; keeps every parameter view 16-byte aligned


@dataclass
class CompressionConfig:
    """Which codec synchronises the gradients, and its parameters.

    algorithm: ``terngrad`` | ``tbq`` | ``graddrop`` | ``dgc`` | ``ecq`` | ``dense``
    (``dense`` is an uncompressed peer-to-peer all-reduce through the same engine).
    """
    algorithm: str = "terngrad"
    bitwidth: int = 2
    enable_random: bool = True
    error_feedback: bool = True
    threshold: float = 2e-3
    sample_rate: float = 0.01
    keep_fraction: float = 0.001
    alpha: float = 1.0
    beta: float = 1.0
    seed: int = 1
    bucket_mb: float = 25.0
    average: bool = True
    flag_timeout_s: float = 20.0
    # engine threads that issue the buckets' kernels: 0 = the backward-hook thread launches them
    # itself; -1 = choose (a worker thread once a step has enough launches to be worth moving
    # off the autograd thread, none for a handful of buckets where the hand-off costs more)
    num_workers: int = -1
    # keep the step's epoch on the device so that the whole step, exchange included, can be
    # captured in a CUDA graph (tbq / terngrad / graddrop / dgc with a fused optimizer; forces
    # inline issue)
    graph_capturable: bool = False
    # sharded exchange (tbq / terngrad): rank j owns 1/world of every bucket; compressed
    # reduce-scatter to the owners, then compressed all-gather of the re-quantised averages.
    # None = decide from the bucket size and the world size (prefer_sharded)
    sharded: Optional[bool] = False
    # DGC extras (algorithm "dgc"): momentum correction with factor masking, local clipping
    momentum_correction: bool = False
    dgc_momentum: float = 0.9
    clip_norm: float = 0.0
    # per-stage device timing (metrics()["stages"]): four one-thread launches per bucket
    trace: bool = False
    # how payloads reach the peers: "p2p" = one store per destination over NVLink (always
    # available); "nvls" = one multicast store through the NVLink switch where the host exposes
    # it (falls back to p2p otherwise; ``wrapper.transport`` says which one runs)
    transport: str = "p2p"

    def engine_dict(self, rank: int, world: int, device: int) -> Dict:
        return dict(rank=rank, world=world, device=device, codec=self.algorithm, bitwidth=self.bitwidth,
                    enable_random=int(self.enable_random), error_feedback=int(self.error_feedback),
                    threshold=float(self.threshold), sample_rate=float(self.sample_rate),
                    keep_fraction=float(self.keep_fraction), alpha=float(self.alpha), beta=float(self.beta),
                    seed=int(self.seed), average=int(self.average), flag_timeout_s=float(self.flag_timeout_s),
                    num_workers=int(self.num_workers), momentum_correction=int(self.momentum_correction),
                    dgc_momentum=float(self.dgc_momentum),
                    dgc_clip=float(self.clip_norm) / max(1.0, float(world)) ** 0.5,
                    trace=int(self.trace))

    @property
    def needs_residual(self) -> bool:
        return self.algorithm in ("tbq", "graddrop", "dgc", "ecq") or (
            self.algorithm == "terngrad" and self.error_feedback)


def prefer_sharded(bucket_bytes: float, world: int) -> bool:
    """Size rule for the form of the tbq / terngrad exchange (used when ``sharded=None``).

    All-gather form: every rank stores its payload into all ``world`` slots and decodes
    ``world`` payloads per element -- two phases, the fewest launches.  Sharded form: compressed
    reduce-scatter to shard owners, then compressed all-gather of the re-quantised averages --
    2 (world-1)/world of one payload on the wire and two table look-ups per element instead of
    ``world``, for a third phase, a second flag wait and a second quantisation.

    Measured on NVSwitch: at 2 and 4 GPUs the all-gather form wins at every size from 256 KB to
    512 MB (512 MB at 4 GPUs: TBQ 0.43 ms against 0.51 ms sharded) -- the switch delivers the
    extra copies of a payload for the cost of one read of the gradient.  At 8 GPUs the sharded
    form wins at 512 MB (TBQ 0.50 against 0.59 ms, TernGrad 0.76 against 0.89 ms), ties at 64 MB
    and loses below.  The rule picks it at 8 ranks from ``SHARDED_MIN_BYTES`` (128 MB, between
    the tie and the win; 25 MB training buckets stay on the all-gather form)."""
    return world >= SHARDED_MIN_WORLD and bucket_bytes >= SHARDED_MIN_BYTES


SHARDED_MIN_BYTES = 128 * (1 << 20)
SHARDED_MIN_WORLD = 8


@dataclass
class BucketPlan:
    offsets: List[int] = field(default_factory=list)      # element offset of each parameter
    buckets: List[tuple] = field(default_factory=list)    # (offset, numel, num_params)
    param_bucket: List[int] = field(default_factory=list)
    total: int = 0


def plan_buckets(numels: Iterable[int], bucket_elems: int) -> BucketPlan:
    """Lay parameters out in *reverse* order (the order backward produces gradients), each
    aligned to 16 bytes, and cut the flat range into buckets of at most ``bucket_elems``."""
    numels = list(numels)
    plan = BucketPlan(offsets=[0] * len(numels), param_bucket=[0] * len(numels))
    cursor, b_start, b_params = 0, 0, 0
    for i in reversed(range(len(numels))):
        size = (numels[i] + ALIGN - 1) // ALIGN * ALIGN
        if b_params > 0 and cursor - b_start + size > bucket_elems:
            plan.buckets.append((b_start, cursor - b_start, b_params))
            b_start, b_params = cursor, 0
        plan.offsets[i] = cursor
        plan.param_bucket[i] = len(plan.buckets)
        cursor += size
        b_params += 1
    if b_params > 0:
        plan.buckets.append((b_start, cursor - b_start, b_params))
    plan.total = cursor
    return plan


def _view_like(flat: torch.Tensor, p: torch.Tensor) -> torch.Tensor:
    """A view of the 1-D slice ``flat`` with ``p``'s shape, keeping a channels-last parameter
    channels-last (so convolutions do not re-layout their weights every step)."""
    if p.dim() == 4 and not p.is_contiguous() and p.is_contiguous(memory_format=torch.channels_last):
        n, c, h, w = p.shape
        return flat.view(n, h, w, c).permute(0, 3, 1, 2)
    return flat.view(p.shape)


class CompressedDataParallel(nn.Module):
    """Wrap ``module`` for data-parallel training with compressed gradient exchange.

    Typical step::

        model = CompressedDataParallel(net, CompressionConfig("terngrad"), lr=0.1, momentum=0.9)
        loss = criterion(model(x), y)
        loss.backward()          # buckets are compressed and exchanged while backward runs
        model.step()             # waits for the exchange; parameters are already updated (fused SGD)

    With ``fused_sgd=False`` the averaged gradients are left in ``p.grad`` for any optimizer.
    """

    def __init__(self, module: nn.Module, config: Optional[CompressionConfig] = None, *, lr: float = 0.1,
                 momentum: float = 0.9, weight_decay: float = 0.0, fused_sgd: bool = True,
                 optimizer: str = "sgd", betas=(0.9, 0.999), eps: float = 1e-8,
                 process_group: Optional[dist.ProcessGroup] = None,
                 symmetric: Optional[SymmetricMemory] = None, rank: Optional[int] = None,
                 world: Optional[int] = None):
        super().__init__()
        self.module = module
        self.config = config or CompressionConfig()
        self.group = process_group
        if rank is None:
            rank = dist.get_rank(process_group) if dist.is_initialized() else 0
        if world is None:
            world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.rank, self.world = rank, world
        self.params = [p for p in module.parameters() if p.requires_grad]
        if not self.params:
            raise ValueError("module has no trainable parameters")
        self.device = self.params[0].device
        if self.device.type != "cuda":
            raise ValueError("CompressedDataParallel needs the module on a CUDA device")
        for p in self.params:
            if p.dtype != torch.float32:
                raise ValueError("parameters must be float32 (use autocast for bf16 compute)")

        bucket_elems = max(ALIGN, int(self.config.bucket_mb * (1 << 20) / 4) // ALIGN * ALIGN)
        self.plan = plan_buckets([p.numel() for p in self.params], bucket_elems)
        n = self.plan.total
        dev = self.device
        self.flat_param = torch.zeros(n, device=dev)
        self.flat_grad = torch.zeros(n, device=dev)
        self.flat_residual = torch.zeros(n, device=dev) if self.config.needs_residual else None
        self.optimizer = optimizer
        if optimizer not in ("sgd", "adamw"):
            raise ValueError("optimizer must be 'sgd' or 'adamw'")
        fused = fused_sgd or optimizer == "adamw"
        self.flat_momentum = torch.zeros(n, device=dev) if fused else None
        self.flat_second = torch.zeros(n, device=dev) if optimizer == "adamw" else None
        self.flat_velocity = torch.zeros(n, device=dev) if self.config.momentum_correction else None
        with torch.no_grad():
            for p, off in zip(self.params, self.plan.offsets):
                view = _view_like(self.flat_param[off:off + p.numel()], p)
                view.copy_(p.data)
                p.data = view
                p.grad = _view_like(self.flat_grad[off:off + p.numel()], p)

        if world > 1 and dist.is_initialized():
            # every replica starts from rank 0's weights
            dist.broadcast(self.flat_param, src=dist.get_global_rank(process_group, 0)
                           if process_group is not None else 0, group=process_group)

        cfg_dict = self.config.engine_dict(rank, world, dev.index)
        # with a fused optimizer nobody reads the averaged gradient: the kernel that applies the
        # update leaves zeros behind, ready for the next backward pass
        cfg_dict["clear_grad"] = 1 if fused else 0
        sharded = self.config.sharded
        if sharded is None:
            sharded = self.config.algorithm in ("tbq", "terngrad") and \
                prefer_sharded(self.config.bucket_mb * (1 << 20), world)
        self.sharded = bool(sharded)
        cfg_dict["sharded"] = 1 if self.sharded else 0
        self.graph_capturable = bool(self.config.graph_capturable)
        if self.graph_capturable:
            if not fused:
                raise ValueError("graph_capturable needs a fused optimizer (the update is part of the captured step)")
            cfg_dict["device_epoch"] = 1
            cfg_dict["num_workers"] = 0
        elif self.config.num_workers < 0:
            per_bucket = {"dgc": 12 + world, "graddrop": 10 + world}.get(self.config.algorithm, 4)
            cfg_dict["num_workers"] = 1 if len(self.plan.buckets) * per_bucket > 200 else 0
        if self.config.transport not in ("p2p", "nvls"):
            raise ValueError("transport must be 'p2p' or 'nvls'")
        cfg_dict["nvls"] = 1 if self.config.transport == "nvls" else 0
        self.engine = _C.DdpEngine(cfg_dict, self.plan.buckets, self.plan.param_bucket)
        self.symmetric = symmetric or SymmetricMemory(self.engine.symmetric_bytes, dev, process_group,
                                                      multicast=self.config.transport == "nvls")
        self.transport = "nvls" if (self.config.transport == "nvls" and self.symmetric.multicast) else "p2p"
        if self.symmetric.nbytes < self.engine.symmetric_bytes:
            raise ValueError("symmetric buffer too small for this model")
        self.engine.set_buffers(self.flat_grad, self.flat_residual, self.flat_param, self.flat_momentum,
                                self.flat_velocity, self.flat_second)
        self.engine.set_symmetric(self.symmetric.buf)
        self.fused_sgd = fused
        self.lr, self.momentum, self.weight_decay = lr, momentum, weight_decay
        self.betas, self.eps = betas, eps
        if optimizer == "adamw":
            self.engine.set_adamw(lr, betas[0], betas[1], eps, weight_decay)
        else:
            self.engine.set_sgd(lr, momentum, weight_decay, fused_sgd)

        self._in_step = False
        self.hooks_enabled = True
        self._hooks = []
        for i, p in enumerate(self.params):
            self._hooks.append(p.register_post_accumulate_grad_hook(self._make_hook(i)))
        self._dev_index = dev.index

    # ------------------------------------------------------------------ hooks
    def _make_hook(self, index: int):
        def hook(_param):
            if self._in_step and self.hooks_enabled:
                self.engine.grad_ready(index, self._dev_index)
        return hook

    def forward(self, *args, **kwargs):
        if self.training and torch.is_grad_enabled() and not self._in_step:
            self.begin_step()
        return self.module(*args, **kwargs)

    def begin_step(self) -> None:
        """Arm the engine for one backward pass (called automatically by ``forward``)."""
        self.engine.begin_step(self._dev_index)
        self._in_step = True

    def step(self) -> None:
        """Wait until every bucket has been exchanged (and, with fused SGD, applied), then clear the
        gradient buffer for the next backward."""
        if not self._in_step:
            raise RuntimeError("step() without a forward/backward since the last step()")
        self.engine.finish_step(self._dev_index)
        self._in_step = False

    def zero_grad(self, set_to_none: bool = False) -> None:  # noqa: D401
        """Gradients live in the flat buffer and are views: they are zeroed, never dropped."""
        self.flat_grad.zero_()

    # ---- whole-step CUDA graph capture (GraphedTrainStep)
    def end_capture(self) -> int:
        """The step issued during a graph capture did not run: undo its host-side accounting."""
        return int(self.engine.end_capture())

    def note_replay(self, launches_per_step: int, count: int = 1) -> None:
        self.engine.note_replay(count, launches_per_step)

    def grad_buffers(self):
        """The buffers a backward pass accumulates into (saved and restored around a graph capture)."""
        return [self.flat_grad]

    def set_lr(self, lr: float) -> None:
        self.lr = lr
        if self.optimizer == "adamw":
            self.engine.set_adamw(lr, self.betas[0], self.betas[1], self.eps, self.weight_decay)
        else:
            self.engine.set_sgd(lr, self.momentum, self.weight_decay, self.fused_sgd)

    def set_keep_fraction(self, keep_fraction: float) -> None:
        """Per-step sparsity (DGC warm-up); must not exceed the configured maximum."""
        self.engine.set_keep_fraction(float(keep_fraction))

    def check(self) -> None:
        """Synchronise and raise if a kernel recorded a flag time-out or a malformed payload."""
        status = self.engine.check_status()
        if status != 0:
            names = {1: "a peer's flag was not published in time", 2: "payload exceeds its slot",
                     3: "malformed payload header"}
            raise RuntimeError(f"hipress engine: {names.get(status, status)}")

    # ------------------------------------------------------------------ state
    def compression_state(self) -> Dict[str, torch.Tensor]:
        """Everything the synchroniser and its fused optimizer carry from step to step, for
        checkpoints: residual / momentum / moment / velocity buffers, the sharded exchange's
        owner-side residual, and the step and epoch counters from which the rounding seeds,
        the slot parity, DGC's position in its warm-up and AdamW's bias correction derive."""
        torch.cuda.synchronize(self.device)
        out = {"steps": torch.tensor(self.engine.steps), "epoch": torch.tensor(self.engine.epoch)}
        if self.flat_residual is not None:
            out["residual"] = self.flat_residual.clone()
        if self.flat_momentum is not None:
            out["momentum"] = self.flat_momentum.clone()
        if self.flat_second is not None:
            out["second_moment"] = self.flat_second.clone()
        if self.flat_velocity is not None:
            out["velocity"] = self.flat_velocity.clone()
        res2 = self.engine.residual2(self._dev_index)
        if res2 is not None:
            out["residual2"] = res2.clone()
        return out

    def load_compression_state(self, state: Dict[str, torch.Tensor]) -> None:
        """Continue from ``compression_state()``: call it on every rank, with the model's
        parameters restored, before the next step."""
        if self._in_step:
            raise RuntimeError("load_compression_state() in the middle of a step")
        torch.cuda.synchronize(self.device)
        for key, buf in (("residual", self.flat_residual), ("momentum", self.flat_momentum),
                         ("second_moment", self.flat_second), ("velocity", self.flat_velocity),
                         ("residual2", self.engine.residual2(self._dev_index))):
            if key in state and buf is not None:
                buf.copy_(state[key])
        if "steps" in state:
            steps = int(state["steps"])
            self.engine.set_progress(steps, int(state.get("epoch", steps)))
        torch.cuda.synchronize(self.device)

    def close(self) -> None:
        """Release the engine and the symmetric memory once no peer can still be reading it.

        Peers read this rank's memory (the dense codec pulls every rank's slot) and write into
        it; freeing it while a slower rank still runs its last step is undefined behaviour with
        CUDA IPC mappings.  ``close`` synchronises this device, waits for every rank at a
        barrier and only then drops the native objects.  Call it on every rank."""
        if getattr(self, "engine", None) is None:
            return
        torch.cuda.synchronize(self.device)
        if self.world > 1 and dist.is_available() and dist.is_initialized():
            dist.barrier(group=self.group)
        for h in self._hooks:
            h.remove()
        self._hooks = []
        self.engine = None
        self.symmetric = None

    def metrics(self) -> Dict[str, float]:
        """Counters of the synchroniser.  ``wait_*`` is the time this rank's flag waits spent
        waiting for peers since the previous call (device-timed; it is what rank skew and the
        transfer itself cost, as opposed to this rank's own kernels).  With
        ``CompressionConfig(trace=True)``, ``stages`` holds, for the last step, the device time in
        microseconds from the step's begin to each bucket's {gradients ready, payload pushed, all
        payloads arrived, update applied}, ``step_us`` the step's length and ``exposed_tail_us``
        the time between the last bucket's gradients being ready (the end of backward) and the
        last update being applied; with a sparse codec also what the last step selected:
        ``selected_k`` elements out of ``candidates`` over the sampled ``thresholds`` (one per
        bucket) and the bytes that put on the wire.  ``residual_norm`` is the L2 norm of the error
        feedback carried into the next step (codecs that keep one).  Synchronises the device."""
        dense = self.engine.dense_bytes_per_step
        wire = self.engine.wire_bytes_per_step
        total_ns, max_ns, waits = self.engine.wait_stats()
        out = {"buckets": len(self.plan.buckets), "dense_bytes_per_step": dense,
               "wire_bytes_per_step": wire,
               "compression_ratio": dense * max(1, self.world - 1) / wire if wire else float("inf"),
               "kernel_launches": self.engine.launches, "steps": self.engine.steps,
               "wait_us_total": total_ns / 1e3, "wait_us_max": max_ns / 1e3, "waits": waits}
        if self.flat_residual is not None:
            # error feedback carried into the next step (for the sparse codecs: the velocity / residual
            # the selection draws from)
            out["residual_norm"] = float(torch.linalg.vector_norm(self.flat_residual))
        times = self.engine.stage_times()
        if times:
            nb = len(self.plan.buckets)
            names = ("ready", "pushed", "arrived", "done")
            stages = [{k: times[4 * b + i] / 1e3 for i, k in enumerate(names)} for b in range(nb)]
            out["stages"] = stages
            out["step_us"] = times[4 * nb] / 1e3
            last_ready = max(s["ready"] for s in stages)
            out["exposed_tail_us"] = max(s["done"] for s in stages) - last_ready
        sparse = self.engine.sparse_stats()
        if sparse:
            import struct
            nb = len(self.plan.buckets)
            ks = [int(sparse[4 * b]) for b in range(nb)]
            out["selected_k"] = sum(ks)
            out["candidates"] = sum(int(sparse[4 * b + 1]) for b in range(nb))
            out["thresholds"] = [struct.unpack("<f", struct.pack("<I", int(sparse[4 * b + 2])))[0] for b in range(nb)]
            out["dropped_candidates"] = max(int(sparse[4 * b + 3]) for b in range(nb))
            # what this rank actually put on the wire in the last step (capacity is in wire_bytes_per_step)
            out["wire_bytes_last_step"] = sum(4 + 8 * k for k in ks) * max(1, self.world - 1)
        return out
