"""CPU restatement of the engine's sharded exchange, shared by the single-GPU emulation test and
the multi-GPU worker: per shard, every rank's payload -> owner's average -> owner's re-compressed
payload -> what every rank decodes."""
import torch

from hipress_b200 import ops

K_EPOCH = 0x9E3779B97F4A7C15
K_BUCKET = 0x632BE59BD9B4E019
K_SHARD = 0xD6E8FEB86659FD93
K_PHASE2 = 0xA24BAED4963EE407


def _signed(seed: int) -> int:
    seed %= 1 << 64
    return seed - (1 << 64) if seed >= (1 << 63) else seed


def shard_elems(n: int, world: int) -> int:
    per = (n + world - 1) // world
    return (per + 4095) // 4096 * 4096


def expected(codec, kw, base_seed, epoch, grads, resid, resid2, world):
    """grads / resid: per-rank CPU tensors (resid updated in place); resid2: per-owner shard residuals
    (updated in place).  Returns the dense tensor every rank ends up with."""
    n = grads[0].numel()
    S = shard_elems(n, world)
    out = torch.zeros(n)
    for j in range(world):
        lo, hi = j * S, min(n, (j + 1) * S)
        if hi <= lo:
            continue
        seed1 = _signed(base_seed + epoch * K_EPOCH + j * K_SHARD)          # bucket 0
        seed2 = _signed(base_seed + epoch * K_EPOCH + K_PHASE2)
        payloads = []
        for r in range(world):
            g, res = grads[r][lo:hi].clone(), resid[r][lo:hi].clone()
            if codec == "tbq":
                payloads.append(ops.tbq_compress(g, res, kw["threshold"]))
            else:
                payloads.append(ops.terngrad_compress(g, kw["bitwidth"], bool(kw["enable_random"]), seed1,
                                                      residual=res if kw["error_feedback"] else None))
            resid[r][lo:hi] = res
        avg = torch.empty(hi - lo)
        res2 = resid2[j][: hi - lo].clone()
        if codec == "tbq":
            ops.tbq_decompress(payloads, avg, kw["threshold"], post_scale=1.0 / world)
            p2 = ops.tbq_compress(avg, res2, kw["threshold"])
            final = torch.empty(hi - lo)
            ops.tbq_decompress([p2], final, kw["threshold"])
        else:
            ops.terngrad_decompress(payloads, avg, post_scale=1.0 / world)
            p2 = ops.terngrad_compress(avg, kw["bitwidth"], bool(kw["enable_random"]), seed2,
                                       residual=res2 if kw["error_feedback"] else None)
            final = torch.empty(hi - lo)
            ops.terngrad_decompress([p2], final)
        resid2[j][: hi - lo] = res2
        out[lo:hi] = final
    return out
