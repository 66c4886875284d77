"""Row sharding of the operator path over several GPUs (one process per GPU).

The B*S token rows are flattened and cut into `world` contiguous blocks; every rank keeps the FULL
[B, H] modulation arrays (they are tiny) and passes its block to the C ABI with `row_start`, so a
block may begin or end in the middle of a sample. FC1 weights are replicated. The only coupling
between ranks is dscale/dshift of a sample whose rows live on more than one rank: each rank then
holds a partial sum, and ONE all-reduce of the packed fp32 [2, B, H] buffer completes them. When
every block boundary falls on a sample boundary no collective is issued at all.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class RowShard:
    """Rows [start, start + count) of the flattened [B*S, H] activation owned by one rank."""

    rank: int
    world: int
    rows_total: int
    seq_len: int
    start: int
    count: int

    @property
    def end(self) -> int:
        return self.start + self.count

    @property
    def first_sample(self) -> int:
        return self.start // self.seq_len

    @property
    def last_sample(self) -> int:
        return (self.end - 1) // self.seq_len if self.count > 0 else self.first_sample - 1

    def samples(self) -> range:
        return range(self.first_sample, self.last_sample + 1)


def boundaries(rows_total: int, world: int) -> list[int]:
    """world + 1 row offsets; block g is [b[g], b[g+1]). Blocks differ in size by at most one row."""
    return [rows_total * g // world for g in range(world + 1)]


def make_shard(rows_total: int, seq_len: int, world: int, rank: int) -> RowShard:
    b = boundaries(rows_total, world)
    return RowShard(rank, world, rows_total, seq_len, b[rank], b[rank + 1] - b[rank])


def straddling_samples(rows_total: int, seq_len: int, world: int) -> list[int]:
    """Samples whose rows are split between ranks (the only ones that need the all-reduce)."""
    out = []
    for cut in boundaries(rows_total, world)[1:-1]:
        if cut % seq_len != 0 and 0 < cut < rows_total:
            out.append(cut // seq_len)
    return sorted(set(out))


def needs_allreduce(rows_total: int, seq_len: int, world: int) -> bool:
    return world > 1 and len(straddling_samples(rows_total, seq_len, world)) > 0


def _capi_backward(kind, dy, x, scale, mean, invstd, shard: RowShard, batch: int, packed: torch.Tensor):
    from . import capi

    dx, _, _ = capi.norm_bwd(kind, dy, x, scale, mean, invstd, row_start=shard.start, seq_len=shard.seq_len,
                             batch=batch, dscale=packed[0], dshift=packed[1])
    return dx


def norm_backward_sharded(kind, dy, x, scale, mean, invstd, shard: RowShard, batch: int, group=None,
                          local_backward=_capi_backward):
    """Backward of AdaLN ("layer") / AdaRMSNorm ("rms") on this rank's row block.

    dy, x: [count, H] local rows; scale: the full [B, H]; mean / invstd: [count] local statistics.
    Returns (dx [count, H], dscale [B, H] fp32, dshift [B, H] fp32). After the call dscale/dshift are
    complete for every sample this rank touches (rows of other samples are zero unless the all-reduce
    ran, in which case they hold the other ranks' sums as well).

    `local_backward(kind, dy, x, scale, mean, invstd, shard, batch, packed)` must write this block's
    partial dscale / dshift into packed[0] / packed[1] for the samples it touches and return dx; the
    default calls the CUDA kernels through the C ABI.
    """
    hidden = x.shape[-1]
    packed = torch.zeros(2, batch, hidden, dtype=torch.float32, device=x.device)  # [dscale | dshift], one buffer
    dx = local_backward(kind, dy, x, scale, mean, invstd, shard, batch, packed)
    if needs_allreduce(shard.rows_total, shard.seq_len, shard.world):
        dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=group)  # one collective, on the compute stream
    return dx, packed[0], packed[1]
