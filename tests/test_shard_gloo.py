"""Row-sharding host logic and the one all-reduce, on CPU ranks (gloo, world_size 2 and 3)."""
from __future__ import annotations

import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from novadit_b200 import shard as sh
from novadit_b200 import synth
from oracle import novadit_oracle as oracle


def test_boundaries_cover_all_rows_evenly():
    for rows, world in [(8192, 8), (10, 3), (7, 8), (1, 2), (0, 4)]:
        b = sh.boundaries(rows, world)
        assert b[0] == 0 and b[-1] == rows and all(x <= y for x, y in zip(b, b[1:]))
        sizes = [y - x for x, y in zip(b, b[1:])]
        assert max(sizes) - min(sizes) <= 1
        parts = [sh.make_shard(rows, 4, world, r) for r in range(world)]
        assert sum(p.count for p in parts) == rows


def test_straddle_detection():
    # workload config 2 on 1/2/4/8 GPUs: 1024 rows per GPU at 8 = 4 whole samples -> no collective
    for world in (1, 2, 4, 8):
        assert not sh.needs_allreduce(32 * 256, 256, world)
    # B=2, S=4096 on 8 GPUs: each sample spans 4 GPUs
    assert sh.needs_allreduce(2 * 4096, 4096, 8)
    assert sh.straddling_samples(2 * 4096, 4096, 8) == [0, 1]
    # more GPUs than samples
    assert sh.straddling_samples(3 * 10, 10, 4) == [0, 1, 2]
    assert sh.straddling_samples(3 * 10, 10, 3) == []
    s = sh.make_shard(30, 10, 4, 1)
    assert (s.start, s.count, s.first_sample, s.last_sample) == (7, 8, 0, 1)


def _oracle_local_backward(kind, dy, x, scale, mean, invstd, shard, batch, packed):
    """CPU stand-in for the kernels: partial sums over this block's rows, sample by sample."""
    h = x.shape[-1]
    dx = torch.empty_like(x)
    for b in shard.samples():
        lo = max(b * shard.seq_len, shard.start) - shard.start
        hi = min((b + 1) * shard.seq_len, shard.end) - shard.start
        fn = oracle.adaln_bwd if kind == "layer" else oracle.adarms_bwd
        kw = dict(mean=mean[lo:hi].unsqueeze(0), invstd=invstd[lo:hi].unsqueeze(0)) if kind == "layer" else \
            dict(inv_rms=invstd[lo:hi].unsqueeze(0))
        d, ds, dh = fn(dy[lo:hi].unsqueeze(0), x[lo:hi].unsqueeze(0), scale[b:b + 1], 1e-6, **kw)
        dx[lo:hi] = d[0]
        packed[0, b] += ds[0]
        packed[1, b] += dh[0]
    return dx


def _worker(rank, world, port, kind, bsz, seq, hid, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        x, scale, shift, dy = synth.norm_inputs(bsz, seq, hid, torch.float32, seed=77)
        if kind == "layer":
            _, mean, invstd = oracle.adaln_fwd(x, scale, shift, 1e-6)
        else:
            _, invstd = oracle.adarms_fwd(x, scale, shift, 1e-6)
            mean = invstd
        s = sh.make_shard(bsz * seq, seq, world, rank)
        sl = slice(s.start, s.end)
        dx, ds, dh = sh.norm_backward_sharded(kind, dy.reshape(-1, hid)[sl], x.reshape(-1, hid)[sl], scale,
                                              mean.reshape(-1)[sl], invstd.reshape(-1)[sl], s, bsz,
                                              local_backward=_oracle_local_backward)
        fn = oracle.adaln_bwd if kind == "layer" else oracle.adarms_bwd
        wdx, wds, wdh = fn(dy, x, scale, 1e-6)
        ok = oracle.rel_l2(dx, wdx.reshape(-1, hid)[sl]) < 1e-6
        mine = list(s.samples())
        ok = ok and oracle.rel_l2(ds[mine], wds[mine]) < 1e-5 and oracle.rel_l2(dh[mine], wdh[mine]) < 1e-5
        if sh.needs_allreduce(bsz * seq, seq, world):  # after the collective every rank holds everything
            ok = ok and oracle.rel_l2(ds, wds) < 1e-5 and oracle.rel_l2(dh, wdh) < 1e-5
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("kind", ["layer", "rms"])
@pytest.mark.parametrize("world,bsz,seq", [(2, 3, 10), (2, 4, 8), (3, 2, 16)])
def test_sharded_backward_allreduce_matches_unsharded(kind, world, bsz, seq):
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = 29600 + (hash((kind, world, bsz, seq)) % 300)
    procs = [ctx.Process(target=_worker, args=(r, world, port, kind, bsz, seq, 24, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert all(ret.get(r) for r in range(world)), dict(ret)
