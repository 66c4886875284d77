"""Row sharding over real GPUs: kernels with row_start on every rank, the one NCCL all-reduce when a sample's rows
span ranks, against the unsharded result of one GPU. Needs at least two GPUs (skipped otherwise)."""
from __future__ import annotations

import os

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, kind, bsz, seq, hid, ret):
    import torch.distributed as dist

    from novadit_b200 import capi, shard as sh, synth
    from oracle import novadit_oracle as oracle

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        x, scale, shift, dy = synth.norm_inputs(bsz, seq, hid, torch.bfloat16, seed=88)
        s = sh.make_shard(bsz * seq, seq, world, rank)
        sl = slice(s.start, s.end)
        xs = x.reshape(-1, hid)[sl].to(dev).contiguous()
        gs = dy.reshape(-1, hid)[sl].to(dev).contiguous()
        sd, hd = scale.to(dev), shift.to(dev)
        out = capi.norm_fwd(kind, xs, sd, hd, 1e-6, row_start=s.start, seq_len=seq)
        mean, inv = (out[1], out[2]) if kind == "layer" else (None, out[1])
        results = []
        for _ in range(2):  # twice: the second run must reproduce the first bit for bit
            dx, ds, dh = sh.norm_backward_sharded(kind, gs, xs, sd, mean, inv, s, bsz)
            torch.cuda.synchronize()
            results.append((dx.clone(), ds.clone(), dh.clone()))
        same = all(torch.equal(a, b) for a, b in zip(*results))
        fn = oracle.adaln_bwd if kind == "layer" else oracle.adarms_bwd
        wdx, wds, wdh = fn(dy, x, scale, 1e-6)
        dx, ds, dh = results[0]
        ok = same and oracle.rel_l2(dx.cpu().float(), wdx.reshape(-1, hid)[sl].float()) < 1e-2
        mine = list(s.samples())
        ok = ok and oracle.rel_l2(ds.cpu()[mine], wds[mine]) < 1e-4 and oracle.rel_l2(dh.cpu()[mine], wdh[mine]) < 1e-4
        if sh.needs_allreduce(bsz * seq, seq, world):  # after the collective every rank holds every sample
            ok = ok and oracle.rel_l2(ds.cpu(), wds) < 1e-4 and oracle.rel_l2(dh.cpu(), wdh) < 1e-4
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("kind", ["layer", "rms"])
@pytest.mark.parametrize("bsz,seq,hid", [
    (3, 1000, 1152),   # the middle sample's rows span both ranks: the all-reduce runs
    (4, 256, 1152),    # whole samples per rank: no collective
    (2, 4096, 768),    # long samples, each on its own rank at two ranks, split at four
])
def test_sharded_backward_over_nccl(kind, bsz, seq, hid):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = 29700 + (hash((kind, bsz, seq, hid)) % 200)
    procs = [ctx.Process(target=_worker, args=(r, world, port, kind, bsz, seq, hid, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert all(ret.get(r) for r in range(world)), dict(ret)
