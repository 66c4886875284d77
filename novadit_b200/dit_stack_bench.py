"""Workload config 5: one training step (forward + backward) of a DiT-XL/2 block stack, fused operators against
the PyTorch definitions of the same stack.

    python -m novadit_b200.dit_stack_bench [--depth 28 --batch 32 --seq 256 --hidden 1152 --heads 16]
    python -m torch.distributed.run --nproc-per-node N ... -m novadit_b200.dit_stack_bench   # one batch per GPU

Latent [B, S, H] ~ N(0, 1), conditioning [B, H] ~ N(0, 1), weights N(0, 0.02) from a seeded CPU generator, bf16;
no dataset or checkpoint is involved. A step computes y = stack(x, c) and the gradients of <y, dy> with respect
to x, c and every parameter. With N ranks every rank steps its own batch (no gradient all-reduce: keeping
replicas in sync is ordinary data parallelism, outside the operator path); the reported tokens/s is the sum over
ranks divided by the slowest rank's time. Prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch


def time_steps(fn, warmup: int, iters: int) -> list[float]:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        out.append(e0.elapsed_time(e1))
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--depth", type=int, default=28)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--seq", type=int, default=256)
    ap.add_argument("--hidden", type=int, default=1152)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--no-ref", action="store_true", help="skip the PyTorch-definition stack")
    ap.add_argument("--zero-init", action="store_true", help="adaLN-Zero initialisation (blocks are identities)")
    args = ap.parse_args()

    from novadit_b200.modules import DiTStack, init_stack_

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("the DiT stack bench needs a CUDA device")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    dt = torch.bfloat16
    gen = torch.Generator().manual_seed(1000 + rank)
    x = torch.randn(args.batch, args.seq, args.hidden, generator=gen).to(dev, dt).requires_grad_(True)
    cond = torch.randn(args.batch, args.hidden, generator=gen).to(dev, dt).requires_grad_(True)
    dy = torch.randn(args.batch, args.seq, args.hidden, generator=gen).to(dev, dt)

    def build(fused: bool):
        stack = DiTStack(args.hidden, args.heads, args.depth, use_fused=fused, zero_init=args.zero_init,
                         device=dev, dtype=dt)
        init_stack_(stack, seed=0, zero_init=args.zero_init)
        targets = (x, cond, *stack.parameters())

        def step():
            y = stack(x, cond)
            return y, torch.autograd.grad(y, targets, dy)

        return stack, step

    result = {"workload": f"config5: DiT stack depth {args.depth}, H {args.hidden}, {args.heads} heads, "
                          f"x [{args.batch},{args.seq},{args.hidden}] bf16 per GPU, fwd+bwd",
              "n_gpus": world, "data": "synthetic"}
    _, fused_step = build(True)
    fused_ms = statistics.median(time_steps(fused_step, args.warmup, args.iters))
    yf, gf = fused_step()
    ref_ms = None
    if not args.no_ref:
        _, ref_step = build(False)
        ref_ms = statistics.median(time_steps(ref_step, args.warmup, args.iters))
        yr, gr = ref_step()

        def rel(a, b):
            a, b = a.detach().float(), b.detach().float()
            return float((a - b).norm() / b.norm().clamp_min(1e-30))

        result["parity_vs_pytorch_stack"] = {
            "y_rel_l2": rel(yf, yr), "dx_rel_l2": rel(gf[0], gr[0]), "dcond_rel_l2": rel(gf[1], gr[1]),
            "param_grads_rel_l2": rel(torch.cat([g.flatten() for g in gf[2:]]), torch.cat([g.flatten() for g in gr[2:]])),
        }
    times = torch.tensor([fused_ms, ref_ms if ref_ms is not None else 0.0], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    fused_ms, ref_max = float(times[0]), float(times[1])
    tokens = world * args.batch * args.seq
    result.update({"fused_ms_per_step": fused_ms, "fused_tokens_per_s": tokens / fused_ms * 1e3})
    if ref_ms is not None:
        result.update({"pytorch_ms_per_step": ref_max, "pytorch_tokens_per_s": tokens / ref_max * 1e3,
                       "speedup": ref_max / fused_ms})
    if rank == 0:
        print(json.dumps(result), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
