"""Host-buffer front end: run an operator step over a stream of batches that live in pinned HOST memory.

The operators themselves take device tensors, like the reference's (`novadit/ops/adaln.py:62-88`). A caller
whose activations sit in host memory pays two PCIe transfers per step, and at the DiT-XL/2 shape those
transfers (tens of MB each way) take ~50x longer than the kernels. `HostPipeline` keeps the three phases of
consecutive steps on three CUDA streams - upload of step i+1, kernels of step i, download of step i-1 - so
that a stream of batches runs at the speed of the slower PCIe direction instead of the sum of all three.

    pipe = HostPipeline(step, device)          # step(*device_inputs) -> tuple of device outputs
    t = pipe.submit(host_inputs)               # pinned host tensors in
    outs = pipe.result(t)                      # pinned host tensors out (valid until `depth` more submits)

There is no CPU path: the pipeline needs a CUDA device and the kernels of `novadit_b200.ops`.
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch


def bind_host_thread_to_gpu(device_index: int) -> bool:
    """Restricts the calling process to the CPU cores the driver reports as closest to the GPU (NVML's CPU
    affinity mask, read-only), so that pinned buffers allocated afterwards are first touched on the GPU's own
    NUMA node and the copies do not cross sockets. Worth it when several ranks drive several GPUs from host
    memory. Returns False (and changes nothing) when NVML or the affinity call is unavailable."""
    try:
        import os

        import pynvml

        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(device_index)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
        cpus = {64 * w + b for w, word in enumerate(mask) for b in range(64) if (word >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return False
        os.sched_setaffinity(0, cpus)
        return True
    except Exception:
        return False


class HostPipeline:
    def __init__(self, step: Callable[..., Sequence[torch.Tensor]], device, depth: int = 3) -> None:
        if not torch.cuda.is_available():
            raise RuntimeError("HostPipeline needs a CUDA device (the operators have no CPU fallback)")
        if depth < 2:
            raise ValueError("depth must be at least 2")
        self.step, self.device, self.depth = step, torch.device(device), depth
        self.s_in = torch.cuda.Stream(self.device)
        self.s_run = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self.slots = [
            {"dev_in": None, "dev_out": None, "host_out": None, "uploaded": torch.cuda.Event(), "ran": torch.cuda.Event(),
             "downloaded": torch.cuda.Event(), "used": False}
            for _ in range(depth)
        ]
        self.next_ticket = 0

    def submit(self, host_inputs: Sequence[torch.Tensor]) -> int:
        """Queues one step; returns a ticket for `result`. Returns without waiting for the GPU unless the
        slot's previous results (ticket - depth) are still being downloaded."""
        ticket = self.next_ticket
        self.next_ticket += 1
        slot = self.slots[ticket % self.depth]
        for t in host_inputs:
            if t.device.type != "cpu" or not t.is_pinned():
                raise ValueError("host inputs must be pinned CPU tensors (torch.Tensor.pin_memory())")
        if slot["dev_in"] is None:
            slot["dev_in"] = [torch.empty(t.shape, dtype=t.dtype, device=self.device) for t in host_inputs]
        with torch.cuda.stream(self.s_in):
            if slot["used"]:
                self.s_in.wait_event(slot["ran"])  # the kernels that read this slot's inputs are done
            for d, h in zip(slot["dev_in"], host_inputs):
                d.copy_(h, non_blocking=True)
            slot["uploaded"].record(self.s_in)
        with torch.cuda.stream(self.s_run):
            self.s_run.wait_event(slot["uploaded"])
            if slot["used"]:
                # The slot's previous outputs were allocated on this stream and read by the download stream.
                # Ordering this stream after that download makes it safe to hand their memory back to this
                # stream's pool here, so the step below reuses it (a steady footprint of `depth` output sets,
                # no allocator bookkeeping across streams).
                self.s_run.wait_event(slot["downloaded"])
                slot["dev_out"] = None
            outs = tuple(self.step(*slot["dev_in"]))
            slot["ran"].record(self.s_run)
        slot["dev_out"] = outs
        if slot["host_out"] is None:
            slot["host_out"] = [torch.empty(o.shape, dtype=o.dtype).pin_memory() for o in outs]
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(slot["ran"])
            for h, o in zip(slot["host_out"], outs):
                h.copy_(o, non_blocking=True)
            slot["downloaded"].record(self.s_out)
        slot["used"] = True
        return ticket

    def result(self, ticket: int) -> list[torch.Tensor]:
        """Blocks until the step's outputs are in host memory and returns them (the slot's pinned buffers)."""
        if not 0 <= ticket < self.next_ticket or ticket < self.next_ticket - self.depth:
            raise ValueError("ticket is not in flight (results are kept for the last `depth` steps)")
        slot = self.slots[ticket % self.depth]
        slot["downloaded"].synchronize()
        return slot["host_out"]

    def drain(self) -> None:
        """Blocks until every queued step has finished downloading."""
        self.s_out.synchronize()
        self.s_run.synchronize()
        self.s_in.synchronize()


def adaln_train_step(eps: float = 1e-6) -> Callable[..., tuple]:
    """step(x, scale, shift, dy) -> (y, dx, dscale, dshift) through `ops.fused_adaln` and autograd."""
    import novadit_b200.ops as ops

    def step(x, scale, shift, dy):
        x = x.detach().requires_grad_(True)
        scale = scale.detach().requires_grad_(True)
        shift = shift.detach().requires_grad_(True)
        y = ops.fused_adaln(x, scale, shift, eps)
        y.backward(dy)
        return y.detach(), x.grad, scale.grad, shift.grad

    return step
