"""Tensor-parallel transformer MLP block: ColumnParallel fc1 (+bias +GeLU) -> RowParallel fc2,
with sequence-sharded input and output — the unit the fused AG+GEMM / GEMM+RS kernels exist
for (GPT-3-175B shape: hidden 12288, ffn 49152)."""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
from torch import nn

from ..parallel.layers import ColumnParallelLinear, RowParallelLinear


class HostStep:
    """Runs ``fn(x_device)`` for a batch that lives in pinned host memory and brings a per-step
    result back: the shard is copied host->device on a side stream into one of two device buffers
    (the upload of a step overlaps the kernels of the step before), ``fn`` runs on the current
    stream, and ``[mean |y|, y[0, :]]`` is copied device->host into a pinned tensor. Works for any
    ``fn`` (the benchmark drives both this library's block and the torch.matmul + NCCL block
    through it, so the two end-to-end numbers differ only in ``fn``)."""

    def __init__(self, fn, device):
        self.fn, self.device = fn, device
        self.copy_stream = torch.cuda.Stream(device=device)
        self.bufs = None
        self.used = [None, None]
        self.step = 0
        self.last_result_event = None

    @torch.no_grad()
    def __call__(self, x_pinned: torch.Tensor, result_pinned: Optional[torch.Tensor] = None):
        if self.bufs is None or self.bufs[0].shape != x_pinned.shape or self.bufs[0].dtype != x_pinned.dtype:
            self.bufs = [torch.empty(x_pinned.shape, dtype=x_pinned.dtype, device=self.device) for _ in range(2)]
            self.used = [None, None]
        main = torch.cuda.current_stream(self.device)
        k = self.step & 1
        self.step += 1
        cs = self.copy_stream
        if self.used[k] is not None:
            cs.wait_event(self.used[k])          # the step that last read this buffer is done with it
        with torch.cuda.stream(cs):
            self.bufs[k].copy_(x_pinned, non_blocking=True)
            up = torch.cuda.Event()
            up.record(cs)
        main.wait_event(up)
        y = self.fn(self.bufs[k])
        res = torch.cat([y.float().abs().mean().reshape(1), y[0].float()])
        done = torch.cuda.Event()
        done.record(main)
        self.used[k] = done
        if result_pinned is None:
            return res.cpu()
        result_pinned.copy_(res, non_blocking=True)
        self.last_result_event = torch.cuda.Event()
        self.last_result_event.record(main)
        return result_pinned


class TPMLP(nn.Module):
    def __init__(self, hidden: int, ffn: int, tp_group=None, bias: bool = True,
                 dtype: torch.dtype = torch.bfloat16, device=None, act: str = "gelu"):
        super().__init__()
        self.group = tp_group if tp_group is not None else dist.group.WORLD
        self.act = act
        self.fc1 = ColumnParallelLinear(hidden, ffn, self.group, bias, dtype, device)
        self.fc2 = RowParallelLinear(ffn, hidden, self.group, bias, dtype, device)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x: [tokens / W, hidden] (this rank's sequence shard) -> [tokens / W, hidden]."""
        if torch.is_grad_enabled() and (x.requires_grad or self.fc1.weight.requires_grad):
            from ..ops.gemm_only import apply_act
            return self.fc2(apply_act(self.fc1(x), self.act))
        h = self.fc1(x, act=self.act)  # activation fused into the AG+GEMM epilogue
        return self.fc2(h)

    @torch.no_grad()
    def forward_host(self, x_pinned: torch.Tensor, result_pinned: Optional[torch.Tensor] = None):
        """End-to-end step for a host-resident batch: copy the shard from pinned host memory, run the
        block, and bring a per-step result (mean |y| and the first output row) back; see
        ``HostStep``. The returned pinned tensor is complete once
        ``torch.cuda.current_stream().synchronize()`` has passed."""
        hs = self.__dict__.get("_host_step")
        if hs is None:
            hs = self.__dict__["_host_step"] = HostStep(self.forward, self.fc1.weight.device)
        return hs(x_pinned, result_pinned)
