"""Tensor-parallel transformer MLP block: ColumnParallel fc1 (+bias +GeLU) -> RowParallel fc2,
with sequence-sharded input and output — the unit the fused AG+GEMM / GEMM+RS kernels exist
for (GPT-3-175B shape: hidden 12288, ffn 49152)."""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
from torch import nn

from ..parallel.layers import ColumnParallelLinear, RowParallelLinear


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
        block, and bring a per-step result (mean |y| and the first output row) back.

        The copies run on a side stream into one of two device buffers, so the upload of this
        step overlaps the kernels of the previous step that are still in flight; the returned
        pinned tensor is complete once ``torch.cuda.current_stream().synchronize()`` (or the
        event in ``self.last_result_event``) has passed."""
        dev = self.fc1.weight.device
        st = self.__dict__.setdefault("_host_state", {})
        if not st or st["shape"] != tuple(x_pinned.shape) or st["dtype"] != x_pinned.dtype:
            st.update(shape=tuple(x_pinned.shape), dtype=x_pinned.dtype, step=0,
                      copy_stream=torch.cuda.Stream(device=dev),
                      bufs=[torch.empty(x_pinned.shape, dtype=x_pinned.dtype, device=dev) for _ in range(2)],
                      used=[None, None])
        main = torch.cuda.current_stream(dev)
        k = st["step"] & 1
        st["step"] += 1
        cs = st["copy_stream"]
        if st["used"][k] is not None:
            cs.wait_event(st["used"][k])          # the step that last read this buffer is done with it
        with torch.cuda.stream(cs):
            st["bufs"][k].copy_(x_pinned, non_blocking=True)
            up = torch.cuda.Event()
            up.record(cs)
        main.wait_event(up)
        y = self.forward(st["bufs"][k])
        res = torch.cat([y.float().abs().mean().reshape(1), y[0].float()])
        done = torch.cuda.Event()
        done.record(main)
        st["used"][k] = done
        if result_pinned is None:
            return res.cpu()
        result_pinned.copy_(res, non_blocking=True)
        self.last_result_event = torch.cuda.Event()
        self.last_result_event.record(main)
        return result_pinned
