"""Failure detection on the host: a rank that never joins makes the others' bounded waits give up
with FluxTimeoutError instead of hanging, and the survivors stay usable. No GPU involved."""
import time

import pytest
import torch
import torch.distributed as dist

from conftest import run_gloo


def _barrier_missing_rank(rank, world):
    import tempname_new_b200 as flux
    gb = flux.GroupBarrier(timeout_s=1.0)
    gb.barrier_all()                      # everybody arrives: passes
    if rank == world - 1:
        time.sleep(2.5)                   # this rank skips the second barrier altogether
        return
    t0 = time.monotonic()
    with pytest.raises(flux.FluxTimeoutError) as e:
        gb.barrier_all()
    assert time.monotonic() - t0 < 2.0
    assert f"[{world - 1}]" in str(e.value)


def _gemm_rs_missing_rank(rank, world):
    import tempname_new_b200 as flux
    op = flux.GemmRS(dist.group.WORLD, 1, 64, 32, torch.float32, timeout_s=1.0)
    a, w = torch.randn(64, 16), torch.randn(32, 16)
    out = op.forward(a, w)                # a healthy call first
    assert out.shape == (64 // world, 32)
    if rank == 0:
        time.sleep(2.5)                   # rank 0 dies between steps (never issues the next call)
        return
    with pytest.raises(flux.FluxTimeoutError) as e:
        op.forward(a, w)
    assert "start handshake" in str(e.value)


def _ag_late_rank_recovers(rank, world):
    """A slow rank inside the limit is not a failure."""
    import tempname_new_b200 as flux
    op = flux.AGKernel(dist.group.WORLD, 1, 32 * world, 8, 16, torch.float32, timeout_s=5.0)
    if rank == 1:
        time.sleep(0.5)
    a, w = torch.full((32, 16), float(rank + 1)), torch.ones(8, 16)
    out = op.forward(a, w)
    for r in range(world):
        assert float(out[32 * r, 0]) == 16.0 * (r + 1)


def _gemm_rs_recovers_after_reset(rank, world):
    """One rank sleeps past the limit: the others time out, the op refuses further calls, every rank
    calls reset(), and the next forward is right again (call numbers re-agreed, counters zeroed)."""
    import tempname_new_b200 as flux
    torch.manual_seed(3 + rank)
    op = flux.GemmRS(dist.group.WORLD, 1, 64, 32, torch.float32, timeout_s=1.0)
    a, w = torch.randn(64, 16), torch.randn(32, 16)

    def reference():
        part = a @ w.t()
        parts = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(parts, part)
        seg = 64 // world
        return sum(parts)[rank * seg:(rank + 1) * seg]

    assert torch.allclose(op.forward(a, w), reference(), atol=1e-4)
    if rank == 0:
        time.sleep(2.0)                   # misses the call the others are making now
    else:
        with pytest.raises(flux.FluxTimeoutError):
            op.forward(a, w)
        with pytest.raises(RuntimeError, match="reset"):
            op.forward(a, w)              # poisoned until reset
    op.reset()                            # collective: rank 0 joins late, the others wait in it
    assert op.poisoned is None
    for _ in range(2):
        assert torch.allclose(op.forward(a, w), reference(), atol=1e-4)


def test_barrier_times_out_when_a_rank_never_arrives():
    run_gloo(_barrier_missing_rank, 3)


def test_gemm_rs_times_out_when_a_rank_leaves_between_steps():
    run_gloo(_gemm_rs_missing_rank, 2)


def test_op_recovers_after_reset():
    run_gloo(_gemm_rs_recovers_after_reset, 2)


def test_late_rank_within_limit_is_fine():
    run_gloo(_ag_late_rank_recovers, 2)
