"""EP dispatch / combine compositions on CPU ranks."""
import torch
import torch.distributed as dist

from conftest import run_gloo


def _ep(rank, world):
    import tempname_new_b200 as flux
    from moe_common import routed_problem
    tpr, H, E, topk = 8, 16, 4, 2
    tokens = tpr * world
    experts, gate, scatter, splits, order = routed_problem(tokens, topk, E, seed=2)
    x_full = torch.randn(tokens, H, generator=torch.Generator().manual_seed(9))
    fwd = flux.DisScatterForward(E, tokens, H, topk, rank, 1, world, world, dtype=torch.float32)
    bwd = flux.DisScatterBackward(E, tokens, H, topk, rank, 1, world, world, dtype=torch.float32)
    rows = fwd.forward(x_full[rank * tpr:(rank + 1) * tpr].contiguous(), experts, scatter, splits)
    E_loc = E // world
    offs = torch.cat([torch.zeros(1, dtype=torch.long), splits.long().cumsum(0)])
    lo, hi = int(offs[rank * E_loc]), int(offs[(rank + 1) * E_loc])
    sorted_tokens = (order // topk)[lo:hi]
    torch.testing.assert_close(rows, x_full[sorted_tokens])
    # combine: every row weighted by its gate, summed per token at the owner
    w = gate.reshape(-1)[order][lo:hi]
    out = bwd.forward(rows * w[:, None], experts, scatter, splits)
    ref = (x_full * gate.sum(1, keepdim=True))[rank * tpr:(rank + 1) * tpr]
    torch.testing.assert_close(out, ref, rtol=1e-5, atol=1e-5)
    import pytest
    with pytest.raises(NotImplementedError):
        flux.AGKernelXNode()
    assert flux.pad_m_to_TPxTile(torch.zeros(5, 3), 2, 4).shape == (8, 3)


def test_ep_dispatch_combine_gloo():
    run_gloo(_ep, 2)
