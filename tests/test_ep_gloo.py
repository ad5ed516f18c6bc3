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
    # the same combine through the stand-alone op, gate weights given as the per-row scale
    tr = flux.TopkReduceScatterOp(dist.group.WORLD, tokens * topk, H, topk, torch.float32, E, world)
    out2 = tr.run([rows], None, rank * E_loc, E_loc, splits, scatter, [w])
    torch.testing.assert_close(out2, ref, rtol=1e-5, atol=1e-5)
    seg = flux.get_gemm_rs_threadblock_segments_info((64 * world, 32), (16, 16), rank, world)
    assert [s.segment_origin for s in seg] == [(rank + 1 + i) % world for i in range(world)]
    assert seg[-1].segment_origin == rank and seg[0].tile_m_start_new == 0 and seg[0].size == 4
    table = torch.zeros(world, 4, dtype=torch.int32)
    assert flux.calc_gemm_rs_threadblock_segments_info(table, (64 * world, 32), (16, 16), rank, world) == world
    assert table[:, 3].tolist() == [4 * i for i in range(world)]
    # routing choices of all ranks, gathered rank after rank (ranks may hold different token counts)
    counts = torch.tensor([3 + r for r in range(world)], dtype=torch.int32)
    mine_i = torch.full((3 + rank, topk), rank, dtype=torch.int32)
    mine_v = torch.full((3 + rank, topk), float(rank) + 0.5)
    all_i = torch.empty(int(counts.sum()), topk, dtype=torch.int32)
    all_v = torch.empty(int(counts.sum()), topk)
    fwd.pre_comm_index(counts, mine_i, mine_v, all_i, all_v, 0)
    exp = torch.cat([torch.full((3 + r, topk), r, dtype=torch.int32) for r in range(world)])
    assert torch.equal(all_i, exp) and torch.equal(all_v, exp.float() + 0.5)
    mine = flux.create_tensor((2, 3), torch.float32)
    assert mine.shape == (2, 3) and len(flux.flux_create_shm_tensor_list((2, 3), torch.float32)) == world
    import pytest
    with pytest.raises(NotImplementedError):
        flux.AGKernelXNode()
    assert flux.pad_m_to_TPxTile(torch.zeros(5, 3), 2, 4).shape == (8, 3)


def test_ep_dispatch_combine_gloo():
    run_gloo(_ep, 2)
