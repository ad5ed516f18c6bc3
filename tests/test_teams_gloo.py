"""Team handles (the ``_nvshmem_team_*`` calling convention over torch process groups) on CPU ranks."""
import torch
import torch.distributed as dist

from conftest import run_gloo


def _teams(rank, world):
    import tempname_new_b200 as flux
    assert flux._nvshmem_team_npes(flux.TEAM_WORLD) == world
    assert flux._nvshmem_team_my_pe(flux.TEAM_WORLD) == rank
    xt, yt = flux._nvshmem_team_split_2d(flux.TEAM_WORLD, 2)            # 2 x 2 grid of the 4 ranks
    assert flux._nvshmem_team_npes(xt) == 2 and flux._nvshmem_team_npes(yt) == 2
    assert flux._nvshmem_team_my_pe(xt) == rank % 2 and flux._nvshmem_team_my_pe(yt) == rank // 2
    cfg = flux._nvshmem_team_get_config(yt)
    assert (cfg.start, cfg.stride, cfg.size) == (rank % 2, 2, 2)
    # my row neighbour, seen from the world and from my column team
    nb = flux._nvshmem_team_translate_pe(xt, 1 - rank % 2, flux.TEAM_WORLD)
    assert nb == (rank // 2) * 2 + (1 - rank % 2)
    assert flux._nvshmem_team_translate_pe(xt, 1 - rank % 2, yt) == -1  # not in my column
    assert flux._nvshmem_team_translate_pe(flux.TEAM_WORLD, rank, yt) == rank // 2
    # the team's process group carries collectives (and therefore the ops of the library)
    t = torch.tensor([float(rank)])
    dist.all_reduce(t, group=flux.team_group(xt))
    assert t.item() == float((rank // 2) * 4 + 1)
    odd = flux._nvshmem_team_split_strided(flux.TEAM_WORLD, 1, 2, 2)    # ranks 1 and 3
    assert (odd == flux.TEAM_INVALID) == (rank % 2 == 0)
    if odd != flux.TEAM_INVALID:
        assert flux._nvshmem_team_my_pe(odd) == rank // 2
        op = flux.GemmRS(flux.team_group(odd), 1, 8, 4, torch.float32)
        a, w = torch.ones(8, 3) * (rank + 1), torch.ones(4, 3)
        out = op.forward(a, w)
        assert torch.allclose(out, torch.full((4, 4), 3.0 * (2 + 4)))
    # node-level groups of a tensor-parallel group laid over two "nodes" of two ranks
    intra = flux.get_intra_node_pg_group(dist.group.WORLD, 2)
    inter = flux.get_inter_node_ag_group(dist.group.WORLD, 2)
    assert dist.get_world_size(intra) == 2 and dist.get_world_size(inter) == 2
    t = torch.tensor([float(rank)])
    dist.all_reduce(t, group=intra)
    assert t.item() == float((rank // 2) * 4 + 1)
    t = torch.tensor([float(rank)])
    dist.all_reduce(t, group=inter)
    assert t.item() == float(2 * (rank % 2) + 2)
    flux.initialize_inter_node_rs_group(dist.group.WORLD, 2)
    assert flux.get_inter_node_rs_group() is inter
    import pytest
    with pytest.raises(NotImplementedError):
        flux.GemmRSTaco()
    dist.barrier()
    flux._nvshmem_team_destroy(odd)
    flux._nvshmem_team_destroy(xt)
    flux._nvshmem_team_destroy(yt)


def test_team_handles_gloo():
    run_gloo(_teams, 4)
