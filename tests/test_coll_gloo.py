"""Stand-alone collectives on CPU ranks."""
import torch
import torch.distributed as dist

from conftest import run_gloo


def _coll(rank, world):
    import tempname_new_b200 as flux
    ag = flux.AllGatherOp(dist.group.WORLD, 1, 4 * world, 8, torch.float32)
    x = torch.full((4, 8), float(rank))
    full = ag.run(x)
    for r in range(world):
        assert float(full[4 * r, 0]) == r
    assert ag.local_input_scale_buffer() is None
    ag.run(x, input_scale=torch.arange(4, dtype=torch.float32).reshape(4, 1) + 10.0 * rank)   # int8 convention
    sc = ag.local_input_scale_buffer()
    assert sc.shape == (4 * world, 1)
    assert sc.reshape(-1).tolist() == [10.0 * r + i for r in range(world) for i in range(4)]
    a2a = flux.All2AllSingle(dist.group.WORLD, 16, 4, world, torch.float32)
    ins = torch.tensor([rank + 1 + d for d in range(world)])       # rows for each destination
    inp = torch.cat([torch.full((int(n), 4), 10.0 * rank + d) for d, n in enumerate(ins.tolist())])
    outs = torch.zeros(world, dtype=torch.int64)
    res = a2a.forward(inp, None, ins, outs)
    assert outs.tolist() == [s + 1 + rank for s in range(world)]
    row = 0
    for s in range(world):
        n = s + 1 + rank
        assert bool((res[row:row + n] == 10.0 * s + rank).all())
        row += n
    sr = flux.AsyncSendRecv(4, 4, rank, world, torch.float32, duplicate=3)
    sr.get_comm_buffer(0).fill_(float(rank + 1))
    dist.barrier()
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    sr.read_comm_buffer(nxt, 1, 0)            # local[1] <- next rank's buffer 0
    assert float(sr.get_comm_buffer(1)[0, 0]) == float(nxt + 1)
    sr.write_comm_buffer(nxt, 0, 2)           # next rank's buffer 2 <- local[0]
    sr.set_signal(nxt, 1, 7)
    sr.wait_signal_eq(1, 7)
    assert float(sr.get_comm_buffer(2)[0, 0]) == float(prv + 1)


def test_collectives_gloo():
    run_gloo(_coll, 2)
