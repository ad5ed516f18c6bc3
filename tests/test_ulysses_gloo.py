"""Ulysses projections on CPU ranks: the op layouts against an index-by-index statement."""
import torch
import torch.distributed as dist

from conftest import run_gloo


def _gather_full(t, world):
    parts = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(parts, t.contiguous())
    return parts


def _pre_attn(rank, world):
    import tempname_new_b200 as flux
    bs, seq, hidden, hd, nh = 2, 8 * world, 32, 8, 4 * world
    ls = seq // world
    torch.manual_seed(0)
    x_full = torch.randn(bs, seq, hidden)
    w = torch.randn(nh * hd, hidden) * 0.2
    x = x_full[:, rank * ls:(rank + 1) * ls].contiguous()
    op = flux.GemmAllToAllTranspose(dist.group.WORLD, 1, world, bs, seq, hidden, hd, nh * hd, torch.float32)
    (out,) = op.forward(x, w)
    y = (x_full @ w.t()).reshape(bs, seq, nh, hd)                       # full projection
    lh = nh // world
    ref = y[:, :, rank * lh:(rank + 1) * lh].permute(0, 2, 1, 3)        # [bs, lh, seq, hd]
    torch.testing.assert_close(out, ref, rtol=1e-5, atol=1e-5)
    # q/k/v packing with grouped-query attention: per rank 2 q heads + 1 k + 1 v
    op2 = flux.GemmAllToAllTranspose(dist.group.WORLD, 1, world, bs, seq, hidden, hd, nh * hd, torch.float32,
                                     gqa=2, comm_op=flux.PreAttnAllToAllCommOp.QKVPackA2A)
    q, k, v = op2.forward(x, w)
    lq, lk = 2, 1
    yq, yk, yv = y[:, :, :lq * world], y[:, :, lq * world:(lq + lk) * world], y[:, :, (lq + lk) * world:]
    torch.testing.assert_close(q, yq[:, :, rank * lq:(rank + 1) * lq], rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(k, yk[:, :, rank * lk:(rank + 1) * lk], rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(v, yv[:, :, rank * lk:(rank + 1) * lk], rtol=1e-5, atol=1e-5)


def _post_attn(rank, world):
    import tempname_new_b200 as flux
    bs, seq, hd, nh, N = 2, 8 * world, 8, 2 * world, 24
    ls, lh = seq // world, nh // world
    torch.manual_seed(1)
    attn_full = torch.randn(bs, nh, seq, hd)                            # all heads, full sequence
    w = torch.randn(N, nh * hd) * 0.2
    mine = attn_full[:, rank * lh:(rank + 1) * lh].contiguous()         # [bs, lh, seq, hd]
    ref_in = attn_full.permute(0, 2, 1, 3).reshape(bs, seq, nh * hd)[:, rank * ls:(rank + 1) * ls]
    ref = ref_in @ w.t()
    for a2a_only in (False, True):
        op = flux.AllToAllTransposeGemm(dist.group.WORLD, 1, world, bs, nh, seq, hd, torch.float32,
                                        a2a_only=a2a_only)
        inp = mine.permute(0, 2, 1, 3).contiguous() if a2a_only else mine
        gi = torch.empty(bs, ls, nh * hd)
        out = op.forward(inp, w, a2a_transpose_output=gi)
        torch.testing.assert_close(gi, ref_in, rtol=0, atol=0)
        torch.testing.assert_close(out, ref, rtol=1e-5, atol=1e-5)


def test_pre_attn_gemm_a2a_gloo():
    run_gloo(_pre_attn, 2)


def test_post_attn_a2a_gemm_gloo():
    run_gloo(_post_attn, 2)


def _varlen(rank, world):
    """Ranks with different sequence lengths (``seq_lens_cpu``): q/k/v packing before attention and
    the out-projection after it, against index-by-index statements over the concatenated sequence."""
    import tempname_new_b200 as flux
    bs, hidden, hd, nh, N = 2, 32, 8, 4 * world, 24
    lens = [5 + 3 * r for r in range(world)]
    offs = [sum(lens[:r]) for r in range(world)]
    total = sum(lens)
    seq_lens_cpu = torch.tensor(lens, dtype=torch.int32)
    torch.manual_seed(2)
    x_full = torch.randn(bs, total, hidden)
    w = torch.randn(nh * hd, hidden) * 0.2
    x = x_full[:, offs[rank]:offs[rank] + lens[rank]].contiguous()
    op = flux.GemmAllToAllTranspose(dist.group.WORLD, 1, world, bs, 8 * world, hidden, hd, nh * hd, torch.float32,
                                    gqa=2, comm_op=flux.PreAttnAllToAllCommOp.QKVPackA2A)
    q, k, v = op.forward(x, w, seq_lens_cpu=seq_lens_cpu)
    y = (x_full @ w.t()).reshape(bs, total, nh, hd)
    lq, lk = 2, 1
    yq, yk, yv = y[:, :, :lq * world], y[:, :, lq * world:(lq + lk) * world], y[:, :, (lq + lk) * world:]
    torch.testing.assert_close(q, yq[:, :, rank * lq:(rank + 1) * lq], rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(k, yk[:, :, rank * lk:(rank + 1) * lk], rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(v, yv[:, :, rank * lk:(rank + 1) * lk], rtol=1e-5, atol=1e-5)
    # post-attention
    nh2 = 2 * world
    lh = nh2 // world
    attn_full = torch.randn(bs, nh2, total, hd)
    wo = torch.randn(N, nh2 * hd) * 0.2
    mine = attn_full[:, rank * lh:(rank + 1) * lh].contiguous()
    ref_in = attn_full.permute(0, 2, 1, 3).reshape(bs, total, nh2 * hd)[:, offs[rank]:offs[rank] + lens[rank]]
    ref = ref_in @ wo.t()
    for a2a_only in (False, True):
        op2 = flux.AllToAllTransposeGemm(dist.group.WORLD, 1, world, bs, nh2, 8 * world, hd, torch.float32,
                                         a2a_only=a2a_only)
        inp = mine.permute(0, 2, 1, 3).contiguous() if a2a_only else mine
        out = op2.forward(inp, wo, seq_lens_cpu=seq_lens_cpu)
        torch.testing.assert_close(out, ref, rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(op2.post_attn_a2a(inp, seq_lens_cpu=seq_lens_cpu), ref_in, rtol=0, atol=0)


def test_per_rank_sequence_lengths_gloo():
    run_gloo(_varlen, 2)


def _sp_subgroups(rank, world):
    """sp_size smaller than the group: two independent sequence-parallel blocks of two ranks each."""
    import tempname_new_b200 as flux
    sp = 2
    block, r = rank // sp, rank % sp
    bs, seq, hidden, hd, nh = 1, 8 * sp, 16, 8, 2 * sp
    ls, lh = seq // sp, nh // sp
    torch.manual_seed(100 + block)                                      # each block has its own data
    x_full = torch.randn(bs, seq, hidden)
    w = torch.randn(nh * hd, hidden) * 0.2
    op = flux.GemmAllToAllTranspose(dist.group.WORLD, 1, sp, bs, seq, hidden, hd, nh * hd, torch.float32)
    assert op.world == sp and op.rank == r
    (out,) = op.forward(x_full[:, r * ls:(r + 1) * ls].contiguous(), w)
    y = (x_full @ w.t()).reshape(bs, seq, nh, hd)
    torch.testing.assert_close(out, y[:, :, r * lh:(r + 1) * lh].permute(0, 2, 1, 3), rtol=1e-5, atol=1e-5)
    attn_full = torch.randn(bs, nh, seq, hd)
    wo = torch.randn(24, nh * hd) * 0.2
    op2 = flux.AllToAllTransposeGemm(dist.group.WORLD, 1, sp, bs, nh, seq, hd, torch.float32)
    out2 = op2.forward(attn_full[:, r * lh:(r + 1) * lh].contiguous(), wo)
    ref_in = attn_full.permute(0, 2, 1, 3).reshape(bs, seq, nh * hd)[:, r * ls:(r + 1) * ls]
    torch.testing.assert_close(out2, ref_in @ wo.t(), rtol=1e-5, atol=1e-5)


def test_sp_size_smaller_than_the_group_gloo():
    run_gloo(_sp_subgroups, 4)
