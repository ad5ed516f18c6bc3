"""Shared MoE test logic: build a routed problem, run layer 0 -> SwiGLU-free activation -> layer 1
through the ops and compare with a dense single-process statement of the same layer."""
import torch
import torch.distributed as dist


def routed_problem(tokens, topk, E, seed=0, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    scores = torch.rand(tokens, E, generator=g)
    gate, experts = scores.topk(topk, dim=1)
    gate = (gate / gate.sum(1, keepdim=True)).float()
    flat = experts.reshape(-1)
    order = torch.argsort(flat, stable=True)
    scatter = torch.empty_like(order)
    scatter[order] = torch.arange(order.numel())
    splits = torch.bincount(flat, minlength=E)
    return (experts.to(device), gate.to(device), scatter.view(tokens, topk).to(torch.int32).to(device),
            splits.to(torch.int32).to(device), order.to(device))


def run_moe_layer(rank, world, ep_size, dtype, device, tpr=16, H=32, ffn=48, E=4, topk=2, tol=1e-4):
    import tempname_new_b200 as flux
    tokens = tpr * world
    experts, gate, scatter, splits, order = routed_problem(tokens, topk, E, seed=3, device=device)
    g = torch.Generator().manual_seed(7)
    x_full = (torch.randn(tokens, H, generator=g) * 0.5).to(dtype).to(device)
    w1_full = (torch.randn(E, ffn, H, generator=g) * 0.2).to(dtype).to(device)
    w2_full = (torch.randn(E, H, ffn, generator=g) * 0.2).to(dtype).to(device)
    pg = dist.group.WORLD
    env = flux.DistEnvTPWithEP(pg, 1, None, ep_size=ep_size)
    tp = world // ep_size
    E_loc = E // ep_size
    e0 = env.ep_rank * E_loc
    fs = ffn // tp
    w1 = w1_full[e0:e0 + E_loc, env.ffn_tp_rank * fs:(env.ffn_tp_rank + 1) * fs].contiguous()
    w2 = w2_full[e0:e0 + E_loc, :, env.ffn_tp_rank * fs:(env.ffn_tp_rank + 1) * fs].contiguous()
    args = flux.MoeArguments(tokens, H, ffn, E, topk, dtype)
    op0 = flux.GemmGroupedV3AGScatter(env, args)
    op1 = flux.GemmGroupedV3GatherRS(E, tokens * topk, H, topk, rank, world, tp, ep_size, tp_group=pg, dtype=dtype)
    x = x_full[rank * tpr:(rank + 1) * tpr].contiguous()
    # gate weight of every sorted row
    row_gate = gate.reshape(-1)[order]
    offs = torch.cat([torch.zeros(1, dtype=torch.long, device=splits.device), splits.long().cumsum(0)])
    lo, hi = int(offs[e0]), int(offs[e0 + E_loc])
    for it in range(2):
        gathered = torch.empty(tokens, H, dtype=dtype, device=device)
        h = op0.forward(x, w1, splits, scatter, allgather_output=gathered)
        assert torch.equal(gathered, x_full)
        assert h.shape == (hi - lo, fs)
        act = torch.nn.functional.silu(h.float()).to(dtype)
        out = op1.forward_gather_rs(act, w2, splits.cpu(), scatter.reshape(-1), output_vec_scale=row_gate[lo:hi])
        # dense statement over all tokens and all experts
        ref = torch.zeros(tokens, H, dtype=torch.float32, device=device)
        for e in range(E):
            for k in range(topk):
                sel = experts[:, k] == e
                if sel.any():
                    hh = torch.nn.functional.silu(x_full[sel].float() @ w1_full[e].float().t())
                    if dtype != torch.float32:      # the ops round the activations to 16 bits
                        hh = hh.to(dtype).float()
                    ref[sel] += gate[sel, k, None] * (hh @ w2_full[e].float().t())
        mine = ref[rank * tpr:(rank + 1) * tpr]
        err = (out.float() - mine).abs().max().item()
        assert err <= tol * max(1.0, mine.abs().max().item()), (err, it)
    op0.check_status()
    op1.check_status()
