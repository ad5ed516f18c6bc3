"""The test-support statements against the ops they describe, on CPU ranks."""
import torch
import torch.distributed as dist

from conftest import run_gloo


def _moe_statements(rank, world):
    import tempname_new_b200 as flux
    from tempname_new_b200.testing import (MoeAgScatterWithTorch, MoeMlp1Ctx, calc_gather_index,
                                           calc_scatter_index_stable_sync, matmul_int8,
                                           moe_gather_rs_forward_torch)
    pg = dist.group.WORLD
    ctx = MoeMlp1Ctx(pg, pg, 2, 8 * world, 16, 24, 4 * world, 2, torch.float32, None, weight_groups=2)
    ref = [o.clone() for o in MoeAgScatterWithTorch.forward(ctx, pg)]
    # the fused op on the same tensors
    env = flux.DistEnvTPWithEP(pg, 1, None, ep_size=world)
    args = flux.MoeArguments(ctx.ntokens, ctx.h, ctx.ffn_size, ctx.nexperts, ctx.topk, torch.float32)
    op = flux.GemmGroupedV3AGScatter(env, args)
    outs = op.forward_multiple_weights(ctx.inputs_shard, ctx.weights, ctx.splits_gpu, ctx.scatter_index)
    for o, r in zip(outs, ref):
        torch.testing.assert_close(o[: r.shape[0]], r, rtol=1e-5, atol=1e-5)
    # index helpers agree with the context's routing tensors
    e0 = ctx.nexperts_ep * ctx.ep_rank
    lo = int(ctx.splits_cpu[:e0].sum())
    gi, ti = calc_gather_index(ctx.scatter_index, lo, lo + ctx.nrows_ep)
    assert torch.equal(gi.long(), ctx.gather_index[lo:lo + ctx.nrows_ep])
    assert torch.equal(ti, ctx.topk_index[lo:lo + ctx.nrows_ep])
    assert torch.equal(calc_scatter_index_stable_sync(ctx.choosed_experts, ctx.splits_gpu), ctx.scatter_index)
    # layer 1: statement against the op
    H = ctx.h
    w2 = (torch.randn(ctx.nexperts_ep, H, ctx.ffn_size_shard, generator=torch.Generator().manual_seed(5 + rank)) * 0.1)
    x2 = ref[0]
    gate = torch.rand(ctx.nrows_ep, generator=torch.Generator().manual_seed(9 + rank))
    M = ctx.ntokens * ctx.topk
    want = moe_gather_rs_forward_torch(pg, M, e0, lo, lo + ctx.nrows_ep, x2, w2, ctx.splits_cpu,
                                       ctx.gather_index, ctx.topk_index, ctx.topk, None, None, gate)
    op1 = flux.GemmGroupedV3GatherRS(ctx.nexperts, M, H, ctx.topk, rank, world, 1, world, tp_group=pg,
                                     dtype=torch.float32)
    got = op1.forward_gather_rs(x2, w2, ctx.splits_cpu, ctx.scatter_index.reshape(-1), output_vec_scale=gate)
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-4)
    a = torch.randint(-100, 100, (4, 8), dtype=torch.int8)
    b = torch.randint(-100, 100, (8, 5), dtype=torch.int8)
    assert torch.equal(matmul_int8(a, b), a.int() @ b.int())


def test_moe_statements_match_the_ops_gloo():
    run_gloo(_moe_statements, 2)


def test_perf_model_and_perf_log_helpers(tmp_path, monkeypatch):
    import tempname_new_b200 as flux
    t = flux.testing
    assert t.is_fp8_dtype(torch.float8_e4m3fn) and not t.is_fp8_dtype(torch.int8)
    bf16 = t.get_max_tensorcore_tflops(torch.bfloat16, 1965e3)
    assert abs(bf16 - 148 * 1.965e9 * 8192 / 1e12) < 1e-6
    assert t.get_max_tensorcore_tflops(torch.float8_e4m3fn, 1965e3) == 2 * bf16
    assert t.get_tensorcore_tflops(None, 74, 4, torch.bfloat16) <= bf16
    assert t.get_dram_gbps_by_device_name("NVIDIA B200") == 7700.0
    tc, tr, tw = t.print_gemm_sol_time(8192, 6144, 12288, torch.bfloat16)
    assert tc > tr > tw > 0
    monkeypatch.setenv("FLUXB_PERF_LOG", str(tmp_path / "perf.jsonl"))
    t.log_perf(t.PerfResult("x", total_ms=1.5))
    assert [r["name"] for r in t.query()] == ["x"] and t.query(delete=True) and t.query() == []
    assert not t.should_log_to_rds()
    t.log_perf_rds(t.PerfResult("y"))          # switch is off: nothing happens
    t.set_global_args(op="gemm_rs", M=8192)
    assert t.get_global_args()["M"] == 8192
