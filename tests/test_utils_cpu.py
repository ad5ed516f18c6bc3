"""CPU checks of the host-side pieces: utilities, routing helpers, tuning table, roofline model."""
import pytest
import torch


def test_torch_allclose_reports_offenders():
    import tempname_new_b200 as flux
    flux.torch_allclose(torch.ones(4, 4), torch.ones(4, 4) + 1e-6, 1e-3, 1e-3)
    y = torch.ones(4, 4)
    y[2, 3] = 5.0
    with pytest.raises(AssertionError) as e:
        flux.torch_allclose(torch.ones(4, 4), y, 1e-3, 1e-3)
    assert "(2, 3)" in str(e.value) and "1 of 16" in str(e.value)


def test_moe_routing_helpers_agree_with_device_free_index_build():
    from tempname_new_b200.ops.misc import calc_scatter_index, moe_index_build
    from tempname_new_b200.testing import gen_moe_gating_args, is_gather_index_stable
    a = gen_moe_gating_args(16, 4, 200, device="cpu", seed=5)
    assert int(a.splits_cpu.sum()) == 800
    splits, offsets, scatter, gather, tki = moe_index_build(a.choosed_experts, 16)
    assert torch.equal(splits, a.splits_gpu)
    assert torch.equal(scatter, a.scatter_index)
    assert torch.equal(gather, a.gather_index) and torch.equal(tki, a.topk_index)
    assert is_gather_index_stable(gather, splits)
    assert torch.equal(calc_scatter_index(a.choosed_experts, a.splits_gpu), a.scatter_index)
    rr = gen_moe_gating_args(8, 2, 64, device="cpu", round_robin=True)
    assert rr.splits_cpu.tolist() == [16] * 8


def test_tuning_table_and_profiling_context(tmp_path, monkeypatch):
    from tempname_new_b200.tuning import table
    from tempname_new_b200.tuning.profiling import ProfilingContext, TuningRecord
    k = table.lookup(8192, 6144, 12288)
    assert k == {"cta_group": 2, "tile_n": 256, "tile_m": 512, "group_m": 8}
    assert table.lookup(8192, 12288, 49152)["group_m"] == 4          # measured entries differ by shape
    cands = table.candidates(8192, 6144, 12288)
    assert {c["tile_m"] for c in cands} == {512, 256, 128} and all("group_m" in c for c in cands)
    assert all(c["tile_m"] != 512 for c in table.candidates(8192, 6144, 12288, segmented_rows=256))
    h = table.lookup(333, 264, 72)
    assert h["cta_group"] == 1 and h["tile_n"] in (128, 256)
    assert table.heuristic(8192, 4096, 32768) == {"cta_group": 2, "tile_n": 256, "group_m": 8}
    f = tmp_path / "extra.json"
    f.write_text('[{"key": [1, 2, 3], "best": {"cta_group": 1, "tile_n": 128, "group_m": 4}}]')
    monkeypatch.setenv("FLUXB_TUNE_FILE", str(f))
    table._EXTRA = None
    assert table.lookup(1, 2, 3)["group_m"] == 4
    table._EXTRA = None
    ctx = ProfilingContext("t")
    ctx.add(TuningRecord("gemm_only", {"m": 1}, {"tile_n": 128}, 0.5))
    assert "gemm_only" in ctx.get_latest_prof_result() and '"tile_n": 128' in ctx.get_code()
    assert len(ctx.get_all_records()) == 1


def test_perf_model_roofline_terms():
    from tempname_new_b200.testing import (estimate_fused_sol_time_ms, estimate_gemm_sol_time_ms, get_nvlink_gbps,
                                           get_tflops, roofline_fraction)
    t = estimate_gemm_sol_time_ms(8192, 12288, 6144)
    assert 0.5 < t < 1.2                                  # ~0.72-0.78 ms at 1.6-1.7 PFLOP/s
    flops = 2.0 * 8192 * 12288 * 6144
    comm = 7 / 8 * 8192 * 12288 * 2
    sol = estimate_fused_sol_time_ms(flops, comm)
    assert sol == pytest.approx(max(flops / (get_tflops() * 1e9), comm / (get_nvlink_gbps() * 1e6)))
    assert roofline_fraction(2 * sol, flops, comm) == pytest.approx(0.5)
    assert get_tflops(torch.float8_e4m3fn) == pytest.approx(2 * get_tflops(torch.bfloat16))


def test_options_and_env_records():
    import tempname_new_b200 as flux
    o = flux.ReduceScatterOption()
    o.use_1d_ring, o.ring_mode = True, flux.RingMode.Ring1D
    assert flux.get_default_rs_ring_mode() == flux.RingMode.All2All
    assert flux.AllGatherOption().mode is None and flux.AllToAllOption().skip_barrier is None
    m = flux.MoeArguments(1024, 256, 512, 8, 2, torch.bfloat16)
    assert m.output_dtype == torch.bfloat16
    with flux.with_torch_deterministic(True):
        assert torch.are_deterministic_algorithms_enabled()


def test_cpu_fallbacks_of_small_ops():
    import tempname_new_b200 as flux
    a = torch.randn(10, 7)
    assert flux.bitwise_check(a, a.clone()) and not flux.bitwise_check(a, a + 1)
    t = torch.empty(1000)
    flux.uniform_initialize(t, 3, -1.0, 1.0)
    assert -1.0 <= float(t.min()) and float(t.max()) < 1.0
    g = flux.GemmOnly(torch.float32, output_dtype=torch.float32)
    x, w = torch.randn(5, 8), torch.randn(6, 8)
    torch.testing.assert_close(g.forward(x, w), x @ w.t())
    out = flux.GemmGroupedV3(torch.randn(2, 4, 8), 2).forward(torch.randn(5, 8), torch.tensor([2, 3]))
    assert out.shape == (5, 4)


def test_topology_probe_with_fake_nvml():
    from tempname_new_b200.parallel import topo

    class FakeNvml:
        def __init__(self, links, switch):
            self.links, self.switch = links, switch

        def nvmlInit(self): pass
        def nvmlShutdown(self): pass
        def nvmlDeviceGetCount(self): return len(self.links)
        def nvmlDeviceGetHandleByIndex(self, i): return i
        def nvmlDeviceGetName(self, h): return b"NVIDIA B200"
        def nvmlDeviceGetNvLinkState(self, h, link): return 1 if link < self.links[h] else 0
        def nvmlDeviceGetNvLinkRemoteDeviceType(self, h, link): return 2 if self.switch else 0
        def nvmlDeviceGetCurrPcieLinkGeneration(self, h): return 5

        def nvmlDeviceGetPciInfo(self, h):
            class P:
                busId = b"00000000:1B:00.0"
            return P()

    t = topo.probe(FakeNvml([18] * 8, True))
    assert t.num_gpus == 8 and t.has_nvlink and t.has_nvswitch and not t.has_heterogeneous_nvlink
    assert t.numa_local_world_size == 8 and t.pcie_gen == [5] * 8
    t = topo.probe(FakeNvml([18, 12, 0, 18], False))
    assert not t.has_nvlink and not t.has_nvswitch and t.has_heterogeneous_nvlink


def test_kernel_timeline_summary_from_stamps():
    """summary() turns raw per-CTA stamps into microseconds since the first CTA started."""
    import torch
    from tempname_new_b200.ops._dense import KernelTimeline, TRACE_SLOTS
    tl = KernelTimeline(device="cpu", ctas=4)
    base = 1_000_000
    for cta in range(3):                      # CTA 3 never ran: all zero
        tl.buf[cta, 0] = base + 100 * cta     # entry
        tl.buf[cta, 3] = base + 5_000 + cta   # first tile loads
        tl.buf[cta, 6] = base + 9_000         # end
        tl.buf[cta, 7] = 2_000 * (cta + 1)    # a duration, not a stamp
    s = tl.summary()
    assert s["entry_us"] == {"min": 0.0, "median": 0.1, "max": 0.2}
    assert s["first_tile_loads_us"]["min"] == 5.0
    assert s["epilogue_done_us"]["max"] == 9.0
    assert s["flag_wait_total_us"] == {"median": 4.0, "max": 6.0}
    assert "handshake_us" not in s and len(TRACE_SLOTS) == 16
    assert KernelTimeline(device="cpu", ctas=2).summary() == {}


def test_tuning_override_pins_knobs_inside_block():
    from tempname_new_b200.tuning.table import lookup, override
    key = (8192, 6144, 12288)
    before = lookup(*key)
    with override(key, {"cta_group": 1, "tile_n": 128, "group_m": 16}):
        assert lookup(*key) == {"cta_group": 1, "tile_n": 128, "group_m": 16}
        with override(key, {"cta_group": 2, "tile_n": 256, "group_m": 2}):
            assert lookup(*key)["group_m"] == 2
        assert lookup(*key)["tile_n"] == 128
    assert lookup(*key) == before


def test_blocked_moe_index_helpers():
    """calc_moe_triton_blocked_gather_a / prepare_moe_ag_scatter_args against a loop statement."""
    import sys, os
    import torch
    import tempname_new_b200 as flux
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from moe_common import routed_problem
    tokens, topk, E, W, tile = 48, 2, 8, 4, 8
    experts, gate, scatter, splits, order = routed_problem(tokens, topk, E, seed=5)
    ep_start, ep_n = 2, 4
    PAD = 2 ** 31 - 1
    sp = splits[ep_start:ep_start + ep_n].tolist()
    n_tiles = sum(-(-s // tile) for s in sp)
    ga = torch.empty(n_tiles * tile, dtype=torch.int32)
    ei = torch.empty(n_tiles, dtype=torch.int32)
    flux.calc_moe_triton_blocked_gather_a(splits, ep_start, ep_n, tile, ga, ei)
    exp_rows, exp_e, m = [], [], 0
    for e, s in enumerate(sp):
        t = -(-s // tile)
        exp_e += [e] * t
        exp_rows += [m + i if i < s else PAD for i in range(t * tile)]
        m += s
    assert ga.tolist() == exp_rows and ei.tolist() == exp_e
    M, M_pad, gA, sD, eidx, r0, r1 = flux.prepare_moe_ag_scatter_args(
        splits, scatter, tokens, topk, 1, ep_start, ep_n, 0, W, tile)
    assert M == sum(sp) and int(M_pad) == n_tiles * tile and eidx.tolist() == exp_e
    base = int(splits[:ep_start].sum())
    token_of_row = (order // topk).tolist()            # sorted row -> token
    tpr = tokens // W
    for pos, row in enumerate(exp_rows):
        if row == PAD:
            assert gA[pos] == PAD and sD[pos] == PAD
        else:
            assert gA[pos] == token_of_row[base + row] and sD[pos] == row
    for t in range(n_tiles):
        srcs = [token_of_row[base + r] // tpr for r in exp_rows[t * tile:(t + 1) * tile] if r != PAD]
        assert r0[t] == min(srcs) and r1[t] == max(srcs)
    # several weight groups repeat the per-group tensors
    out2 = flux.prepare_moe_ag_scatter_args(splits, scatter, tokens, topk, 2, ep_start, ep_n, 0, W, tile)
    assert out2[2].numel() == 2 * gA.numel() and out2[4].tolist() == exp_e * 2


def test_grouped_gemm_v2_constructor_and_scales():
    import torch
    import tempname_new_b200 as flux
    w = torch.randn(3, 4, 8)
    x = torch.randn(10, 8)
    sp = torch.tensor([3, 5, 2])
    op = flux.GemmGroupedV2(w, 3, torch.float32, torch.float32)
    y = op.forward(x, sp, input_scale=torch.tensor([2.0]), weight_scale=torch.tensor([1.0, 0.5, 3.0]))
    ref = torch.cat([x[:3] @ w[0].t() * 2, x[3:8] @ w[1].t(), x[8:] @ w[2].t() * 6])
    torch.testing.assert_close(y, ref, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(flux.GemmGroupedV3(w, 3).forward(x, sp), torch.cat(
        [x[:3] @ w[0].t(), x[3:8] @ w[1].t(), x[8:] @ w[2].t()]), rtol=1e-5, atol=1e-5)
    import pytest
    with pytest.raises(TypeError):
        flux.GemmGroupedV2(w, 3, torch.bfloat16)


def test_tune_file_and_load_tuning_record(tmp_path, monkeypatch):
    import json
    import tempname_new_b200 as flux
    from tempname_new_b200.tuning import table
    f = tmp_path / "tune.json"
    f.write_text(json.dumps([{"key": [1234, 512, 256], "best": {"cta_group": 1, "tile_n": 128, "group_m": 4}}]))
    monkeypatch.setenv("FLUXB_TUNE_FILE", str(f))
    monkeypatch.setattr(table, "_EXTRA", None)
    assert table.lookup(1234, 512, 256) == {"cta_group": 1, "tile_n": 128, "group_m": 4}
    flux.load_tuning_record({"key": [77, 256, 128], "best": {"cta_group": 2, "tile_n": 256, "group_m": 2}})
    assert table.lookup(77, 256, 128)["group_m"] == 2
    monkeypatch.setattr(table, "_EXTRA", None)


def test_source_hygiene_of_the_tree():
    """The formatter / content check that the pre-commit hook runs passes on the tree itself, and
    it does find what it is meant to find."""
    from pathlib import Path
    from tempname_new_b200.utils import hygiene
    assert hygiene.main(["--check"]) == 0
    bad = hygiene.check_text(Path("x.py"), "a = 1 \n\tb = 2\n# see DESIGN" + ".md\nlast")
    kinds = {what for _, what in bad}
    assert {"trailing whitespace", "tab character", "no newline at end of file"} <= kinds
    assert any("outside the source tree" in k for k in kinds)
    assert hygiene.fix_text("a = 1  \n\n\n") == "a = 1\n"


def test_weight_layout_helper_and_per_expert_block_scaled_cpu_path():
    """``as_nk`` hands the kernels [N, K]: a [K, N] weight is a free transposed view when it can be read
    in place (16-bit, CUDA, aligned) and a re-laid-out copy otherwise; the per-expert block-scaled forms
    fall back to the PyTorch statement, expert by expert, on CPU tensors."""
    import torch
    import tempname_new_b200 as flux
    from tempname_new_b200.ops import _dense
    from tempname_new_b200.ops.gemm_only import as_nk
    w_kn = torch.randn(64, 48).bfloat16()                      # [K, N]
    v = as_nk(w_kn, True)
    assert v.shape == (48, 64) and v.stride(-1) == 1           # CPU: copied into the K-major layout
    assert torch.equal(v, w_kn.t())
    assert as_nk(v, False) is v                                # already [N, K] with contiguous K
    # the in-place rule itself: N contiguous, N and pitch multiples of 8, 16-byte aligned, 16-bit
    assert _dense.kn_in_place(torch.empty(64, 48, dtype=torch.bfloat16).t())
    assert not _dense.kn_in_place(torch.empty(64, 44, dtype=torch.bfloat16).t())          # N % 8
    assert not _dense.kn_in_place(torch.empty(64, 48, dtype=torch.float8_e4m3fn).t())     # 8-bit
    assert not _dense.kn_in_place(torch.empty(64, 48, dtype=torch.bfloat16))              # K contiguous already
    # block-scaled per-expert forms on CPU tensors
    E, N, K = 2, 128, 256
    x = torch.randn(256, K)
    w = torch.randn(E * N, K) * 0.1
    qz = flux.Quantization(torch.float32, torch.float8_e4m3fn)
    xq, sx, _, _ = qz.quantize_vector_blockwise(x, False)
    wq, sw, _, _ = qz.quantize_square_blockwise(w, False)
    op = flux.BlockScaleGemm(num_streams=3)
    out = op.forward_multi_stream(xq, [128, 128], wq.view(E, N, K), input_scale=sx, weight_scale=sw.view(E, 1, K // 128))
    for e in range(E):
        ref = flux.blockscale_gemm_torch(xq[e * 128:(e + 1) * 128], wq.view(E, N, K)[e], sx[e:e + 1],
                                         sw.view(E, 1, K // 128)[e], torch.float32)
        assert (out[e * 128:(e + 1) * 128].float() - ref).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item())
