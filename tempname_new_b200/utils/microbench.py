"""Single-GPU micro-benchmarks of the library's kernels, usable on their own or under ncu:

    python -m tempname_new_b200.utils.microbench gemm --m 8192 --n 8192 --k 8192 --cta-group 2
    python -m tempname_new_b200.utils.microbench quant --m 8192 --k 8192

Each prints one JSON line with the CUDA-event time (median, L2 flushed between iterations),
achieved TFLOP/s or GB/s and the fraction of the measured peak in ``MEASURED_PEAKS.json``
(fallback 1590 TFLOP/s / 6650 GB/s when that file is absent).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return p["bf16_tflops"], p["hbm_gbs"], "measured"
    except (OSError, KeyError):
        return 1590.0, 6650.0, "fallback"


def timed(fn, iters: int, warmup: int, flush: bool = True):
    dev = torch.device("cuda")
    scratch = torch.empty(256 << 20, dtype=torch.int8, device=dev) if flush else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if scratch is not None:
            scratch.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts) // 2]


def cmd_gemm(a):
    from ..ops import _dense
    dev = torch.device("cuda")
    dt = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp8": torch.float8_e4m3fn}[a.dtype]
    x = torch.randn(a.m, a.k, device=dev).to(dt)
    w = (torch.randn(a.n, a.k, device=dev) * 0.02).to(dt)
    if a.weight_kn:
        w = w.t().contiguous().t()   # [N, K] view of [K, N] memory: read in place as MN-major tiles
    out = torch.empty(a.m, a.n, device=dev, dtype=torch.bfloat16 if dt != torch.float16 else dt)
    if a.impl == "torch":
        fn = lambda: torch.matmul(x, w.t(), out=out)  # noqa: E731
    else:
        fn = lambda: _dense.plain_gemm(x, w, out, tile_n=a.tile_n, group_m=a.group_m,  # noqa: E731
                                       cta_group=a.cta_group, tile_m=a.tile_m)
    ms = timed(fn, a.iters, a.warmup, not a.no_flush)
    tf = 2.0 * a.m * a.n * a.k / ms / 1e9
    pk, _, src = peaks()
    print(json.dumps({"op": "gemm", "impl": a.impl, "m": a.m, "n": a.n, "k": a.k, "dtype": a.dtype,
                      "cta_group": a.cta_group, "tile_n": a.tile_n, "group_m": a.group_m,
                      "weight_kn": bool(a.weight_kn), "ms": ms,
                      "tflops": tf, "frac_of_bf16_peak": tf / pk, "peak": src}))


def cmd_quant(a):
    import tempname_new_b200 as flux
    dev = torch.device("cuda")
    x = torch.randn(a.m, a.k, device=dev).bfloat16()
    q = flux.Quantization(torch.bfloat16, torch.float8_e4m3fn)
    fn = (lambda: q.quantize_vector_blockwise(x, a.transpose)) if a.kind == "1x128" else \
        (lambda: q.quantize_square_blockwise(x, a.transpose))
    ms = timed(fn, a.iters, a.warmup, not a.no_flush)
    nbytes = a.m * a.k * (2 + 1 + (1 if a.transpose else 0))
    gbs = nbytes / ms / 1e6
    _, pk, src = peaks()
    print(json.dumps({"op": "quant_" + a.kind, "m": a.m, "k": a.k, "transpose": a.transpose, "ms": ms,
                      "gbs": gbs, "frac_of_hbm_peak": gbs / pk, "peak": src}))


def cmd_blockscale(a):
    import tempname_new_b200 as flux
    dev = torch.device("cuda")
    x = torch.randn(a.m, a.k, device=dev).bfloat16()
    w = (torch.randn(a.n, a.k, device=dev) * 0.05).bfloat16()
    qz = flux.Quantization(torch.bfloat16, torch.float8_e4m3fn)
    xq, sx, _, _ = qz.quantize_vector_blockwise(x, False)
    wq, sw, _, _ = qz.quantize_square_blockwise(w, False)
    op = flux.BlockScaleGemm()
    out = torch.empty(a.m, a.n, device=dev, dtype=torch.bfloat16)
    ms = timed(lambda: op.forward(xq, wq, output=out, input_scale=sx, weight_scale=sw), a.iters, a.warmup,
               not a.no_flush)
    tf = 2.0 * a.m * a.n * a.k / ms / 1e9
    pk, _, src = peaks()
    rec = {"op": "blockscale_gemm", "m": a.m, "n": a.n, "k": a.k, "ms": ms, "tflops": tf,
           "frac_of_bf16_peak": tf / pk, "peak": src}
    if a.phases:
        # phase clocks of the promotion (self-checking build only: FLUXB_DEBUG=1), cycles per k-block, median
        # over the CTAs: timeline slots 8 / 9 / 10 = promotion warp 4 waiting for MMAs / reading TMEM / in all,
        # 11 = its k-blocks, 12 / 13 = the MMA issuer waiting for a free TMEM buffer / for operands
        from ..ops import _dense
        with _dense.KernelTimeline(dev) as tl:
            op.forward(xq, wq, output=out, input_scale=sx, weight_scale=sw)
            torch.cuda.synchronize()
            t = tl.buf.cpu()
        t = t[t[:, 11] > 0].double()
        if t.numel() == 0:
            rec["phases"] = "no phase clocks: load the self-checking build (FLUXB_DEBUG=1)"
        else:
            kb = t[:, 11]
            rec["phases"] = {name: round(float((t[:, col] / kb).median()), 1) for name, col in
                             (("promotion_waits_for_mma", 8), ("promotion_reads_tmem", 9), ("promotion_all", 10),
                              ("issuer_waits_for_tmem", 12), ("issuer_waits_for_operands", 13))}
    print(json.dumps(rec))


def cmd_grouped(a):
    """Per-expert GEMM over `rows` expert-sorted rows, contiguous or gathered from a token matrix."""
    import os
    import torch.distributed as dist
    import tempname_new_b200 as flux
    dev = torch.device("cuda", torch.cuda.current_device())
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29561")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    E, topk = a.experts, a.topk
    tokens = a.rows // topk
    g = flux.testing.gen_moe_gating_args(E, topk, tokens, device=dev, seed=1)
    dt = torch.float8_e4m3fn if a.dtype == "fp8" else torch.bfloat16
    w = (torch.randn(E, a.n, a.k, device=dev) * (0.5 if a.dtype == "fp8" else 0.02)).to(dt)
    out = torch.empty(a.rows, a.n, device=dev, dtype=torch.bfloat16)
    if a.gathered:
        if a.dtype == "fp8":
            raise SystemExit("--gathered is measured on bf16 tokens")
        x = torch.randn(tokens, a.k, device=dev).bfloat16()
        env = flux.DistEnvTPWithEP(dist.group.WORLD, 1, None, ep_size=1)
        op = flux.GemmGroupedV3AGScatter(env, flux.MoeArguments(tokens, a.k, a.n, E, topk, torch.bfloat16))
        fn = lambda: op.forward(x, w, g.splits_gpu, g.scatter_index, outputs_buf=out)  # noqa: E731
    else:
        x = torch.randn(a.rows, a.k, device=dev).to(dt)
        op = flux.GemmGroupedV3(w, E)
        fn = lambda: op.forward(x, g.splits_gpu)  # noqa: E731
    ms = timed(fn, a.iters, a.warmup, not a.no_flush)
    tf = 2.0 * a.rows * a.n * a.k / ms / 1e9
    pk, _, src = peaks()
    print(json.dumps({"op": "grouped_gemm", "dtype": a.dtype, "gathered": bool(a.gathered), "rows": a.rows, "n": a.n,
                      "k": a.k,
                      "experts": E, "ms": ms, "tflops": tf, "frac_of_bf16_peak": tf / pk, "peak": src}))


def _single_rank_group():
    import os
    import torch.distributed as dist
    dev = torch.device("cuda", torch.cuda.current_device())
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29561")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    return dist.group.WORLD, dev


def cmd_ulysses(a):
    """World-size-1 run of the Ulysses kernels: the GEMM plus the layout change done by the
    epilogue (pre) or by the communication warps feeding the K loop (post)."""
    import tempname_new_b200 as flux
    pg, dev = _single_rank_group()
    hidden = a.heads * a.head_dim
    if a.which == "pre":
        op = flux.GemmAllToAllTranspose(pg, 1, 1, 1, a.seq, hidden, a.head_dim, hidden, torch.bfloat16)
        x = torch.randn(1, a.seq, hidden, device=dev).bfloat16()
        w = (torch.randn(hidden, hidden, device=dev) * 0.02).bfloat16()
        fn = lambda: op.forward(x, w)  # noqa: E731
    else:
        op = flux.AllToAllTransposeGemm(pg, 1, 1, 1, a.heads, a.seq, a.head_dim, torch.bfloat16)
        x = torch.randn(1, a.heads, a.seq, a.head_dim, device=dev).bfloat16()
        w = (torch.randn(hidden, hidden, device=dev) * 0.02).bfloat16()
        fn = lambda: op.forward(x, w)  # noqa: E731
    ms = timed(fn, a.iters, a.warmup, not a.no_flush)
    tf = 2.0 * a.seq * hidden * hidden / ms / 1e9
    pk, _, src = peaks()
    print(json.dumps({"op": "ulysses_" + a.which, "seq": a.seq, "heads": a.heads, "head_dim": a.head_dim, "ms": ms,
                      "tflops": tf, "frac_of_bf16_peak": tf / pk, "peak": src}))


def cmd_combine(a):
    """World-size-1 run of the MoE top-k combine kernel (grouped GEMM excluded)."""
    import tempname_new_b200 as flux
    pg, dev = _single_rank_group()
    E, topk, H = a.experts, a.topk, a.hidden
    g = flux.testing.gen_moe_gating_args(E, topk, a.tokens, device=dev, seed=1)
    op = flux.DisScatterBackward(E, a.tokens, H, topk, 0, 1, 1, 1, pg=pg)
    rows = torch.randn(a.tokens * topk, H, device=dev).bfloat16()
    fn = lambda: op.forward_gpu(rows, None, g.scatter_index, g.splits_gpu)  # noqa: E731
    ms = timed(fn, a.iters, a.warmup, not a.no_flush)
    nbytes = a.tokens * H * 2 * (topk + 1 + 1 + 1)   # rows read, partial written, partial read, output written
    _, pk, src = peaks()
    print(json.dumps({"op": "moe_combine", "tokens": a.tokens, "topk": topk, "hidden": H, "ms": ms,
                      "gbs": nbytes / ms / 1e6, "frac_of_hbm_peak": nbytes / ms / 1e6 / pk, "peak": src}))


def cmd_moe_l1(a):
    """World-size-1 run of MoE layer 1 with the combine fused in: grouped GEMM whose epilogue sends the
    gate-weighted rows to their [token][k] slots, and the top-k sum in the tail of the same kernel."""
    import tempname_new_b200 as flux
    pg, dev = _single_rank_group()
    E, topk, H, ffn = a.experts, a.topk, a.hidden, a.ffn
    g = flux.testing.gen_moe_gating_args(E, topk, a.tokens, device=dev, seed=1)
    rows = a.tokens * topk
    act = (torch.randn(rows, ffn, device=dev) * 0.5).bfloat16()
    w2 = (torch.randn(E, H, ffn, device=dev) * 0.02).bfloat16()
    gate_rows = g.gate_weight.reshape(-1)[torch.argsort(g.choosed_experts.reshape(-1), stable=True)].contiguous()
    op = flux.GemmGroupedV3GatherRS(E, rows, H, topk, 0, 1, 1, 1, tp_group=pg)
    fn = lambda: op.forward_gather_rs(act, w2, g.splits_gpu, g.scatter_index.reshape(-1),  # noqa: E731
                                      output_vec_scale=gate_rows)
    ms = timed(fn, a.iters, a.warmup, not a.no_flush)
    op.check_status()
    tf = 2.0 * rows * H * ffn / ms / 1e9
    pk, _, src = peaks()
    print(json.dumps({"op": "moe_layer1_fused", "tokens": a.tokens, "topk": topk, "experts": E, "hidden": H,
                      "ffn": ffn, "ms": ms, "tflops": tf, "frac_of_bf16_peak": tf / pk, "peak": src}))


def cmd_small(a):
    """In-place cast, routing-index build and row all-gather (world size 1) in one go."""
    import tempname_new_b200 as flux
    pg, dev = _single_rank_group()
    _, pk, src = peaks()
    n = a.elems
    t = torch.rand(n, device=dev)
    op = flux.InplaceCast(n, dev)
    ms = timed(lambda: op.from_fp32_to_bf16(t), a.iters, a.warmup, not a.no_flush)
    print(json.dumps({"op": "inplace_cast", "elems": n, "ms": ms, "gbs": n * 6 / ms / 1e6,
                      "frac_of_hbm_peak": n * 6 / ms / 1e6 / pk, "peak": src}))
    ce = torch.randint(0, 64, (65536, 8), device=dev, dtype=torch.int32)
    ms = timed(lambda: flux.moe_index_build(ce, 64), a.iters, a.warmup, not a.no_flush)
    print(json.dumps({"op": "moe_index_build", "entries": ce.numel(), "experts": 64, "ms": ms}))
    ag = flux.AllGatherOp(pg, 1, 16384, 4096, torch.bfloat16)
    x = torch.randn(16384, 4096, device=dev).bfloat16()
    ms = timed(lambda: ag.run(x), a.iters, a.warmup, not a.no_flush)
    print(json.dumps({"op": "a2a_rows(all-gather, W=1)", "bytes": x.numel() * 2, "ms": ms,
                      "gbs": x.numel() * 4 / ms / 1e6, "frac_of_hbm_peak": x.numel() * 4 / ms / 1e6 / pk, "peak": src}))


def main(argv=None):
    ap = argparse.ArgumentParser(prog="microbench")
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=8192)
    g.add_argument("--n", type=int, default=8192)
    g.add_argument("--k", type=int, default=8192)
    g.add_argument("--dtype", default="bf16", choices=["bf16", "fp16", "fp8"])
    g.add_argument("--impl", default="fluxb", choices=["fluxb", "torch"])
    g.add_argument("--cta-group", type=int, default=0)
    g.add_argument("--tile-n", type=int, default=0)
    g.add_argument("--tile-m", type=int, default=0)
    g.add_argument("--weight-kn", action="store_true", help="hold the weight as [K, N] (read in place)")
    m1 = sub.add_parser("moe_l1")
    m1.add_argument("--tokens", type=int, default=8192)
    m1.add_argument("--topk", type=int, default=8)
    m1.add_argument("--experts", type=int, default=8)
    m1.add_argument("--hidden", type=int, default=4096)
    m1.add_argument("--ffn", type=int, default=1536)
    m1.set_defaults(fn=cmd_moe_l1)
    g.add_argument("--group-m", type=int, default=0)
    g.set_defaults(fn=cmd_gemm)
    q = sub.add_parser("quant")
    q.add_argument("--m", type=int, default=8192)
    q.add_argument("--k", type=int, default=8192)
    q.add_argument("--kind", default="1x128", choices=["1x128", "128x128"])
    q.add_argument("--transpose", action="store_true")
    q.set_defaults(fn=cmd_quant)
    b = sub.add_parser("blockscale")
    b.add_argument("--m", type=int, default=8192)
    b.add_argument("--n", type=int, default=8192)
    b.add_argument("--k", type=int, default=8192)
    b.add_argument("--phases", action="store_true", help="print the promotion phase clocks (FLUXB_DEBUG=1)")
    b.set_defaults(fn=cmd_blockscale)
    gg = sub.add_parser("grouped")
    gg.add_argument("--rows", type=int, default=65536)
    gg.add_argument("--n", type=int, default=3072)
    gg.add_argument("--k", type=int, default=4096)
    gg.add_argument("--experts", type=int, default=8)
    gg.add_argument("--topk", type=int, default=8)
    gg.add_argument("--gathered", action="store_true")
    gg.add_argument("--dtype", default="bf16", choices=["bf16", "fp8"])
    gg.set_defaults(fn=cmd_grouped)
    u = sub.add_parser("ulysses")
    u.add_argument("--which", default="pre", choices=["pre", "post"])
    u.add_argument("--seq", type=int, default=4096)
    u.add_argument("--heads", type=int, default=32)
    u.add_argument("--head-dim", type=int, default=128)
    u.set_defaults(fn=cmd_ulysses)
    c = sub.add_parser("combine")
    c.add_argument("--tokens", type=int, default=8192)
    c.add_argument("--topk", type=int, default=8)
    c.add_argument("--experts", type=int, default=64)
    c.add_argument("--hidden", type=int, default=4096)
    c.set_defaults(fn=cmd_combine)
    sm = sub.add_parser("small")
    sm.add_argument("--elems", type=int, default=1 << 26)
    sm.set_defaults(fn=cmd_small)
    for p in (g, q, b, gg, u, c, sm, m1):
        p.add_argument("--iters", type=int, default=10)
        p.add_argument("--warmup", type=int, default=3)
        p.add_argument("--no-flush", action="store_true")
    a = ap.parse_args(argv)
    try:
        a.fn(a)
    finally:
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized():
            torch.cuda.synchronize()
            dist.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main())
