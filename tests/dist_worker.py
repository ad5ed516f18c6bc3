"""Multi-GPU checks of the fused ops, run as one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node W --master-addr 127.0.0.1 \
        --master-port P tests/dist_worker.py [dense] [blockscale] [ulysses] [moe] [--perf]

Every op is compared with a PyTorch fp32 statement built from NCCL collectives. With ``--perf``
the headline shapes are also timed against torch.matmul + NCCL (CUDA events, max over ranks).
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import tempname_new_b200 as flux  # noqa: E402

rank = int(os.environ["RANK"])
W = int(os.environ["WORLD_SIZE"])
lr = int(os.environ.get("LOCAL_RANK", rank))
torch.cuda.set_device(lr)
dev = torch.device("cuda", lr)
dist.init_process_group("nccl", device_id=dev)
pg = dist.group.WORLD
flux.init_flux_shm(pg)
torch.manual_seed(1234 + rank)
what = [a for a in sys.argv[1:] if not a.startswith("--")] or ["dense", "blockscale", "ulysses", "moe", "coll"]
perf = "--perf" in sys.argv


def p0(*a):
    if rank == 0:
        print(*a, flush=True)


SUSTAIN_S = float(next((a.split("=")[1] for a in sys.argv if a.startswith("--sustain=")), "0"))


def timeit(fn, iters=10, warm=3):
    """Mean time of ``iters`` back-to-back calls, maximum over ranks. With ``--sustain=S`` every
    measurement runs for about S seconds instead (the same count on every rank), so that the power
    cap, not the boost clock of a short burst, sets the clock of all the numbers being compared."""
    for _ in range(warm):
        fn()
    if SUSTAIN_S > 0:
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(3):
            fn()
        e.record()
        torch.cuda.synchronize()
        n = torch.tensor([SUSTAIN_S * 3e3 / max(s.elapsed_time(e), 1e-3)], device=dev)
        dist.all_reduce(n, op=dist.ReduceOp.MIN)
        iters = max(iters, int(n.item()))
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def close(out, ref, what_, tol=2e-2):
    err = (out.float() - ref.float()).abs().max().item()
    lim = tol * max(1.0, ref.float().abs().max().item())
    assert err <= lim, f"[rank {rank}] {what_}: max err {err} > {lim}"
    return err


# ------------------------------------------------------------------------------------------
def check_dense():
    # (the 1024-row segments run as 512-row CTA-pair tiles with a split last wave; the last shape gives
    # every CTA pair several tiles, remote ones followed by tiles of the own segment)
    for (M, Nn, K) in [(256 * W, 256, 64 * W), (512 * W, 768, 512 * W), (200 * W, 264, 72 * W),
                       (1024 * W, 1280, 256 * W), (4096 * W, 4096, 128 * W)]:
        Kl = K // W
        a = (torch.randn(M, Kl, device=dev) * 0.5).bfloat16()
        w = (torch.randn(Nn, Kl, device=dev) * 0.05).bfloat16()
        op = flux.GemmRS(pg, 1, M, Nn, torch.bfloat16)
        ref32 = torch.empty(M // W, Nn, device=dev)
        dist.reduce_scatter_tensor(ref32, a.float() @ w.float().t())
        for _ in range(2):
            close(op.forward(a, w), ref32, f"GemmRS {M}x{Nn}x{K}")
        op.check_status()
        seg = M // W
        a = (torch.randn(seg, K, device=dev) * 0.5).bfloat16()
        w = (torch.randn(Nn, K, device=dev) * 0.05).bfloat16()
        op = flux.AGKernel(pg, 1, M, Nn, K, torch.bfloat16)
        full = torch.empty(M, K, device=dev, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(full, a)
        gi = torch.empty_like(full)
        for _ in range(2):
            close(op.forward(a, w, gathered_input=gi), full.float() @ w.float().t(), f"AGKernel {M}x{Nn}x{K}")
            assert torch.equal(gi, full)
        op.check_status()
    # signed 8-bit operands (s32 accumulation), dequantised by two per-tensor scales
    M, Nn, K = 256 * W, 512, 256 * W
    g = torch.Generator(device="cpu").manual_seed(7 + rank)
    a8 = torch.randint(-127, 128, (M, K // W), generator=g, dtype=torch.int8).to(dev)
    w8 = torch.randint(-127, 128, (Nn, K // W), generator=g, dtype=torch.int8).to(dev)
    sa, sb = torch.tensor([0.02], device=dev), torch.tensor([0.01], device=dev)
    op = flux.GemmRS(pg, 1, M, Nn, torch.int8, output_dtype=torch.bfloat16)
    part = (a8.float() @ w8.float().t()) * 2e-4          # exact in fp32: |sum| < 2^24
    ref32 = torch.empty(M // W, Nn, device=dev)
    dist.reduce_scatter_tensor(ref32, part.bfloat16().float())
    close(op.forward(a8, w8, input_scale=sa, weight_scale=sb), ref32, "GemmRS int8")
    op.check_status()
    a8 = torch.randint(-127, 128, (M // W, K), generator=g, dtype=torch.int8).to(dev)
    w8 = torch.randint(-127, 128, (Nn, K), generator=g, dtype=torch.int8).to(dev)
    op = flux.AGKernel(pg, 1, M, Nn, K, torch.int8, output_dtype=torch.bfloat16)
    full8 = torch.empty(M, K, device=dev, dtype=torch.int8)
    dist.all_gather_into_tensor(full8, a8)
    close(op.forward(a8, w8, input_scale=sa, weight_scale=sb), (full8.float() @ w8.float().t()) * 2e-4,
          "AGKernel int8")
    # one scale per input row (this rank's [M/W, 1]) and per output column ([1, N]), fp16 output with bias
    sa_r = torch.rand(M // W, 1, device=dev) * 0.02 + 0.001
    sb_c = torch.rand(1, Nn, device=dev) * 0.02 + 0.001
    dist.broadcast(sb_c, 0)
    sa_all = torch.empty(M, 1, device=dev)
    dist.all_gather_into_tensor(sa_all, sa_r)
    close(op.forward(a8, w8, input_scale=sa_r, weight_scale=sb_c), (full8.float() @ w8.float().t()) * sa_all * sb_c,
          "AGKernel int8, per-row x per-column scales", tol=1e-2)
    op.check_status()
    # 16-bit extras on more than one rank: fp16, bias, weights given as [K, N]
    Mh, Nh, Kh = 512 * W, 512, 256 * W
    ah = (torch.randn(Mh // W, Kh, device=dev) * 0.5).half()
    wh = (torch.randn(Nh, Kh, device=dev) * 0.05).half()
    bh = torch.randn(1, Nh, device=dev).half()
    oph = flux.AGKernel(pg, 1, Mh, Nh, Kh, torch.float16)
    fullh = torch.empty(Mh, Kh, device=dev, dtype=torch.float16)
    dist.all_gather_into_tensor(fullh, ah)
    close(oph.forward(ah, wh.t().contiguous(), bias=bh, transpose_weight=True),
          fullh.float() @ wh.float().t() + bh.float(), "AGKernel fp16 + bias + transpose_weight", tol=1e-2)
    oph.check_status()
    ar = (torch.randn(Mh, Kh // W, device=dev) * 0.5).half()
    wr = (torch.randn(Nh, Kh // W, device=dev) * 0.05).half()
    br = torch.randn(Mh, Nh, device=dev).half()          # [M, N] bias: added on every rank, as in the reference
    opr = flux.GemmRS(pg, 1, Mh, Nh, torch.float16, transpose_weight=True)
    refh = torch.empty(Mh // W, Nh, device=dev)
    dist.reduce_scatter_tensor(refh, (ar.float() @ wr.float().t() + br.float()).half().float())
    close(opr.forward(ar, wr.t().contiguous(), bias=br), refh, "GemmRS fp16 + bias + transpose_weight", tol=1e-2)
    opr.check_status()
    gb = flux.GroupBarrier(pg)
    for _ in range(3):
        gb.barrier_all()
    torch.cuda.synchronize()
    gb.check()
    p0(f"dense ok (W={W})")
    if perf:
        M, N, K = 8192, 12288, 49152
        a = (torch.randn(M, K // W, device=dev) * 0.5).bfloat16()
        w = (torch.randn(N, K // W, device=dev) * 0.02).bfloat16()
        op = flux.GemmRS(pg, 1, M, N, torch.bfloat16)
        ref = torch.empty(M // W, N, device=dev, dtype=torch.bfloat16)

        def torch_rs():
            dist.reduce_scatter_tensor(ref, torch.matmul(a, w.t()))
        t_f, t_t, t_g = timeit(lambda: op.forward(a, w)), timeit(torch_rs), timeit(lambda: torch.matmul(a, w.t()))
        t_p = timeit(lambda: flux.GemmOnly(torch.bfloat16, torch.bfloat16).forward(a, w))
        p0(f"GEMM-RS M={M} N={N} K={K} W={W}: fluxb {t_f:.3f} ms | torch+nccl {t_t:.3f} ms | matmul {t_g:.3f} ms"
           f" | fluxb plain GEMM {t_p:.3f} ms")
        if "--timeline" in sys.argv:
            with flux.KernelTimeline(dev) as tl:   # the last of twelve back-to-back calls: steady state
                dist.barrier(pg)
                for _ in range(12):
                    op.forward(a, w)
                torch.cuda.synchronize()
            p0(f"GEMM-RS timeline (us; slice0 = first own tile reached, slice1 / slice2 = reduce tail entered / left): "
               f"{tl.summary()}")
        op.check_status()
        M, N, K = 8192, 49152, 12288
        a = (torch.randn(M // W, K, device=dev) * 0.5).bfloat16()
        w = (torch.randn(N // W, K, device=dev) * 0.02).bfloat16()
        op = flux.AGKernel(pg, 1, M, N // W, K, torch.bfloat16)
        full = torch.empty(M, K, device=dev, dtype=torch.bfloat16)
        out = torch.empty(M, N // W, device=dev, dtype=torch.bfloat16)

        def torch_ag():
            dist.all_gather_into_tensor(full, a)
            torch.matmul(full, w.t(), out=out)
        t_f, t_t = timeit(lambda: op.forward(a, w, output=out)), timeit(torch_ag)
        t_g = timeit(lambda: torch.matmul(full, w.t(), out=out))
        t_p = timeit(lambda: flux.GemmOnly(torch.bfloat16, torch.bfloat16).forward(full, w, output_buf=out))
        p0(f"AG-GEMM M={M} N={N} K={K} W={W}: fluxb {t_f:.3f} ms | torch+nccl {t_t:.3f} ms | matmul {t_g:.3f} ms"
           f" | fluxb plain GEMM {t_p:.3f} ms")
        if "--timeline" in sys.argv:
            with flux.KernelTimeline(dev) as tl:   # the last of twelve back-to-back calls: steady state
                dist.barrier(pg)
                for _ in range(12):
                    op.forward(a, w, output=out)
                torch.cuda.synchronize()
            p0(f"AG-GEMM timeline (us): {tl.summary()}")
        op.check_status()


# ------------------------------------------------------------------------------------------
def check_blockscale():
    qz = flux.Quantization(torch.bfloat16, torch.float8_e4m3fn)
    shapes = [(256 * W, 256, 256)] + ([(16384, 28672 // W, 8192)] if perf else [(1024 * W, 512, 1024)])
    for (M, Nl, K) in shapes:          # AG + GEMM: M sharded, N local
        seg = M // W
        x = torch.randn(seg, K, device=dev).bfloat16() * (1 + rank)
        w = (torch.randn(Nl, K, device=dev) * 0.05).bfloat16()
        xq, sx, _, _ = qz.quantize_vector_blockwise(x, False)
        wq, sw, _, _ = qz.quantize_square_blockwise(w, False)
        op = flux.AGKernel(pg, 1, M, Nl, K, torch.float8_e4m3fn, torch.bfloat16)
        full_q = torch.empty(M, K, device=dev, dtype=torch.uint8)
        dist.all_gather_into_tensor(full_q, xq.view(torch.uint8))
        full_s = torch.empty(M // 128, K // 128, 128, device=dev)
        dist.all_gather_into_tensor(full_s, sx)
        ref = flux.blockscale_gemm_torch(full_q.view(torch.float8_e4m3fn)[:2048], wq, full_s[:16], sw, torch.float32)
        for _ in range(2):
            out = op.forward(xq, wq, input_scale=sx, weight_scale=sw)
            close(out[:2048], ref, f"blockscale AG {M}x{Nl}x{K}")
        op.check_status()
        if perf and M >= 8192:
            t = timeit(lambda: op.forward(xq, wq, input_scale=sx, weight_scale=sw))
            p0(f"fp8 block-scaled AG-GEMM M={M} N={Nl * W} K={K} W={W}: {t:.3f} ms "
               f"({2.0 * M * Nl * K / t / 1e9:.0f} TFLOPS/GPU)")
    shapes = [(256 * W, 256, 128 * W)] + ([(16384, 8192, 28672)] if perf else [(512 * W, 512, 256 * W)])
    for (M, N, K) in shapes:           # GEMM + RS: K sharded
        Kl = (K // W) // 128 * 128
        x = torch.randn(M, Kl, device=dev).bfloat16()
        w = (torch.randn(N, Kl, device=dev) * 0.05).bfloat16()
        xq, sx, _, _ = qz.quantize_vector_blockwise(x, False)
        wq, sw, _, _ = qz.quantize_square_blockwise(w, False)
        op = flux.GemmRS(pg, 1, M, N, torch.float8_e4m3fn, torch.bfloat16)
        part = flux.blockscale_gemm_torch(xq[: 256 * W], wq, sx[: 2 * W], sw, torch.float32) if M > 256 * W else \
            flux.blockscale_gemm_torch(xq, wq, sx, sw, torch.float32)
        rows = part.shape[0] // W
        # reduce-scatter of the first rows only needs matching row ranges per rank: use all_reduce
        dist.all_reduce(part)
        for _ in range(2):
            out = op.forward(xq, wq, input_scale=sx, weight_scale=sw)
            seg = M // W
            lo = rank * seg
            if lo < part.shape[0]:
                n = min(seg, part.shape[0] - lo)
                close(out[:n], part[lo:lo + n], f"blockscale RS {M}x{N}x{K}")
        op.check_status()
        if perf and M >= 8192:
            t = timeit(lambda: op.forward(xq, wq, input_scale=sx, weight_scale=sw))
            p0(f"fp8 block-scaled GEMM-RS M={M} N={N} K={Kl * W} W={W}: {t:.3f} ms "
               f"({2.0 * M * N * Kl / t / 1e9:.0f} TFLOPS/GPU)")
    p0(f"blockscale ok (W={W})")


# ------------------------------------------------------------------------------------------
def check_ulysses():
    from tempname_new_b200.ops.ulysses import (post_attn_a2a_torch, pre_attn_a2a_torch,
                                               pre_attn_qkv_pack_a2a_torch)
    cfgs = [(1, 64 * W, 256, 64, 2 * W), (2, 128 * W, 512, 128, 4 * W)]
    if perf:
        cfgs.append((1, 4096 * W, 4096, 128, 32))
    for (bs, seq, hidden, hd, nh) in cfgs:
        ls = seq // W
        x = (torch.randn(bs, ls, hidden, device=dev) * 0.5).bfloat16()
        w = (torch.randn(nh * hd, hidden, device=dev) * 0.05).bfloat16()
        y = (x.reshape(-1, hidden).float() @ w.float().t()).bfloat16()
        op = flux.GemmAllToAllTranspose(pg, 1, W, bs, seq, hidden, hd, nh * hd, torch.bfloat16)
        ref = pre_attn_a2a_torch(y, pg, bs, ls, nh, hd)[0]
        for _ in range(2):
            (out,) = op.forward(x, w)
            close(out, ref, f"gemm_a2a_transpose bs{bs} seq{seq}")
        op.check_status()
        if (nh // W) % 4 == 0:
            op2 = flux.GemmAllToAllTranspose(pg, 1, W, bs, seq, hidden, hd, nh * hd, torch.bfloat16, gqa=2,
                                             comm_op=flux.PreAttnAllToAllCommOp.QKVPackA2A)
            refs = pre_attn_qkv_pack_a2a_torch(y, pg, bs, ls, nh, hd, 2)
            for o, r, n in zip(op2.forward(x, w), refs, "qkv"):
                close(o, r, f"qkv_pack {n} bs{bs} seq{seq}")
            op2.check_status()
        # post-attention
        N = hidden
        attn = (torch.randn(bs, nh // W, seq, hd, device=dev) * 0.5).bfloat16()
        wo = (torch.randn(N, nh * hd, device=dev) * 0.05).bfloat16()
        for a2a_only in (False, True):
            inp = attn.permute(0, 2, 1, 3).contiguous() if a2a_only else attn
            gi_ref = post_attn_a2a_torch(inp, pg, a2a_only)
            ref = gi_ref.reshape(-1, nh * hd).float() @ wo.float().t()
            op3 = flux.AllToAllTransposeGemm(pg, 1, W, bs, nh, seq, hd, torch.bfloat16, a2a_only=a2a_only)
            gi = torch.empty_like(gi_ref)
            for _ in range(2):
                out = op3.forward(inp, wo, a2a_transpose_output=gi)
                assert torch.equal(gi, gi_ref), f"[rank {rank}] a2a_transpose_gemm gathered input differs"
                close(out.reshape(-1, N), ref, f"a2a_transpose_gemm bs{bs} seq{seq} a2a_only={a2a_only}")
            for _ in range(2):   # own slice read in place from the attention output
                out = op3.forward(inp, wo)
                close(out.reshape(-1, N), ref, f"a2a_transpose_gemm (in place) bs{bs} seq{seq} a2a_only={a2a_only}")
            # the exchange alone, on the strided-exchange kernel
            for _ in range(2):
                assert torch.equal(op3.post_attn_a2a(inp), gi_ref), f"[rank {rank}] post_attn_a2a differs"
            op3.check_status()
        # stand-alone seq -> heads exchanges against the collective statement
        ref_pre = pre_attn_a2a_torch(y, pg, bs, ls, nh, hd)[0]
        for _ in range(2):
            assert torch.equal(op.pre_attn_a2a(y.reshape(bs, ls, nh, hd)), ref_pre), "pre_attn_a2a differs"
        if (nh // W) % 4 == 0:
            for o, r in zip(op2.pre_attn_qkv_pack_a2a(y.reshape(bs, ls, nh, hd)), refs):
                assert torch.equal(o, r), "pre_attn_qkv_pack_a2a differs"
            op2.check_status()
        op.check_status()
        if perf and seq >= 8192:
            full_flops = 2.0 * bs * ls * hidden * nh * hd
            t_f = timeit(lambda: op.forward(x, w))

            def torch_pre():
                yy = torch.matmul(x.reshape(-1, hidden), w.t())
                pre_attn_a2a_torch(yy, pg, bs, ls, nh, hd)
            t_t = timeit(torch_pre)
            p0(f"gemm_a2a_transpose seq={seq} W={W}: fluxb {t_f:.3f} ms ({full_flops / t_f / 1e9:.0f} TF/GPU) | "
               f"torch+nccl {t_t:.3f} ms")
            op3 = flux.AllToAllTransposeGemm(pg, 1, W, bs, nh, seq, hd, torch.bfloat16)
            t_f = timeit(lambda: op3.forward(attn, wo))

            def torch_post():
                g = post_attn_a2a_torch(attn, pg, False)
                torch.matmul(g.reshape(-1, nh * hd), wo.t())
            t_t = timeit(torch_post)
            p0(f"a2a_transpose_gemm seq={seq} W={W}: fluxb {t_f:.3f} ms | torch+nccl {t_t:.3f} ms")
            if "--timeline" in sys.argv:
                with flux.KernelTimeline(dev) as tl:
                    dist.barrier(pg)
                    op3.forward(attn, wo)
                    torch.cuda.synchronize()
                p0(f"a2a_transpose_gemm timeline (us): {tl.summary()}")
    # ---- per-rank sequence lengths: projection kernel + strided exchange, exchange + projection
    from tempname_new_b200.ops.ulysses import post_attn_a2a_varlen_torch, pre_attn_a2a_varlen_torch
    bs, hidden, hd, nh = 2, 256, 64, 4 * W
    lens = [32 + 16 * r for r in range(W)]
    seq_cap = sum(lens) + 64
    seq_cap += (-seq_cap) % W
    lens_cpu = torch.tensor(lens, dtype=torch.int32)
    x = (torch.randn(bs, lens[rank], hidden, device=dev) * 0.5).bfloat16()
    w = (torch.randn(nh * hd, hidden, device=dev) * 0.05).bfloat16()
    y = (x.reshape(-1, hidden).float() @ w.float().t()).bfloat16().reshape(bs, lens[rank], nh, hd)
    opv = flux.GemmAllToAllTranspose(pg, 1, W, bs, seq_cap, hidden, hd, nh * hd, torch.bfloat16, gqa=2,
                                     comm_op=flux.PreAttnAllToAllCommOp.QKVPackA2A)
    lq, lk = 2, 1
    parts = (y[:, :, :lq * W], y[:, :, lq * W:(lq + lk) * W], y[:, :, (lq + lk) * W:])
    refs = [pre_attn_a2a_varlen_torch(t.contiguous(), pg, lens) for t in parts]
    for _ in range(2):
        for o, r, n in zip(opv.forward(x, w, seq_lens_cpu=lens_cpu), refs, "qkv"):
            close(o, r, f"varlen qkv_pack {n}")
    opv.check_status()
    attn = (torch.randn(bs, nh // W, sum(lens), hd, device=dev) * 0.5).bfloat16()
    wo = (torch.randn(hidden, nh * hd, device=dev) * 0.05).bfloat16()
    for a2a_only in (False, True):
        inp = attn.permute(0, 2, 1, 3).contiguous() if a2a_only else attn
        gi_ref = post_attn_a2a_varlen_torch(inp, pg, a2a_only, lens)
        opw = flux.AllToAllTransposeGemm(pg, 1, W, bs, nh, seq_cap, hd, torch.bfloat16, a2a_only=a2a_only)
        for _ in range(2):
            assert torch.equal(opw.post_attn_a2a(inp, seq_lens_cpu=lens_cpu), gi_ref), "varlen post_attn_a2a differs"
            out = opw.forward(inp, wo, seq_lens_cpu=lens_cpu)
            close(out.reshape(-1, hidden), gi_ref.reshape(-1, nh * hd).float() @ wo.float().t(),
                  f"varlen a2a_transpose_gemm a2a_only={a2a_only}")
        opw.check_status()
    p0(f"ulysses ok (W={W})")


def check_coll():
    ag = flux.AllGatherOp(pg, 1, 1024 * W, 512, torch.bfloat16)
    x = torch.randn(1024, 512, device=dev).bfloat16()
    ref = torch.empty(1024 * W, 512, device=dev, dtype=torch.bfloat16)
    dist.all_gather_into_tensor(ref, x)
    for _ in range(2):
        assert torch.equal(ag.run(x), ref)
    ag.check_status()
    # per-row scales of an int8 shard ride along (rows not a multiple of four: padded rows of 16 bytes)
    xs = torch.randint(-100, 100, (1022, 512), device=dev, dtype=torch.int8)
    ss = torch.rand(1022, 1, device=dev) + rank
    ag8 = flux.AllGatherOp(pg, 1, 1024 * W, 512, torch.int8)
    got = ag8.run(xs, input_scale=ss)
    ref8 = torch.empty(1022 * W, 512, device=dev, dtype=torch.int8)
    dist.all_gather_into_tensor(ref8, xs)
    refs = torch.empty(1022 * W, 1, device=dev)
    dist.all_gather_into_tensor(refs, ss)
    assert torch.equal(got, ref8) and torch.equal(ag8.local_input_scale_buffer(), refs)
    ag8.check_status()
    a2a = flux.All2AllSingle(pg, 4096, 256, W, torch.bfloat16)
    ins = torch.tensor([64 * (1 + (rank + d) % 3) for d in range(W)], device=dev, dtype=torch.int32)
    inp = torch.randn(int(ins.sum()), 256, device=dev).bfloat16()
    outs64 = torch.empty(W, dtype=torch.int64, device=dev)
    dist.all_to_all_single(outs64, ins.long())
    ref = torch.empty(int(outs64.sum()), 256, device=dev, dtype=torch.bfloat16)
    dist.all_to_all_single(ref, inp, outs64.tolist(), ins.tolist())
    osp = torch.empty(W, dtype=torch.int32, device=dev)
    for _ in range(2):
        res = a2a.forward(inp, None, ins, osp)
        assert torch.equal(osp.long(), outs64)
        assert torch.equal(res[: ref.shape[0]], ref)
    a2a.check_status()
    sr = flux.AsyncSendRecv(16, 64, rank, W, torch.bfloat16, duplicate=3, pg=pg)
    sr.get_comm_buffer(0).fill_(float(rank + 1))
    torch.cuda.synchronize()
    dist.barrier()
    nxt, prv = (rank + 1) % W, (rank - 1) % W
    sr.write_comm_buffer(nxt, 0, 2)
    sr.set_signal(nxt, 1, 7)
    sr.wait_signal_eq(1, 7)
    torch.cuda.synchronize()
    assert float(sr.get_comm_buffer(2)[0, 0]) == float(prv + 1)
    # expert-parallel dispatch / combine
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from moe_common import routed_problem
    tpr, H, E, topk = 256, 512, 8 * W, 2
    tokens = tpr * W
    experts, gate, scatter, splits, order = routed_problem(tokens, topk, E, seed=2, device=dev)
    x_full = torch.randn(tokens, H, generator=torch.Generator().manual_seed(9)).to(dev).bfloat16()
    fwd = flux.DisScatterForward(E, tokens, H, topk, rank, 1, W, W, pg=pg)
    bwd = flux.DisScatterBackward(E, tokens, H, topk, rank, 1, W, W, pg=pg)
    rows = fwd.forward(x_full[rank * tpr:(rank + 1) * tpr].contiguous(), experts, scatter, splits)
    offs = torch.cat([torch.zeros(1, dtype=torch.long, device=dev), splits.long().cumsum(0)])
    E_loc = E // W
    lo, hi = int(offs[rank * E_loc]), int(offs[(rank + 1) * E_loc])
    assert torch.equal(rows, x_full[(order // topk)[lo:hi]])
    wrow = gate.reshape(-1)[order][lo:hi]
    out = bwd.forward((rows.float() * wrow[:, None]).bfloat16(), experts, scatter, splits)
    close(out, (x_full.float() * gate.sum(1, keepdim=True))[rank * tpr:(rank + 1) * tpr], "ep combine")
    bwd.op.check_status()
    p0(f"coll ok (W={W})")
    if perf:
        rows_, K_ = 1024, 12288          # the activation shard of the TP-MLP step
        agp = flux.AllGatherOp(pg, 1, rows_ * W, K_, torch.bfloat16)
        xs = torch.randn(rows_, K_, device=dev).bfloat16()
        full_ = torch.empty(rows_ * W, K_, device=dev, dtype=torch.bfloat16)
        t_f = timeit(lambda: agp.run(xs))
        t_t = timeit(lambda: dist.all_gather_into_tensor(full_, xs))
        recv = (W - 1) * xs.numel() * 2 / 1e6
        p0(f"AllGatherOp {rows_}x{K_} bf16 per rank, W={W}: fluxb {t_f:.3f} ms ({recv / t_f:.0f} GB/s in per GPU) | "
           f"nccl {t_t:.3f} ms ({recv / t_t:.0f} GB/s)")
        agp.check_status()


def check_moe():
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from moe_common import run_moe_layer
    for ep in sorted({W, 1, max(W // 2, 1)}):
        run_moe_layer(rank, W, ep, torch.bfloat16, dev, tpr=256, H=512, ffn=768 * W // ep // max(W // ep, 1),
                      E=8 * ep if ep > 1 else 8, topk=2, tol=3e-2)
    p0(f"moe ok (W={W})")
    if perf:
        moe_perf()


def moe_perf(E=64, topk=8, H=4096, ffn=1536, tpr=8192):
    """64 experts, top-8, hidden 4096, expert FFN 1536 (gate and up fused into one 3072-wide GEMM),
    8192 tokens per rank, expert parallel over all ranks."""
    from tempname_new_b200.testing import gen_moe_gating_args
    tokens = tpr * W
    g = gen_moe_gating_args(E, topk, tokens, device=dev, seed=1)
    env = flux.DistEnvTPWithEP(pg, 1, None, ep_size=W)
    E_loc, e0 = E // W, rank * (E // W)
    x = (torch.randn(tpr, H, device=dev) * 0.5).bfloat16()
    w1 = (torch.randn(E_loc, 2 * ffn, H, device=dev) * 0.02).bfloat16()
    w2 = (torch.randn(E_loc, H, ffn, device=dev) * 0.02).bfloat16()
    offs = torch.cat([torch.zeros(1, dtype=torch.long), g.splits_cpu.long().cumsum(0)])
    lo, hi = int(offs[e0]), int(offs[e0 + E_loc])
    rows = hi - lo
    op0 = flux.GemmGroupedV3AGScatter(env, flux.MoeArguments(tokens, H, 2 * ffn, E, topk, torch.bfloat16))
    op1 = flux.GemmGroupedV3GatherRS(E, tokens * topk, H, topk, rank, W, 1, W, tp_group=pg)
    h = torch.empty(rows, 2 * ffn, device=dev, dtype=torch.bfloat16)
    act = (torch.randn(rows, ffn, device=dev) * 0.5).bfloat16()
    gate_rows = g.gate_weight.reshape(-1)[torch.argsort(g.choosed_experts.reshape(-1), stable=True)][lo:hi].contiguous()
    t0 = timeit(lambda: op0.forward(x, w1, g.splits_gpu, g.scatter_index, outputs_buf=h), 5, 2)
    t1 = timeit(lambda: op1.forward_gather_rs(act, w2, g.splits_gpu, g.scatter_index.reshape(-1),
                                              output_vec_scale=gate_rows), 5, 2)
    op0.check_status()
    op1.check_status()
    # torch statement of the same layers (all_gather + index_select + per-expert matmul; per-expert
    # matmul + scatter + top-k sum + reduce_scatter)
    full = torch.empty(tokens, H, device=dev, dtype=torch.bfloat16)
    gidx = g.gather_index.long()
    sl = g.splits_cpu.tolist()
    ridx = g.scatter_index.reshape(-1).long()

    def torch_l0():
        dist.all_gather_into_tensor(full, x)
        a = full[gidx[lo:hi]]
        r = 0
        for el in range(E_loc):
            n = sl[e0 + el]
            torch.matmul(a[r:r + n], w1[el].t(), out=h[r:r + n])
            r += n

    yrows = torch.empty(rows, H, device=dev, dtype=torch.bfloat16)
    out = torch.empty(tpr, H, device=dev, dtype=torch.bfloat16)

    def torch_l1():
        r = 0
        for el in range(E_loc):
            n = sl[e0 + el]
            torch.matmul(act[r:r + n], w2[el].t(), out=yrows[r:r + n])
            r += n
        y = yrows * gate_rows[:, None].bfloat16()
        fullrows = torch.zeros(tokens * topk, H, device=dev, dtype=torch.bfloat16)
        fullrows[lo:hi] = y
        red = fullrows[ridx].view(tokens, topk, H).sum(1)
        dist.reduce_scatter_tensor(out, red)
    tt0, tt1 = timeit(torch_l0, 3, 1), timeit(torch_l1, 3, 1)
    f0, f1 = 2.0 * rows * H * 2 * ffn, 2.0 * rows * H * ffn
    p0(f"MoE E={E} top{topk} H={H} ffn={ffn} {tpr} tok/rank EP{W}: layer0 fluxb {t0:.3f} ms ({f0 / t0 / 1e9:.0f} TF/GPU)"
       f" | torch+nccl {tt0:.3f} ms ; layer1 fluxb {t1:.3f} ms ({f1 / t1 / 1e9:.0f} TF/GPU) | torch+nccl {tt1:.3f} ms")


def check_failure():
    """A rank that stops taking part between steps: the others' device waits give up after their
    limit, the status record says where, and the context stays usable. Runs with plain peer
    stores (no multicast objects are in use anywhere in the library)."""
    M, N, K = 256 * W, 256, 128 * W
    a = (torch.randn(M, K // W, device=dev) * 0.5).bfloat16()
    w = (torch.randn(N, K // W, device=dev) * 0.05).bfloat16()
    op = flux.GemmRS(pg, 1, M, N, torch.bfloat16, timeout_s=1.0)
    ref32 = torch.empty(M // W, N, device=dev)
    dist.reduce_scatter_tensor(ref32, a.float() @ w.float().t())
    close(op.forward(a, w), ref32, "GemmRS before the failure")
    op.check_status()
    torch.cuda.synchronize()
    dist.barrier()
    if rank == W - 1:
        p0("")                                  # the last rank leaves between steps: no launch
    else:
        op.forward(a, w)                        # peers wait for the missing rank, bounded
        try:
            op.check_status()
            raise AssertionError("the missing rank went unnoticed")
        except flux.FluxTimeoutError as e:
            assert "start handshake" in str(e) or "tile counter" in str(e), str(e)
        # the device still works
        x = torch.randn(512, 512, device=dev).bfloat16()
        g = flux.GemmOnly(torch.bfloat16).forward(x, x)
        close(g, x.float() @ x.float().t(), "GemmOnly after the timeout")
        # ... and the op itself refuses to run on half-counted state
        try:
            op.forward(a, w)
            raise AssertionError("a poisoned op accepted a call")
        except RuntimeError as e:
            assert "reset" in str(e), str(e)
    torch.cuda.synchronize()
    # every rank (the one that sat out too) resets the op; then it is right again, twice
    op.reset()
    for _ in range(2):
        close(op.forward(a, w), ref32, "GemmRS after reset")
    op.check_status()
    torch.cuda.synchronize()
    print(f"[rank {rank}] failure ok", flush=True)


if "dense" in what:
    check_dense()
if "blockscale" in what:
    check_blockscale()
if "ulysses" in what:
    check_ulysses()
if "moe" in what:
    check_moe()
if "coll" in what:
    check_coll()
if "failure" in what:
    check_failure()
p0("ALL OK")
dist.barrier()
dist.destroy_process_group()
