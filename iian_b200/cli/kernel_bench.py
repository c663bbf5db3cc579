"""Times one of the engine's kernels alone, at the Qwen3-8B layer sizes by default.

    python -m iian_b200.cli.kernel_bench gemm_skinny --shape gate_up --rows 8
    python -m iian_b200.cli.kernel_bench gemm_tcgen05 --shape gate_up --rows 2048 --epilogue swiglu
    python -m iian_b200.cli.kernel_bench attention_decode --batch 8 --ctx 1152
    python -m iian_b200.cli.kernel_bench attention_prefill --tokens 2048
    python -m iian_b200.cli.kernel_bench rope --rows 2048
    python -m iian_b200.cli.kernel_bench norm --rows 2048
    python -m iian_b200.cli.kernel_bench layer_decode --batch 8 --ctx 1152 --graph

Timing: CUDA events around ``--iters`` launches after ``--warmup`` launches, on the launching stream;
the operands rotate through copies that together exceed the 126 MB L2, so every launch reads from HBM.
With ``--graph`` the timed launches are captured into one CUDA graph and the graph is replayed: the
engine's decode steps run that way, and kernels of a few microseconds are otherwise timed by the host's
launch rate.  The same command under ``ncu`` (with small ``--iters``) gives the counters kept under
``profiles/``.
"""
from __future__ import annotations

import argparse
import math
import sys

SHAPES = {  # name -> (out features, in features) at the Qwen3-8B sizes
    "qkv": (6144, 4096), "o": (4096, 4096), "gate_up": (24576, 4096), "down": (4096, 12288), "head": (151936, 4096),
}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="kernel_bench", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("kernel", choices=["gemm_skinny", "gemm_stream", "gemm_tcgen05", "gemm_library", "attention_decode", "attention_prefill",
                                       "rope", "norm", "swiglu", "layer_decode"])
    ap.add_argument("--shape", default="gate_up", choices=sorted(SHAPES))
    ap.add_argument("--rows", type=int, default=8, help="rows of activations (tokens in the step)")
    ap.add_argument("--epilogue", default="store", choices=["store", "swiglu"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=1152)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--prefix", type=int, default=0, help="attention_prefill: tokens of the sequence already in the cache before the portion")
    ap.add_argument("--seqs", type=int, default=1, help="attention_prefill: sequences that each bring such a portion")
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--splits", type=int, default=0, help="key splits of decode attention (0: the engine's choice)")
    ap.add_argument("--stages", type=int, default=0, help="decode attention: shared-memory tiles per CTA (2 or 3; 0: the default)")
    ap.add_argument("--unsplit-stages", type=int, default=0, help="decode attention with unsplit keys: 2 or 3 tiles per CTA (0: the kernel's rule)")
    ap.add_argument("--tc", action="store_true", help="attention_prefill: the tcgen05 kernel instead of the mma.sync kernel")
    ap.add_argument("--no-cluster", action="store_true", help="decode attention: merge key splits through scratch memory")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--graph", action="store_true", help="time the launches as one replayed CUDA graph")
    ap.add_argument("--cfg", type=int, default=0, help="gemm_skinny: tile configuration (0: the kernel's choice)")
    ap.add_argument("--bn", type=int, default=0, help="gemm_tcgen05: columns of a tile, 128 or 256 (0: the engine's choice)")
    ap.add_argument("--ksplit", type=int, default=0, help="gemm_skinny: CTAs that share K for one row block (0: the engine's choice)")
    args = ap.parse_args(argv)

    import torch
    from ..ops.cuda_backend import CudaKernels

    if not torch.cuda.is_available():
        print("kernel_bench: no CUDA device", file=sys.stderr)
        return 2
    k = CudaKernels()
    if args.stages and args.kernel != "gemm_stream":
        k.set_decode_stages(args.stages)
    if args.unsplit_stages:
        from ..ops.cuda_backend import _fn
        from ctypes import c_int
        if _fn("attention_mma", "iian_attention_unsplit_stages", [c_int])(args.unsplit_stages) != 0:
            raise SystemExit("kernel_bench: --unsplit-stages takes 2 or 3")
    dev = torch.device("cuda:0")
    bf = torch.bfloat16
    gen = torch.Generator(device=dev).manual_seed(0)

    def rnd(*shape, std=1.0, dtype=bf):
        return (torch.randn(*shape, device=dev, generator=gen, dtype=torch.float32) * std).to(dtype)

    def timeit(fn):
        for i in range(args.warmup):
            fn(i)
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if args.graph:
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side), torch.cuda.graph(graph, stream=side):
                for i in range(args.iters):
                    fn(i)
            graph.replay()
            torch.cuda.synchronize()
            reps = 5
            s.record()
            for _ in range(reps):
                graph.replay()
            e.record()
            torch.cuda.synchronize()
            return s.elapsed_time(e) / (args.iters * reps) * 1e3
        s.record()
        for i in range(args.iters):
            fn(i)
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) / args.iters * 1e3       # microseconds

    class Meta:
        pass

    if args.kernel.startswith("gemm"):
        m, kd = SHAPES[args.shape]
        n = args.rows
        copies = max(2, int(300e6 // (m * kd * 2)) + 1)
        ws = [rnd(m, kd, std=0.02) for _ in range(copies)]
        x = rnd(n, kd)
        swiglu = args.epilogue == "swiglu"
        out = torch.empty(n, m // 2 if swiglu else m, device=dev, dtype=bf)
        if args.kernel == "gemm_skinny":
            us = timeit(lambda i: k.gemm_skinny(x, ws[i % copies], out, cfg=args.cfg, ksplit=args.ksplit, epilogue=1 if swiglu else 0))
        elif args.kernel == "gemm_stream":       # (--stages 6 or 12: depth of the ring of shared-memory stages)
            if args.stages:
                type(k).STREAM_STAGES = args.stages
            us = timeit(lambda i: k._gemm_stream(x, ws[i % copies], out, n, m, kd, 1 if swiglu else 0))
            k.tcgen05_check(dev)
        elif args.kernel == "gemm_tcgen05":
            us = timeit(lambda i: k.gemm_tcgen05(x, ws[i % copies], out, epilogue=1 if swiglu else 0, bn=args.bn))
            k.tcgen05_check(dev)
        else:
            us = timeit(lambda i: torch.mm(x, ws[i % copies].t(), out=out))
        gb, tf = m * kd * 2 / 1e9, 2.0 * n * m * kd / 1e12
        print(f"{args.kernel} {args.shape} [{m} x {kd}] rows {n} epilogue {args.epilogue}: {us:.1f} us, "
              f"{gb / (us * 1e-6):.0f} GB/s of weights, {tf / (us * 1e-6):.0f} TFLOP/s")
        return 0

    nh, nkv, hd, ps = args.heads, args.kv_heads, args.head_dim, args.page_size
    if args.kernel == "layer_decode":
        # the kernels of one decoder layer of a decode step in their order, on buffers of the right sizes;
        # the weights rotate through copies like above
        b, ctx_len = args.batch, args.ctx
        hidden, inter = SHAPES["o"][0], SHAPES["down"][1]
        per_layer = sum(SHAPES[n][0] * SHAPES[n][1] * 2 for n in ("qkv", "o", "gate_up", "down"))
        copies = max(2, int(300e6 // per_layer) + 1)
        ws = [{n: rnd(*SHAPES[n], std=0.02) for n in ("qkv", "o", "gate_up", "down")} for _ in range(copies)]
        blocks = math.ceil((ctx_len + 1) / ps)
        n_pages = b * blocks
        caches = [(rnd(n_pages, nkv, ps, hd), rnd(n_pages, nkv, ps, hd)) for _ in range(copies)]
        meta = Meta()
        perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(1)).to(torch.int32)
        meta.block_table = perm.view(b, blocks).to(dev).contiguous()
        meta.cu_q = torch.arange(0, b + 1, dtype=torch.int32, device=dev)
        meta.ctx_len = torch.full((b,), ctx_len, dtype=torch.int32, device=dev)
        meta.positions = torch.full((b,), ctx_len - 1, dtype=torch.int32, device=dev)
        meta.seq_of_token = torch.arange(b, dtype=torch.int32, device=dev)
        meta.num_seqs, meta.num_tokens, meta.max_q_len, meta.max_ctx, meta.decode_only = b, b, 1, ctx_len, True
        slots = (meta.block_table[:, (ctx_len - 1) // ps].to(torch.int64) * ps + (ctx_len - 1) % ps).to(torch.int32)
        res = rnd(b, hidden, dtype=torch.float32)
        delta = rnd(b, hidden, std=0.01)
        h = torch.empty(b, hidden, device=dev, dtype=bf)
        qkv = torch.empty(b, (nh + 2 * nkv) * hd, device=dev, dtype=bf)
        qh = torch.empty(b, nh, hd, device=dev, dtype=bf)
        attn = torch.empty(b, nh * hd, device=dev, dtype=bf)
        act = torch.empty(b, inter, device=dev, dtype=bf)
        nw, qw = torch.ones(hidden, device=dev), torch.ones(hd, device=dev)
        inv = torch.pow(torch.tensor(1e6, dtype=torch.float64), -2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd).float().to(dev)
        table = torch.empty(b, hd // 2, 2, device=dev)
        k.rotary_table(inv, meta.positions, hd // 2, table)

        def layer(i):
            w, (kc, vc) = ws[i % copies], caches[i % copies]
            k.add_rms_norm(res, delta, nw, 1e-6, h)
            k.linear(h, w["qkv"], qkv)
            k.qk_norm_rope_store(qkv, qh, kc, vc, num_heads=nh, num_kv_heads=nkv, head_dim=hd, q_weight=qw, k_weight=qw,
                                 eps=1e-6, inv_freq=inv, rot_dim=hd, rope_style=0, positions=meta.positions, slots=slots,
                                 write_kv=True, table=table)
            k.paged_attention_mma(qh, kc, vc, attn, meta, num_heads=nh, num_kv_heads=nkv, head_dim=hd,
                                  scale=1 / math.sqrt(hd), window=None)
            k.linear(attn, w["o"], delta)
            k.add_rms_norm(res, delta, nw, 1e-6, h)
            if k.can_fuse_swiglu(h, w["gate_up"], 8):
                k.linear_swiglu(h, w["gate_up"], act)
            else:
                gu = torch.empty(b, 2 * inter, device=dev, dtype=bf)
                k.linear(h, w["gate_up"], gu)
                k.swiglu(gu, act, 8)
            k.linear(act, w["down"], delta)

        us = timeit(layer)
        gb = (per_layer + b * ctx_len * nkv * hd * 4) / 1e9
        print(f"layer_decode batch {b} ctx {ctx_len}: {us:.1f} us a layer, {gb / (us * 1e-6):.0f} GB/s of weights and K/V")
        return 0
    if args.kernel in ("attention_decode", "attention_prefill"):
        decode = args.kernel == "attention_decode"
        seqs = args.batch if decode else args.seqs
        ctx_len = args.ctx if decode else args.tokens + args.prefix
        q_len = 1 if decode else args.tokens
        blocks = math.ceil(ctx_len / ps)
        n_pages = seqs * blocks
        copies = max(2, int(300e6 // (n_pages * nkv * ps * hd * 4)) + 1) if decode else 1
        caches = [(rnd(n_pages, nkv, ps, hd), rnd(n_pages, nkv, ps, hd)) for _ in range(copies)]
        perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(1)).to(torch.int32)
        meta = Meta()
        meta.block_table = perm.view(seqs, blocks).to(dev).contiguous()
        meta.cu_q = torch.arange(0, seqs * q_len + 1, q_len, dtype=torch.int32, device=dev)
        meta.ctx_len = torch.full((seqs,), ctx_len, dtype=torch.int32, device=dev)
        meta.positions = torch.cat([torch.arange(ctx_len - q_len, ctx_len, dtype=torch.int32) for _ in range(seqs)]).to(dev)
        meta.seq_of_token = torch.arange(seqs, dtype=torch.int32).repeat_interleave(q_len).to(dev)
        meta.num_seqs, meta.num_tokens, meta.max_q_len, meta.max_ctx, meta.decode_only = seqs, seqs * q_len, q_len, ctx_len, decode
        q = rnd(seqs * q_len, nh, hd)
        out = torch.empty(seqs * q_len, nh * hd, device=dev, dtype=bf)
        kw = dict(num_heads=nh, num_kv_heads=nkv, head_dim=hd, scale=1 / math.sqrt(hd), window=None)
        if decode and args.splits:
            kw.update(n_split=args.splits, small_tiles=True)
        if args.no_cluster:
            kw.update(cluster=False)
        if not decode and args.tc:
            us = timeit(lambda i: k.paged_attention_tc(q, caches[i % copies][0], caches[i % copies][1], out, meta, **kw))
            k.tcgen05_check(dev)
        else:
            us = timeit(lambda i: k.paged_attention_mma(q, caches[i % copies][0], caches[i % copies][1], out, meta, **kw))
        if decode:
            gb = seqs * ctx_len * nkv * hd * 2 * 2 / 1e9
            print(f"attention_decode batch {seqs} ctx {ctx_len} heads {nh}/{nkv} x {hd}: {us:.1f} us, {gb / (us * 1e-6):.0f} GB/s of K/V "
                  f"(splits {args.splits or k.attention_splits(seqs, nkv, ctx_len)})")
        else:
            tf = seqs * 4.0 * nh * hd * (q_len * (q_len + 1) / 2 + q_len * args.prefix) / 1e12
            print(f"attention_prefill {seqs} x {q_len} tokens after {args.prefix} heads {nh}/{nkv} x {hd}: {us:.1f} us, "
                  f"{tf / (us * 1e-6):.0f} TFLOP/s (causal)")
        return 0

    n = args.rows
    hidden = SHAPES["o"][0]
    if args.kernel == "norm":
        res = [rnd(n, hidden, dtype=torch.float32) for _ in range(4)]
        delta, w = rnd(n, hidden), torch.ones(hidden, device=dev)
        out = torch.empty(n, hidden, device=dev, dtype=bf)
        us = timeit(lambda i: k.add_rms_norm(res[i % 4], delta, w, 1e-6, out))
        gb = n * hidden * (4 + 2 + 4 + 2) / 1e9
        print(f"add_rms_norm rows {n} width {hidden}: {us:.1f} us, {gb / (us * 1e-6):.0f} GB/s")
    elif args.kernel == "swiglu":
        f = SHAPES["down"][1]
        gu = rnd(n, 2 * f)
        out = torch.empty(n, f, device=dev, dtype=bf)
        us = timeit(lambda i: k.swiglu(gu, out, 8))
        print(f"swiglu rows {n} width {f}: {us:.1f} us, {n * f * 6 / 1e9 / (us * 1e-6):.0f} GB/s")
    else:
        width = (nh + 2 * nkv) * hd
        qkv = rnd(n, width)
        n_pages = math.ceil(n / ps) + 1
        kc, vc = torch.zeros(n_pages, nkv, ps, hd, device=dev, dtype=bf), torch.zeros(n_pages, nkv, ps, hd, device=dev, dtype=bf)
        q_out = torch.empty(n, nh, hd, device=dev, dtype=bf)
        qw, kw_ = torch.ones(hd, device=dev), torch.ones(hd, device=dev)
        inv = torch.pow(torch.tensor(1e6, dtype=torch.float64), -2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd).float().to(dev)
        pos = torch.arange(n, dtype=torch.int32, device=dev)
        table = torch.empty(n, hd // 2, 2, device=dev)
        k.rotary_table(inv, pos, hd // 2, table)
        us = timeit(lambda i: k.qk_norm_rope_store(qkv, q_out, kc, vc, num_heads=nh, num_kv_heads=nkv, head_dim=hd, q_weight=qw,
                                                   k_weight=kw_, eps=1e-6, inv_freq=inv, rot_dim=hd, rope_style=0, positions=pos,
                                                   slots=pos, write_kv=True, table=table))
        print(f"qk_norm_rope_store rows {n} heads {nh}+2x{nkv} x {hd}: {us:.1f} us, {n * width * 4 / 1e9 / (us * 1e-6):.0f} GB/s")
    return 0


if __name__ == "__main__":
    sys.exit(main())
