"""Time one kernel of the package on synthetic data of a given shape: the cases that the
summaries under ``profiles/`` were measured and captured with.

    python -m miniserve_b200.tools.kernel_bench attn_decode --batch 64 --context 2048
    python -m miniserve_b200.tools.kernel_bench attn_prefill --tokens 2048
    python -m miniserve_b200.tools.kernel_bench skinny --m 8 --n 4096 --k 1024
    python -m miniserve_b200.tools.kernel_bench sample --batch 8 --top-p 0.9
    python -m miniserve_b200.tools.kernel_bench decay_scan --tokens 2048 --heads 8 --key-dim 64 --value-dim 128 [--delta]
    python -m miniserve_b200.tools.kernel_bench attn_prefill --tokens 2048 --softcap 30 --chunk 1024 --learned-sink
    python -m miniserve_b200.tools.kernel_bench add_rmsnorm --m 2048 --n 1024 --offset
    python -m miniserve_b200.tools.kernel_bench pointwise --op channel_gate --tokens 2048 --heads 16 --head-dim 128

Each case rotates over enough copies of its inputs to exceed the L2 cache, captures one pass over
all copies in a CUDA graph, and reports the time per launch with the bytes or flops it implies.
``--launches N`` instead runs N plain launches (what a profiler attaches to).
"""

from __future__ import annotations

import argparse
import json
import random
import sys
from types import SimpleNamespace

import torch

L2_BYTES = 160e6


def _paged(rows, page, nkv, d, seed, device):
    rng = random.Random(seed)
    need = [-(-(s + n) // page) for s, n in rows]
    order = list(range(sum(need) + 3))
    rng.shuffle(order)
    tables, at = [], 0
    for n in need:
        tables.append(order[at:at + n])
        at += n
    i32 = dict(dtype=torch.int32, device=device)
    k = torch.randn((len(order), nkv, page, d), device=device).bfloat16()
    v = torch.randn((len(order), nkv, page, d), device=device).bfloat16()
    indptr = [0]
    for t in tables:
        indptr.append(indptr[-1] + len(t))
    cu = [0]
    for _, n in rows:
        cu.append(cu[-1] + n)
    ctx = SimpleNamespace(
        num_rows=len(rows), num_tokens=cu[-1], cu_q=torch.tensor(cu, **i32),
        q_start=torch.tensor([s for s, _ in rows], **i32), kv_len=torch.tensor([s + n for s, n in rows], **i32),
        page_indptr=[torch.tensor(indptr, **i32)], page_indices=[torch.tensor([p for t in tables for p in t], **i32)],
        max_q_len=max(n for _, n in rows), max_kv_len=max(s + n for s, n in rows),
        decode_only=all(n == 1 for _, n in rows), host_q_start=[s for s, _ in rows], host_q_len=[n for _, n in rows],
        leading_single_rows=next((i for i, (_, n) in enumerate(rows) if n != 1), len(rows)), graph_bucket=0, scratch={}, step_cache={},
        sm_count=torch.cuda.get_device_properties(0).multi_processor_count, stream=0)
    return k, v, ctx


def _time(calls, copies, launches):
    """calls(i, stream) launches the kernel on input copy i."""
    s = torch.cuda.Stream()
    if launches:
        with torch.cuda.stream(s):
            for i in range(launches):
                calls(i % copies, s.cuda_stream)
        s.synchronize()
        return None
    with torch.cuda.stream(s):
        for i in range(copies):
            calls(i, s.cuda_stream)
    s.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        for i in range(copies):
            calls(i, torch.cuda.current_stream().cuda_stream)
    for _ in range(2):
        g.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(7):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) * 1000 / copies)
    return sorted(times)[len(times) // 2]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("kernel", choices=["attn_decode", "attn_prefill", "skinny", "add_rmsnorm", "gemm", "gate_up", "sample", "decay_scan", "pointwise", "experts"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--prefix", type=int, default=0, help="attn_prefill: tokens already in the cache before the portion")
    ap.add_argument("--m", type=int, default=8)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=1024)
    ap.add_argument("--gemm", choices=["auto", "tcgen05", "library"], default="auto",
                    help="gemm, gate_up: this package's tcgen05 kernels, the vendor library, or the engine's choice")
    ap.add_argument("--vocab", type=int, default=151936, help="sample: tokens in a row of logits")
    ap.add_argument("--temperature", type=float, default=0.8, help="sample: 0 is greedy")
    ap.add_argument("--top-p", type=float, default=1.0, help="sample: below 1, the nucleus is found first")
    ap.add_argument("--key-dim", type=int, default=64, help="decay_scan: key channels of a head")
    ap.add_argument("--value-dim", type=int, default=128, help="decay_scan: value channels of a head")
    ap.add_argument("--delta", action="store_true", help="decay_scan: the delta rule instead of the decay rule")
    ap.add_argument("--softcap", type=float, default=0.0, help="attn_*: scores capped at this (0: none)")
    ap.add_argument("--chunk", type=int, default=0, help="attn_*: a query sees only its own block of this many positions (0: all)")
    ap.add_argument("--learned-sink", action="store_true", help="attn_*: a sink with a score per head")
    ap.add_argument("--offset", action="store_true", help="add_rmsnorm: the kernel with a float32 weight stored around zero and a factor on the addend")
    ap.add_argument("--distance-bias", action="store_true", help="attn_*: r1 ln(1 + r2 distance) taken off the scores, numbers per head")
    ap.add_argument("--keep-first", type=int, default=0, help="attn_*: this many first keys stay visible behind --window")
    ap.add_argument("--window", type=int, default=0, help="attn_*: a query sees only this many keys back (0: all)")
    ap.add_argument("--op", choices=["channel_gate", "head_gate", "relu_squared", "gelu_tanh", "latent_prepare", "qkv_prepare",
                                     "layernorm", "layernorm_pair", "token_shift", "clamped_glu", "sum_bias", "act_mul", "axpby"],
                    default="channel_gate", help="pointwise: which kernel (--tokens rows; --heads x --head-dim, or --n, columns)")
    ap.add_argument("--experts", type=int, default=14, help="experts: how many experts")
    ap.add_argument("--top", type=int, default=4, help="experts: choices per token")
    ap.add_argument("--launches", type=int, default=0, help="run this many plain launches and report nothing")
    args = ap.parse_args(argv)

    from .. import ops

    dev = torch.device("cuda:0")
    out = dict(kernel=args.kernel)
    if args.kernel in ("attn_decode", "attn_prefill"):
        nq, nkv, d = args.heads, args.kv_heads, args.head_dim
        if args.kernel == "attn_decode":
            rows = [(args.context, 1)] * args.batch
            byts = args.batch * (args.context + 1) * nkv * d * 2 * 2
            work = dict(bytes=byts)
        else:
            rows = [(args.prefix, args.tokens)]  # a portion of a prompt behind `prefix` cached tokens
            pairs = args.tokens * (args.tokens + 1) / 2 + args.tokens * args.prefix
            if args.window:
                pairs = sum(min(p + 1, args.window) + min(args.keep_first, max(p + 1 - args.window, 0))
                            for p in range(args.prefix, args.prefix + args.tokens))
            if args.chunk:
                pairs = sum(p % args.chunk + 1 for p in range(args.prefix, args.prefix + args.tokens))
            flops = 4.0 * nq * d * pairs
            byts = (args.prefix + args.tokens) * nkv * d * 4
            work = dict(flops=flops)
        copies = max(2, int(L2_BYTES // byts) + 1)
        sets = [_paged(rows, args.page_size, nkv, d, i, dev) for i in range(copies)]
        q = torch.randn(sum(n for _, n in rows), nq, d, device=dev).bfloat16()
        o = torch.empty_like(q)
        if args.kernel == "attn_decode" and args.chunk:
            work = dict(bytes=args.batch * (args.context % args.chunk + 1) * nkv * d * 2 * 2)
        if args.kernel == "attn_decode" and args.window:
            work = dict(bytes=args.batch * (min(args.context + 1, args.window) + args.keep_first) * nkv * d * 2 * 2)
        extras = ops.AttentionExtras(torch.randn(nq, device=dev) if args.learned_sink else None, args.softcap, args.chunk,
                                     torch.randn(nq, device=dev) if args.distance_bias else None,
                                     torch.rand(nq, device=dev) + 0.1 if args.distance_bias else None, args.keep_first)

        def calls(i, stream):
            k, v, ctx = sets[i]
            ctx.stream = stream
            ops.attention(o, q, k, v, ctx, 0, d ** -0.5, args.window or args.chunk or None, extras=extras)
    elif args.kernel in ("gemm", "gate_up"):
        # gemm: x [m, k] times w [n, k]^T; gate_up: silu(x Wg^T) * (x Wu^T) with the stacked weight [2 n, k]
        ops.TC_GEMM = {"auto": "auto", "tcgen05": "1", "library": "0"}[args.gemm]
        rows = args.n * (2 if args.kernel == "gate_up" else 1)
        work = dict(flops=2.0 * args.m * rows * args.k)
        copies = max(2, int(L2_BYTES // (rows * args.k * 2)) + 1)
        ws = [(torch.randn(rows, args.k, device=dev) * args.k ** -0.5).bfloat16() for _ in range(copies)]
        x = torch.randn(args.m, args.k, device=dev).bfloat16()
        o = torch.empty(args.m, args.n, device=dev, dtype=torch.bfloat16)
        scratch = torch.empty(args.m, rows, device=dev, dtype=torch.bfloat16)

        def calls(i, stream):
            if args.kernel == "gemm":
                ops.linear(x, ws[i], out=o, stream=stream)
            else:
                ops.linear_silu_mul(x, ws[i], o, scratch=scratch, stream=stream)
    elif args.kernel == "experts":
        # both products of a routed feed-forward over --tokens tokens with --top choices each among --experts experts of
        # --n channels (--k the model's width), the choices uniform; --gemm tcgen05 (grouped kernel) or library (here: mma.sync)
        from ..ops import experts as xo

        t, e, top, inter, width = args.tokens, args.experts, args.top, args.n, args.k
        slots = t * top
        tc = args.gemm != "library"
        tile_rows = xo.TC_TILE_ROWS if tc else xo.TILE_ROWS
        work = dict(flops=2.0 * slots * 3 * inter * width)
        copies = max(2, int(L2_BYTES // (e * 3 * inter * width * 2)) + 1)
        wg = [(torch.randn(e, 2 * inter, width, device=dev) * width ** -0.5).bfloat16() for _ in range(copies)]
        wd = [(torch.randn(e, width, inter, device=dev) * inter ** -0.5).bfloat16() for _ in range(copies)]
        x = torch.randn(t, width, device=dev).bfloat16()
        idx = torch.stack([torch.randperm(e, device=dev)[:top] for _ in range(t)]).to(torch.int32).contiguous()
        i32 = dict(dtype=torch.int32, device=dev)
        pos, perm, offsets = torch.empty(slots, **i32), torch.empty(slots, **i32), torch.empty(e + 1, **i32)
        tiles, meta = torch.empty(xo.expert_max_tiles(slots, e, tile_rows), 2, **i32), torch.empty(2, **i32)
        xo.expert_plan(pos, perm, offsets, tiles, meta, idx, e, tile_rows=tile_rows)
        xs = torch.zeros(slots, width, device=dev, dtype=torch.bfloat16)
        act = torch.empty(slots, inter, device=dev, dtype=torch.bfloat16)
        y = torch.empty(slots, width, device=dev, dtype=torch.float32)

        def calls(i, stream):
            if tc:
                xo.expert_gather(xs, x, perm, meta, top, stream=stream)
                xo.expert_products_tc(act, xs, wg[i], tiles, meta, offsets, True, stream=stream)
                xo.expert_products_tc(y, act, wd[i], tiles, meta, offsets, False, stream=stream)
            else:
                xo.expert_gate_up(act, x, wg[i], perm, top, tiles, meta, offsets, "silu", stream=stream)
                xo.expert_down(y, act, wd[i], tiles, meta, offsets, stream=stream)
    elif args.kernel == "sample":
        # --batch rows of float32 logits, each row with its own seed
        byts = args.batch * args.vocab * 4
        work = dict(bytes=byts)
        copies = max(2, min(16, int(L2_BYTES // byts) + 1))
        logits = [torch.randn(args.batch, args.vocab, device=dev) * 3 for _ in range(copies)]
        tokens = torch.empty(args.batch, dtype=torch.int32, device=dev)
        temp = torch.full((args.batch,), args.temperature, device=dev)
        top_p = torch.full((args.batch,), args.top_p, device=dev) if args.top_p < 1 else None
        seed = torch.arange(args.batch, dtype=torch.int64, device=dev)
        counter = torch.full((args.batch,), 5, dtype=torch.int64, device=dev)
        nucleus = torch.empty(args.batch * ops.nucleus_bytes(), dtype=torch.uint8, device=dev)

        def calls(i, stream):
            if args.temperature == 0:
                ops.sample(tokens, logits[i], stream=stream)
            else:
                ops.sample(tokens, logits[i], temperature=temp, top_p=top_p, seed=seed, counter=counter,
                           scratch=nucleus if top_p is not None else None, stream=stream)
    elif args.kernel == "skinny":
        byts = args.n * args.k * 2
        work = dict(bytes=byts)
        copies = max(2, int(L2_BYTES // byts) + 1)
        ws = [torch.randn(args.n, args.k, device=dev).bfloat16() for _ in range(copies)]
        x = torch.randn(args.m, args.k, device=dev).bfloat16()
        o = torch.empty(args.m, args.n, device=dev, dtype=torch.bfloat16)

        def calls(i, stream):
            ops.linear(x, ws[i], out=o, stream=stream)
    elif args.kernel == "add_rmsnorm":
        h = args.n
        byts = args.m * h * 10
        work = dict(bytes=byts)
        copies = 16
        res = torch.randn(args.m, h, device=dev)
        delta = torch.randn(args.m, h, device=dev).bfloat16()
        w = torch.ones(h, device=dev).bfloat16()
        o = torch.empty(args.m, h, device=dev, dtype=torch.bfloat16)

        wf = torch.zeros(h, device=dev)

        def calls(i, stream):
            if args.offset:
                ops.add_rmsnorm_scaled(o, res, delta, 0.5, wf, 1.0, 1e-6, stream=stream)
            else:
                ops.add_rmsnorm(o, res, delta, w, 1e-6, stream=stream)
    elif args.kernel == "pointwise":
        t, nq, d = args.tokens, args.heads, args.head_dim
        width = nq * d
        bf = dict(device=dev, dtype=torch.bfloat16)
        per_set = t * width * 2 * 6
        copies = max(2, int(L2_BYTES // per_set) + 1)
        # a projection's rows (operands are column ranges of it), attention's output, and the row that features are written into
        sets = [(torch.randn(t, nq, d, **bf), torch.randn(t, 3 * width + 8, **bf), torch.empty(t, 2 * width, **bf)) for _ in range(copies)]
        pool, _, pctx = _paged([(0, t)], args.page_size, 1, d, 0, dev)
        kpool, vpool, kctx = _paged([(0, t)], args.page_size, nq, d, 1, dev)
        i32 = dict(dtype=torch.int32, device=dev)
        positions, row_of = torch.arange(t, **i32), torch.zeros(t, **i32)
        status = torch.zeros(1, **i32)
        wn = torch.ones(d, device=dev)
        table = torch.randn(t, d, device=dev)
        qo = torch.empty(t, nq, d, **bf)
        # the block's kernels: rows of --n channels (the model's width; the gated activation reads 2 n and writes n)
        n = args.n
        res, delta = torch.randn(t, n, device=dev), torch.randn(t, n, **bf)
        lw, lb = (torch.randn(n, device=dev) for _ in range(2))
        ln_a, ln_b = torch.empty(t, n, **bf), torch.empty(t, n, **bf)
        gate_up, glu_bias = torch.randn(t, 2 * n, **bf), torch.randn(2 * n, device=dev)
        slots = torch.zeros(2, n, **bf)
        sctx = SimpleNamespace(row_of_token=row_of, cu_q=torch.tensor([0, t], **i32), q_start=torch.zeros(1, **i32),
                               state_slot=torch.zeros(1, **i32), num_rows=1, stream=0)
        byts = {"layernorm": t * n * 12, "layernorm_pair": t * n * 14, "token_shift": t * n * 4, "clamped_glu": t * n * 6,
                "sum_bias": t * n * 6, "act_mul": t * n * 6, "axpby": t * n * 6,
                "channel_gate": 3 * t * width * 2, "head_gate": 2 * t * width * 2, "relu_squared": 2 * t * width * 2,
                "gelu_tanh": 2 * t * width * 2, "latent_prepare": 2 * t * d * 2, "qkv_prepare": 2 * 3 * t * width * 2}[args.op]
        work = dict(bytes=byts)

        def calls(i, stream):
            att, wide, feat = sets[i]
            if args.op == "layernorm":
                ops.add_layernorm(ln_a, res, delta, lw, lb, 1e-5, stream=stream)
            elif args.op == "layernorm_pair":
                ops.add_layernorm(ln_a, res, delta, lw, lb, 1e-5, out2=ln_b, weight2=lb, bias2=lw, stream=stream)
            elif args.op == "token_shift":
                sctx.stream = stream
                ops.token_shift(ln_b, ln_a, slots, lw, sctx)
            elif args.op == "clamped_glu":
                ops.clamped_glu(ln_a, gate_up, glu_bias, 7.0, 1.702, 1.0, stream=stream)
            elif args.op == "act_mul":
                ops.act_mul(ln_a, gate_up, "gelu_tanh", stream=stream)
            elif args.op == "sum_bias":
                ops.sum_bias(ln_a, delta, ln_b, lw, stream=stream)
            elif args.op == "axpby":
                ops.axpby(ln_a, delta, ln_b, 1.0, 1.0, stream=stream)
            elif args.op == "channel_gate":
                ops.channel_gate(feat[:, :width], att, wide[:, width:2 * width], d, 1.0, stream=stream)
            elif args.op == "head_gate":
                ops.head_gate(feat[:, :width], att, wide[:, width:width + nq], d, 1.0, stream=stream)
            elif args.op == "relu_squared":
                ops.relu_squared(feat[:, width:], wide[:, :width], stream=stream)
            elif args.op == "gelu_tanh":
                ops.gelu_tanh(qo, att, stream=stream)
            elif args.op == "latent_prepare":
                ops.latent_prepare(pool, wide[:, width:width + d], wn, 1e-6, positions, row_of, pctx.page_indptr[0], pctx.page_indices[0],
                                   args.page_size, status, stream=stream)
            else:
                ops.qkv_prepare(qo, kpool, vpool, wide[:, :width], wide[:, width:2 * width], wide[:, 2 * width:3 * width], None, None, table,
                                d, False, 1e-6, positions, row_of, kctx.page_indptr[0], kctx.page_indices[0], args.page_size, status,
                                stream=stream)
    else:
        # the linear-attention recurrence: `batch` requests of `tokens` tokens each (1: a decode step), from zero state
        t, hh, dk, dv, rows = args.tokens * args.batch, args.heads, args.key_dim, args.value_dim, args.batch
        i32 = dict(dtype=torch.int32, device=dev)
        bufs = {}

        def buffer(role, shape, dt, device):
            return bufs.setdefault((role, shape, dt), torch.empty(shape, dtype=dt, device=device))

        ctx = SimpleNamespace(cu_q=torch.arange(0, t + 1, args.tokens, **i32), q_start=torch.zeros(rows, **i32),
                              state_slot=torch.arange(rows, **i32), num_rows=rows, decode_only=args.tokens == 1, buffer=buffer, stream=0)
        kind = torch.float32 if args.delta else torch.bfloat16  # the delta rule's q, k, v come from the convolution in float32
        q, k = (torch.randn(t, hh * dk, device=dev).to(kind) for _ in range(2))
        v = torch.randn(t, hh * dv, device=dev).to(kind)
        z = torch.randn(t, hh * dk, device=dev).bfloat16()
        beta = torch.randn(t, hh, device=dev).bfloat16() if args.delta else None
        bias, coef = torch.zeros(hh * dk, device=dev), torch.full((hh,), 0.1, device=dev)
        state, o = torch.zeros(rows + 1, hh, dv, dk, device=dev), torch.empty(t, hh, dv, device=dev)
        item = 4 if args.delta else 2
        work = dict(bytes=t * hh * ((2 * dk + dv) * item + dk * 2 + dv * 4) + 2 * rows * hh * dk * dv * 4)
        copies = 2

        def calls(i, stream):
            ctx.stream = stream
            ops.decay_scan(o, state, q, k, v, z, bias, coef, -1.0, beta, ctx, hh, dk, dv, dk ** -0.5, delta=args.delta)
    us = _time(calls, copies, args.launches)
    if us is not None:
        out.update(us_per_launch=round(us, 2), copies=copies)
        if "bytes" in work:
            out.update(bytes=work["bytes"], tb_per_s=round(work["bytes"] / us / 1e6, 3))
        if "flops" in work:
            out.update(flops=work["flops"], tflops=round(work["flops"] / us / 1e6, 1))
    out.update({k: v for k, v in vars(args).items() if k != "kernel"})
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
