"""Micro-benchmarks of single kernels, in the manner of the reference's benchmarks/bench_kernels.py
(which times its two Triton kernels against eager PyTorch): each kernel of this package alone, at
the shapes of a model preset, timed on the device inside a captured CUDA graph with inputs that
rotate through more memory than the L2 holds, next to the vendor-library product where there is one.

    python -m mini_inference_engine_b200.kernels.microbench gemm --tokens 1 8 64
    python -m mini_inference_engine_b200.kernels.microbench decode-attention --batch 8 --context 512
    python -m mini_inference_engine_b200.kernels.microbench prefill-attention --tokens 2048
    python -m mini_inference_engine_b200.kernels.microbench small --batch 8

``--once`` runs every kernel a few times without a graph and exits: the form to put under a profiler.
"""
from __future__ import annotations

import argparse
import math

import torch

from ..config import load_preset
from . import gemm_tc, ops

DEV = "cuda"
L2_BYTES = 126e6


def graph_time_us(fn, calls: int, replays: int = 3) -> float:
    """Mean microseconds per call of ``fn(i)``, i = 0..calls-1, captured once and replayed."""
    for i in range(min(calls, 2)):
        fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(calls):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(replays):
        g.replay()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / (calls * replays) * 1e3


def run_plain(fn, calls: int) -> None:
    for i in range(calls):
        fn(i)
    torch.cuda.synchronize()


def cmd_gemm(args):
    cfg = load_preset(args.preset)
    h, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    qkv = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim
    shapes = [("qkv", qkv, h, False), ("o", h, cfg.num_attention_heads * cfg.head_dim, False),
              ("gate_up+swiglu", 2 * I, h, True), ("down", h, I, False), ("lm_head", V, h, False)]
    for name, N, K, swiglu in shapes:
        if args.only and args.only not in name:
            continue
        copies = max(2, int(4 * L2_BYTES / (N * K * 2)))
        ws = [torch.randn(N, K, device=DEV).bfloat16() for _ in range(copies)]
        for M in args.tokens:
            x = torch.randn(M, K, device=DEV).bfloat16()
            y = torch.empty(M, N // 2 if swiglu else N, device=DEV, dtype=torch.bfloat16)
            y_lib = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
            ours = lambda i: gemm_tc.gemm(x, ws[i % copies], y, swiglu=swiglu)        # noqa: E731
            pair = lambda i: gemm_tc.gemm_pair(x, ws[i % copies], y, swiglu=swiglu)   # noqa: E731
            lib = lambda i: torch.mm(x, ws[i % copies].t(), out=y_lib)              # noqa: E731
            if args.once:
                run_plain(pair if args.pair else ours, 3)
                continue
            t_ours, t_lib = graph_time_us(ours, copies), graph_time_us(lib, copies)
            gemm_tc.check_error()
            byts, flops = N * K * 2 + M * K * 2 + M * N * 2, 2 * M * N * K
            print(f"{name:15s} M={M:5d} N={N:6d} K={K:5d}  tcgen05 {t_ours:8.1f} us ({byts / t_ours / 1e3:6.0f} GB/s, "
                  f"{flops / t_ours / 1e6:7.1f} TFLOP/s)  library {t_lib:8.1f} us  plan {gemm_tc.plan(M, N, K)}", flush=True)
            if M >= 256:                 # the product on pairs of SMs (csrc/gemm_pair_tc.cu)
                t_pair = graph_time_us(pair, copies)
                gemm_tc.check_error()
                print(f"{name:15s} M={M:5d} on pairs of SMs {t_pair:8.1f} us ({flops / t_pair / 1e6:7.1f} TFLOP/s)", flush=True)
            H, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
            if name == "qkv" and gemm_tc.can_fuse_rope(x, ws[0], H, Hkv, D, D):
                # the same product with the rotation and the cache write in its epilogue, against product + rotation kernel
                inv = (1.0 / (cfg.rope_theta ** (torch.arange(0, D, 2).float() / D))).to(DEV)
                cos, sin = ops.rope_tables(inv, cfg.max_position_embeddings)
                kc = torch.zeros(M + 2, Hkv, 16, D, device=DEV, dtype=torch.bfloat16)
                vc = torch.zeros_like(kc)
                pos = torch.full((M,), 100, dtype=torch.int32, device=DEV)
                slots = (torch.arange(M, dtype=torch.int32, device=DEV) + 1) * 16
                fused = lambda i: gemm_tc.gemm_qkv_rope(x, ws[i % copies], y, None, pos, slots, cos, sin, kc, vc, H, Hkv, D, D, 16)  # noqa: E731

                def two(i):
                    gemm_tc.gemm(x, ws[i % copies], y)
                    ops.rope_cache_write(y, pos, slots, cos, sin, kc, vc, H, Hkv, D, D, 16)
                print(f"{'qkv + rotation':15s} M={M:5d} fused epilogue {graph_time_us(fused, copies):8.1f} us   "
                      f"product then rotation kernel {graph_time_us(two, copies):8.1f} us", flush=True)
        del ws


def _paged(batch: int, ctx: int, cfg, page: int):
    Hkv, D = cfg.num_key_value_heads, cfg.head_dim
    pages_per = -(-ctx // page)
    num_pages = batch * pages_per + 1
    perm = torch.randperm(num_pages - 1) + 1
    bt = perm[:batch * pages_per].view(batch, pages_per).to(torch.int32).to(DEV)
    k = torch.randn(num_pages, Hkv, page, D, device=DEV).bfloat16()
    return bt, k, torch.randn_like(k)


def cmd_decode_attention(args):
    cfg = load_preset(args.preset)
    H, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    stride = (H + 2 * Hkv) * D
    for B in args.batch:
        bt, k, v = _paged(B, args.context, cfg, args.page)
        qkv = torch.randn(B, stride, device=DEV).bfloat16()
        rows = torch.arange(B, dtype=torch.int32, device=DEV)
        ones = torch.ones(B, dtype=torch.int32, device=DEV)
        ctx = torch.full((B,), args.context, dtype=torch.int32, device=DEV)
        out = torch.empty(B, H, D, device=DEV, dtype=torch.bfloat16)
        fn = lambda i: ops.decode_attention(qkv, stride, k, v, bt, rows, ones, ctx, out, H, Hkv, D, args.page,   # noqa: E731
                                            1 / math.sqrt(D), max_ctx=args.max_context or args.context, splits=args.splits,
                                            merge=args.merge if args.merge or args.splits is None else "cluster",
                                            stages=args.stages, tma={'auto': None, 'on': True, 'off': False}[args.tma])
        if args.rope:
            # the rotation with the cache write as a kernel of its own in front of the attention, against both inside it
            inv = (1.0 / (cfg.rope_theta ** (torch.arange(0, D, 2).float() / D))).to(DEV)
            cos, sin = ops.rope_tables(inv, max(args.context, 16))
            pos = ctx - 1
            slots = (bt[rows.long(), ((args.context - 1) // args.page)] * args.page + (args.context - 1) % args.page).to(torch.int32)
            attend = fn

            def apart(i):
                ops.rope_cache_write(qkv, pos, slots, cos, sin, k, v, H, Hkv, D, D, args.page)
                attend(i)
            inside = lambda i: ops.decode_attention(qkv, stride, k, v, bt, rows, ones, ctx, out, H, Hkv, D, args.page,   # noqa: E731
                                                    1 / math.sqrt(D), max_ctx=args.max_context or args.context, rope=(cos, sin))
            ta, ti = graph_time_us(apart, 20), graph_time_us(inside, 20)
            print(f"decode attention B={B:4d} ctx={args.context}: rotation kernel + attention {ta:7.2f} us, rotation inside {ti:7.2f} us", flush=True)
            continue
        if args.once:
            run_plain(fn, 3)
            continue
        t = graph_time_us(fn, 20)
        byts = B * args.context * Hkv * D * 2 * 2
        plan = args.splits or "%d by %s" % ops.decode_plan(B, Hkv * -(-(H // Hkv) // 16), args.max_context or args.context, True, D)[:2]
        print(f"decode attention B={B:4d} ctx={args.context} splits={plan}{' ' + args.merge if args.merge else ''}: {t:7.2f} us  "
              f"({byts / t / 1e3:6.0f} GB/s of cache)", flush=True)


def cmd_prefill_attention(args):
    cfg = load_preset(args.preset)
    H, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    stride = (H + 2 * Hkv) * D
    for T in args.tokens:
        bt, k, v = _paged(1, T, cfg, args.page)
        qkv = torch.randn(T, stride, device=DEV).bfloat16()
        z = torch.zeros(1, dtype=torch.int32, device=DEV)
        n = torch.full((1,), T, dtype=torch.int32, device=DEV)
        out = torch.empty(T, H, D, device=DEV, dtype=torch.bfloat16)
        flops = 4 * H * D * T * (T + 1) / 2
        for name, kernel in (("tcgen05", ops.prefill_attention_tc), ("tcgen05 x2", ops.prefill_attention_tc),
                             ("mma.sync", ops.prefill_attention)):
            if args.only and args.only != name.split()[0]:
                continue
            if name.startswith("tcgen05"):                 # one query tile a block, or two side by side (head_dim 64)
                if name.endswith("x2") and D != 64:
                    continue
                ops.set_prefill_pairs(1 if name.endswith("x2") else 0)
            fn = lambda i: kernel(qkv, stride, k, v, bt, z, n, n, T, out, H, Hkv, D, args.page, 1 / math.sqrt(D), min_q_len=1)  # noqa: E731
            if args.once:
                run_plain(fn, 3)
                continue
            t = graph_time_us(fn, 5)
            print(f"prefill attention {name:10s} T={T:5d}: {t:8.1f} us  ({flops / t / 1e6:6.1f} TFLOP/s causal)", flush=True)
        ops.set_prefill_pairs(-1)
        ops.check_tc_errors()


def cmd_small(args):
    cfg = load_preset(args.preset)
    h, H, Hkv, D, I, V = (cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                          cfg.intermediate_size, cfg.vocab_size)
    for B in args.batch:
        res = torch.randn(B, h, device=DEV)
        delta = torch.randn(B, h, device=DEV).bfloat16()
        w = torch.ones(h, device=DEV).bfloat16()
        y = torch.empty(B, h, device=DEV, dtype=torch.bfloat16)
        qkv = torch.randn(B, (H + 2 * Hkv) * D, device=DEV).bfloat16()
        inv = (1.0 / (cfg.rope_theta ** (torch.arange(0, D, 2).float() / D))).to(DEV)
        cos, sin = ops.rope_tables(inv, cfg.max_position_embeddings)
        kc = torch.zeros(B + 2, Hkv, 16, D, device=DEV, dtype=torch.bfloat16)
        vc = torch.zeros_like(kc)
        pos = torch.full((B,), 100, dtype=torch.int32, device=DEV)
        slots = (torch.arange(B, dtype=torch.int32, device=DEV) + 1) * 16
        gu = torch.randn(B, 2 * I, device=DEV).bfloat16()
        act = torch.empty(B, I, device=DEV, dtype=torch.bfloat16)
        lg = torch.randn(B, V, device=DEV)
        tok = torch.empty(B, dtype=torch.int32, device=DEV)
        zf, zl, zi = torch.zeros(B, device=DEV), torch.zeros(B, dtype=torch.int64, device=DEV), torch.zeros(B, dtype=torch.int32, device=DEV)
        table = torch.randn(V, h, device=DEV).bfloat16()
        r2 = torch.empty(B, h, device=DEV)
        kernels = {
            "add_rmsnorm": lambda i: ops.add_rmsnorm(delta, res, w, cfg.rms_norm_eps, y),
            "rope_cache_write": lambda i: ops.rope_cache_write(qkv, pos, slots, cos, sin, kc, vc, H, Hkv, D, D, 16),
            "swiglu": lambda i: ops.swiglu(gu, act),
            "sample": lambda i: ops.sample(lg, zf, zl, zi, 0, tok),
            "embedding": lambda i: ops.embedding(table, zi, r2),
        }
        for name, fn in kernels.items():
            if args.once:
                run_plain(fn, 3)
            else:
                print(f"{name:18s} rows={B:5d}: {graph_time_us(fn, 20):7.2f} us", flush=True)


def main(argv=None):
    ap = argparse.ArgumentParser(prog="mini_inference_engine_b200.kernels.microbench", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--preset", default="tinyllama-1.1b")
    ap.add_argument("--once", action="store_true", help="run each kernel a few times without timing (for a profiler)")
    sub = ap.add_subparsers(dest="command", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--tokens", type=int, nargs="+", default=[1, 8, 64, 2048])
    g.add_argument("--only", default=None, help="substring of the projection's name")
    g.add_argument("--pair", action="store_true", help="with --once: run the product on pairs of SMs instead")
    g.set_defaults(fn=cmd_gemm)
    d = sub.add_parser("decode-attention")
    d.add_argument("--batch", type=int, nargs="+", default=[1, 8, 64])
    d.add_argument("--context", type=int, default=512)
    d.add_argument("--max-context", type=int, default=0)
    d.add_argument("--splits", type=int, default=None)
    d.add_argument("--merge", choices=["cluster", "scratch"], default=None,
                   help="how the parts are merged (default with no --splits: the wrapper's plan)")
    d.add_argument("--stages", type=int, default=None)
    d.add_argument("--page", type=int, default=16)
    d.add_argument("--tma", choices=["auto", "on", "off"], default="auto", help="key/value copies by TMA (default: the wrapper's choice)")
    d.add_argument("--rope", action="store_true", help="time the rotation kernel in front of the attention against the rotation inside it")
    d.set_defaults(fn=cmd_decode_attention)
    p = sub.add_parser("prefill-attention")
    p.add_argument("--tokens", type=int, nargs="+", default=[512, 2048, 8192])
    p.add_argument("--only", default=None, choices=[None, "tcgen05", "mma.sync"])
    p.add_argument("--page", type=int, default=16)
    p.set_defaults(fn=cmd_prefill_attention)
    s = sub.add_parser("small")
    s.add_argument("--batch", type=int, nargs="+", default=[8, 2048])
    s.set_defaults(fn=cmd_small)
    args = ap.parse_args(argv)
    args.fn(args)


if __name__ == "__main__":
    main()
