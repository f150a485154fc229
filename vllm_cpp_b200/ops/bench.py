"""Kernel micro-benchmarks: ``python -m vllm_cpp_b200.ops.bench [--json out.json]``.

Each case is timed with CUDA events on the launching stream after warm-up, with an L2 flush
(a write larger than L2) between timed iterations, and reported as achieved TFLOP/s or GB/s
next to the same shape run through ``torch.matmul`` (cuBLAS) where that is meaningful.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import reference as ref
from .. import ops


def _time(fn, iters=10, warmup=3, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    return times[len(times) // 2]


def small_case(name: str):
    """One kernel on a small input (a few hundred MB at most), three launches."""
    dev = torch.device("cuda")
    Hq, Hkv, D, bs = 32, 8, 128, 16
    if name == "gemm_small":
        a = torch.randn(4096, 4096, device=dev, dtype=torch.bfloat16)
        w = torch.randn(6144, 4096, device=dev, dtype=torch.bfloat16) * 0.05
        fn = lambda: ops.gemm(a, w)
    elif name == "gemm_decode_small":
        a = torch.randn(64, 4096, device=dev, dtype=torch.bfloat16)
        w = torch.randn(28672, 4096, device=dev, dtype=torch.bfloat16) * 0.05
        fn = lambda: ops.gemm(a, w)
    elif name == "prefill_small":
        B, ql = 4, 1024
        nb = ql // bs
        cache = torch.randn(B * nb + 1, 2, bs, Hkv, D, device=dev, dtype=torch.bfloat16)
        bt = torch.arange(B * nb, device=dev, dtype=torch.int32).reshape(B, nb)
        sl = torch.full((B,), ql, dtype=torch.int32, device=dev)
        qs = torch.arange(B + 1, device=dev, dtype=torch.int32) * ql
        treq, tq0 = ref.build_prefill_tiles([ql] * B)
        treq = torch.tensor(treq, dtype=torch.int32, device=dev)
        tq0 = torch.tensor(tq0, dtype=torch.int32, device=dev)
        q = torch.randn(B * ql, Hq * D, device=dev, dtype=torch.bfloat16)
        fn = lambda: ops.attn_prefill(q, cache, block_table=bt, seq_lens=sl, q_start=qs,
                                      tile_req=treq, tile_q0=tq0, num_q_heads=Hq,
                                      num_kv_heads=Hkv, head_dim=D, block_size=bs,
                                      scale=D ** -0.5)
    elif name == "decode_small":
        B, ctx = 128, 1024
        nb = ctx // bs
        cache = torch.randn(B * nb + 1, 2, bs, Hkv, D, device=dev, dtype=torch.bfloat16)
        bt = torch.arange(B * nb, device=dev, dtype=torch.int32).reshape(B, nb)
        sl = torch.full((B,), ctx, dtype=torch.int32, device=dev)
        q = torch.randn(B, Hq * D, device=dev, dtype=torch.bfloat16)
        fn = lambda: ops.attn_decode(q, cache, block_table=bt, seq_lens=sl, num_q_heads=Hq,
                                     num_kv_heads=Hkv, head_dim=D, block_size=bs, scale=D ** -0.5)
    elif name == "gdn_scan_small":
        from . import gdn as G
        T, Hk, Hv = 16384, 2, 6          # one 16k-token prompt at the TP=8 head counts of Qwen3.6-27B
        xc = torch.randn(T, 2 * Hk * 128 + Hv * 128, device=dev).to(torch.bfloat16)
        q = torch.nn.functional.normalize(torch.randn(T, Hk, 128, device=dev), dim=-1).to(torch.bfloat16)
        k = torch.nn.functional.normalize(torch.randn(T, Hk, 128, device=dev), dim=-1).to(torch.bfloat16)
        g = -torch.rand(T, Hv, device=dev) * 0.1
        beta = torch.rand(T, Hv, device=dev)
        lens = [2048] * 8
        qsl = [0]
        for n in lens:
            qsl.append(qsl[-1] + n)
        state = torch.zeros(len(lens), Hv, 128, 128, device=dev)
        slots = torch.arange(len(lens), dtype=torch.int32, device=dev)
        hi = torch.zeros(len(lens), dtype=torch.int32, device=dev)
        out = torch.empty(T, Hv, 128, device=dev, dtype=torch.bfloat16)
        ws = G.GdnWorkspace(dev, T, len(lens), Hv)
        fn = lambda: G.chunk_scan(q, k, xc, g, beta, state, qsl, slots, hi, out, ws, v_col0=2 * Hk * 128)
    elif name == "gdn_decode_small":
        from . import gdn as G
        B, Hk, Hv = 256, 2, 6
        xc = torch.randn(B, 2 * Hk * 128 + Hv * 128, device=dev).to(torch.bfloat16)
        a = torch.randn(B, Hv, device=dev).to(torch.bfloat16)
        b = torch.randn(B, Hv, device=dev).to(torch.bfloat16)
        A_log = torch.zeros(Hv, device=dev)
        dtb = torch.zeros(Hv, device=dev)
        state = torch.zeros(B, Hv, 128, 128, device=dev)     # 100 MB read + written per launch
        slots = torch.arange(B, dtype=torch.int32, device=dev)
        out = torch.empty(B, Hv, 128, device=dev, dtype=torch.bfloat16)
        fn = lambda: G.packed_decode(xc, a, b, A_log, dtb, state, slots, out, Hk, Hv)
    elif name == "moe_small":
        from . import moe as M
        T, E, k, H, I = 2048, 128, 8, 2048, 768
        x = torch.randn(T, H, device=dev).to(torch.bfloat16)
        wgu = (torch.randn(E, 2 * I, H, device=dev) * 0.05).to(torch.bfloat16)
        ids, w = M.router_topk(torch.randn(T, E, device=dev), k)
        ws = M.MoeWorkspace(dev, T, k, E, H, I)
        M.moe_sort(ids, 0, E, ws)
        M.moe_gather(x, ws, E, T * k)
        fn = lambda: M.grouped_gemm(ws.xs, wgu, ws.gu, ws, T * k)
    elif name == "gemm_streamk_small":
        # Llama-8B down projection at a mixed-step batch: 80 pair tiles on 74 CTA pairs, so the six
        # tiles of the ragged wave run as stream-K
        a = torch.randn(1280, 14336, device=dev, dtype=torch.bfloat16)
        w = torch.randn(4096, 14336, device=dev, dtype=torch.bfloat16) * 0.05
        fn = lambda: ops.gemm(a, w)
    elif name == "gemm_gated_small":
        a = torch.randn(1280, 4096, device=dev, dtype=torch.bfloat16)
        wg = torch.randn(14336, 4096, device=dev, dtype=torch.bfloat16) * 0.05
        wu = torch.randn(14336, 4096, device=dev, dtype=torch.bfloat16) * 0.05
        wil = ops.interleave_gate_up(wg, wu)
        del wg, wu
        fn = lambda: ops.gemm_gated(a, wil, 0)
    elif name == "gemm_fp8_small":
        from . import quant as Q
        a8 = torch.randn(4096, 4096, device=dev).to(torch.float8_e4m3fn)
        w8 = (torch.randn(6144, 4096, device=dev) * 0.05).to(torch.float8_e4m3fn)
        sa = torch.ones(4096, device=dev)      # one scale per token and per output channel, as the
        sw = torch.ones(6144, device=dev)      # W8A8 linear layers run it
        fn = lambda: Q.gemm_fp8(a8, w8, sa, sw)
    elif name == "gemm_w4a16_small":
        from . import quant as Q
        a = torch.randn(64, 4096, device=dev, dtype=torch.bfloat16)
        packed = torch.randint(0, 256, (28672, 2048), device=dev, dtype=torch.uint8)
        sf = torch.full((28672, 256), 0x38, device=dev, dtype=torch.uint8)     # e4m3 1.0
        g = torch.full((1,), 0.01, device=dev)
        fn = lambda: Q.gemm_w4a16(a, packed, sf, g)
    elif name == "gemm_nvfp4_small":
        # W4A4 on kind::mxf4nvf4, decode-sized batch against the widest projection of a 27B model
        from . import quant as Q
        M, N, K = 64, 34816, 5120
        aq = torch.randint(0, 256, (M, K // 2), device=dev, dtype=torch.uint8)
        wq = torch.randint(0, 256, (N, K // 2), device=dev, dtype=torch.uint8)
        sfa = torch.full((128 * K // 16,), 0x38, device=dev, dtype=torch.uint8)        # e4m3 1.0
        sfw = torch.full((N * K // 16,), 0x38, device=dev, dtype=torch.uint8)
        one = torch.ones(1, device=dev)
        fn = lambda: Q.gemm_nvfp4(aq, sfa, one, wq, sfw, one)
    elif name == "gemm_nvfp4_prefill_small":
        from . import quant as Q
        M, N, K = 4096, 8192, 5120
        aq = torch.randint(0, 256, (M, K // 2), device=dev, dtype=torch.uint8)
        wq = torch.randint(0, 256, (N, K // 2), device=dev, dtype=torch.uint8)
        sfa = torch.full((M * K // 16,), 0x38, device=dev, dtype=torch.uint8)
        sfw = torch.full((N * K // 16,), 0x38, device=dev, dtype=torch.uint8)
        one = torch.ones(1, device=dev)
        fn = lambda: Q.gemm_nvfp4(aq, sfa, one, wq, sfw, one)
    elif name == "decode_d256_small":
        # tensor-core decode attention at head_dim 256 (hybrid-attention layers of the 27B shape)
        B, ctx_len, Hq2, Hkv2, D2, bs2 = 64, 4096, 24, 4, 256, 32
        nb = ctx_len // bs2
        cache = torch.randn(B * nb + 1, 2, bs2, Hkv2, D2, device=dev, dtype=torch.bfloat16)
        bt = torch.arange(B * nb, device=dev, dtype=torch.int32).reshape(B, nb)
        sl = torch.full((B,), ctx_len, dtype=torch.int32, device=dev)
        q = torch.randn(B, Hq2 * D2, device=dev, dtype=torch.bfloat16)
        fn = lambda: ops.attn_decode(q, cache, block_table=bt, seq_lens=sl, num_q_heads=Hq2,
                                     num_kv_heads=Hkv2, head_dim=D2, block_size=bs2, scale=D2 ** -0.5)
    elif name == "mla_decode_small":
        from . import mla as MLA
        B, H, ctx, mbs = 128, 16, 1024, 64
        nb = ctx // mbs
        cache = torch.randn(B * nb + 1, mbs, 576, device=dev, dtype=torch.bfloat16)
        bt = torch.arange(B * nb, device=dev, dtype=torch.int32).reshape(B, nb)
        sl = torch.full((B,), ctx, dtype=torch.int32, device=dev)
        qabs = torch.randn(B, H, 576, device=dev, dtype=torch.bfloat16)
        out = torch.empty(B, H, 512, device=dev, dtype=torch.bfloat16)
        fn = lambda: MLA.mla_decode(qabs, cache, bt, sl, out, 576 ** -0.5, mbs)
    else:
        raise SystemExit(f"unknown case {name}")
    ms = _time(fn, iters=3, warmup=1)
    print(f"{name}: {ms:.4f} ms  status={ops.read_status()}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default=None)
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--case", default=None,
                    help="run one small case only (for profiler captures): "
                         "gemm_small | gemm_decode_small | prefill_small | decode_small | gdn_scan_small | "
                         "gdn_decode_small | moe_small | gemm_streamk_small | gemm_gated_small | "
                         "gemm_fp8_small | gemm_w4a16_small | gemm_nvfp4_small | gemm_nvfp4_prefill_small | "
                         "decode_d256_small | mla_decode_small")
    args = ap.parse_args()
    if args.case:
        return small_case(args.case)
    dev = torch.device("cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows = []

    def gemm_case(M, N, K, tag):
        a = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.05
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        t_ours = _time(lambda: ops.gemm(a, w, out=out), flush=flush)
        t_lib = _time(lambda: torch.matmul(a, w.t(), out=out), flush=flush)
        fl = 2.0 * M * N * K
        by = 2.0 * (M * K + N * K + M * N)
        rows.append(dict(kind="gemm_bf16", tag=tag, M=M, N=N, K=K, ms=t_ours, cublas_ms=t_lib,
                         tflops=fl / t_ours / 1e9, cublas_tflops=fl / t_lib / 1e9,
                         gbs=by / t_ours / 1e6, cublas_gbs=by / t_lib / 1e6))
        print(f"gemm {tag:>10} M={M:5d} N={N:6d} K={K:5d}: ours {t_ours:8.4f} ms "
              f"({fl / t_ours / 1e9:7.1f} TF, {by / t_ours / 1e6:6.0f} GB/s) | cuBLAS {t_lib:8.4f} ms "
              f"({fl / t_lib / 1e9:7.1f} TF)", flush=True)

    # Llama-3.1-8B projections: prefill (M=8192) and decode (M=1..256)
    shapes = [("qkv", 6144, 4096), ("o", 4096, 4096), ("gate_up", 28672, 4096),
              ("down", 4096, 14336)]
    for tag, N, K in shapes:
        for M in ([8192, 64] if args.quick else [8192, 2048, 256, 64, 8, 1]):
            gemm_case(M, N, K, tag)
    if not args.quick:
        gemm_case(256, 128256, 4096, "lm_head")
        gemm_case(8192, 8192, 8192, "square")

    # attention
    Hq, Hkv, D, bs = 32, 8, 128, 16
    for B, ctx in ([(64, 1024)] if args.quick else [(256, 1152), (64, 1024), (8, 4096), (1, 8192)]):
        nb = (ctx + bs - 1) // bs
        cache = torch.randn(B * nb + 1, 2, bs, Hkv, D, device=dev, dtype=torch.bfloat16)
        bt = torch.arange(B * nb, device=dev, dtype=torch.int32).reshape(B, nb)
        sl = torch.full((B,), ctx, dtype=torch.int32, device=dev)
        q = torch.randn(B, Hq * D, device=dev, dtype=torch.bfloat16)
        out = torch.empty_like(q)
        t = _time(lambda: ops.attn_decode(q, cache, block_table=bt, seq_lens=sl, num_q_heads=Hq,
                                          num_kv_heads=Hkv, head_dim=D, block_size=bs,
                                          scale=D ** -0.5, out=out), flush=flush)
        by = 2.0 * B * ctx * 2 * Hkv * D
        rows.append(dict(kind="attn_decode", B=B, ctx=ctx, ms=t, gbs=by / t / 1e6))
        print(f"attn_decode B={B:4d} ctx={ctx:5d}: {t:8.4f} ms ({by / t / 1e6:6.0f} GB/s)", flush=True)
        del cache
    for B, ql in ([(4, 1024)] if args.quick else [(8, 1024), (2, 4096), (1, 8192)]):
        nb = (ql + bs - 1) // bs
        cache = torch.randn(B * nb + 1, 2, bs, Hkv, D, device=dev, dtype=torch.bfloat16)
        bt = torch.arange(B * nb, device=dev, dtype=torch.int32).reshape(B, nb)
        sl = torch.full((B,), ql, dtype=torch.int32, device=dev)
        qs = torch.arange(B + 1, device=dev, dtype=torch.int32) * ql
        treq, tq0 = ref.build_prefill_tiles([ql] * B)
        treq = torch.tensor(treq, dtype=torch.int32, device=dev)
        tq0 = torch.tensor(tq0, dtype=torch.int32, device=dev)
        q = torch.randn(B * ql, Hq * D, device=dev, dtype=torch.bfloat16)
        out = torch.empty_like(q)
        t = _time(lambda: ops.attn_prefill(q, cache, block_table=bt, seq_lens=sl, q_start=qs,
                                           tile_req=treq, tile_q0=tq0, num_q_heads=Hq,
                                           num_kv_heads=Hkv, head_dim=D, block_size=bs,
                                           scale=D ** -0.5, out=out), flush=flush)
        fl = 4.0 * B * Hq * D * ql * ql / 2
        rows.append(dict(kind="attn_prefill", B=B, q_len=ql, ms=t, tflops=fl / t / 1e9))
        print(f"attn_prefill B={B} q_len={ql}: {t:8.4f} ms ({fl / t / 1e9:7.1f} TF causal)", flush=True)
        del cache
    st = ops.read_status()
    print("status word:", st)
    if args.json:
        with open(args.json, "w") as f:
            json.dump(dict(rows=rows, status=st), f, indent=1)


if __name__ == "__main__":
    main()
