"""Per-kernel timing at the shapes of the served workloads, with roofline fractions.

    python -m acache_b200.microbench [name ...] [--iters N] [--json]

Each case builds seeded synthetic inputs on the GPU (working sets larger than the 126 MB
L2 where the kernel is bandwidth-bound, or an L2 flush between iterations), warms up,
times ``iters`` launches with CUDA events on the launching stream and prints the
algorithmic bytes or FLOPs per launch, the achieved rate and its fraction of the
measured peak (``MEASURED_PEAKS.json`` beside the repository root when present).
It is also the small, single-kernel program used for profiler captures.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

from . import _lib, ops
from .model import acache_attention as aa
from .model import attention as att
from .model.modeling_common import build_rope_table

ROOT = Path(__file__).resolve().parents[1]
DEV = "cuda"


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def _time(fn, iters, flush=None, warmup=3):
    for _ in range(warmup):
        if flush is not None:
            flush.zero_()
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters * 1e-3


def _flush_buffer():
    return torch.empty(256 << 20, dtype=torch.uint8, device=DEV)


def case_relocate(L, A, hkv, D, R, dtype, shifts_hi, Bk=256):
    """Affix relocation + RoPE for R requests: source read once, R rotated copies written."""
    nb = -(-A // Bk) * (R + 1)
    k = torch.randn(L, nb * Bk, hkv, D, device=DEV, dtype=dtype)
    v = torch.randn_like(k)
    cos, sin = build_rope_table(shifts_hi + 1, D, 500000.0, torch.float32, DEV)
    g = torch.Generator().manual_seed(0)
    shifts = torch.randint(1, shifts_hi, (R,), generator=g).to(torch.int32).to(DEV)
    per = -(-A // Bk)
    tables = torch.arange(per, per * (R + 1), dtype=torch.int32, device=DEV).view(R, per)
    es = k.element_size()
    nbytes = 2 * L * A * hkv * D * es * (1 + R)
    fn = lambda: aa.relocate_affix_batched(k, v, cos, sin, A, shifts, dst_block_tables=tables, block_size=Bk)
    return fn, dict(bytes=nbytes, unit_bytes_per_request=4 * L * A * hkv * D * es)


def case_store(N, hkv, D, dtype):
    nb = N // 256 + 2
    key = torch.randn(N, hkv, D, device=DEV, dtype=dtype)
    val = torch.randn_like(key)
    kc = torch.zeros(nb, 256, hkv, D, device=DEV, dtype=dtype)
    vc = torch.zeros_like(kc)
    slots = torch.randperm(nb * 256, device=DEV)[:N].to(torch.int32)
    fn = lambda: att.store_kvcache(key, val, kc, vc, slots)
    return fn, dict(bytes=4 * N * hkv * D * key.element_size())


def case_attention(B, q_len, kv_lo, kv_hi, nh, hkv, D, dtype=torch.bfloat16, affix=0, seed=0, layout="logical",
                   grouped=False):
    """``affix`` > 0: slots 0..affix-1 are the shared span, every 5th of its tokens is an anchor
    with a private copy.  layout "logical": keys in position order (anchors interrupt the span
    every 5 slots); "runs": the span as one run with holes, then the private slots (what the
    engine hands over in block decode, together with ``grouped``: the span is staged once per
    four requests)."""
    g = torch.Generator().manual_seed(seed)
    kv_lens = torch.randint(kv_lo, kv_hi + 1, (B,), generator=g).tolist()
    Bk = 256
    k_anchor = len(range(2, affix, 5)) if affix else 0
    nb = sum(-(-(n + k_anchor) // Bk) for n in kv_lens) + 8
    kc = torch.randn(nb, Bk, hkv, D, device=DEV, dtype=dtype)
    vc = torch.randn_like(kc)
    q = torch.randn(B * q_len, nh, D, device=DEV, dtype=dtype)
    cu_q = torch.arange(0, (B + 1) * q_len, q_len, dtype=torch.int32, device=DEV)
    maps, spans, blk = [], [], -(-affix // Bk) if affix else 0
    for n in kv_lens:
        own = n - affix
        c = -(-(own + k_anchor) // Bk)
        private = (torch.arange(c * Bk) + blk * Bk)[: own + k_anchor]
        blk += c
        span = torch.arange(affix)
        if layout == "runs":
            span[2:affix:5] = -1
            maps.append(torch.cat([span, private]))
        else:
            span[2:affix:5] = private[:k_anchor]
            maps.append(torch.cat([span, private[k_anchor:]]))
        spans.append(affix)
    cu_k = torch.zeros(B + 1, dtype=torch.int32)
    cu_k[1:] = torch.cumsum(torch.tensor([m.numel() for m in maps]), 0)
    rsm = torch.cat(maps).to(torch.int32).to(DEV)
    split = torch.tensor(spans, dtype=torch.int32, device=DEV) if (affix and layout == "runs") else None
    es = q.element_size()
    flops = sum(4.0 * q_len * n * nh * D for n in kv_lens)
    nbytes = sum(2.0 * n * hkv * D * es + 2.0 * q_len * nh * D * es for n in kv_lens)
    cu_k = cu_k.to(DEV)
    fn = lambda: aa.acache_attention(q, kc, vc, cu_q, cu_k, rsm, None, 0, split, max_seqlen_q=q_len,
                                     max_seqlen_k=max(kv_lens), group_shared_span=grouped)
    return fn, dict(bytes=nbytes, flops=flops)


def case_topk(B, A, k):
    s = torch.randn(B, A, device=DEV)
    fn = lambda: ops.anchor_topk(s, k, True)
    return fn, dict(bytes=B * (4 * A + 8 * k))


def case_importance(nq, nh, hkv, D, A, shift):
    q = torch.randn(nq + 160, nh, D, device=DEV, dtype=torch.bfloat16)
    rows = torch.arange(160, 160 + nq, dtype=torch.int32, device=DEV)
    kc = torch.randn(A, hkv, D, device=DEV, dtype=torch.bfloat16)
    cos, sin = build_rope_table(max(shift + 1, 2), D, 500000.0, torch.float32, DEV)
    imp = torch.zeros(A, device=DEV)
    fn = lambda: ops.anchor_importance(q, rows, kc, shift, cos, sin, D ** -0.5, imp)
    return fn, dict(flops=2.0 * 2 * nh * nq * A * D)  # two passes over the scores


def case_transfer(R, T, V):
    logits = torch.randn(R * T, V, device=DEV, dtype=torch.bfloat16)
    blocks = torch.full((R, T), 126336, dtype=torch.int64, device=DEV)
    work = blocks.clone()

    def fn():
        work.copy_(blocks)
        ops.transfer_tokens(logits, work, 126336, 0.9)

    return fn, dict(bytes=R * T * V * 2)


def case_rope_store(n, nh, hkv, D):
    qkv = torch.randn(n, (nh + 2 * hkv) * D, device=DEV, dtype=torch.bfloat16)
    q, k, v = (qkv[:, : nh * D].view(n, nh, D), qkv[:, nh * D: (nh + hkv) * D].view(n, hkv, D),
               qkv[:, (nh + hkv) * D:].view(n, hkv, D))
    pos = torch.randint(0, 1300, (n,), device=DEV)
    cos, sin = build_rope_table(2048, D, 500000.0, torch.float32, DEV)
    nb = n // 256 + 2
    kc = torch.zeros(nb, 256, hkv, D, device=DEV, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    slots = torch.randperm(nb * 256, device=DEV)[:n].to(torch.int32)
    fn = lambda: ops.rope_store(q, k, v, pos, cos, sin, kc, vc, slots)
    return fn, dict(bytes=n * D * 2 * (2 * nh + 2 * hkv + 2 * hkv + hkv))  # q,k rw; k,v cache w; v r


def case_act_mul(n, ffn):
    gate = torch.randn(n, ffn, device=DEV, dtype=torch.bfloat16)
    up = torch.randn_like(gate)
    fn = lambda: ops.act_mul(gate, up, "silu")
    return fn, dict(bytes=3 * n * ffn * 2)


def case_add_rmsnorm(n, hidden):
    x = torch.randn(n, hidden, device=DEV, dtype=torch.bfloat16)
    d = torch.randn_like(x)
    w = torch.ones(hidden, device=DEV, dtype=torch.bfloat16)
    fn = lambda: ops.add_rmsnorm(x, d, w, 1e-5)
    return fn, dict(bytes=4 * n * hidden * 2)


def case_qkv(n, hidden, nh, hkv, D, fused):
    import torch.nn.functional as F

    x = torch.randn(n, hidden, device=DEV, dtype=torch.bfloat16)
    w = torch.randn((nh + 2 * hkv) * D, hidden, device=DEV, dtype=torch.bfloat16) * hidden ** -0.5
    pos = torch.randint(0, 1300, (n,), device=DEV)
    cos, sin = build_rope_table(2048, D, 500000.0, torch.float32, DEV)
    nb = n // 256 + 2
    kc = torch.zeros(nb, 256, hkv, D, device=DEV, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    slots = torch.randperm(nb * 256, device=DEV)[:n].to(torch.int32)

    def unfused():
        qkv = F.linear(x, w)
        q, k, v = (qkv[:, : nh * D].view(n, nh, D), qkv[:, nh * D: (nh + hkv) * D].view(n, hkv, D),
                   qkv[:, (nh + hkv) * D:].view(n, hkv, D))
        ops.rope_store(q, k, v, pos, cos, sin, kc, vc, slots)

    fn = (lambda: ops.qkv_rope_scatter(x, w, None, nh, hkv, D, pos, cos, sin, kc, vc, slots)) if fused else unfused
    return fn, dict(flops=2.0 * n * hidden * (nh + 2 * hkv) * D, bytes=2.0 * (nh + 2 * hkv) * D * hidden)


def case_linear(kind, M, K=4096, nh=32, hkv=32, D=128, ffn=12288, vocab=126464):
    """One fused projection of this package at the LLaDA-8B sizes: "qkv" (+ RoPE + cache scatter),
    "gate_up" (+ gated activation), "head" (+ arg-max statistics), "plain" (K -> 4096), "sliced"
    (K -> 4096 with the K range cut into the planned number of slices, fp32 partial sums)."""
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    if kind == "qkv":
        N = (nh + 2 * hkv) * D
        w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * K ** -0.5
        pos = torch.randint(0, 1300, (M,), device=DEV)
        cos, sin = build_rope_table(2048, D, 500000.0, torch.float32, DEV)
        nb = M // 256 + 2
        kc = torch.zeros(nb, 256, hkv, D, device=DEV, dtype=torch.bfloat16)
        vc = torch.zeros_like(kc)
        slots = torch.randperm(nb * 256, device=DEV)[:M].to(torch.int32)
        fn = lambda: ops.linear_qkv_rope_scatter(x, w, None, nh, hkv, D, pos, cos, sin, kc, vc, slots)
    elif kind == "gate_up":
        N = 2 * ffn
        w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * K ** -0.5
        fn = lambda: ops.linear_swiglu(x, w, "silu")
    elif kind == "head":
        N = vocab
        w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * K ** -0.5
        fn = lambda: ops.linear_argmax(x, w)
    elif kind == "sliced":
        N = 4096
        w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * K ** -0.5
        fn = lambda: ops.linear_partials(x, w)
    else:
        N = 4096
        w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * K ** -0.5
        fn = lambda: ops.linear(x, w)
    return fn, dict(flops=2.0 * M * N * K, bytes=2.0 * N * K + 2.0 * M * K)


def gemm_sweep(iters=10, shapes=None, tiles=None):
    """Projection shapes of the served models: this package's CTA-pair GEMM at several tile
    shapes against the library GEMM.  Back-to-back launches over 8 rotating weight copies (so the
    weights come from HBM, as in a model), one event pair around ``8 * iters`` launches."""
    import torch.nn.functional as F

    shapes = shapes or [("qkv/gate/up decode", 512, 4096, 12288), ("attn_out decode", 512, 4096, 4096),
                        ("ff_out decode", 512, 12288, 4096), ("gate+up decode", 512, 4096, 24576),
                        ("qkv refresh", 2304, 4096, 12288), ("ff_out refresh", 2304, 12288, 4096),
                        ("head decode", 512, 4096, 126464), ("qkv dream decode", 1024, 3584, 4608),
                        ("ff_out dream decode", 1024, 18944, 3584)]
    tiles = tiles or [(0, 0), (1, 256), (1, 176), (1, 128), (1, 112), (2, 256), (2, 176), (2, 128), (2, 112)]
    _, tf, src = peaks()
    for name, M, K, N in shapes:
        copies = max(2, min(8, int((1 << 30) // (N * K * 2))))
        x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
        ws = [torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * K ** -0.5 for _ in range(copies)]
        flops = 2.0 * M * N * K

        def timeit(fn):
            for w in ws[:2]:
                fn(w)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                for w in ws:
                    fn(w)
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) * 1e-3 / (iters * copies)

        t_lib = timeit(lambda w: F.linear(x, w))
        print(f"{name:22s} M={M} K={K} N={N}  library {t_lib * 1e6:8.1f} us {flops / t_lib / 1e12:7.1f} TFLOP/s", flush=True)
        for tile in tiles:
            ops.GEMM_TILE = tile
            try:
                t = timeit(lambda w: ops.linear(x, w))
                print(f"    tile {tile}: {t * 1e6:8.1f} us {flops / t / 1e12:7.1f} TFLOP/s  {t_lib / t:5.2f}x library"
                      f"  {flops / t / 1e12 / tf:5.2f} of {src} burst peak", flush=True)
            except (NotImplementedError, _lib.AcacheError) as exc:
                print(f"    tile {tile}: {exc}", flush=True)
            finally:
                ops.GEMM_TILE = (0, 0)
        del ws, x
        torch.cuda.empty_cache()
    _lib.check_device_errors()


def sliced_sweep(iters=10):
    """The plain projections of a block at block-decode row counts, each followed by the
    residual-add + RMSNorm kernel that consumes it: library GEMM against this package's GEMM with
    the K range cut into slices (``ops.linear_partials``) at several slice counts and tiles.
    Back-to-back launches over rotating weight copies, replayed as a CUDA graph, one event pair
    around all replays."""
    import torch.nn.functional as F

    shapes = [("attn_out decode", 512, 4096, 4096), ("ff_out decode", 512, 12288, 4096),
              ("attn_out decode, 8 requests", 256, 4096, 4096), ("ff_out decode, 8 requests", 256, 12288, 4096),
              ("o_proj dream decode", 1024, 3584, 3584), ("down_proj dream decode", 1024, 18944, 3584)]
    for name, M, K, N in shapes:
        copies = max(2, min(8, int((1 << 30) // (N * K * 2))))
        x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
        ws = [torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * K ** -0.5 for _ in range(copies)]
        res = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
        nw = torch.ones(N, device=DEV, dtype=torch.bfloat16)

        def timeit(fn):
            # the launches of one pass over the weight copies as a CUDA graph: two small kernels per
            # projection would otherwise be timed at the host's launch rate
            for w in ws[:2]:
                fn(w)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for w in ws:
                    fn(w)
            graph.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) * 1e-3 / (iters * copies)

        t_lib = timeit(lambda w: F.linear(x, w))
        t_lib2 = timeit(lambda w: ops.add_rmsnorm(res, F.linear(x, w), nw, 1e-5))
        planned = ops.linear_partials_splits(M, K, N)
        print(f"{name:30s} M={M} K={K} N={N}  library {t_lib * 1e6:7.1f} us, + add_rmsnorm {t_lib2 * 1e6:7.1f} us;"
              f" planned slices {planned}", flush=True)
        for tile in ((1, 256), (1, 240), (2, 256)):
            if tile[0] == 2 and M <= 256:
                continue
            for s in (1, 2, 4):
                try:
                    t = timeit(lambda w: ops.linear_partials(x, w, s, tile))
                    t2 = timeit(lambda w: ops.add_rmsnorm(res, ops.linear_partials(x, w, s, tile), nw, 1e-5))
                    print(f"    tile {tile} slices {s}: {t * 1e6:7.1f} us ({t_lib / t:4.2f}x library), "
                          f"+ add_rmsnorm {t2 * 1e6:7.1f} us ({t_lib2 / t2:4.2f}x)", flush=True)
                except (NotImplementedError, _lib.AcacheError) as exc:
                    print(f"    tile {tile} slices {s}: {exc}", flush=True)
        del ws, x
        torch.cuda.empty_cache()
    _lib.check_device_errors()


def mma_rate():
    """Rate at which one issuing thread's tcgen05.mma stream is retired (no memory traffic): per
    product width N, CTA group, number of alternating accumulators, commits and k steps per loop."""
    lib = _lib.load()
    out = torch.zeros(4, dtype=torch.int64, device=DEV)
    for cg in (1, 2):
        for n in (64, 128, 256):
            for nacc in (1, 2):
                for ce in (0, 1):
                    for kper in (4, 8):
                        _lib.check(lib.acache_diag_mma_rate(cg, n, nacc, ce, kper, 2000, _lib.ptr(out), _lib.stream_ptr()),
                                   "diag_mma_rate")
                        clk, ns, issued, done = out.tolist()
                        units = 74 if cg == 2 else 148
                        flop = issued * 2.0 * (256 if cg == 2 else 128) * n * 16
                        print(f"cta_group {cg} N={n:3d} accumulators {nacc} commit every {ce} k steps {kper}: "
                              f"{clk / issued:6.1f} cycles and {ns / issued:6.1f} ns per product at {clk / ns:.2f} GHz"
                              f" = {flop / (ns * 1e-9) / 1e12 * units:7.1f} TFLOP/s over the GPU"
                              f"{'' if done else '  (final wait ran out)'}", flush=True)


def fused_sweep(iters=10):
    """The fused projections of a block against the library GEMM followed by the separate kernel,
    at the decode (512 rows) and refresh (2304 rows) sizes of the LLaDA-8B workload; back-to-back
    launches over rotating weight copies, one event pair around all of them."""
    import torch.nn.functional as F

    D, nh, hkv, hidden, ffn, vocab = 128, 32, 32, 4096, 12288, 126464
    cos, sin = build_rope_table(2048, D, 500000.0, torch.float32, DEV)

    def timeit(fn, ws):
        for w in ws[:2]:
            fn(w)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            for w in ws:
                fn(w)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / (iters * len(ws))

    for M in (512, 2304):
        x = torch.randn(M, hidden, device=DEV, dtype=torch.bfloat16)
        pos = torch.randint(0, 1300, (M,), device=DEV)
        nb = M // 256 + 2
        kc = torch.zeros(nb, 256, hkv, D, device=DEV, dtype=torch.bfloat16)
        vc = torch.zeros_like(kc)
        slots = torch.randperm(nb * 256, device=DEV)[:M].to(torch.int32)
        # --- QKV
        ws = [torch.randn((nh + 2 * hkv) * D, hidden, device=DEV, dtype=torch.bfloat16) * hidden ** -0.5 for _ in range(8)]

        def lib_qkv(w):
            qkv = F.linear(x, w)
            q, k, v = (qkv[:, : nh * D].view(M, nh, D), qkv[:, nh * D: (nh + hkv) * D].view(M, hkv, D),
                       qkv[:, (nh + hkv) * D:].view(M, hkv, D))
            ops.rope_store(q, k, v, pos, cos, sin, kc, vc, slots)

        t_lib = timeit(lib_qkv, ws)
        print(f"M={M} qkv + rope + scatter: library GEMM + kernel {t_lib:7.1f} us", flush=True)
        for tile in [(0, 0), (1, 256), (2, 176), (1, 176), (2, 128)]:
            ops.GEMM_TILE = tile
            t = timeit(lambda w: ops.linear_qkv_rope_scatter(x, w, None, nh, hkv, D, pos, cos, sin, kc, vc, slots), ws)
            print(f"    fused, tile {tile}: {t:7.1f} us  {t_lib / t:5.2f}x", flush=True)
        ops.GEMM_TILE = (0, 0)
        del ws
        # --- gate / up
        ws = [torch.randn(2 * ffn, hidden, device=DEV, dtype=torch.bfloat16) * hidden ** -0.5 for _ in range(4)]
        t_lib = timeit(lambda w: ops.act_mul_halves(F.linear(x, w), "silu"), ws)
        print(f"M={M} gate/up + activation: library GEMM + kernel {t_lib:7.1f} us", flush=True)
        for tile in [(0, 0), (1, 256), (1, 224), (2, 176), (2, 128)]:
            ops.GEMM_TILE = tile
            t = timeit(lambda w: ops.linear_swiglu(x, w, "silu"), ws)
            print(f"    fused, tile {tile}: {t:7.1f} us  {t_lib / t:5.2f}x", flush=True)
        ops.GEMM_TILE = (0, 0)
        del ws
        torch.cuda.empty_cache()
    # --- output head on 512 rows
    M = 512
    x = torch.randn(M, hidden, device=DEV, dtype=torch.bfloat16)
    ws = [torch.randn(vocab, hidden, device=DEV, dtype=torch.bfloat16) * hidden ** -0.5 for _ in range(2)]
    blocks = torch.full((16, 32), 126336, dtype=torch.int64, device=DEV)

    def lib_head(w):
        ops.transfer_tokens(F.linear(x, w), blocks.clone(), 126336, 0.9)

    def own_head(w):
        x0, conf = ops.linear_argmax(x, w)
        ops.apply_transfer(x0, conf, blocks.clone(), 126336, 0.9)

    t_lib = timeit(lib_head, ws)
    print(f"M={M} output head + unmasking: library GEMM + kernels {t_lib:7.1f} us", flush=True)
    for tile in [(0, 0), (2, 256), (1, 256), (2, 128)]:
        ops.GEMM_TILE = tile
        t = timeit(own_head, ws)
        print(f"    fused, tile {tile}: {t:7.1f} us  {t_lib / t:5.2f}x", flush=True)
    ops.GEMM_TILE = (0, 0)
    _lib.check_device_errors()


CASES = {
    # name: (builder, bound)
    "relocate_cfg1_fp32": (lambda: case_relocate(2, 512, 8, 128, 4, torch.float32, 1024), "hbm"),
    "relocate_dream_infix": (lambda: case_relocate(28, 600, 4, 128, 32, torch.bfloat16, 128), "hbm"),
    "relocate_llada_800": (lambda: case_relocate(32, 800, 32, 128, 4, torch.bfloat16, 1024), "hbm"),
    "relocate_llada_8192_1req": (lambda: case_relocate(8, 8192, 32, 128, 1, torch.bfloat16, 4104), "hbm"),
    "store_refresh_llada": (lambda: case_store(4 * 576, 32, 128, torch.bfloat16), "hbm"),
    "rope_store_decode_llada": (lambda: case_rope_store(512, 32, 32, 128), "hbm"),
    "rope_store_refresh_llada": (lambda: case_rope_store(4 * 576, 32, 32, 128), "hbm"),
    "attention_decode_llada": (lambda: case_attention(16, 32, 1120, 1312, 32, 32, 128, affix=800, layout="runs",
                                                      grouped=True), "hbm"),
    "attention_decode_llada_per_request": (lambda: case_attention(16, 32, 1120, 1312, 32, 32, 128, affix=800), "hbm"),
    "attention_decode_llada_runs_per_request": (lambda: case_attention(16, 32, 1120, 1312, 32, 32, 128, affix=800,
                                                                       layout="runs"), "hbm"),
    "attention_decode_dream": (lambda: case_attention(32, 32, 920, 1112, 28, 4, 128, affix=600), "hbm"),
    "attention_decode_long": (lambda: case_attention(64, 8, 9224, 12296, 32, 32, 128, affix=8192, layout="runs",
                                                     grouped=True), "hbm"),
    "attention_decode_long_per_request": (lambda: case_attention(64, 8, 9224, 12296, 32, 32, 128, affix=8192), "hbm"),
    "attention_refresh_llada": (lambda: case_attention(4, 576, 1120, 1312, 32, 32, 128, affix=800), "tensor"),
    "attention_refresh_long": (lambda: case_attention(2, 3400, 9224, 12296, 32, 32, 128, affix=8192), "tensor"),
    "attention_prefill_8192": (lambda: case_attention(1, 8192, 8192, 8192, 32, 32, 128), "tensor"),
    "qkv_fused_decode_llada": (lambda: case_qkv(512, 4096, 32, 32, 128, True), "tensor"),
    "qkv_cublas_decode_llada": (lambda: case_qkv(512, 4096, 32, 32, 128, False), "tensor"),
    "qkv_fused_refresh_llada": (lambda: case_qkv(2304, 4096, 32, 32, 128, True), "tensor"),
    "qkv_cublas_refresh_llada": (lambda: case_qkv(2304, 4096, 32, 32, 128, False), "tensor"),
    "qkv_fused_decode_dream": (lambda: case_qkv(1024, 3584, 28, 4, 128, True), "tensor"),
    "qkv_cublas_decode_dream": (lambda: case_qkv(1024, 3584, 28, 4, 128, False), "tensor"),
    "linear_qkv_decode_llada": (lambda: case_linear("qkv", 512), "tensor"),
    "linear_qkv_refresh_llada": (lambda: case_linear("qkv", 2304), "tensor"),
    "linear_gate_up_decode_llada": (lambda: case_linear("gate_up", 512), "tensor"),
    "linear_gate_up_refresh_llada": (lambda: case_linear("gate_up", 2304), "tensor"),
    "linear_head_decode_llada": (lambda: case_linear("head", 512), "tensor"),
    "linear_plain_decode_llada": (lambda: case_linear("plain", 512), "tensor"),
    "linear_sliced_ff_out_decode_llada": (lambda: case_linear("sliced", 512, K=12288), "tensor"),
    "act_mul_decode_llada": (lambda: case_act_mul(512, 12288), "hbm"),
    "add_rmsnorm_decode_llada": (lambda: case_add_rmsnorm(512, 4096), "hbm"),
    "topk_cfg1": (lambda: case_topk(4, 512, 103), "latency"),
    "topk_llada_bs16": (lambda: case_topk(16, 800, 160), "latency"),
    "topk_long_bs64": (lambda: case_topk(64, 8192, 820), "latency"),
    "importance_llada": (lambda: case_importance(256, 32, 32, 128, 800, 0), "tensor"),
    "importance_long": (lambda: case_importance(8, 32, 32, 128, 8192, 2000), "tensor"),
    "transfer_tokens_llada": (lambda: case_transfer(16, 32, 126464), "hbm"),
}


def run(names, iters, as_json=False):
    hbm, tf, src = peaks()
    flush = _flush_buffer()
    results = {}
    for name in names:
        build, bound = CASES[name]
        fn, work = build()
        sec = _time(fn, iters, flush)
        rec = dict(us=sec * 1e6, bound=bound)
        if "bytes" in work:
            rec["GBps"] = work["bytes"] / sec / 1e9
            rec["hbm_frac"] = rec["GBps"] / hbm
        if "flops" in work:
            rec["TFLOPs"] = work["flops"] / sec / 1e12
            rec["tensor_frac"] = rec["TFLOPs"] / tf
        rec.update({k: v for k, v in work.items()})
        results[name] = rec
        if not as_json:
            extra = " ".join(f"{k}={v:.4g}" for k, v in rec.items() if isinstance(v, float))
            print(f"{name:28s} {extra}  [{bound}, peaks {src}]", flush=True)
        del fn
        torch.cuda.empty_cache()
    _lib.check_device_errors()
    if as_json:
        print(json.dumps(dict(peaks=dict(hbm_gbs=hbm, bf16_tflops=tf, source=src), results=results)))
    return results


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("names", nargs="*")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--mma-rate", action="store_true", help="issue rate of a stream of tcgen05.mma without memory traffic")
    ap.add_argument("--sliced-sweep", action="store_true",
                    help="plain projections with the K range cut into slices (+ the norm kernel that adds them)")
    ap.add_argument("--fused-sweep", action="store_true", help="fused projections against library GEMM + separate kernel")
    ap.add_argument("--gemm-sweep", action="store_true", help="projection GEMMs at several tile shapes against the library")
    args = ap.parse_args(argv)
    if args.gemm_sweep:
        gemm_sweep(args.iters)
        return
    if args.sliced_sweep:
        sliced_sweep(args.iters)
        return
    if args.fused_sweep:
        fused_sweep(args.iters)
        return
    if args.mma_rate:
        mma_rate()
        return
    names = args.names or list(CASES)
    for n in names:
        if n not in CASES:
            sys.exit(f"unknown case {n}; choose from {', '.join(CASES)}")
    run(names, args.iters, args.json)


if __name__ == "__main__":
    main()
