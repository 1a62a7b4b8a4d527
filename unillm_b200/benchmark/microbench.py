"""Device-timed micro-benchmarks of the hot kernels (CUDA events, warm-up, L2 flush between runs).

``python -m unillm_b200.benchmark.microbench [gemm|attn|norm|all] [--json PATH]`` prints one line per
case with the achieved TFLOP/s or GB/s and the fraction of the measured peak (MEASURED_PEAKS.json
when present at the repository root).
"""
from __future__ import annotations

import argparse
import json
import math
import os
from pathlib import Path

import torch

from ..ops import cuda_ops


def _peaks():
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d.get("hbm_gbs", 6650.0), d.get("bf16_tflops", 1590.0), "measured"
    return 6650.0, 1590.0, "fallback"


_flush = None


def flush_l2():
    global _flush
    if _flush is None:
        _flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    _flush.zero_()


def time_ms(fn, iters=10, warmup=3, flush=True, reps=8):
    """Median and best device time of ``fn`` in ms, L2 flushed before every call.

    The call is captured in a CUDA graph as ``reps`` x (flush, fn) and timed against a graph of ``reps`` x flush, so
    host-side launch cost (ctypes, tensor-map encoding) never sits between the two events.  Falls back to eager
    timing when capture is not possible."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    try:
        flush_l2()
        torch.cuda.synchronize()
        s_ = torch.cuda.Stream()
        g_both, g_flush = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        with torch.cuda.stream(s_):
            with torch.cuda.graph(g_both, stream=s_):
                for _ in range(reps):
                    if flush:
                        flush_l2()
                    fn()
            with torch.cuda.graph(g_flush, stream=s_):
                for _ in range(reps):
                    if flush:
                        flush_l2()
        torch.cuda.synchronize()

        def run(g):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            g.replay()
            e.record()
            torch.cuda.synchronize()
            return s.elapsed_time(e)

        run(g_both), run(g_flush)
        ts = []
        for _ in range(iters):
            ts.append((run(g_both) - run(g_flush)) / reps)
        ts.sort()
        return ts[len(ts) // 2], ts[0]
    except Exception:
        torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush:
            flush_l2()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts) // 2], ts[0]


def bench_gemm(results, only=None, tile=0, pair=0):
    hbm, tf, how = _peaks()
    shapes = [only] if only else [
        # up to 16 tokens: the weight-streaming kernel (Llama-3-8B layer shapes, 70B shard of 8-way tensor parallelism)
        (1, 6144, 4096, 0), (1, 14336, 4096, 1), (1, 4096, 14336, 0), (4, 6144, 4096, 0), (8, 6144, 4096, 0),
        (8, 14336, 4096, 1), (16, 6144, 4096, 0), (16, 14336, 4096, 1), (16, 4096, 14336, 0), (32, 6144, 4096, 0),
        (1, 1280, 8192, 0), (1, 3584, 8192, 1), (1, 8192, 3584, 0), (1, 128256, 4096, 0),
        # (M, N, K, dual) : Llama-3-8B decode / prefill shapes
        (64, 6144, 4096, 0), (256, 6144, 4096, 0), (256, 4096, 4096, 0),
        (256, 14336, 4096, 1), (256, 4096, 14336, 0), (256, 128256, 4096, 0),
        # tensor-parallel (TP=8) per-rank decode shapes: few tiles -> cluster split-K
        (256, 768, 4096, 0), (256, 4096, 512, 0), (256, 1792, 4096, 1), (256, 4096, 1792, 0), (256, 16032, 4096, 0),
        (2048, 6144, 4096, 0), (2048, 14336, 4096, 1), (2048, 4096, 14336, 0), (8192, 8192, 8192, 0),
        # mixed decode + prefill step of the serving benchmark (about 512 token rows)
        (512, 6144, 4096, 0), (512, 4096, 4096, 0), (512, 14336, 4096, 1), (512, 4096, 14336, 0),
    ]
    for M, N, K, dual in shapes:
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(N * (2 if dual else 1), K, device="cuda", dtype=torch.bfloat16) * 0.02
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        fn = (lambda: cuda_ops.gemm_tn(x, w, dual_rows=N, act="silu", out=out, tile_tokens=tile, cta_pair=pair)) if dual else (lambda: cuda_ops.gemm_tn(x, w, out=out, tile_tokens=tile, cta_pair=pair))
        med, best = time_ms(fn)
        flops = 2.0 * M * N * K * (2 if dual else 1)
        byts = 2.0 * (w.numel() + x.numel() + out.numel())
        ref = (lambda: torch.nn.functional.silu(x @ w[:N].t()) * (x @ w[N:].t())) if dual else (lambda: x @ w.t())
        rmed, _ = time_ms(ref)
        r = dict(kind="gemm", M=M, N=N, K=K, dual=dual, ms=med, best_ms=best, tflops=flops / med / 1e9,
                 gbs=byts / med / 1e6, frac_tflops=flops / med / 1e9 / tf, frac_hbm=byts / med / 1e6 / hbm,
                 cublas_ms=rmed, peaks=how)
        results.append(r)
        print(json.dumps(r))


def gemm_timeline(shape: str, pair: int = 0, tile: int = 0):
    """Per-CTA timeline of one 1-CTA GEMM launch (needs ``UB_GEMM_DEBUG=4`` in the environment before the library is
    loaded): microseconds from the first CTA's entry to set-up done, first operand stage landed, last MMA issued,
    accumulator complete, split-K barriers / pushes / finish, and exit; mean / min / max over the CTAs of the launch."""
    import ctypes as C

    import numpy as np

    from ..ops._native import cuda_lib

    M, N, K = [int(v) for v in shape.split(",")[:3]]
    names = ["entry", "setup done", "1st stage landed", "last MMA issued", "accumulator ready", "epilogue stores issued",
             "split-K finish done", "exit", "cluster barrier 1", "partials pushed", "cluster barrier 2"]
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(3):
        flush.fill_(1)
        cuda_ops.gemm_tn(x, w, out=out, tile_tokens=tile, cta_pair=pair or 1)
        torch.cuda.synchronize()
    buf = np.zeros((512, 12), dtype=np.uint64)
    rc = cuda_lib().ub_gemm_debug_timeline(buf.ctypes.data_as(C.c_void_p))
    if rc != 0 or not (buf[:, 0] > 0).any():
        raise RuntimeError("no timeline recorded: set UB_GEMM_DEBUG=4 (the 2-CTA kernel records none: use --pair 1)")
    t = buf.astype(np.float64)
    used = (t[:, 0] > 0) & (t[:, 0] > t[:, 0].max() - 2e5)          # the CTAs of the last launch
    t0 = t[used, 0].min()
    rows = {}
    for k in (0, 1, 2, 3, 4, 5, 8, 9, 10, 6, 7):
        col = t[used, k]
        ok = col > 0
        if ok.any():
            rows[names[k]] = [round(float((col[ok].mean() - t0) / 1e3), 2), round(float((col[ok].min() - t0) / 1e3), 2),
                              round(float((col[ok].max() - t0) / 1e3), 2)]
    r = dict(kind="gemm_timeline", M=M, N=N, K=K, ctas=int(used.sum()), us_mean_min_max=rows)
    print(json.dumps(r))
    return r


def bench_attn(results, case="all"):
    hbm, tf, how = _peaks()
    decode_cases = [(256, 1152, 32, 8, 128), (64, 4096, 32, 8, 128), (256, 1152, 4, 1, 128), (8, 4096, 8, 1, 128)]
    for B, ctx, Hq, Hkv, D in (decode_cases if case in ("all", "decode") else []):
        bs = 16
        nblk = B * ((ctx + bs - 1) // bs)
        kc = torch.randn(nblk, Hkv, bs, D, device="cuda", dtype=torch.bfloat16)
        vc = torch.randn_like(kc)
        bt = torch.randperm(nblk, device="cuda").to(torch.int32).view(B, -1)
        sl = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
        q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16)
        out = torch.empty_like(q)
        scratch = torch.empty(B * Hq * 16 * (D + 2), dtype=torch.float32, device="cuda")
        med, best = time_ms(lambda: cuda_ops.attn_decode(q, kc, vc, bt, sl, out=out, scratch=scratch, max_seq_len=ctx))
        byts = 2.0 * 2 * B * ctx * Hkv * D
        r = dict(kind="attn_decode", B=B, ctx=ctx, Hq=Hq, Hkv=Hkv, D=D, ms=med, best_ms=best, gbs=byts / med / 1e6,
                 frac_hbm=byts / med / 1e6 / hbm, peaks=how)
        results.append(r)
        print(json.dumps(r))
        # one pipeline per warp, no KV split
        med, best = time_ms(lambda: cuda_ops.attn_decode(q, kc, vc, bt, sl, out=out, splits=1, kernel="warp"))
        r = dict(kind="attn_decode", kernel="warp", B=B, ctx=ctx, Hq=Hq, Hkv=Hkv, D=D, ms=med, best_ms=best,
                 gbs=byts / med / 1e6, frac_hbm=byts / med / 1e6 / hbm, peaks=how)
        results.append(r)
        print(json.dumps(r))
        # the same problem through the prefill kernels (one query token per sequence)
        qs1 = torch.arange(B + 1, dtype=torch.int32, device="cuda")
        med, best = time_ms(lambda: cuda_ops.attn_prefill(q, kc, vc, bt, sl, qs1, 1, out=out, causal=True))
        r = dict(kind="attn_decode_via_prefill", B=B, ctx=ctx, Hq=Hq, Hkv=Hkv, D=D, ms=med, best_ms=best, gbs=byts / med / 1e6,
                 frac_hbm=byts / med / 1e6 / hbm, path=cuda_ops.attn_prefill_last_path(), peaks=how)
        results.append(r)
        print(json.dumps(r))
    if case in ("all", "decode", "suffix"):
        # the suffix pass of the cascade in the serving benchmark: 256 sequences, 1024 shared keys skipped, 128..256 own
        # keys each, the shared-prefix partial folded into the output
        B, Hq, Hkv, D, bs, pre = 256, 32, 8, 128, 16, 1024
        lens = [pre + 128 + (i * 128) // B for i in range(B)]
        per = (max(lens) + bs - 1) // bs
        nblk = B * per
        kc = torch.randn(nblk, Hkv, bs, D, device="cuda", dtype=torch.bfloat16)
        vc = torch.randn_like(kc)
        bt = torch.randperm(nblk, device="cuda").to(torch.int32).view(B, per)
        sl = torch.tensor(lens, dtype=torch.int32, device="cuda")
        q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16)
        out = torch.empty_like(q)
        oa = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16)
        la = torch.randn(B, Hq, device="cuda", dtype=torch.float32)
        med, best = time_ms(lambda: cuda_ops.attn_decode(q, kc, vc, bt, sl, out=out, kv_start=pre, splits=1, merge=(oa, la)))
        byts = 2.0 * 2 * sum(l - pre for l in lens) * Hkv * D
        r = dict(kind="attn_decode_suffix", B=B, prefix=pre, suffix="128..256", Hq=Hq, Hkv=Hkv, D=D, ms=med, best_ms=best,
                 gbs=byts / med / 1e6, frac_hbm=byts / med / 1e6 / hbm, peaks=how)
        results.append(r)
        print(json.dumps(r))
        med, best = time_ms(lambda: cuda_ops.attn_decode(q, kc, vc, bt, sl, out=out, kv_start=pre, splits=1, merge=(oa, la),
                                                         kernel="warp"))
        r = dict(kind="attn_decode_suffix", kernel="warp", B=B, prefix=pre, suffix="128..256", Hq=Hq, Hkv=Hkv, D=D, ms=med,
                 best_ms=best, gbs=byts / med / 1e6, frac_hbm=byts / med / 1e6 / hbm, peaks=how)
        results.append(r)
        print(json.dumps(r))
    prefill_cases = [(2048, 2048, 32, 8, 128, True), (8192, 8192, 4, 1, 128, True), (256, 1024, 32, 8, 128, False),
                     (512, 1024, 32, 8, 128, False)]
    for T, ctx, Hq, Hkv, D, causal in (prefill_cases if case in ("all", "prefill") else []):
        bs = 16
        nblk = (ctx + bs - 1) // bs
        kc = torch.randn(nblk, Hkv, bs, D, device="cuda", dtype=torch.bfloat16)
        vc = torch.randn_like(kc)
        bt = torch.arange(nblk, device="cuda", dtype=torch.int32).view(1, -1)
        sl = torch.tensor([ctx], dtype=torch.int32, device="cuda")
        qs = torch.tensor([0, T], dtype=torch.int32, device="cuda")
        q = torch.randn(T, Hq, D, device="cuda", dtype=torch.bfloat16)
        out = torch.empty_like(q)
        med, best = time_ms(lambda: cuda_ops.attn_prefill(q, kc, vc, bt, sl, qs, T, out=out, causal=causal))
        flops = 4.0 * T * ctx * Hq * D / (2 if causal else 1)
        r = dict(kind="attn_prefill", T=T, ctx=ctx, Hq=Hq, Hkv=Hkv, D=D, causal=causal, ms=med, best_ms=best,
                 tflops=flops / med / 1e9, frac_tflops=flops / med / 1e9 / tf, path=cuda_ops.attn_prefill_last_path(),
                 peaks=how)
        results.append(r)
        print(json.dumps(r))
        if os.environ.get("UB_ATTN_DEBUG"):
            # per-tile stamps of CTA (0, 0, 0) of the last launch, SM cycles relative to the first stamp
            import ctypes as C

            import numpy as np

            from ..ops._native import cuda_lib

            buf = np.zeros((16, 10), dtype=np.uint64)
            rc = cuda_lib().ub_attn_debug_timeline(buf.ctypes.data_as(C.c_void_p))
            if rc != 0 or not buf.any():
                print(json.dumps(dict(kind="attn_prefill_timeline", error=f"nothing recorded (rc {rc})")))
            else:
                t = buf.astype(np.int64)[: min(16, (ctx + 127) // 128)]
                t0 = t[t > 0].min()
                names = ["S ready", "S in registers", "exponentials done", "previous PV done", "P published",
                         "next K landed", "next QK issued", "V landed", "P half 0 seen", "P half 1 seen"]
                tl = {n: [int(t[j, k] - t0) if t[j, k] > 0 else None for j in range(min(16, (ctx + 127) // 128))]
                      for k, n in enumerate(names)}
                print(json.dumps(dict(kind="attn_prefill_timeline", T=T, ctx=ctx, cycles=tl)))


def bench_fill(results):
    """Rate at which an SM fills its shared memory from L2 with 16 KB operand tiles: linear bulk copies against the
    tensor-map tile copies the GEMM producers issue (``csrc/common/fill_probe.cu``)."""
    import ctypes as C

    from ..ops._native import cuda_lib

    lib = cuda_lib()
    lib.ub_fill_probe.restype = C.c_int
    lib.ub_fill_probe.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
    rows, K, steps = 6144, 4096, 512                           # 50 MB: stays in L2
    buf = torch.ones(rows, K, device="cuda", dtype=torch.bfloat16)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    cyc = torch.zeros(sms, dtype=torch.int64, device="cuda")
    err = cuda_ops.err_word("cuda")
    names = ["linear bulk copy, 16 KB contiguous", "tensor-map tile {64, 128}, row pitch 8 KB", "tensor-map tile {64, 128}, tiles contiguous"]
    for mode in range(3):
        best = None
        for _ in range(4):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            n = lib.ub_fill_probe(buf.data_ptr(), rows, K, mode, steps, err.data_ptr(), cyc.data_ptr(),
                                  C.c_void_p(torch.cuda.current_stream().cuda_stream))
            e1.record()
            torch.cuda.synchronize()
            if n <= 0:
                raise RuntimeError(f"ub_fill_probe failed: {n}")
            ms = e0.elapsed_time(e1)
            best = ms if best is None else min(best, ms)
        cuda_ops.check_device_errors()
        r = dict(kind="smem_fill", mode=names[mode], ctas=n, tile_bytes=16384, tiles_per_cta=steps, us=best * 1e3,
                 tb_per_s=n * steps * 16384 / best / 1e9, bytes_per_clk_per_sm=16384.0 * steps / float(cyc.float().mean()))
        results.append(r)
        print(json.dumps(r))


def bench_fused_emulated(results, world=8, batch=512, only=None):
    """The fused tensor-parallel kernels of one layer at the serving step's per-rank shapes, with all ``world`` ranks
    emulated on ONE GPU: the peers' buffers are plain local tensors, the chain runs once for every rank (producers before
    consumers, one stream), then rank 0's kernels are timed alone -- their counters stay satisfied, so no kernel waits.
    What this measures is the kernels' own cost with the peer stores landing in local HBM instead of crossing NVLink;
    beside each one the same shape without the collective part.  ``only``: run just that kernel a few times (for ncu)."""
    from ..dist.fused import FusedComm

    hbm, tf, how = _peaks()
    H, I = 4096, 14336 // world
    Kq = (32 // world) * 128                    # o_proj: this rank's slice of the attention output
    P = max(1, batch // 128)
    T = (batch - P + P * 128) // world * world  # rows of a steady-state step, a multiple of the world size
    R = T // world
    comms = FusedComm.emulated(world, H, T, "cuda")
    g = torch.Generator(device="cpu").manual_seed(0)
    rnd = lambda *sh, sc=1.0: (torch.randn(*sh, generator=g) * sc).to(torch.bfloat16).cuda()   # noqa: E731
    a_o, w_o = rnd(T, Kq), rnd(H, Kq, sc=Kq ** -0.5)
    a_d, w_d = rnd(T, I), rnd(H, I, sc=I ** -0.5)
    w_qkv, w_gu = rnd(Kq + 2 * max(1, 8 // world) * 128, H, sc=H ** -0.5), rnd(2 * I, H, sc=H ** -0.5)
    ln = torch.ones(H, dtype=torch.bfloat16, device="cuda")
    res = rnd(R, H)
    # one pass of the whole chain for every rank: every counter that rank 0's kernels wait on is satisfied afterwards
    for c in comms:
        cuda_ops.gemm_tn(a_o, w_o, out=c.rs_local_tensor(0, R).view(world * R, H), rs=c.gemm_rs(0, R))
    for c in comms:
        cuda_ops.norm(c.rs_local_tensor(0, R), ln, residual=res, eps=1e-5, want_residual_out=True, no_out=True, T=R,
                      rs=c.norm_rs(0), ag=c.norm_ag(1), reset=c.reset_after_ag(1))
    for c in comms:
        cuda_ops.gemm_tn(a_d, w_d, out=c.rs_local_tensor(1, R).view(world * R, H), rs=c.gemm_rs(1, R))
    for c in comms:
        cuda_ops.norm(c.rs_local_tensor(1, R), ln, residual=res, eps=1e-5, want_residual_out=True, no_out=True, T=R,
                      rs=c.norm_rs(1), ag=c.norm_ag(0), reset=c.reset_after_ag(0))
    torch.cuda.synchronize()
    cuda_ops.check_device_errors()
    c0 = comms[0]
    # the pipeline zeroes every counter after its use; leave rank 0's satisfied so that each kernel can be timed alone
    from ..dist.fused import AG0, AG1, RS0, RS1

    fl = c0.buf[c0.flags.offset:c0.flags.offset + 1024].view(torch.int32)
    fl[RS0], fl[RS1] = world, world
    fl[AG0:AG0 + world] = 1
    fl[AG1:AG1 + world] = 1
    out_o = c0.rs_local_tensor(0, R).view(world * R, H)
    out_d = c0.rs_local_tensor(1, R).view(world * R, H)
    plain = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
    x1 = c0.ag_local_tensor(1, T)
    x0 = c0.ag_local_tensor(0, T)
    cases = {
        "o_proj + reduce-scatter push": (lambda: cuda_ops.gemm_tn(a_o, w_o, out=out_o, rs=c0.gemm_rs(0, R)),
                                         lambda: cuda_ops.gemm_tn(a_o, w_o, out=plain), 2.0 * T * H * Kq),
        "down + reduce-scatter push": (lambda: cuda_ops.gemm_tn(a_d, w_d, out=out_d, rs=c0.gemm_rs(1, R)),
                                       lambda: cuda_ops.gemm_tn(a_d, w_d, out=plain), 2.0 * T * H * I),
        "all-gather wait + QKV": (lambda: cuda_ops.gemm_tn(x0, w_qkv, ag=c0.gemm_ag(0, R)),
                                  lambda: cuda_ops.gemm_tn(x0, w_qkv), 2.0 * T * w_qkv.shape[0] * H),
        "all-gather wait + gate/up": (lambda: cuda_ops.gemm_tn(x1, w_gu, dual_rows=I, act="silu", ag=c0.gemm_ag(1, R)),
                                      lambda: cuda_ops.gemm_tn(x1, w_gu, dual_rows=I, act="silu"), 4.0 * T * I * H),
        "norm: sum 8 slots + residual, all-gather push": (
            lambda: cuda_ops.norm(c0.rs_local_tensor(0, R), ln, residual=res, eps=1e-5, want_residual_out=True, no_out=True,
                                  T=R, rs=c0.norm_rs(0), ag=c0.norm_ag(1)),
            lambda: cuda_ops.norm(c0.rs_local_tensor(0, R)[0], ln, residual=res, eps=1e-5, want_residual_out=True, T=R), 0.0),
    }
    if only is not None:
        fn = cases[only][0]
        for _ in range(6):
            flush_l2()
            fn()
        torch.cuda.synchronize()
        cuda_ops.check_device_errors()
        print(json.dumps(dict(kind="fused_emulated_once", case=only, world=world, T=T)))
        return
    for name, (fused, base, flops) in cases.items():
        med, best = time_ms(fused)
        bmed, _ = time_ms(base)
        r = dict(kind="fused_emulated", world=world, T=T, rows_per_rank=R, case=name, us=med * 1e3, best_us=best * 1e3,
                 unfused_us=bmed * 1e3, tflops=(flops / med / 1e9 if flops else None), peaks=how)
        results.append(r)
        print(json.dumps(r))
    torch.cuda.synchronize()
    cuda_ops.check_device_errors()


def bench_quant(results):
    """Block-quantised weights: the GEMV on Q4_K / Q8_0 blocks (1 - 8 tokens) and dequantise + tcgen05 GEMM (more tokens),
    against the bf16 kernels on the expanded matrix.  Bytes = the quantised blocks."""
    from ..ops import quant as Q
    from ..weights.gguf import Q4_K, Q8_0, quantize_blocks

    hbm, tf, how = _peaks()
    for qname, qt, bits in (("q4_k", Q4_K, 4.5), ("q8_0", Q8_0, 8.5)):
        for M, N, K in ((1, 4096, 4096), (1, 14336, 4096), (8, 6144, 4096), (1, 4096, 14336)):
            w = torch.randn(N, K) * 0.05
            raw = quantize_blocks(w, qt)
            blocks = torch.from_numpy(raw.copy()).cuda()
            x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
            med, best = time_ms(lambda: Q.qgemv_cuda(blocks, x, N, qt))
            wd = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
            out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
            dmed, _ = time_ms(lambda: cuda_ops.gemm_tn(x, wd, out=out))
            byts = float(blocks.numel() * blocks.element_size())
            r = dict(kind="qgemv", qtype=qname, M=M, N=N, K=K, ms=med, best_ms=best, gbs=byts / med / 1e6,
                     frac_hbm=byts / med / 1e6 / hbm, bf16_ms=dmed, speedup_vs_bf16=dmed / med, bits_per_weight=bits, peaks=how)
            results.append(r)
            print(json.dumps(r))


def bench_norm(results):
    hbm, tf, how = _peaks()
    for T, H in [(256, 4096), (8192, 4096), (8192, 8192)]:
        x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
        r_ = torch.randn_like(x)
        w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
        out, ro = torch.empty_like(x), torch.empty_like(x)
        med, best = time_ms(lambda: cuda_ops.norm(x, w, residual=r_, out=out, residual_out=ro))
        byts = 2.0 * 4 * T * H
        r = dict(kind="rmsnorm_residual", T=T, H=H, ms=med, best_ms=best, gbs=byts / med / 1e6,
                 frac_hbm=byts / med / 1e6 / hbm, peaks=how)
        results.append(r)
        print(json.dumps(r))


def bench_tp_layer(results, world=8, batch=512, variants=False):
    """Every kernel of one decoder layer at the per-rank shapes of ``world``-way tensor parallelism (Llama-3-8B
    architecture, the serving benchmark's steady-state step: ``batch`` decode rows that share a 1024-token prefix +
    batch/128 prefill chunks of 128 tokens), each timed alone through a CUDA graph with L2 flushed.  No communication:
    this is the compute a rank has to get through per layer."""
    hbm, tf, how = _peaks()
    H, D, bs, pre = 4096, 128, 16, 1024
    Hq, Hkv, I = 32 // world, max(1, 8 // world), 14336 // world
    P = max(1, batch // 128)
    T = batch - P + P * 128                     # rows of a steady-state step
    dev = "cuda"

    def rec(name, med, best, **kw):
        r = dict(kind="tp_layer", world=world, batch=batch, op=name, us=med * 1e3, best_us=best * 1e3, **kw)
        results.append(r)
        print(json.dumps(r))

    # ---- GEMMs ----
    gem = [("qkv", T, (Hq + 2 * Hkv) * D, H, 0), ("o_proj", T, H, Hq * D, 0), ("gate_up", T, I, H, 1), ("down", T, H, I, 0)]
    for name, M, N, K, dual in gem:
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N * (2 if dual else 1), K, device=dev, dtype=torch.bfloat16) * 0.02
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        opts = [dict()]
        if variants:
            opts += [dict(tile_tokens=t, cta_pair=1) for t in (64, 128, 256)] + [dict(cta_pair=2)] + \
                    [dict(tile_tokens=t, cta_pair=1, splits=sp) for t in (128, 256) for sp in (2, 4)] + \
                    [dict(cta_pair=2, pair_splits=sp) for sp in (2, 4)] + \
                    [dict(cta_pair=2, tile_tokens=128), dict(cta_pair=2, tile_tokens=128, pair_splits=2)]
        for o in opts:
            try:
                fn = (lambda: cuda_ops.gemm_tn(x, w, dual_rows=N, act="silu", out=out, **o)) if dual else \
                     (lambda: cuda_ops.gemm_tn(x, w, out=out, **o))
                med, best = time_ms(fn)
            except Exception as e:        # a variant the kernel does not have (e.g. split-K of a 2 x 256 gated tile)
                print(json.dumps(dict(op=name, opts=o, error=str(e)[:80])))
                continue
            flops = 2.0 * M * N * K * (2 if dual else 1)
            rec(name, med, best, M=M, N=N, K=K, dual=dual, opts=o, tflops=flops / med / 1e9,
                ctas=cuda_ops.gemm_num_ctas(M, N, K, bool(dual), o.get("tile_tokens", 0), o.get("splits", 0), o.get("cta_pair", 0)))
        ref = (lambda: torch.nn.functional.silu(x @ w[:N].t()) * (x @ w[N:].t())) if dual else (lambda: x @ w.t())
        rmed, rbest = time_ms(ref)
        rec(name + " (cuBLAS)", rmed, rbest, M=M, N=N, K=K, dual=dual)
    # ---- attention ----
    B = batch - P
    lens = [pre + 128 + (i * 128) // max(B, 1) for i in range(B)]
    per = (max(lens) + bs - 1) // bs
    nblk = pre // bs + (B + P) * (per - pre // bs) + 8
    kc = torch.randn(nblk, Hkv, bs, D, device=dev, dtype=torch.bfloat16)
    vc = torch.randn_like(kc)
    shared = torch.arange(pre // bs, dtype=torch.int32)
    own = torch.randperm(nblk - pre // bs)[: (B + P) * (per - pre // bs)].to(torch.int32).view(B + P, -1) + pre // bs
    bt = torch.cat([shared[None].expand(B + P, -1), own], 1).contiguous().to(dev)
    qkv = torch.randn(T, Hq + 2 * Hkv, D, device=dev, dtype=torch.bfloat16)
    q = qkv[:, :Hq]
    out = torch.empty(T, Hq, D, device=dev, dtype=torch.bfloat16)
    oa = torch.empty(T, Hq, D, device=dev, dtype=torch.bfloat16)
    la = torch.empty(T, Hq, device=dev, dtype=torch.float32)
    plen = torch.tensor([pre], dtype=torch.int32, device=dev)
    qs_all = torch.tensor([0, T], dtype=torch.int32, device=dev)
    G = Hq // Hkv
    ctas = -(-T // (128 // G)) * Hkv
    auto = max(1, min(pre // 128, 148 // ctas, 8))
    for kvs in sorted({1, 2, 4, 8, auto}):
        scratch = torch.empty(cuda_ops.attn_prefill_split_scratch_floats(T, Hq, D, kvs), dtype=torch.float32, device=dev)
        med, best = time_ms(lambda: cuda_ops.attn_prefill(q, kc, vc, bt[:1], plen, qs_all, T, causal=False, out=oa, lse=la,
                                                          return_lse=True, kv_splits=kvs, scratch=scratch))
        rec("attn_shared_prefix", med, best, rows=T, keys=pre, kv_splits=kvs, ctas=ctas * kvs, auto=(kvs == auto),
            tflops=4.0 * T * pre * Hq * D / med / 1e9)
    sl_d = torch.tensor(lens, dtype=torch.int32, device=dev)
    med, best = time_ms(lambda: cuda_ops.attn_decode(q[:B], kc, vc, bt[:B], sl_d, out=out[:B], kv_start=pre, splits=1,
                                                     merge=(oa[:B], la[:B])))
    byts = 2.0 * 2 * sum(l - pre for l in lens) * Hkv * D
    rec("attn_decode_suffix", med, best, B=B, gbs=byts / med / 1e6, frac_hbm=byts / med / 1e6 / hbm)
    for kern in ("warp",) if variants else ():
        med, best = time_ms(lambda: cuda_ops.attn_decode(q[:B], kc, vc, bt[:B], sl_d, out=out[:B], kv_start=pre, splits=1,
                                                         merge=(oa[:B], la[:B]), kernel=kern))
        rec("attn_decode_suffix", med, best, B=B, kernel=kern, gbs=byts / med / 1e6, frac_hbm=byts / med / 1e6 / hbm)
    sl_p = torch.full((P,), pre + 128, dtype=torch.int32, device=dev)
    qs_p = (torch.arange(P + 1, dtype=torch.int32) * 128).to(dev)
    med, best = time_ms(lambda: cuda_ops.attn_prefill(q[B:], kc, vc, bt[B:], sl_p, qs_p, 128, causal=True, kv_start=pre,
                                                      out=out[B:], merge=(oa[B:], la[B:])))
    rec("attn_prefill_suffix", med, best, seqs=P, q_len=128)
    # ---- norm, RoPE + append ----
    x = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
    r_ = torch.randn_like(x)
    w = torch.ones(H, device=dev, dtype=torch.bfloat16)
    o1, o2 = torch.empty_like(x), torch.empty_like(x)
    med, best = time_ms(lambda: cuda_ops.norm(x, w, residual=r_, out=o1, residual_out=o2))
    rec("rmsnorm_residual (all rows)", med, best, T=T, gbs=2.0 * 4 * T * H / med / 1e6)
    R = -(-T // world)
    med, best = time_ms(lambda: cuda_ops.norm(x[:R], w, residual=r_[:R], out=o1[:R], residual_out=o2[:R]))
    rec("rmsnorm_residual (rows of one rank)", med, best, T=R)
    pos = torch.randint(0, 1280, (T,), dtype=torch.int32, device=dev)
    slots = torch.randperm(nblk * bs, device=dev)[:T].to(torch.int32)
    qkv2 = qkv.view(T, -1).contiguous()
    med, best = time_ms(lambda: cuda_ops.rope_kv_append(qkv2, pos, slots, kc, vc, num_q_heads=Hq, num_kv_heads=Hkv,
                                                        head_dim=D, theta=500000.0))
    rec("rope_kv_append", med, best, T=T)
    tot = {}
    for r in results:
        if r.get("kind") == "tp_layer" and "cuBLAS" not in r["op"] and not r.get("opts") and r.get("auto", True) and \
                "all rows" not in r["op"]:
            tot[r["op"]] = r["us"]
    norm_us = tot.pop("rmsnorm_residual (rows of one rank)", 0.0)
    layer = sum(tot.values()) + 2 * norm_us
    print(json.dumps(dict(kind="tp_layer_total", world=world, batch=batch, us_per_layer=layer, ms_per_32_layers=layer * 32e-3,
                          ops=tot, norm_us_each=norm_us)))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("what", nargs="?", default="all", choices=["gemm", "attn", "norm", "tp", "quant", "fused", "fill", "all"])
    ap.add_argument("--fused-case", default=None, help="fused only: run just this kernel a few times (for a profiler)")
    ap.add_argument("--world", type=int, default=8, help="tp only: tensor-parallel size whose per-rank shapes are timed")
    ap.add_argument("--batch", type=int, default=512, help="tp only: concurrent sequences of the serving step")
    ap.add_argument("--variants", action="store_true", help="tp only: also time forced tile / pair / split-K choices")
    ap.add_argument("--attn-case", default="all", choices=["all", "decode", "prefill", "suffix"], help="subset of the attention shapes")
    ap.add_argument("--json", default=None)
    ap.add_argument("--shape", default=None, help="gemm only: M,N,K,dual -- run just this shape")
    ap.add_argument("--tile", type=int, default=0, help="gemm only: force the token-tile width")
    ap.add_argument("--timeline", default=None, help="gemm only: M,N,K -- per-CTA timeline of one launch (UB_GEMM_DEBUG=4)")
    ap.add_argument("--pair", type=int, default=0, help="gemm only: 0 auto, 1 never, 2 always use the 2-CTA kernel")
    a = ap.parse_args(argv)
    results = []
    if a.timeline:
        results.append(gemm_timeline(a.timeline, a.pair, a.tile))
        return
    if a.what == "tp":
        bench_tp_layer(results, a.world, a.batch, a.variants)
    if a.what in ("gemm", "all"):
        bench_gemm(results, tuple(int(v) for v in a.shape.split(",")) if a.shape else None, a.tile, a.pair)
    if a.what in ("attn", "all"):
        bench_attn(results, a.attn_case)
    if a.what in ("norm", "all"):
        bench_norm(results)
    if a.what == "quant":
        bench_quant(results)
    if a.what == "fused":
        bench_fused_emulated(results, a.world, a.batch, a.fused_case)
    if a.what == "fill":
        bench_fill(results)
    if a.json:
        os.makedirs(os.path.dirname(a.json) or ".", exist_ok=True)
        Path(a.json).write_text(json.dumps(results, indent=1))


if __name__ == "__main__":
    main()
