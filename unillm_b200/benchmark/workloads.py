"""The five benchmark workloads (one request mix each) and a runner that reports output tok/s, p50 TTFT / TPOT and
the engine's cache statistics as one JSON line per run.

    python -m unillm_b200.benchmark.workloads --config 1                      # CPU, TinyLlama architecture, fp32
    python -m torch.distributed.run --nproc-per-node 8 -m unillm_b200.benchmark.workloads --config 2
    ... --config 3 (Mixtral, expert parallel), 4 (shared-prefix), 5 (70B decode sweep)

``--scale`` shrinks request counts (and, below 0.05, the models) so that every workload also runs as a smoke test.
Multi-GPU numbers are timed on the device (CUDA events around every engine step, max over ranks); the CPU workload
is timed with the wall clock.  Results are appended to ``--out`` (JSON lines) so that a sweep can resume.

The reference's own harness measures one prompt at a time on the CPU (``benchmark/runner.rs:51-130``); these
workloads measure the serving engine.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from typing import Dict, List, Optional

import torch

ARCH = {
    "tinyllama": dict(vocab_size=32000, hidden_size=2048, intermediate_size=5632, num_hidden_layers=22, num_attention_heads=32,
                      num_key_value_heads=4, rope_theta=10000.0, rms_norm_eps=1e-5, max_position_embeddings=2048),
    "llama2-7b": dict(vocab_size=32000, hidden_size=4096, intermediate_size=11008, num_hidden_layers=32, num_attention_heads=32,
                      num_key_value_heads=32, rope_theta=10000.0, rms_norm_eps=1e-5, max_position_embeddings=4096),
    "llama3-8b": dict(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32,
                      num_key_value_heads=8, rope_theta=500000.0, rms_norm_eps=1e-5, max_position_embeddings=8192),
    "llama3-70b": dict(vocab_size=128256, hidden_size=8192, intermediate_size=28672, num_hidden_layers=80, num_attention_heads=64,
                       num_key_value_heads=8, rope_theta=500000.0, rms_norm_eps=1e-5, max_position_embeddings=8192),
    "mixtral-8x7b": dict(vocab_size=32000, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32,
                         num_key_value_heads=8, rope_theta=1000000.0, rms_norm_eps=1e-5, max_position_embeddings=32768,
                         num_experts=8, num_experts_per_tok=2, sliding_window=32768),
}


def shrink(arch: dict, world: int) -> dict:
    """A small model of the same family (smoke tests)."""
    a = dict(arch)
    a.update(vocab_size=4096, hidden_size=512, intermediate_size=1024, num_hidden_layers=2, num_attention_heads=8,
             num_key_value_heads=8 if arch["num_key_value_heads"] == arch["num_attention_heads"] else max(world, 4))
    return a


def percentile(xs: List[float], q: float) -> Optional[float]:
    if not xs:
        return None
    s = sorted(xs)
    return s[min(len(s) - 1, int(q * len(s)))]


def build_engine(arch_name: str, world: int, rank: int, group, device: str, *, max_seqs: int, max_len: int, blocks: int,
                 max_tokens: int = 8192, small: bool = False, fused: bool = True, graphs: bool = True,
                 async_scheduling: bool = True):
    from ..engine.llm_engine import LLMEngine
    from ..engine.runner import GpuModelRunner, RunnerWeights, TpContext
    from ..models import configs as C
    from ..models.families import LlamaModel, MixtralModel

    arch = shrink(ARCH[arch_name], world) if small else ARCH[arch_name]
    moe = "num_experts" in arch
    cfg = (C.MixtralConfig if moe else C.LlamaConfig)(**arch)
    spec = (MixtralModel if moe else LlamaModel).spec_from_config(cfg)
    tp = TpContext(rank, world, group, fused=fused)
    w = RunnerWeights.random(spec, device, rank, world, seed=1234, expert_parallel=moe)
    if tp.fused:
        from ..dist.fused import FusedComm

        tp.comm = FusedComm.create(spec, rank, world, group, max_tokens=max_tokens + max_seqs, device=device)
    runner = GpuModelRunner(spec, w, num_blocks=blocks, block_size=16, max_num_seqs=max_seqs, max_num_batched_tokens=max_tokens,
                            max_model_len=max_len, tp=tp, device=device, use_cuda_graphs=graphs)
    eng = LLMEngine(runner, num_blocks=blocks, block_size=16, max_num_seqs=max_seqs, max_num_batched_tokens=max_tokens,
                    max_model_len=max_len, enable_prefix_caching=True, async_scheduling=async_scheduling)
    return eng, runner, cfg, w


def serve(eng, requests: List[dict], device: Optional[str], dist_group=None, world: int = 1, health=None) -> Dict:
    """Runs the requests (dicts: prompt, max_tokens, arrival seconds) to completion; returns aggregate metrics.

    ``health``: an optional ``dist.health.FailureDetector``; its ``check()`` runs on the host before every step, so a
    peer whose heartbeat has stopped ends the run with ``RankFailure`` before the next launch."""
    from ..sampling import SamplingParams

    cuda = device is not None and device.startswith("cuda")
    pending = sorted(requests, key=lambda r: r.get("arrival", 0.0))
    t0 = time.perf_counter()
    ids, evs, nxt, steps = [], [], 0, 0
    while nxt < len(pending) or eng.has_unfinished():
        now = time.perf_counter() - t0
        while nxt < len(pending) and pending[nxt].get("arrival", 0.0) <= now:
            r = pending[nxt]
            ids.append(eng.add_request(r["prompt"], SamplingParams(temperature=0.0, max_tokens=r["max_tokens"], ignore_eos=True)))
            nxt += 1
        if not eng.has_unfinished():
            time.sleep(min(0.001, max(0.0, pending[nxt]["arrival"] - now)))
            continue
        e = None
        if cuda:
            e = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            eng.step_events = e
        if health is not None:
            health.check()
        eng.step()
        if e is not None and eng.step_events is None:
            evs.append(e)                    # recorded: the step launched work (a drain-only step does not)
        steps += 1
    if cuda:
        torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    eng.step_events = None
    dev_s = sum(a.elapsed_time(b) for a, b in evs) / 1e3 if cuda else wall
    if world > 1:
        import torch.distributed as dist

        t = torch.tensor([dev_s, wall], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=dist_group)
        dev_s, wall = t.tolist()
    seqs = [eng.seqs[i] for i in ids]
    out_tokens = sum(len(s.output_ids) for s in seqs)
    ttft = [s.first_token_time - s.arrival for s in seqs if s.first_token_time is not None]
    tpot = [(s.token_times[-1] - s.token_times[0]) / (len(s.token_times) - 1) for s in seqs if len(s.token_times) > 1]
    st = eng.stats
    return {"output_tokens": out_tokens, "device_s": dev_s, "wall_s": wall, "steps": steps,
            "tok_s_device": out_tokens / dev_s if dev_s > 0 else None, "tok_s_wall": out_tokens / wall,
            "ttft_p50_ms": 1e3 * percentile(ttft, 0.5) if ttft else None, "ttft_p99_ms": 1e3 * percentile(ttft, 0.99) if ttft else None,
            "tpot_p50_ms": 1e3 * percentile(tpot, 0.5) if tpot else None, "tpot_p99_ms": 1e3 * percentile(tpot, 0.99) if tpot else None,
            "prefill_tokens": st.prefill_tokens, "decode_tokens": st.decode_tokens, "prefix_hit_tokens": st.cached_tokens,
            "preemptions": st.preemptions, "device_errors": st.device_errors}


def rand_ids(g, n: int, vocab: int) -> List[int]:
    return torch.randint(0, vocab, (n,), generator=g).tolist()


# ------------------------------------------------------------------------------------------------
def config1(scale: float) -> Dict:
    """TinyLlama architecture, CPU fp32, 32 prompt tokens + 32 greedy tokens through the paged cache (block 16)."""
    from ..engine.cpu_runner import CpuModelRunner
    from ..engine.llm_engine import LLMEngine
    from ..models import configs as C
    from ..models.families import LlamaModel

    arch = dict(ARCH["tinyllama"])
    if scale < 1.0:
        arch.update(num_hidden_layers=max(1, int(22 * scale)))
    cfg = C.LlamaConfig(**arch)
    t0 = time.perf_counter()
    m = LlamaModel.new(cfg, init="random", seed=0)
    load_s = time.perf_counter() - t0
    eng = LLMEngine(CpuModelRunner(m, num_blocks=64, block_size=16, max_model_len=256), num_blocks=64, block_size=16,
                    max_num_seqs=1, max_num_batched_tokens=256, max_model_len=256)
    g = torch.Generator().manual_seed(1234)
    res = serve(eng, [{"prompt": rand_ids(g, 32, cfg.vocab_size), "max_tokens": 32}], None)
    res.update(model="tinyllama", dtype="fp32", device="cpu", layers=arch["num_hidden_layers"], init_s=load_s,
               threads=torch.get_num_threads())
    return res


def gpu_config(n: int, scale: float, env, fused: bool = True, health=None, warm: bool = True) -> Dict:
    rank, world, group, device = env
    small = scale < 0.05
    g = torch.Generator().manual_seed(99)
    build = lambda *a, **k: build_engine(*a, fused=fused, **k)      # noqa: E731
    if n == 2:
        nreq = max(8, int(1024 * scale))
        rate = 64.0                                    # requests per second
        eng, runner, cfg, w = build("llama2-7b", world, rank, group, device, max_seqs=256, max_len=2048 + 512 + 16,
                                           blocks=max(4096, min(60000, nreq * 170)), small=small)
        lens = torch.randint(128, 2049, (nreq,), generator=g).tolist()
        outs = torch.randint(64, 513, (nreq,), generator=g).tolist()
        gaps = torch.empty(nreq).exponential_(rate, generator=g).cumsum(0).tolist()
        if small:
            lens, outs = [l // 8 for l in lens], [o // 8 for o in outs]
        reqs = [{"prompt": rand_ids(g, l, cfg.vocab_size), "max_tokens": o, "arrival": a} for l, o, a in zip(lens, outs, gaps)]
        extra = {"model": "llama2-7b", "requests": nreq, "arrival": f"poisson {rate}/s", "prompt": "U[128,2048]", "output": "U[64,512]"}
    elif n == 3:
        nreq = max(8, int(256 * scale))
        pl, ol = (1024, 256) if not small else (128, 32)
        eng, runner, cfg, w = build("mixtral-8x7b", world, rank, group, device, max_seqs=256, max_len=pl + ol + 16,
                                           blocks=nreq * ((pl + ol) // 16 + 2) + 64, small=small)
        mk = lambda: [{"prompt": rand_ids(g, pl, cfg.vocab_size), "max_tokens": ol} for _ in range(nreq)]   # noqa: E731
        reqs = mk()
        extra = {"model": "mixtral-8x7b", "requests": nreq, "prompt": pl, "output": ol, "expert_parallel": w.ep}
    elif n == 4:
        nreq = max(8, int(512 * scale))
        pl, sl, ol = (1024, 128, 128) if not small else (128, 32, 16)
        eng, runner, cfg, w = build("llama3-8b", world, rank, group, device, max_seqs=min(512, nreq),
                                           max_len=pl + sl + ol + 16, blocks=pl // 16 + nreq * ((sl + ol) // 16 + 2) + 64, small=small)

        def mk():
            prefix = rand_ids(g, pl, cfg.vocab_size)
            return [{"prompt": prefix + rand_ids(g, sl, cfg.vocab_size), "max_tokens": ol} for _ in range(nreq)]

        reqs = mk()
        extra = {"model": "llama3-8b", "requests": nreq, "shared_prefix": pl, "suffix": sl, "output": ol}
    else:
        raise ValueError(n)
    warmed = False
    if warm and n in (3, 4) and runner.use_cuda_graphs:
        # Fixed-length workloads walk through the same step shapes on every run: one untimed pass over requests of
        # the same shape (other token ids, so nothing of it is a prefix-cache hit later) captures the CUDA graphs,
        # and the timed pass then measures serving, not graph capture.
        serve(eng, reqs, device, group, world, health)
        import dataclasses

        for f in dataclasses.fields(eng.stats):
            setattr(eng.stats, f.name, 0)
        reqs = mk()
        warmed = True
    cap0 = runner.captures
    res = serve(eng, reqs, device, group, world, health)
    comm = runner.tp.comm
    if comm is not None:
        torch.cuda.synchronize()
        res.update(symmetric_heap="own" if comm.heap is not None else "torch", nvswitch_multicast=bool(comm.multimem))
        comm.close()
    res.update(extra, n_gpus=world, dtype="bf16",
               parallelism=f"tp{world}" + (f"+ep{world}" if w.ep else "") + ("" if fused or world == 1 else "-nccl-baseline"),
               graphs=len(runner.graphs), graph_captures_in_timed_run=runner.captures - cap0, warm_pass=warmed,
               fused_steps=runner.fused_steps, unfused_steps=runner.unfused_steps, small_model=small)
    return res


def config5(scale: float, env, fused: bool = True, model: str = "llama3-70b", context: int = 4096) -> List[Dict]:
    """Llama-3-70B decode sweep.  The KV cache is filled with random values at the target context (decode time does not
    depend on the values), then ``steps`` decode steps run through the runner with CUDA graphs.  ``model`` / ``context``
    run the same sweep on another architecture (e.g. ``llama3-8b`` on one GPU: single-stream decode latency)."""
    from ..engine.runner import StepBatch

    rank, world, group, device = env
    small = scale < 0.05
    ctx, steps = (context, 256) if not small else (256, 16)
    batches = [b for b in (1, 8, 32, 128, 256) if b <= max(1, int(256 * scale)) or small and b <= 8] or [1]
    bmax = max(batches)
    max_len = ctx + steps + 16
    per = (max_len + 15) // 16                       # block-table width of the runner
    blocks = bmax * per + 16
    eng, runner, cfg, w = build_engine(model, world, rank, group, device, max_seqs=bmax, max_len=max_len,
                                       blocks=blocks, small=small, fused=fused)
    for kc in runner.k_cache:
        kc.normal_(0, 0.5)
    for vc in runner.v_cache:
        vc.normal_(0, 0.5)
    out = []
    for B in batches:
        tables = [list(range(1 + i * per, 1 + (i + 1) * per)) for i in range(B)]
        toks = [1] * B

        def step(k):
            L = ctx + k
            sb = StepBatch(toks, [L] * B, [tables[i][L // 16] * 16 + L % 16 for i in range(B)], B, [L + 1] * B, tables, [],
                           list(range(B)))
            runner.launch(sb)
            return runner.fetch()

        for k in range(4):
            step(k)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for k in range(4, 4 + steps):
            toks = step(k)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if world > 1:
            import torch.distributed as dist

            t = torch.tensor([ms], dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
            ms = float(t[0])
        wbytes = w.nbytes()
        out.append({"model": model, "weight_gb_per_gpu": round(wbytes / 1e9, 2),
                    "weight_stream_floor_ms": round(wbytes / 6.54e12 * 1e3, 3), "n_gpus": world, "batch": B, "context": ctx, "decode_steps": steps,
                    "tpot_ms": ms / steps, "tok_s_device": B * steps / (ms / 1e3), "kv": "random values at the target context",
                    "small_model": small, "dtype": "bf16",
                    "parallelism": f"tp{world}" + ("" if fused or world == 1 else "-nccl-baseline")})
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=int, required=True, choices=[1, 2, 3, 4, 5])
    ap.add_argument("--scale", type=float, default=1.0)
    ap.add_argument("--model", default="llama3-70b", help="config 5: architecture of the decode sweep")
    ap.add_argument("--context", type=int, default=4096, help="config 5: context length of the decode sweep")
    ap.add_argument("--out", default=None, help="append JSON lines here")
    ap.add_argument("--nccl-baseline", action="store_true",
                    help="tensor parallel through NCCL all-reduce between separate kernels instead of the fused kernels")
    ap.add_argument("--no-warm-pass", action="store_true", help="configs 3 / 4: time the first pass, graph captures included")
    ap.add_argument("--health", action="store_true",
                    help="start a heartbeat per rank (TCP store on MASTER_PORT + 17) and check the peers before every step")
    a = ap.parse_args(argv)
    if a.config == 1:
        results = [config1(a.scale)]
        rank = 0
    else:
        from ..dist.launch import init_distributed, shutdown

        env = init_distributed(control_group=False)
        rank = env.rank
        e = (env.rank, env.world, env.group, env.device)
        health = hb = None
        if a.health:
            from ..dist.health import FailureDetector, Heartbeat, StepWatchdog

            if env.world > 1:
                import datetime

                from torch.distributed import TCPStore

                store = TCPStore(os.environ.get("MASTER_ADDR", "127.0.0.1"), int(os.environ.get("MASTER_PORT", "29500")) + 17,
                                 env.world, is_master=(env.rank == 0), timeout=datetime.timedelta(seconds=120))
            else:
                from ..dist.health import DictStore

                store = DictStore()
            hb = Heartbeat(store, env.rank, env.world, interval=0.2, timeout=5.0).start()
            health = FailureDetector(hb, StepWatchdog(hb, max_lag=1 << 30))
        try:
            if a.config == 5:
                results = config5(a.scale, e, fused=not a.nccl_baseline, model=a.model, context=a.context)
            else:
                results = [gpu_config(a.config, a.scale, e, fused=not a.nccl_baseline, health=health, warm=not a.no_warm_pass)]
        finally:
            if hb is not None:
                hb.stop()
        from ..ops import cuda_ops

        cuda_ops.check_device_errors()
        shutdown()
    if rank == 0:
        for r in results:
            r["config"] = a.config
            line = json.dumps(r)
            print(line)
            if a.out:
                with open(a.out, "a") as f:
                    f.write(line + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
