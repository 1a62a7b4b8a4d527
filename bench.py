"""Headline benchmark: output tokens/s of the Llama-3-8B architecture served by the engine.

``python bench.py --gpus N --steps K --warmup W`` (for N > 1 launched under ``torch.distributed.run``,
one rank per GPU, tensor parallel over all N ranks).

Workload (the prefix-sharing serving configuration, in steady state): ``--batch`` concurrent requests
(default 512), every request = a 1024-token prefix shared by all requests + a unique 128-token suffix
(random ids), 128 greedy output tokens, random-init bf16 weights, paged KV with 16-token blocks and the
radix prefix cache on.  The request stream never dries up: whenever a request finishes a new one is
queued, and the first wave gets staggered output budgets so that from the first timed step on, every
step retires and admits about batch/128 requests.  One "step" is one engine iteration: decode of all
running sequences + chunked prefill of the newly admitted suffixes + sampling.

Two timings of the same K steps are reported:
  * ``value``  : output tokens / device time, device time = sum over steps of the CUDA-event interval
                 around the step's metadata upload + kernels, maximum over ranks;
  * ``e2e``    : output tokens / wall time of ``LLMEngine.step()`` (scheduler, pinned-host -> device copy
                 of the step's inputs, kernels, device -> host read of the sampled tokens), barrier and
                 synchronize on both sides, maximum over ranks.
Model weights (16 GB) are far larger than L2, so every step streams its inputs from HBM.

Before the timed steps the engine runs untimed until every CUDA graph that the steady state needs has been
captured (one whole output period without a new capture); during the timed steps a shape that still has no
graph runs as plain launches instead of being captured, and the line says how many such steps there were.
The line also carries the per-step device times (median / min / max), every rank's device and host time,
the count of fused and NCCL-path steps, and the latency of the requests that lived inside the timed steps.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import subprocess
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

MODELS = {
    "llama3-8b": dict(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                      num_attention_heads=32, num_key_value_heads=8, rope_theta=500000.0, rms_norm_eps=1e-5,
                      max_position_embeddings=8192),
    "llama2-7b": dict(vocab_size=32000, hidden_size=4096, intermediate_size=11008, num_hidden_layers=32,
                      num_attention_heads=32, num_key_value_heads=32, rope_theta=10000.0, rms_norm_eps=1e-5,
                      max_position_embeddings=4096),
    "llama3-70b": dict(vocab_size=128256, hidden_size=8192, intermediate_size=28672, num_hidden_layers=80,
                       num_attention_heads=64, num_key_value_heads=8, rope_theta=500000.0, rms_norm_eps=1e-5,
                       max_position_embeddings=8192),
    "mixtral-8x7b": dict(vocab_size=32000, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                         num_attention_heads=32, num_key_value_heads=8, rope_theta=1000000.0, rms_norm_eps=1e-5,
                         max_position_embeddings=32768, num_experts=8, num_experts_per_tok=2, sliding_window=32768),
    "tiny-moe": dict(vocab_size=4096, hidden_size=1024, intermediate_size=1024, num_hidden_layers=4,
                     num_attention_heads=8, num_key_value_heads=8, rope_theta=10000.0, rms_norm_eps=1e-5,
                     max_position_embeddings=4096, num_experts=8, num_experts_per_tok=2, sliding_window=4096),
    "tiny": dict(vocab_size=4096, hidden_size=1024, intermediate_size=2048, num_hidden_layers=4,
                 num_attention_heads=8, num_key_value_heads=8, rope_theta=10000.0, rms_norm_eps=1e-5,
                 max_position_embeddings=4096),
}


class ClockSampler:
    """SM clock and throttle reasons of one GPU, sampled every 20 ms while the timed region runs.

    NVML is opened and the device handle looked up BEFORE the timed region (``prepare``), inside this process, so
    that nothing but two cheap queries per sample happens while the steps are timed.  (Starting one ``nvidia-smi``
    process per rank at the start of the timed region put eight NVML initialisations, each enumerating all GPUs of
    the box, inside a window of a few hundred milliseconds.)  ``nvidia-smi`` remains the fallback when the NVML
    binding cannot be imported; it is then started early, in ``prepare``."""

    REASONS = ((0x8, "hw_slowdown"), (0x40, "hw_thermal_slowdown"), (0x20, "sw_thermal_slowdown"),
               (0x4, "sw_power_cap"), (0x80, "hw_power_brake_slowdown"))
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, torch_index: int):
        self.index, self.nvml, self.handle, self.proc = torch_index, None, None, None
        self.samples, self.lines, self.max_mhz = [], [], None
        self._stop = threading.Event()
        self._on = False
        self.thread = None

    def prepare(self):
        try:
            import pynvml
            import torch

            pynvml.nvmlInit()
            h = None
            try:
                uuid = str(torch.cuda.get_device_properties(self.index).uuid)
                h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
            except Exception:
                vis = os.environ.get("CUDA_VISIBLE_DEVICES")
                phys = self.index
                if vis:
                    try:
                        phys = int(vis.split(",")[self.index])
                    except ValueError:
                        phys = self.index
                h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
            self.nvml, self.handle = pynvml, h
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
        except Exception:
            self.nvml = None
            try:
                self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                              "--format=csv,noheader,nounits", "-lms", "50"],
                                             stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
                self.thread = threading.Thread(target=self._read, daemon=True)
                self.thread.start()
            except Exception:
                self.proc = None

    def _poll(self):
        n, h = self.nvml, self.handle
        reasons = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or n.nvmlDeviceGetCurrentClocksThrottleReasons
        while not self._stop.is_set():
            if self._on:
                try:
                    self.samples.append((float(n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM)), int(reasons(h))))
                except Exception:
                    pass
            self._stop.wait(0.02)

    def _read(self):
        for line in self.proc.stdout:
            if self._on:
                self.lines.append(line.strip())

    def start(self):
        self._on = True

    def stop(self):
        self._on = False
        self._stop.set()
        if self.nvml is not None:
            sm = sorted(s for s, _ in self.samples)
            bits = 0
            for _, b in self.samples:
                bits |= b
            return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.max_mhz,
                    "reasons": sorted(name for bit, name in self.REASONS if bits & bit), "samples": len(sm),
                    "source": "nvml, sampled in-process every 20 ms during the timed steps"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=3)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx = float(f[1])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm), "source": "nvidia-smi -lms 50, started before the warm-up"}


def reference_arm(args):
    # The reference is a Rust workspace with no Python packaging: an offline `pip install --no-index` of its source
    # tree answers "neither setup.py nor pyproject.toml found", and there is no cargo / rustc available to build it
    # another way.
    if int(os.environ.get("RANK", "0")) != 0:
        return 0                                   # under torchrun only rank 0 reports
    print(json.dumps({"impl": "reference", "unavailable":
                      "reference is a Rust/Candle CPU workspace: not pip-installable (no setup.py/pyproject.toml) "
                      "and no Rust toolchain offline; it has no GPU or multi-GPU path to run"}))
    return 0


def _median(xs):
    xs = sorted(xs)
    n = len(xs)
    if n == 0:
        return None
    return xs[n // 2] if n % 2 else 0.5 * (xs[n // 2 - 1] + xs[n // 2])


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama3-8b", choices=sorted(MODELS))
    ap.add_argument("--batch", type=int, default=512)
    ap.add_argument("--prefix-len", type=int, default=1024)
    ap.add_argument("--suffix-len", type=int, default=128)
    ap.add_argument("--output-len", type=int, default=128)
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--sync-scheduling", action="store_true",
                    help="read every step's tokens before scheduling the next one (default: the host runs one step ahead)")
    ap.add_argument("--profile-ops", action="store_true", help="print device ms per op over the timed steps (eager mode)")
    ap.add_argument("--baseline-collectives", action="store_true",
                    help="tensor parallel with NCCL all-reduce between separate kernels instead of the fused path")
    ap.add_argument("--library-baseline", action="store_true",
                    help="N > 1: also time the NCCL + separate-kernel path in the same process group (before the fused "
                         "path) and report it under 'library_baseline'")
    ap.add_argument("--emulate-shard", type=int, default=0, metavar="W",
                    help="1 GPU: run the per-rank shapes of W-way tensor parallelism (heads, KV heads, MLP width and "
                         "vocabulary divided by W) without any communication -- the compute floor of one rank; "
                         "the token counts it prints are not a throughput of the full model")
    args = ap.parse_args(argv)
    if args.impl == "reference":
        return reference_arm(args)
    args.warmup = max(args.warmup, 3)

    import torch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        args.gpus = world
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    group = None
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device(dev))
        group = dist.group.WORLD

    from unillm_b200.engine.llm_engine import LLMEngine
    from unillm_b200.engine.runner import GpuModelRunner, RunnerWeights, TpContext
    from unillm_b200.models import configs as C
    from unillm_b200.models.families import LlamaModel, MixtralModel
    from unillm_b200.ops import cuda_ops
    from unillm_b200.sampling import SamplingParams

    moe = "num_experts" in MODELS[args.model]
    if moe:
        cfg = C.MixtralConfig(**MODELS[args.model])
        spec = MixtralModel.spec_from_config(cfg)
    else:
        cfg = C.LlamaConfig(**MODELS[args.model])
        spec = LlamaModel.spec_from_config(cfg)
    if args.emulate_shard > 1:
        if world > 1 or moe:
            raise SystemExit("--emulate-shard is a 1-GPU mode for dense models")
        W = args.emulate_shard
        spec = dataclasses.replace(spec, num_heads=spec.num_heads // W, num_kv_heads=max(1, spec.num_kv_heads // W),
                                   intermediate_size=spec.intermediate_size // W, vocab_size=spec.vocab_size // W)
    B, PL, SL, OL = args.batch, args.prefix_len, args.suffix_len, args.output_len
    bs = 16
    max_len = PL + SL + OL + bs
    blocks_needed = PL // bs + (B + 8) * ((SL + OL) // bs + 2)
    num_blocks = max(2 * blocks_needed, 1024)
    # MoE models: attention tensor parallel + expert parallel (whole experts per rank) when the ranks divide the experts
    weights = RunnerWeights.random(spec, dev, rank, world, seed=1234, expert_parallel=moe)
    V = spec.vocab_size
    sampler = ClockSampler(local)
    sampler.prepare()

    def setup(fused: bool):
        """Engine in steady state with its CUDA graphs captured (all untimed)."""
        tp = TpContext(rank, world, group, fused=fused)
        if tp.fused:
            from unillm_b200.dist.fused import FusedComm

            tp.comm = FusedComm.create(spec, rank, world, group, max_tokens=8192 + B, device=dev)
        runner = GpuModelRunner(spec, weights, num_blocks=num_blocks, block_size=bs, max_num_seqs=B,
                                max_num_batched_tokens=8192, max_model_len=max_len, tp=tp, device=dev,
                                use_cuda_graphs=not args.no_graphs)
        eng = LLMEngine(runner, num_blocks=num_blocks, block_size=bs, max_num_seqs=B, max_num_batched_tokens=8192,
                        max_model_len=max_len, enable_prefix_caching=True, async_scheduling=not args.sync_scheduling)
        eng.max_device_errors = 0        # a step that reports a device error ends the run (or sends it to the fallback path)

        g = torch.Generator().manual_seed(2024)
        prefix = torch.randint(0, V, (PL,), generator=g).tolist()

        def new_prompt():
            return prefix + torch.randint(0, V, (SL,), generator=g).tolist()

        # first wave: staggered budgets put the engine in steady state (about B/OL requests retire per step)
        for i in range(B):
            eng.add_request(new_prompt(), SamplingParams(temperature=0.0, max_tokens=1 + (i * OL) // B, ignore_eos=True))
        params = SamplingParams(temperature=0.0, max_tokens=OL, ignore_eos=True)

        def top_up():
            while len(eng.waiting) < 8:
                eng.add_request(new_prompt(), params)

        top_up()
        # setup (untimed): run until every request of the first wave has produced its first token
        first_wave = [eng.seqs[i] for i in range(B)]
        while any(s.first_token_time is None for s in first_wave) and eng.stats.steps < 400:
            eng.step()
            top_up()
        if eng.stats.device_errors:
            raise RuntimeError(f"{eng.stats.device_errors} steps reported a device error during setup")
        # setup (untimed): CUDA-graph capture is a one-time cost per step shape.  The workload repeats with the
        # output length as its period, so the set of shapes is complete once a whole period (and a margin) has
        # passed without a new capture.
        stable = guard = 0
        while runner.use_cuda_graphs and stable < OL + 16 and guard < 6 * OL:
            n_graphs = len(runner.graphs)
            eng.step()
            top_up()
            stable = stable + 1 if len(runner.graphs) == n_graphs else 0
            guard += 1
        for _ in range(args.warmup):
            eng.step()
            top_up()
        eng.flush()                      # nothing launched before the timed steps is read inside them
        torch.cuda.synchronize()
        cuda_ops.check_device_errors()
        if eng.stats.device_errors:
            raise RuntimeError(f"{eng.stats.device_errors} steps reported a device error during setup")
        return tp, runner, eng, top_up

    def timed(state, K, clocks=None):
        """K engine steps between barrier + synchronize on both sides; returns this job's numbers (max over ranks)."""
        tp, runner, eng, top_up = state
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
        runner.capture_new_graphs = False          # an unseen shape runs as plain launches, never a capture, from here on
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        if clocks is not None:
            clocks.start()
        c0 = dict(l=runner.launches, h=runner.h2d_bytes, d=runner.d2h_bytes, cap=runner.captures, eag=runner.eager_steps,
                  fu=runner.fused_steps, un=runner.unfused_steps, wait=runner.wait_s, err=eng.stats.device_errors)
        tokens = 0
        host_s = 0.0
        t_first = time.perf_counter()
        for k in range(K):
            eng.step_events = evs[k]
            ts = time.perf_counter()
            outs = eng.step()
            host_s += time.perf_counter() - ts
            tokens += len(outs)
            top_up()
        tokens += len(eng.flush())           # the last step's tokens are read inside the timed region as well
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t_last = time.perf_counter()
        wall = t_last - t_first
        clk = clocks.stop() if clocks is not None else None
        eng.step_events = None
        runner.capture_new_graphs = True
        per_step = [a.elapsed_time(b) for a, b in evs]
        dev_ms = sum(per_step)
        cuda_ops.check_device_errors()
        host_busy_ms = (host_s - (runner.wait_s - c0["wait"])) * 1e3 / K     # scheduler + packing + launch, per step
        res = {
            "tokens": tokens, "dev_ms": dev_ms, "wall": wall, "per_step": per_step, "clocks": clk,
            "launches": runner.launches - c0["l"], "h2d": (runner.h2d_bytes - c0["h"]) / K,
            "d2h": (runner.d2h_bytes - c0["d"]) / K, "captures": runner.captures - c0["cap"],
            "eager_steps": runner.eager_steps - c0["eag"], "fused_steps": runner.fused_steps - c0["fu"],
            "unfused_steps": runner.unfused_steps - c0["un"], "device_errors": eng.stats.device_errors - c0["err"],
            "host_busy_ms": host_busy_ms, "window": (t_first, t_last),
        }
        if world > 1:
            # every rank's device time, host time and per-step maxima, so that a straggler is visible in the line
            mine = torch.tensor([dev_ms, wall, host_busy_ms, max(per_step), _median(per_step)], dtype=torch.float64, device=dev)
            allr = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(allr, mine)
            allr = torch.stack(allr).tolist()
            res["ranks"] = {"dev_ms": [r[0] for r in allr], "wall_s": [r[1] for r in allr],
                            "host_busy_ms_per_step": [r[2] for r in allr], "step_ms_max": [r[3] for r in allr],
                            "step_ms_p50": [r[4] for r in allr]}
            res["dev_ms"] = max(r[0] for r in allr)
            res["wall"] = max(r[1] for r in allr)
            ps = torch.tensor(per_step, dtype=torch.float64, device=dev)
            dist.all_reduce(ps, op=dist.ReduceOp.MAX)
            res["per_step"] = ps.tolist()
        return res

    K = args.steps
    library = None
    if args.library_baseline and world > 1 and not args.baseline_collectives:
        st = setup(False)
        r = timed(st, K)
        library = {"value": r["tokens"] / (r["dev_ms"] / 1e3), "unit": "tok/s", "ms_per_step": r["dev_ms"] / K,
                   "ms_per_step_p50": _median(r["per_step"]),
                   "what": "same engine and kernels, separate launches with NCCL all-reduce between them (no CUDA graph)"}
        del st, r
        torch.cuda.empty_cache()

    fused = world > 1 and not args.baseline_collectives
    fallback_reason = None
    state = None
    if fused:
        # The fused path is the product; if it cannot run on this box (a bounded device wait gave up, a peer mapping
        # failed) every rank agrees to measure the NCCL path instead and the JSON line says so.
        ok, why = 1, ""
        try:
            state = setup(True)
        except Exception as e:          # noqa: BLE001 - any failure means "fall back", the reason is reported
            ok, why = 0, repr(e)[:200]
        flag = torch.tensor([ok], dtype=torch.int32, device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag[0]) == 0:
            fallback_reason = why or "another rank failed in the fused path"
            state = None
            torch.cuda.empty_cache()
            fused = False
    if state is None:
        state = setup(False)
    tp, runner, eng, top_up = state

    if args.profile_ops:
        runner.use_cuda_graphs = False
        runner.profile = True
    r = timed(state, K, sampler)
    if args.profile_ops and rank == 0:
        rep = runner.profile_report()
        tot = sum(rep.values())
        for name, ms in sorted(rep.items(), key=lambda kv: -kv[1]):
            print(f"  {name:40s} {ms / K:9.3f} ms/step {100 * ms / tot:5.1f}%", file=sys.stderr)
    # latency of the requests that lived inside the timed steps (host clock, this rank)
    t_first, t_last = r["window"]
    ttft, tpot = [], []
    for s in eng.seqs.values():
        if s.first_token_time is not None and t_first <= s.first_token_time <= t_last and s.arrival >= t_first:
            ttft.append((s.first_token_time - s.arrival) * 1e3)
        tt = [t for t in s.token_times if t_first <= t <= t_last]
        if len(tt) >= 2:
            tpot.append((tt[-1] - tt[0]) * 1e3 / (len(tt) - 1))
    if rank == 0:
        tokens, dev_ms, wall = r["tokens"], r["dev_ms"], r["wall"]
        value = tokens / (dev_ms / 1e3)
        e2e = tokens / wall
        ps = r["per_step"]
        par = f"tp{world}" + (f"+ep{world}" if weights.ep else "") + ("" if tp.fused or world == 1 else "-nccl-baseline")
        if args.emulate_shard > 1:
            par = f"1 GPU running the per-rank shapes of tp{args.emulate_shard} without communication"
        out = {
            "metric": f"output tok/s, {args.model} architecture, engine steady state (device-timed, max over ranks)",
            "value": value, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": args.warmup,
            "ms_per_step": dev_ms / K, "ms_per_step_p50": _median(ps), "ms_per_step_min": min(ps),
            "ms_per_step_max": max(ps), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic (random token ids, random-init weights)",
            "config": {"model": args.model, "global_batch": B, "seq_len": PL + SL + OL,
                       "parallelism": par,
                       "fused_fallback": fallback_reason,
                       "workload": f"{B} concurrent requests: {PL}-token shared prefix + {SL} unique + {OL} greedy outputs, "
                                   "continuous batching in steady state",
                       "kv_block": bs, "prefix_cache": True, "cuda_graphs": not args.no_graphs,
                       "symmetric_heap": (None if tp.comm is None else ("own" if tp.comm.heap is not None else "torch")),
                       "nvswitch_multicast": (None if tp.comm is None else bool(tp.comm.multimem)),
                       "reduce_scatter": (None if tp.comm is None else
                                          "owner reads rows summed by the switch (multimem.ld_reduce)" if tp.comm.multimem_rs
                                          else "GEMM epilogue stores rows into the owners' slots (peer stores)"),
                       "scheduling": "synchronous" if args.sync_scheduling else "host one step ahead of the device",
                       "l2": "inputs larger than L2: each step streams the model weights (>= 2 GB per GPU) from HBM",
                       "output_tokens_timed": tokens},
            "e2e": {"value": e2e, "unit": "tok/s", "ms_per_step": wall * 1e3 / K, "h2d_bytes_per_step": r["h2d"],
                    "d2h_bytes_per_step": r["d2h"]},
            "gpu_launches": r["launches"],
            "clocks": r["clocks"],
            "captures_in_timed_region": r["captures"], "eager_steps_in_timed_region": r["eager_steps"],
            "fused_steps": r["fused_steps"], "unfused_steps": r["unfused_steps"],
            "device_errors_in_timed_region": r["device_errors"],
            "host_busy_ms_per_step": r["host_busy_ms"],
            "latency": {"ttft_ms_p50": _median(ttft), "tpot_ms_p50": _median(tpot), "requests_admitted": len(ttft),
                        "note": "requests inside the timed steps, host clock of rank 0; a request is queued when a "
                                "slot of the closed loop is about to free up, so TTFT = queue wait + its prefill step"},
            "engine": {"prefill_tokens": eng.stats.prefill_tokens, "decode_tokens": eng.stats.decode_tokens,
                       "cached_tokens": eng.stats.cached_tokens, "preemptions": eng.stats.preemptions,
                       "graphs": len(runner.graphs)},
        }
        if "ranks" in r:
            out["ranks"] = r["ranks"]
        if library is not None:
            out["library_baseline"] = library
            out["vs_library_baseline"] = value / library["value"]
        print(json.dumps(out))
    if world > 1:
        # orderly teardown: every rank unbinds its memory from the multicast object before any rank frees its block
        torch.cuda.synchronize()
        if tp.comm is not None:
            tp.comm.close()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
