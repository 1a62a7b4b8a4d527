"""Fused compute + collective kernels.

Single-GPU part: all ranks are emulated on one device with ``FusedComm.emulated`` (their "peer pointers"
are ordinary buffers of the same GPU) and kernels are launched producer-before-consumer on one stream,
so no kernel ever waits for a kernel that has not been launched yet.

Multi-GPU part (needs >= 2 GPUs): a tiny LLaMA runs through the engine with tensor parallel 2 in child
processes, once with the fused kernels and once with the NCCL baseline, and must produce the same
tokens as the single-GPU run.
"""
import math
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rand(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16).cuda()


@pytest.mark.parametrize("world,T", [(2, 64), (4, 256), (8, 512)])
def test_gemm_rs_norm_ag_gemm_chain_emulated(world, T):
    from unillm_b200.dist.fused import FusedComm
    from unillm_b200.ops import cuda_ops as K

    H, Kfull, I = 512, 1024, 768
    R = T // world
    comms = FusedComm.emulated(world, H, T, "cuda")
    x = _rand(T, Kfull, seed=1)
    wo = _rand(H, Kfull, scale=1 / math.sqrt(Kfull), seed=2)
    res = _rand(T, H, seed=3)
    ln = _rand(H, seed=4)
    wup = _rand(I * world, H, scale=1 / math.sqrt(H), seed=5)
    Kr = Kfull // world
    for rep in range(2):      # twice: the counters must be reset correctly between uses
        # ---- F1 producer on every rank: partial GEMM, rows pushed to their owner ----
        for r, c in enumerate(comms):
            xr = x[:, r * Kr:(r + 1) * Kr].contiguous()
            wr = wo[:, r * Kr:(r + 1) * Kr].contiguous()
            out = c.rs_local_tensor(0, R).view(world * R, H)
            K.gemm_tn(xr, wr, out=out, rs=c.gemm_rs(0, R))
        # ---- F1 consumer + F3 producer on every rank ----
        new_res = []
        for r, c in enumerate(comms):
            _, h = K.norm(c.rs_local_tensor(0, R), ln, residual=res[r * R:(r + 1) * R].contiguous(), eps=1e-5,
                          want_residual_out=True, no_out=True, T=R, rs=c.norm_rs(0), ag=c.norm_ag(1),
                          reset=c.reset_after_ag(1))
            new_res.append(h)
        # ---- F3 consumer: column-parallel GEMM on the gathered rows ----
        ys = []
        for r, c in enumerate(comms):
            ys.append(K.gemm_tn(c.ag_local_tensor(1, T), wup[r * I:(r + 1) * I].contiguous(), ag=c.gemm_ag(1, R)))
        # the gated GEMM waits on the same counters (for >= 256 tokens it runs on CTA pairs)
        wgu = _rand(2 * 256, H, scale=1 / math.sqrt(H), seed=6)
        act = K.gemm_tn(comms[0].ag_local_tensor(1, T), wgu, dual_rows=256, act="silu", ag=comms[0].gemm_ag(1, R))
        # a second norm kernel (the "next layer" one) resets the counters used above, as in the layer pipeline
        for r, c in enumerate(comms):
            K.norm(new_res[r], ln, eps=1e-5, T=R, reset=c.reset_after_ag(0))
        torch.cuda.synchronize()
        K.check_device_errors()
        hsum = (x.float() @ wo.float().t()).to(torch.bfloat16).float()   # order of rounding differs slightly
        href = x.float() @ wo.float().t() + res.float()
        got_res = torch.cat(new_res).float()
        assert (got_res - href).abs().max().item() < 0.06 * max(1.0, href.abs().max().item())
        hn = got_res * torch.rsqrt(got_res.pow(2).mean(-1, keepdim=True) + 1e-5) * ln.float()
        yref = hn.to(torch.bfloat16).float() @ wup.float().t()
        ygot = torch.cat(ys, dim=1).float()
        assert (ygot - yref).abs().max().item() < 0.05 * max(1.0, yref.abs().max().item())
        hb = hn.to(torch.bfloat16).float()
        aref = torch.nn.functional.silu(hb @ wgu[:256].float().t()) * (hb @ wgu[256:].float().t())
        assert (act.float() - aref.cuda()).abs().max().item() < 0.05 * max(1.0, aref.abs().max().item())
        for c in comms:   # counters of the other phase were zeroed, and the last CTA of every launch zeroed its local one
            flags = c.buf[c.flags.offset:c.flags.offset + 256].view(torch.int32)
            assert int(flags[16:25].abs().sum()) == 0
            assert int(flags[40:44].abs().sum()) == 0


def test_flag_wait_times_out_without_hanging():
    """A counter that nothing bumps: the bounded wait gives up, records status 2 and the context stays usable."""
    from unillm_b200.ops import cuda_ops as K

    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    K.wait_flags(flags.data_ptr(), 2, 5, "cuda")
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="flag wait timed out"):
        K.check_device_errors()
    K.check_device_errors()      # the word was cleared
    assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0


_CHILD = r"""
import os, sys, json, torch
import torch.distributed as dist
sys.path.insert(0, os.environ["REPO"])
from unillm_b200.engine.llm_engine import LLMEngine
from unillm_b200.engine.runner import GpuModelRunner, RunnerWeights, TpContext
from unillm_b200.models import configs as C
from unillm_b200.models.families import LlamaModel, MixtralModel
from unillm_b200.ops import cuda_ops
from unillm_b200.sampling import SamplingParams
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device(f"cuda:{rank}"))
moe = os.environ.get("MODEL", "llama") == "mixtral"
if moe:
    cfg = C.MixtralConfig(vocab_size=1024, hidden_size=512, intermediate_size=512, num_hidden_layers=3,
                          num_attention_heads=8, num_key_value_heads=4, num_experts=4, sliding_window=4096)
    spec = MixtralModel.spec_from_config(cfg)
else:
    cfg = C.LlamaConfig(vocab_size=1024, hidden_size=512, intermediate_size=1024, num_hidden_layers=3,
                        num_attention_heads=8, num_key_value_heads=4, rms_norm_eps=1e-5)
    spec = LlamaModel.spec_from_config(cfg)
g = torch.Generator().manual_seed(0)
shared = torch.randint(0, 1024, (48,), generator=g).tolist()
prompts = [shared + torch.randint(0, 1024, (n,), generator=g).tolist() for n in (16, 48, 32, 64, 16, 80, 8, 24)]
out = {}
from unillm_b200.dist.fused import FusedComm
comm = FusedComm.create(spec, rank, world, dist.group.WORLD, max_tokens=512, device=f"cuda:{rank}")
out["heap"] = "own" if comm.heap is not None else "torch"
out["multimem"] = bool(comm.multimem)
# one fixed prefill step for the logit comparison: 3 sequences, 112 token rows (a multiple of the world size)
from unillm_b200.engine.runner import StepBatch
def logit_batch():
    toks, pos, slots, lens, tables, qlens, rows = [], [], [], [], [], [], []
    nxt = 1
    gg = torch.Generator().manual_seed(5)
    for n in (40, 24, 48):
        p = torch.randint(0, 1024, (n,), generator=gg).tolist()
        nb = n // 16 + 2
        blocks = list(range(nxt, nxt + nb)); nxt += nb
        for i, t in enumerate(p):
            toks.append(t); pos.append(i); slots.append(blocks[i // 16] * 16 + i % 16)
        lens.append(n); tables.append(blocks); qlens.append(n); rows.append(len(toks) - 1)
    return StepBatch(toks, pos, slots, 0, lens, tables, qlens, rows)
logits = {}
modes = ("tp1", "nccl", "fused", "fused_graph") + (("fused_replicated",) if moe else ())
for mode in modes:
    # mixtral: "fused" sends each (token, expert) pair to the rank of its expert; "fused_replicated" is the layout in
    # which every rank sees all rows after the all-gather and keeps the pairs of its experts
    os.environ["UB_MOE_SPARSE"] = "0" if mode == "fused_replicated" else "1"
    tpw = 1 if mode == "tp1" else world
    tp = TpContext(rank if tpw > 1 else 0, tpw, dist.group.WORLD if tpw > 1 else None, fused=mode.startswith("fused"))
    w = RunnerWeights.random(spec, f"cuda:{rank}", tp.rank, tp.world, seed=7, expert_parallel=moe)
    assert w.ep == (moe and tp.world > 1)
    if tp.fused:
        tp.comm = comm
    runner = GpuModelRunner(spec, w, num_blocks=128, max_num_seqs=8, max_num_batched_tokens=256, max_model_len=256,
                            tp=tp, use_cuda_graphs=(mode == "fused_graph"))
    eng = LLMEngine(runner, num_blocks=128, max_num_seqs=8, max_num_batched_tokens=256, max_model_len=256)
    out[mode] = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10))
    torch.cuda.synchronize()
    cuda_ops.check_device_errors()
    if mode != "fused_graph":
        lg = runner.logits_for(logit_batch()).float()
        if tpw > 1:                                  # vocabulary shards -> full rows
            parts = [torch.empty_like(lg) for _ in range(world)]
            dist.all_gather(parts, lg.contiguous())
            lg = torch.cat(parts, dim=-1)
        logits[mode] = lg
        torch.cuda.synchronize()
        cuda_ops.check_device_errors()
        assert runner.fused_steps > 0 or mode != "fused"
        if moe and mode.startswith("fused"):
            assert bool(getattr(runner, "_moe_sparse", False)) == (mode == "fused")
        if moe and mode == "fused":
            # token conservation: the pairs received over all ranks in the last MoE call are all pairs of the step
            d = list(runner._moe_dispatch_state.values())[-1]
            n = d.offsets[d.experts_local:d.experts_local + 1].clone().to(torch.int64)
            dist.all_reduce(n)
            out["pairs_received"], out["pairs_sent"] = int(n), d.R * world * d.K
    dist.barrier()
# one-shot all-reduce and pair gather over peer memory against NCCL: exchanges of different sizes, i.e. with different
# numbers of CTAs (each CTA index keeps its own arrival count), parity slots alternating
ar_err = 0.0
for it in range(5):
    t = (torch.randn((16, 17, 4, 30, 9)[it], spec.hidden_size, generator=torch.Generator().manual_seed(100 * rank + it)) * 2).to(torch.bfloat16).cuda()
    ref_t = t.float().clone()
    dist.all_reduce(ref_t)
    got_t = comm.all_reduce(t.clone())
    torch.cuda.synchronize()
    ar_err = max(ar_err, float((got_t.float() - ref_t).abs().max()) / max(1.0, float(ref_t.abs().max())))
    pv = torch.randn(5 + it, 24, generator=torch.Generator().manual_seed(7 * rank + it)).cuda()
    pi = torch.randint(0, 1000, (5 + it, 24), generator=torch.Generator().manual_seed(9 * rank + it)).to(torch.int32).cuda()
    gv, gi = comm.gather_pairs(pv, pi)
    lv = [torch.empty_like(pv) for _ in range(world)]
    li = [torch.empty_like(pi) for _ in range(world)]
    dist.all_gather(lv, pv)
    dist.all_gather(li, pi)
    ev, ei = torch.cat(lv, 1), torch.cat(li, 1)
    if not (torch.equal(gv, ev) and torch.equal(gi, ei)):
        bad = ((gv != ev) | (gi != ei)).nonzero()
        raise AssertionError(f"pair gather differs from NCCL on rank {rank}, exchange {it}: {bad.shape[0]} of {gv.numel()} "
                             f"entries, first {bad[:4].tolist()}, got {gv[tuple(bad[0].tolist())].item()} want {ev[tuple(bad[0].tolist())].item()}")
cuda_ops.check_device_errors()
out["all_reduce_err"] = ar_err
# top-k / top-p sampling over vocabulary shards: candidate pairs gathered through peer memory against whole rows of
# logits gathered by NCCL -- same logits, same Philox draws, so the tokens have to be identical
tp = TpContext(rank, world, dist.group.WORLD, fused=True)
tp.comm = comm
w = RunnerWeights.random(spec, f"cuda:{rank}", rank, world, seed=7, expert_parallel=moe)
sampled = {}
for how in ("pairs", "nccl"):
    os.environ["UB_SAMPLE_PAIRS"] = "1" if how == "pairs" else "0"
    runner = GpuModelRunner(spec, w, num_blocks=128, max_num_seqs=8, max_num_batched_tokens=256, max_model_len=256,
                            tp=tp, use_cuda_graphs=False)
    eng = LLMEngine(runner, num_blocks=128, max_num_seqs=8, max_num_batched_tokens=256, max_model_len=256)
    sps = [SamplingParams(temperature=0.8, top_k=40, max_tokens=6, seed=11), SamplingParams(temperature=1.0, top_p=0.9, max_tokens=6, seed=12),
           SamplingParams(temperature=0.0, max_tokens=6), SamplingParams(temperature=1.2, top_k=5, top_p=0.7, max_tokens=6, seed=13)]
    ids = [eng.add_request(p, sp) for p, sp in zip(prompts[:4], sps)]
    eng.run_to_completion()
    sampled[how] = [list(eng.seqs[i].output_ids) for i in ids]
    # temperature only: the draw from the whole vocabulary, split over the shards
    ids = [eng.add_request(p, SamplingParams(temperature=0.9, max_tokens=6)) for p in prompts[4:8]]
    eng.run_to_completion()
    sampled[how + "_whole"] = [list(eng.seqs[i].output_ids) for i in ids]
    torch.cuda.synchronize()
    cuda_ops.check_device_errors()
    dist.barrier()
out["sampled"] = sampled
ref = logits["tp1"]
scale = float(ref.abs().max())
cmp = ("nccl", "fused") + (("fused_replicated",) if moe else ())
out["logit_err"] = {m: float((logits[m] - ref).abs().max()) / scale for m in cmp}
out["argmax_agree"] = {m: float((logits[m].argmax(-1) == ref.argmax(-1)).float().mean()) for m in cmp}
comm.close()
if rank == 0:
    print("RESULT " + json.dumps(out))
dist.destroy_process_group()
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("heap", ["own", "own-peer-only", "torch"])
@pytest.mark.parametrize("model", ["llama", "mixtral"])
def test_tensor_parallel_engine_fused_matches_baseline(tmp_path, model, heap):
    """llama: tensor parallel 2.  mixtral: attention tensor parallel 2 + expert parallel 2 (two experts per rank).
    ``heap``: the library's symmetric heap with the NVSwitch multicast paths (multimem.ld_reduce / multimem.st) when the
    GPUs have multicast, the same heap with plain peer stores only, or torch's symmetric memory."""
    import json

    script = tmp_path / "child.py"
    script.write_text(_CHILD)
    env = dict(os.environ, REPO=os.path.dirname(os.path.dirname(os.path.abspath(__file__))), NCCL_NVLS_ENABLE="0", MODEL=model,
               UB_SYMM_HEAP="torch" if heap == "torch" else "own", UB_MULTIMEM="0" if heap == "own-peer-only" else "1")
    port = 29731 + 10 * ["llama", "mixtral"].index(model) + ["own", "own-peer-only", "torch"].index(heap)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), str(script)]
    p = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    line = [l for l in p.stdout.splitlines() if l.startswith("RESULT ")][-1]
    out = json.loads(line[7:])
    total = sum(len(r) for r in out["tp1"])

    def agreement(a, b):
        """Greedy tokens of a random-weight model flip on near-ties, and everything after a flip differs: count the
        sequences that agree on their first tokens and the tokens that agree overall."""
        first = sum(ra[:3] == rb[:3] for ra, rb in zip(out[a], out[b]))
        same = sum(x == y for ra, rb in zip(out[a], out[b]) for x, y in zip(ra, rb))
        return first, same

    summary = {k: out[k] for k in ("logit_err", "argmax_agree", "heap", "multimem")}
    summary["agreement"] = {f"{a}/{b}": agreement(a, b) for a, b in
                            [("fused", "fused_graph"), ("tp1", "nccl"), ("tp1", "fused"), ("tp1", "fused_graph")]}
    print(summary)
    # The graph path pads the step to bucketed shapes, so its GEMMs may pick other tiles and K splits than the eager
    # path: same math, different rounding.  With routed experts a near-tie in the router moves a token to another
    # expert, which changes its row by far more than rounding does, hence the wider margin there.
    # The logit comparison below is the numerical check; the token comparison guards against a path that derails.
    floor = 0.75 if model == "mixtral" else 0.9
    slack = 2 if model == "mixtral" else 1
    first, same = agreement("fused", "fused_graph")
    assert first >= len(out["tp1"]) - slack and same / total > floor, summary
    for mode in ("nccl", "fused", "fused_graph"):
        first, agree = agreement("tp1", mode)
        assert first >= len(out["tp1"]) - slack and agree / total > min(floor, 0.8), (mode, summary)
    assert out["heap"] == ("torch" if heap == "torch" else "own")
    if heap != "own":
        assert not out["multimem"]
    # logits of one prefill step, every vocabulary column, against the single-GPU run: bf16 activations with other
    # summation orders (K split over the ranks, partial sums rounded to bf16 before the reduction)
    assert out["all_reduce_err"] < 0.01, out["all_reduce_err"]        # bf16 rounding of the sum
    assert out["sampled"]["pairs"] == out["sampled"]["nccl"], out["sampled"]
    assert all(len(t) == 6 for t in out["sampled"]["pairs"])
    wa, wb = out["sampled"]["pairs_whole"], out["sampled"]["nccl_whole"]
    assert all(len(t) == 6 for t in wa)
    # same logits and uniform numbers; shard-wise and whole-row sums round differently, so allow one boundary flip
    # (everything after a flip in that sequence differs)
    assert sum(a == b for a, b in zip(wa, wb)) >= 3, (wa, wb)
    if model == "mixtral":
        assert out["pairs_received"] == out["pairs_sent"] > 0
    for mode in out["logit_err"]:
        assert out["logit_err"][mode] < 0.04, summary
        assert out["argmax_agree"][mode] == 1.0 or out["logit_err"][mode] < 0.02, summary


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_symmetric_heap_peer_and_multicast_access(tmp_path):
    """The library's own symmetric heap on 2 GPUs: a peer sees what its neighbour stored, a multicast store lands on
    every rank and a multicast load returns the sum of the ranks' copies (the last two where the GPUs support
    multicast); the probe also reports the copy bandwidths."""
    import json

    out_file = tmp_path / "links.json"
    env = dict(os.environ, PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))), NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29769", "-m", "unillm_b200.dist.probe_links", "--mb", "16", "--json", str(out_file)]
    p = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    res = json.loads(out_file.read_text())
    assert res["all_ranks_ok"] and res["checks"]["peer_store"] and res["checks"]["peer_load"]
    if res["multicast"]:
        assert res["checks"]["multimem_st"] and res["checks"]["multimem_ld_reduce"]
    assert all(v["peer_store"] > 1.0 for v in res["gbs"].values())


def _gpu_elastic_worker(rank, world, port, q, exit_rank, exit_step):
    """One rank of the GPU recovery test: fused tensor parallelism over the own symmetric heap WITHOUT a multicast
    binding, a gloo control group (no NCCL anywhere), failures made on the host only."""
    import datetime
    import time

    os.environ.update(UB_SYMM_HEAP="own", UB_MULTIMEM="0", NCCL_NVLS_ENABLE="0")
    import torch
    from torch.distributed import TCPStore

    from unillm_b200.dist.elastic import serve_elastic
    from unillm_b200.dist.fused import FusedComm
    from unillm_b200.dist.health import FaultInjector
    from unillm_b200.engine.llm_engine import LLMEngine
    from unillm_b200.engine.runner import GpuModelRunner, RunnerWeights, TpContext
    from unillm_b200.models import configs as C
    from unillm_b200.models.families import LlamaModel
    from unillm_b200.ops import cuda_ops
    from unillm_b200.sampling import SamplingParams

    torch.cuda.set_device(rank)
    dev = f"cuda:{rank}"
    store = TCPStore("127.0.0.1", port, world, is_master=(rank == 0), wait_for_workers=True,
                     timeout=datetime.timedelta(seconds=120))
    cfg = C.LlamaConfig(vocab_size=1024, hidden_size=512, intermediate_size=1024, num_hidden_layers=3,
                        num_attention_heads=8, num_key_value_heads=4, rms_norm_eps=1e-5)
    spec = LlamaModel.spec_from_config(cfg)
    g = torch.Generator().manual_seed(0)
    params = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    reqs = [{"id": i, "prompt": torch.randint(0, 1024, (n,), generator=g).tolist(), "params": params}
            for i, n in enumerate((16, 48, 32, 64))]
    built = []

    def build_engine(g_rank, g_world, group):
        tp = TpContext(g_rank, g_world, group if g_world > 1 else None, fused=g_world > 1)
        w = RunnerWeights.random(spec, dev, g_rank, g_world, seed=7)
        if tp.fused:
            tp.comm = FusedComm.create(spec, g_rank, g_world, group, max_tokens=512, device=dev, heap="own")
            assert tp.comm.heap is not None and not tp.comm.multimem        # plain peer stores / loads only
        runner = GpuModelRunner(spec, w, num_blocks=128, max_num_seqs=8, max_num_batched_tokens=256, max_model_len=256,
                                tp=tp, use_cuda_graphs=False, device=dev)
        built.append((g_world, runner))
        return LLMEngine(runner, num_blocks=128, max_num_seqs=8, max_num_batched_tokens=256, max_model_len=256)

    ref = None
    if rank == 0:                                   # the undisturbed single-GPU tokens, for the comparison at the end
        ref = build_engine(0, 1, None).generate([r["prompt"] for r in reqs], params)
        built.clear()
    inj = FaultInjector()
    if rank == exit_rank:
        inj.exit_at_step(exit_step)
    res = serve_elastic(rank, world, store, build_engine, reqs, num_heads=8, num_kv_heads=4, hb_interval=0.05,
                        hb_timeout=1.5, injector=inj, backend="gloo")
    torch.cuda.synchronize()
    err = None
    try:
        cuda_ops.check_device_errors()
    except RuntimeError as e:       # noqa: BLE001 - reported to the parent
        err = str(e)
    fused_steps = [(wd, r.fused_steps, r.unfused_steps) for wd, r in built]
    q.put((rank, res.role, res.outputs, res.generations, res.final_world, res.recovered_from, res.steps, ref, fused_steps, err))
    if rank == 0:
        time.sleep(2.0)             # the store lives in this process: keep it until the other rank has reported


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_gpu_rank_leaves_between_steps_and_the_survivor_finishes():
    """Two GPU ranks serve four requests with the fused tensor-parallel kernels (own symmetric heap, no multicast
    binding, gloo control group, no NCCL); rank 1 exits between steps with nothing of its own in flight.  Rank 0 learns of
    it on the host (heartbeat + step gate) before its next launch, so none of its kernels ever waits for the dead peer;
    it rebuilds a single-GPU engine, restores the request log and finishes.  No device wait times out."""
    import multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    import socket

    with socket.socket() as s_:
        s_.bind(("127.0.0.1", 0))
        port = s_.getsockname()[1]
    procs = [ctx.Process(target=_gpu_elastic_worker, args=(r, 2, port, q, 1, 5)) for r in range(2)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(2):
        r = q.get(timeout=240)
        got[r[0]] = r[1:]
    for p in procs:
        p.join(timeout=60)
    assert got[1][0] == "exited"
    role, outs, gens, final_world, recovered, steps, ref, fused_steps, err = got[0]
    assert err is None and got[1][8] is None, (err, got[1][8])
    assert role == "finished" and gens == 2 and final_world == 1 and recovered == [[1]], got[0][:6]
    assert fused_steps[0][0] == 2 and fused_steps[0][1] > 0              # the first generation ran the fused kernels
    assert all(len(outs[i]) == 12 for i in range(4))
    # tensor parallel 2 rounds differently from 1 GPU, so a near-tie may flip a token; the history up to the failure was
    # generated at TP 2, the rest on one GPU
    agree = sum(a == b for i in range(4) for a, b in zip(outs[i], ref[i]))
    assert agree >= 0.7 * 48, (agree, outs, ref)
