"""Host-side distributed logic on CPU: heartbeat / watchdog / fault injection (threads and gloo-free TCPStore
processes), tensor-parallel shard arithmetic over a gloo group, engine snapshot / restore."""
import json
import socket
import time

import pytest
import torch
import torch.multiprocessing as mp

from unillm_b200.dist.health import (DictStore, FailureDetector, FaultInjector, Heartbeat, RankFailure, RecoveryPlan,
                                     StepWatchdog)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_heartbeat_watchdog_in_process():
    store = DictStore()
    hbs = [Heartbeat(store, r, 3, interval=0.02, timeout=0.6).start() for r in range(3)]
    try:
        for step in range(3):
            for h in hbs:
                h.set_step(step)
        time.sleep(0.1)
        det = FailureDetector(hbs[0], StepWatchdog(hbs[0], max_lag=1, stall_timeout=10))
        rep = det.poll()
        assert rep.healthy and rep.status() == "healthy" and not rep.dead
        inj = FaultInjector(hbs[2])
        inj.mute_heartbeat()
        hbs[0].set_step(5), hbs[1].set_step(5)
        time.sleep(0.9)
        rep = det.poll()
        assert rep.dead == [2] and rep.status() == "unhealthy"
        with pytest.raises(RankFailure) as e:
            det.check()
        assert e.value.ranks == [2]
        inj.mute_heartbeat(False)
        time.sleep(0.1)
        rep = det.poll()
        assert rep.dead == [] and rep.lagging == [2] and rep.status() == "degraded"
        det2 = FailureDetector(hbs[1], device_error_check=lambda: "flag wait timed out (peer 3)")
        assert det2.poll().device_error and not det2.poll().healthy
    finally:
        for h in hbs:
            h.stop()


def test_fault_injector_and_recovery_plan():
    inj = FaultInjector()
    inj.fail_at_step(2)
    inj.before_step(1, 0)
    with pytest.raises(RankFailure):
        inj.before_step(2, 0)
    inj2 = FaultInjector()
    inj2.exhaust_allocator_after(2)
    assert [inj2.on_alloc() for _ in range(4)] == [False, False, True, True]
    reqs = [{"id": 0, "prompt": [1, 2, 3], "output": [7, 8], "max_tokens": 5}, {"id": 1, "prompt": [4], "output": [9] * 4, "max_tokens": 4}]
    plan = RecoveryPlan.make(8, dead=[5], num_heads=32, num_kv_heads=8, requests=reqs)
    assert plan.new_world == 4 and plan.survivors == [0, 1, 2, 3, 4, 6, 7] and plan.new_ranks == {0: 0, 1: 1, 2: 2, 3: 3}
    assert plan.requeue == [{"prompt": [1, 2, 3, 7, 8], "done": 2, "max_tokens": 3, "id": 0}]
    assert RecoveryPlan.make(8, [0, 1, 2, 3, 4, 5], 32, 8).new_world == 2
    assert RecoveryPlan.make(2, [1], 32, 8).new_world == 1


def _hb_worker(rank, world, port, q):
    from torch.distributed import TCPStore

    store = TCPStore("127.0.0.1", port, world, is_master=(rank == 0), wait_for_workers=True, timeout=__import__("datetime").timedelta(seconds=30))
    hb = Heartbeat(store, rank, world, interval=0.05, timeout=2.0).start()
    inj = FaultInjector(hb)
    if rank == 2:
        inj.exit_at_step(3)
    det = FailureDetector(hb, StepWatchdog(hb, max_lag=100))
    try:
        for step in range(200):
            inj.before_step(step, rank)
            hb.set_step(step)
            time.sleep(0.02)            # the "step"
            det.check()
        q.put((rank, "no failure seen", None))
    except RankFailure as e:
        plan = RecoveryPlan.make(world, e.ranks, num_heads=4, num_kv_heads=2)
        q.put((rank, "detected", (e.ranks, plan.new_world, hb._step)))
        if rank == 0:
            time.sleep(1.0)             # keep the store alive until the other observer has reported
    except SystemExit:
        q.put((rank, "exited", hb._step))
    finally:
        hb.stop()


def test_rank_exit_is_detected_by_peers():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_hb_worker, args=(r, 3, port, q)) for r in range(3)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(3):
        r, what, info = q.get(timeout=60)
        got[r] = (what, info)
    for p in procs:
        p.join(timeout=30)
    assert got[2][0] == "exited"
    for r in (0, 1):
        assert got[r][0] == "detected", got
        ranks, new_world, step = got[r][1]
        assert ranks == [2] and new_world == 2 and step >= 3


def _tp_worker(rank, world, port, q):
    import torch.distributed as dist

    from unillm_b200.engine.runner import RunnerWeights
    from unillm_b200.models import configs as C
    from unillm_b200.models.families import LlamaModel

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        cfg = C.LlamaConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=4,
                            num_key_value_heads=2)
        m = LlamaModel.new(cfg, init="random", seed=3)
        m.p = {k: v.to(torch.bfloat16).float() for k, v in m.p.items()}
        w = RunnerWeights(m.spec, m.p, "cpu", rank, world)
        h = torch.randn(5, 32, generator=torch.Generator().manual_seed(0)).to(torch.bfloat16).float()
        # column-parallel gate/up, row-parallel down, one all-reduce
        gu = w.t["layers.0.w_gate_up"].float()
        I = gu.shape[0] // 2
        a = torch.nn.functional.silu(h @ gu[:I].t()) * (h @ gu[I:].t())
        y = a @ w.t["layers.0.w_down"].float().t()
        dist.all_reduce(y)
        full = m.p["layers.0.w_gate_up"]
        If = full.shape[0] // 2
        ref = (torch.nn.functional.silu(h @ full[:If].t()) * (h @ full[If:].t())) @ m.p["layers.0.w_down"].t()
        err_mlp = (y - ref).abs().max().item()
        # head-parallel attention projections: q/k/v rows of this rank's heads, o columns
        D = m.spec.head_dim
        qkv = w.t["layers.0.wqkv"].float()
        assert qkv.shape[0] == (w.hq + 2 * w.hkv) * D and w.hq == 2 and w.hkv == 1
        o_part = (h @ qkv[:w.hq * D].t()) @ w.t["layers.0.wo"].float().t()
        dist.all_reduce(o_part)
        qfull = m.p["layers.0.wqkv"][:4 * D]
        err_o = (o_part - (h @ qfull.t()) @ m.p["layers.0.wo"].t()).abs().max().item()
        # vocab-parallel greedy sampling: local (max, argmax) pairs merged across ranks
        logits = h @ w.t["lm_head"].float().t()
        v, i = logits.max(-1)
        pairs = torch.stack([v, (i + rank * w.vocab_shard).float()], -1)
        allp = [torch.empty_like(pairs) for _ in range(world)]
        dist.all_gather(allp, pairs)
        st = torch.stack(allp)                         # [world, T, 2]
        best = st[..., 0].argmax(0)
        merged = st[best, torch.arange(5), 1].long()
        ref_ids = (h @ m.p["lm_head"].t()).argmax(-1)
        q.put((rank, err_mlp, err_o, bool((merged == ref_ids).all())))
    finally:
        dist.destroy_process_group()


def test_tensor_parallel_shards_over_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_tp_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(2)]
    for p in procs:
        p.join(timeout=30)
    for rank, e1, e2, ok in res:
        assert e1 < 1e-4 and e2 < 1e-4 and ok, res


def test_engine_snapshot_restore_continues_identically():
    from unillm_b200.engine.cpu_runner import CpuModelRunner
    from unillm_b200.engine.llm_engine import LLMEngine
    from unillm_b200.models import configs as C
    from unillm_b200.models.families import LlamaModel
    from unillm_b200.sampling import SamplingParams

    cfg = C.LlamaConfig(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2)
    m = LlamaModel.new(cfg, init="random", seed=3)

    def engine():
        return LLMEngine(CpuModelRunner(m, num_blocks=64, block_size=4, max_model_len=128), num_blocks=64, block_size=4,
                         max_num_seqs=4, max_num_batched_tokens=16, max_model_len=128)

    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 128, (n,), generator=g).tolist() for n in (9, 14, 3, 21, 6)]
    params = SamplingParams(temperature=0.0, max_tokens=10)
    ref = engine().generate(prompts, params)
    e1 = engine()
    ids = [e1.add_request(p, params) for p in prompts]
    for _ in range(6):
        e1.step()
    snap = json.loads(json.dumps(e1.snapshot()))
    assert any(r["output"] for r in snap["requests"]) and any(r["status"] != "finished" for r in snap["requests"])
    e2 = engine()
    requeued = e2.restore(snap)
    assert requeued
    out = e2.run_to_completion()
    assert [out[i] for i in ids] == ref
    with pytest.raises(Exception):
        e2.restore(snap)


def _elastic_worker(rank, world, port, q, exit_rank, exit_step):
    import datetime

    from torch.distributed import TCPStore

    from unillm_b200.dist.elastic import serve_elastic
    from unillm_b200.engine.cpu_runner import TpCpuModelRunner
    from unillm_b200.engine.llm_engine import LLMEngine
    from unillm_b200.models import configs as C
    from unillm_b200.models.families import LlamaModel
    from unillm_b200.sampling import SamplingParams

    torch.set_num_threads(1)
    store = TCPStore("127.0.0.1", port, world, is_master=(rank == 0), wait_for_workers=True,
                     timeout=datetime.timedelta(seconds=60))
    cfg = C.LlamaConfig(vocab_size=96, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2)
    m = LlamaModel.new(cfg, init="random", seed=11)
    m.p = {k: v.to(torch.bfloat16).float() for k, v in m.p.items()}
    g = torch.Generator().manual_seed(4)
    params = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    reqs = [{"id": i, "prompt": torch.randint(0, 96, (n,), generator=g).tolist(), "params": params}
            for i, n in enumerate((7, 12, 3, 9))]

    def build_engine(g_rank, g_world, group):
        runner = TpCpuModelRunner(m, g_rank, g_world, group, num_blocks=64, block_size=4, max_model_len=64)
        return LLMEngine(runner, num_blocks=64, block_size=4, max_num_seqs=4, max_num_batched_tokens=16, max_model_len=64)

    inj = FaultInjector()
    if rank == exit_rank:
        inj.exit_at_step(exit_step)
    res = serve_elastic(rank, world, store, build_engine, reqs, num_heads=4, num_kv_heads=2, hb_interval=0.05,
                        hb_timeout=1.5, injector=inj)
    q.put((rank, res.role, res.outputs, res.generations, res.final_world, res.recovered_from, res.steps))
    if rank == 0:
        time.sleep(2.0)             # the store lives in this process: keep it until the others have reported


def test_rank_loss_is_survived_at_a_smaller_tensor_parallel_size():
    """Four CPU ranks serve four requests tensor parallel (4 query heads, 2 KV heads: every KV head is replicated on two
    ranks); rank 3 exits between steps.  The others notice on the host (heartbeat + step gate) before their next
    collective, re-form a 2-rank group (the largest size that divides the 4 heads), prefill the token history again
    and finish with the tokens of an undisturbed single-rank run."""
    from unillm_b200.engine.cpu_runner import CpuModelRunner
    from unillm_b200.engine.llm_engine import LLMEngine
    from unillm_b200.models import configs as C
    from unillm_b200.models.families import LlamaModel
    from unillm_b200.sampling import SamplingParams

    cfg = C.LlamaConfig(vocab_size=96, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2)
    m = LlamaModel.new(cfg, init="random", seed=11)
    m.p = {k: v.to(torch.bfloat16).float() for k, v in m.p.items()}
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, 96, (n,), generator=g).tolist() for n in (7, 12, 3, 9)]
    eng = LLMEngine(CpuModelRunner(m, num_blocks=64, block_size=4, max_model_len=64), num_blocks=64, block_size=4,
                    max_num_seqs=4, max_num_batched_tokens=16, max_model_len=64)
    ref = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_elastic_worker, args=(r, 4, port, q, 3, 4)) for r in range(4)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(4):
        r = q.get(timeout=180)
        got[r[0]] = r[1:]
    for p in procs:
        p.join(timeout=60)
    assert got[3][0] == "exited"
    assert got[2][0] == "spare" and got[2][4] == [[3]]
    for r in (0, 1):
        role, outs, gens, final_world, recovered, steps = got[r]
        assert role == "finished" and gens == 2 and final_world == 2 and recovered == [[3]], got[r]
        assert [outs[i] for i in range(4)] == ref


def test_kv_heads_are_replicated_when_ranks_outnumber_them():
    from unillm_b200.engine.runner import RunnerWeights
    from unillm_b200.models import configs as C
    from unillm_b200.models.families import LlamaModel

    cfg = C.LlamaConfig(vocab_size=64, hidden_size=64, intermediate_size=64, num_hidden_layers=1, num_attention_heads=8,
                        num_key_value_heads=2)
    m = LlamaModel.new(cfg, init="random", seed=1)
    D = m.spec.head_dim
    q, k, v = m.p["layers.0.wqkv"].split([8 * D, 2 * D, 2 * D], 0)
    for rank in range(8):
        w = RunnerWeights(m.spec, m.p, "cpu", rank, 8)
        assert (w.hq, w.hkv, w.kv_lo) == (1, 1, rank // 4)
        got = w.t["layers.0.wqkv"].float()
        assert torch.equal(got[:D], q[rank * D:(rank + 1) * D].to(torch.bfloat16).float())
        assert torch.equal(got[D:2 * D], k[w.kv_lo * D:(w.kv_lo + 1) * D].to(torch.bfloat16).float())
        assert torch.equal(got[2 * D:], v[w.kv_lo * D:(w.kv_lo + 1) * D].to(torch.bfloat16).float())
    assert RunnerWeights.kv_layout(8, 3, 4) == (2, 6)
    with pytest.raises(Exception):
        RunnerWeights.kv_layout(3, 0, 2)


def test_fused_comm_layout_has_no_overlap_and_matches_its_size():
    """The symmetric buffer of the fused tensor-parallel kernels: every area (reduce-scatter / all-gather rows, counters,
    greedy-merge pairs, one-shot all-reduce slots, sampling pair slots, MoE dispatch / combine areas) lies inside the
    allocation, none overlaps another, and ``nbytes`` is exactly the end of the last one."""
    import torch

    from unillm_b200.dist import fused as F

    for world, hidden, max_tokens, k, e in ((2, 512, 512, 0, 0), (8, 4096, 8704, 0, 0), (8, 4096, 2304, 2, 8), (4, 1024, 100, 6, 64)):
        n = F.FusedComm.nbytes(world, hidden, max_tokens, k, e)
        c = F.FusedComm(0, world, hidden, max_tokens, torch.empty(0, dtype=torch.uint8), [0] * world, moe_top_k=k, moe_experts=e)
        names = ["flags", "am_vals", "am_ids", "ar_slots", "sg_vals", "sg_ids"] + (["disp_rows", "disp_meta", "disp_counts", "comb"] if k else [])
        areas = list(c.rs) + list(c.ag) + [getattr(c, nm) for nm in names]
        spans = sorted((a.offset, a.offset + a.nbytes) for a in areas)
        assert spans[0][0] == 0 and spans[-1][1] == n
        for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
            assert a1 <= b0, (world, hidden, (a0, a1), (b0, b1))
        assert all(a.offset % 16 == 0 for a in areas)
        words = [F.AG0, F.RS1, F.AG1, F.RS0, F.ARGMAX_FLAG, F.ARGMAX_ROUND, F.LOCAL_RS0, F.LOCAL_RS1, F.LOCAL_AG0, F.LOCAL_AG1,
                 F.AR_ROUND, F.AR_DONE, F.DISP_FLAG, F.DISP_ROUND, F.LOCAL_DISP, F.SG_ROUND, F.SG_DONE]
        ranges = [(F.AG0, 8), (F.AG1, 8), (F.AR_FLAGS, 64), (F.SG_FLAGS, 64), (F.AR_CTA_ROUNDS, 64), (F.SG_CTA_ROUNDS, 64)]
        used = set()
        for w_ in words:
            if not any(lo <= w_ < lo + cnt for lo, cnt in ranges):
                assert w_ not in used, w_
                used.add(w_)
        for lo, cnt in ranges:
            for w_ in range(lo, lo + cnt):
                assert w_ not in used and w_ < F.FLAG_WORDS, w_
                used.add(w_)


def test_candidate_count_of_a_tensor_parallel_draw():
    from unillm_b200.engine.runner import GpuModelRunner as R

    assert R.candidate_count([0.0, 0.0], None, None) == 1                       # greedy rows: the shard's winner
    assert R.candidate_count([0.7, 0.0, 1.0], [40, 0, 8], [1.0, 1.0, 1.0]) == 40
    assert R.candidate_count([0.7, 1.0], [0, 5], [0.9, 1.0]) == 1024               # top-p keeps 1024 survivors
    assert R.candidate_count([0.7, 1.0], [5000, 5], None) == 1024                  # capped like the sampler
    assert R.candidate_count([0.7, 1.0], None, None) == 0                          # whole-vocabulary draw: gather logits
    assert R.candidate_count([0.7, 1.0], [0, 5], [1.0, 0.5]) == 0
