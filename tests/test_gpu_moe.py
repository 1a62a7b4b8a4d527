"""MoE kernels (route / sort / gather / grouped GEMM / combine) against plain PyTorch fp32, and a Mixtral-style and a
DeepSeek-style model through the GPU runner against the CPU oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref_route(x, rw, K, norm_topk):
    logits = x.float() @ rw.float().t()
    if norm_topk:
        v, idx = torch.topk(logits, K, dim=-1)
        w = torch.softmax(v, dim=-1)
    else:
        w, idx = torch.topk(torch.softmax(logits, dim=-1), K, dim=-1)
    return logits, idx, w


@pytest.mark.parametrize("T,E,K,H,norm", [(37, 8, 2, 256, True), (300, 64, 6, 512, False), (1, 16, 4, 128, True),
                                          (64, 128, 2, 256, True)])
def test_route_sort_tables(T, E, K, H, norm):
    from unillm_b200.ops import cuda_ops as ops

    g = torch.Generator().manual_seed(T + E)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    rw = (torch.randn(E, H, generator=g) * 0.2).to(torch.bfloat16)
    logits, idx, w = _ref_route(x, rw, K, norm)
    r = ops.moe_route(x.cuda(), rw.cuda(), K, norm_topk=norm, round_logits_bf16=False)
    torch.cuda.synchronize()
    ops.check_device_errors()
    ids = r.topk_ids.cpu().long()
    # a near-tie may be ordered differently; compare by logit value
    sel = torch.gather(logits, 1, ids)
    assert (sel - torch.gather(logits, 1, idx)).abs().max() < 2e-2
    same = (ids == idx).all(dim=1)
    assert same.float().mean() > 0.9
    assert (r.topk_w.cpu()[same] - w[same]).abs().max() < 2e-3
    counts = torch.bincount(ids.flatten(), minlength=E)
    assert torch.equal(r.counts.cpu().long(), counts)
    off = torch.cat([torch.zeros(1, dtype=torch.long), counts.cumsum(0)])
    assert torch.equal(r.offsets.cpu().long(), off)
    sr, rs = r.sorted_rows.cpu().long(), r.row_slot.cpu().long()
    assert torch.equal(sr[rs], torch.arange(T * K))
    assert sorted(sr.tolist()) == list(range(T * K))
    for e in range(E):
        rows = sr[off[e]:off[e + 1]]
        assert (ids.flatten()[rows] == e).all()
    tiles = r.tiles.cpu()
    valid = tiles[tiles[:, 0] >= 0]
    assert int(((counts + r.tile_tokens - 1) // r.tile_tokens).sum()) == valid.shape[0]
    for e_, r0, r1, _ in valid.tolist():
        assert off[e_] <= r0 < r1 == off[e_ + 1] and (r0 - off[e_]) % r.tile_tokens == 0


@pytest.mark.parametrize("T,E,K,H,I,gated", [(64, 8, 2, 256, 384, True), (500, 8, 2, 512, 256, True),
                                             (33, 16, 4, 256, 200, False), (7, 64, 6, 128, 128, True)])
def test_moe_block_matches_fp32(T, E, K, H, I, gated):
    from unillm_b200.ops import cuda_ops as ops

    g = torch.Generator().manual_seed(T * 3 + E)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    res = torch.randn(T, H, generator=g).to(torch.bfloat16)
    rw = (torch.randn(E, H, generator=g) * 0.2).to(torch.bfloat16)
    gu = (torch.randn(E, (2 if gated else 1) * I, H, generator=g) * H ** -0.5).to(torch.bfloat16)
    dn = (torch.randn(E, H, I, generator=g) * I ** -0.5).to(torch.bfloat16)
    xd = x.cuda()
    r = ops.moe_route(xd, rw.cuda(), K, norm_topk=True, round_logits_bf16=False)
    xs = ops.moe_gather(xd, r)
    a = ops.grouped_gemm(xs, gu.cuda(), r, dual_rows=I if gated else 0, act="silu")
    y = ops.grouped_gemm(a, dn.cuda(), r)
    out = ops.moe_combine(y, r, residual=res.cuda())
    torch.cuda.synchronize()
    ops.check_device_errors()
    ids, w = r.topk_ids.cpu().long(), r.topk_w.cpu()
    assert torch.equal(xs.cpu(), x[r.sorted_rows.cpu().long() // K])
    ref = res.float().clone()
    for t in range(T):
        for k in range(K):
            e = int(ids[t, k])
            hcol = x[t].float() @ gu[e].float().t()
            hcol = torch.nn.functional.silu(hcol[:I]) * hcol[I:] if gated else torch.nn.functional.silu(hcol)
            ref[t] += w[t, k] * (hcol.to(torch.bfloat16).float() @ dn[e].float().t())
    err = (out.float().cpu() - ref).abs().max().item()
    assert err < 0.05 * max(1.0, ref.abs().max().item()), err


@pytest.mark.parametrize("kind", ["mixtral", "deepseek"])
def test_moe_model_runner_vs_cpu(kind):
    from unillm_b200.engine.cpu_runner import CpuModelRunner
    from unillm_b200.engine.llm_engine import LLMEngine
    from unillm_b200.engine.runner import GpuModelRunner, RunnerWeights
    from unillm_b200.models import configs as C
    from unillm_b200.models.families import DECODER_FAMILIES
    from unillm_b200.ops import cuda_ops
    from unillm_b200.sampling import SamplingParams

    if kind == "mixtral":
        cls = DECODER_FAMILIES["mixtral"]
        cfg = C.MixtralConfig(vocab_size=512, hidden_size=256, intermediate_size=256, num_hidden_layers=2,
                              num_attention_heads=4, num_key_value_heads=2, num_experts=8, sliding_window=4096)
    else:
        cls = DECODER_FAMILIES["deepseek_moe"]
        cfg = cls.config_class().replace(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                                         num_attention_heads=4, num_key_value_heads=4, moe_intermediate_size=128, num_experts=16,
                                         num_experts_per_tok=4)
    m = cls.new(cfg, init="random", seed=9)
    m.p = {k: v.to(torch.bfloat16).float() for k, v in m.p.items()}
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (21, 40, 7, 33)]
    outs = {}
    for name in ("cpu", "eager", "graph"):
        if name == "cpu":
            runner = CpuModelRunner(m, num_blocks=128, block_size=16, max_model_len=256)
        else:
            runner = GpuModelRunner(m.spec, RunnerWeights(m.spec, m.p, "cuda"), num_blocks=128, block_size=16, max_num_seqs=8,
                                    max_num_batched_tokens=256, max_model_len=256, use_cuda_graphs=(name == "graph"))
        eng = LLMEngine(runner, num_blocks=128, block_size=16, max_num_seqs=8, max_num_batched_tokens=256, max_model_len=256)
        outs[name] = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10))
        if name != "cpu":
            torch.cuda.synchronize()
            cuda_ops.check_device_errors()
    assert outs["eager"] == outs["graph"]
    agree = sum(a == b for ra, rb in zip(outs["cpu"], outs["eager"]) for a, b in zip(ra, rb))
    assert agree / 40 > 0.6, agree


def test_expert_parallel_partials_and_fused_combine():
    """Expert parallelism emulated on one GPU: each 'rank' routes with its expert range; partial rows summed over the
    ranks equal the single-rank result, both through plain combine and through the combine that pushes into the
    owners' receive slots (all slots live on this GPU here; ranks run one after another on one stream)."""
    from unillm_b200.ops import cuda_ops as ops

    T, E, K, H, I, W = 96, 8, 2, 256, 128, 4
    g = torch.Generator().manual_seed(11)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).cuda()
    rw = (torch.randn(E, H, generator=g) * 0.2).to(torch.bfloat16).cuda()
    gu = (torch.randn(E, 2 * I, H, generator=g) * H ** -0.5).to(torch.bfloat16).cuda()
    dn = (torch.randn(E, H, I, generator=g) * I ** -0.5).to(torch.bfloat16).cuda()

    def run(lo, n, rs=None):
        r = ops.moe_route(x, rw, K, round_logits_bf16=False, expert_lo=lo, num_local_experts=n)
        xs = ops.moe_gather(x, r)
        a = ops.grouped_gemm(xs, gu[lo:lo + (n or E)].contiguous(), r, dual_rows=I, act="silu")
        y = ops.grouped_gemm(a, dn[lo:lo + (n or E)].contiguous(), r)
        if rs is None:
            return ops.moe_combine(y, r), r
        ops.moe_combine_rs(y, r, rs)
        return None, r

    full, r_full = run(0, 0)
    parts = []
    for rank in range(W):
        out, r = run(rank * (E // W), E // W)
        parts.append(out.float())
        slots = r.row_slot.cpu()
        ids = r.topk_ids.cpu().flatten()
        local = (ids >= rank * (E // W)) & (ids < (rank + 1) * (E // W))
        assert ((slots >= 0) == local).all()
    total = torch.stack(parts).sum(0)
    assert (total - full.float()).abs().max().item() < 0.03 * max(1.0, full.float().abs().max().item())
    # fused combine + reduce-scatter: rows_per_rank R, owner o receives [W][R][H]
    R = T // W
    recv = [torch.zeros(W, R, H, dtype=torch.bfloat16, device="cuda") for _ in range(W)]
    flags = torch.zeros(W, dtype=torch.int32, device="cuda")
    local = torch.zeros(W, dtype=torch.int32, device="cuda")          # one arrival counter per emulated rank
    for rank in range(W):
        rs = {"world": W, "rank": rank, "rows_per_rank": R, "peer_out": [t.data_ptr() for t in recv],
              "peer_flag": [flags[o:o + 1].data_ptr() for o in range(W)], "local_count": local[rank:rank + 1].data_ptr()}
        run(rank * (E // W), E // W, rs)
    torch.cuda.synchronize()
    ops.check_device_errors()
    assert flags.cpu().tolist() == [W] * W                            # one arrival per source rank
    assert local.cpu().tolist() == [0] * W                            # the last CTA of each launch zeroed its counter
    got = torch.cat([recv[o].float().sum(0) for o in range(W)], 0)
    assert (got - full.float()).abs().max().item() < 0.05 * max(1.0, full.float().abs().max().item())


@pytest.mark.parametrize("T,E,K,H,I,W", [(96, 8, 2, 256, 128, 4), (64, 4, 2, 512, 256, 2), (120, 64, 6, 256, 128, 8)])
def test_sparse_dispatch_and_combine_emulated_ranks(T, E, K, H, I, W):
    """Sparse expert-parallel dispatch / combine with all ranks emulated on one GPU (every sender runs before any
    receiver on one stream, so each bounded wait finds its counter complete): every (token, expert) pair reaches
    exactly one rank, the combine area of a token's owner ends up with the K weighted expert outputs, their sum equals
    the single-rank MoE block, and a second exchange (counted, not reset, arrival words) works as well."""
    from unillm_b200.dist.fused import RS1, FusedComm
    from unillm_b200.ops import cuda_ops as ops

    g = torch.Generator().manual_seed(T + E)
    rw = (torch.randn(E, H, generator=g) * 0.2).to(torch.bfloat16).cuda()
    gu = (torch.randn(E, 2 * I, H, generator=g) * H ** -0.5).to(torch.bfloat16).cuda()
    dn = (torch.randn(E, H, I, generator=g) * I ** -0.5).to(torch.bfloat16).cuda()
    comms = FusedComm.emulated(W, H, T, "cuda", moe_top_k=K, moe_experts=E)
    R, EL = T // W, E // W
    states = [ops.MoeDispatch(R, K, E, W, "cuda") for _ in range(W)]
    for it in range(2):
        x = torch.randn(T, H, generator=g).to(torch.bfloat16).cuda()
        r_full = ops.moe_route(x, rw, K, round_logits_bf16=False)
        xs = ops.moe_gather(x, r_full)
        full = ops.moe_combine(ops.grouped_gemm(ops.grouped_gemm(xs, gu, r_full, dual_rows=I, act="silu"), dn, r_full), r_full)
        for rank in range(W):                                   # senders
            own = x[rank * R:(rank + 1) * R].contiguous()
            ops.moe_route(own, rw, K, round_logits_bf16=False, routing=states[rank].route)
            ops.moe_dispatch(own, states[rank], comms[rank].moe_dispatch_args())
        received = 0
        for rank in range(W):                                   # receivers: experts [rank * EL, (rank + 1) * EL)
            d, c = states[rank], comms[rank]
            ops.moe_recv_build(d, c.moe_recv_args(), "cuda")
            rows = ops.gather_rows(c.moe_recv_rows(d.slots), d.sorted_rows)
            a = ops.grouped_gemm(rows, gu[rank * EL:(rank + 1) * EL].contiguous(), d, dual_rows=I, act="silu")
            y = ops.grouped_gemm(a, dn[rank * EL:(rank + 1) * EL].contiguous(), d)
            ops.moe_combine_push(y, d, c.moe_return_args())
            torch.cuda.synchronize()
            ops.check_device_errors()
            n = int(d.offsets[EL])
            received += n
            # the rows that arrived are the rows of the tokens that chose this rank's experts, in expert order
            meta = d.slot_meta[:n].cpu()
            pair = meta[:, 0].long()
            ids = r_full.topk_ids.cpu().flatten()
            assert ((ids[pair] >= rank * EL) & (ids[pair] < (rank + 1) * EL)).all()
            assert (ids[pair][1:] >= ids[pair][:-1]).all()
            assert torch.equal(rows[:n].cpu(), x.cpu()[pair // K])
            assert torch.equal(meta[:, 1].long(), (pair // K) // R)            # return address: the token's owner
        assert received == T * K                                               # token conservation
        got = torch.cat([comms[o].moe_comb_tensor(R).float().sum(0) for o in range(W)], 0)
        assert (got - full.float()).abs().max().item() < 0.05 * max(1.0, full.float().abs().max().item())
        for o in range(W):
            fl = comms[o].buf[comms[o].flags.offset:comms[o].flags.offset + 256].view(torch.int32)
            assert int(fl[RS1]) == W                                           # one combine arrival per rank
            fl[RS1] = 0                                                        # what the next norm kernel does in the pipeline
