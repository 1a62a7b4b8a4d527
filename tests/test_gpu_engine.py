"""End-to-end checks of the GPU model runner and engine against the fp32 CPU oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _tiny(kind="llama"):
    from unillm_b200.models import configs as C
    from unillm_b200.models.families import LlamaModel, MixtralModel, GPT2Model, FalconModel

    if kind == "llama":
        cfg = C.LlamaConfig(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                            num_attention_heads=4, num_key_value_heads=2, rms_norm_eps=1e-5)
        cls = LlamaModel
    elif kind == "gpt2":
        cfg = C.GPT2Config().replace(vocab_size=512, hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
                                     num_key_value_heads=4, intermediate_size=1024, max_position_embeddings=256)
        cls = GPT2Model
    elif kind == "falcon":
        cfg = C.FalconConfig().replace(vocab_size=512, hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
                                       num_key_value_heads=2, intermediate_size=1024, new_decoder_architecture=True)
        cls = FalconModel
    else:
        raise ValueError(kind)
    m = cls.new(cfg, init="random", seed=5)
    # the oracle uses the bf16-rounded weights in fp32 so that only activation rounding differs
    m.p = {k: v.to(torch.bfloat16).float() for k, v in m.p.items()}
    return m


def _runners(m, num_blocks=128, block_size=16, graphs=False):
    from unillm_b200.engine.cpu_runner import CpuModelRunner
    from unillm_b200.engine.runner import GpuModelRunner, RunnerWeights

    cpu = CpuModelRunner(m, num_blocks=num_blocks, block_size=block_size, max_model_len=512)
    w = RunnerWeights(m.spec, m.p, "cuda")
    gpu = GpuModelRunner(m.spec, w, num_blocks=num_blocks, block_size=block_size, max_num_seqs=16,
                         max_num_batched_tokens=512, max_model_len=512, use_cuda_graphs=graphs)
    return cpu, gpu


def _prefill_batch(prompts, block_size=16):
    from unillm_b200.engine.runner import StepBatch

    toks, pos, slots, lens, tables, qlens, rows = [], [], [], [], [], [], []
    nxt = 1
    for p in prompts:
        nb = (len(p) + block_size) // block_size + 1
        blocks = list(range(nxt, nxt + nb))
        nxt += nb
        for i, t in enumerate(p):
            toks.append(t), pos.append(i), slots.append(blocks[i // block_size] * block_size + i % block_size)
        lens.append(len(p)), tables.append(blocks), qlens.append(len(p)), rows.append(len(toks) - 1)
    return StepBatch(toks, pos, slots, 0, lens, tables, qlens, rows)


@pytest.mark.parametrize("kind", ["llama", "gpt2", "falcon"])
def test_runner_logits_match_cpu_oracle(kind):
    from unillm_b200.engine.runner import StepBatch
    from unillm_b200.ops import cuda_ops

    m = _tiny(kind)
    cpu, gpu = _runners(m)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (37, 5, 64)]
    b = _prefill_batch(prompts)
    ref = cpu.forward_logits(b)
    got = gpu.logits_for(b).float().cpu()
    torch.cuda.synchronize()
    cuda_ops.check_device_errors()
    err = (got - ref).abs().max().item()
    assert err < 0.08 * max(1.0, ref.abs().max().item()), err
    assert (got.argmax(-1) == ref.argmax(-1)).float().mean() >= 0.66
    # one decode step on top of the prefilled caches
    nxt = ref.argmax(-1).tolist()
    toks, pos, slots, lens = [], [], [], []
    for i, p in enumerate(prompts):
        l = len(p)
        toks.append(nxt[i]), pos.append(l), lens.append(l + 1)
        slots.append(b.block_tables[i][l // 16] * 16 + l % 16)
    d = StepBatch(toks, pos, slots, 3, lens, b.block_tables, [], [0, 1, 2])
    ref2 = cpu.forward_logits(d)
    got2 = gpu.logits_for(d).float().cpu()
    cuda_ops.check_device_errors()
    assert (got2 - ref2).abs().max().item() < 0.08 * max(1.0, ref2.abs().max().item())


def test_engine_tokens_gpu_vs_cpu_and_graph_vs_eager():
    from unillm_b200.engine.llm_engine import LLMEngine
    from unillm_b200.sampling import SamplingParams
    from unillm_b200.ops import cuda_ops

    m = _tiny("llama")
    g = torch.Generator().manual_seed(1)
    shared = torch.randint(0, 512, (70,), generator=g).tolist()
    prompts = [shared + torch.randint(0, 512, (n,), generator=g).tolist() for n in (3, 40, 17, 9, 25, 1, 33, 12, 5, 8)]
    results = {}
    for name in ("cpu", "eager", "graph", "eager-async", "graph-async"):
        cpu, gpu = _runners(m, graphs=name.startswith("graph"))
        eng = LLMEngine(cpu if name == "cpu" else gpu, num_blocks=128, block_size=16, max_num_seqs=16,
                        max_num_batched_tokens=128, max_model_len=512, async_scheduling=name.endswith("async"))
        results[name] = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12))
        if name != "cpu":
            torch.cuda.synchronize()
            cuda_ops.check_device_errors()
            assert eng.stats.cached_tokens > 0
    assert results["eager"] == results["graph"]
    # the host running one step ahead (input tokens fed from the device buffer of the previous step's samples)
    assert results["eager-async"] == results["eager"]
    assert results["graph-async"] == results["graph"]
    agree = sum(a == b for ra, rb in zip(results["cpu"], results["eager"]) for a, b in zip(ra, rb))
    total = sum(len(r) for r in results["cpu"])
    assert agree / total > 0.7, (agree, total)


def test_engine_shared_prefix_cascade_matches_plain():
    """Decode over a radix-shared prefix (cascade: prefix pass + suffix pass + merge) equals the plain path."""
    from unillm_b200.engine.runner import StepBatch
    from unillm_b200.ops import cuda_ops

    m = _tiny("llama")
    _, gpu = _runners(m, num_blocks=256)
    g = torch.Generator().manual_seed(2)
    shared = torch.randint(0, 512, (96,), generator=g).tolist()
    B = 10
    shared_blocks = list(range(1, 7))
    toks, pos, slots, lens, tables, qlens, rows = [], [], [], [], [], [], []
    nxt = 10
    # prefill: first sequence computes the shared prefix; all sequences have unique suffix blocks
    suffixes = [torch.randint(0, 512, (5 + i,), generator=g).tolist() for i in range(B)]
    full = shared + suffixes[0]
    blocks0 = shared_blocks + [nxt, nxt + 1]
    nxt += 2
    for i, t in enumerate(full):
        toks.append(t), pos.append(i), slots.append(blocks0[i // 16] * 16 + i % 16)
    lens.append(len(full)), tables.append(blocks0), qlens.append(len(full)), rows.append(len(toks) - 1)
    for j in range(1, B):
        bl = shared_blocks + [nxt, nxt + 1]
        nxt += 2
        for i, t in enumerate(suffixes[j]):
            p = 96 + i
            toks.append(t), pos.append(p), slots.append(bl[p // 16] * 16 + p % 16)
        lens.append(96 + len(suffixes[j])), tables.append(bl), qlens.append(len(suffixes[j])), rows.append(len(toks) - 1)
    gpu.logits_for(StepBatch(toks, pos, slots, 0, lens, tables, qlens, rows))
    dt, dp, ds, dl = [], [], [], []
    for j in range(B):
        l = lens[j]
        dt.append(7 + j), dp.append(l), dl.append(l + 1), ds.append(tables[j][l // 16] * 16 + l % 16)
    plain = gpu.logits_for(StepBatch(dt, dp, ds, B, dl, tables, [], list(range(B)), shared_prefix_len=0)).clone()
    casc = gpu.logits_for(StepBatch(dt, dp, ds, B, dl, tables, [], list(range(B)), shared_prefix_len=96))
    torch.cuda.synchronize()
    cuda_ops.check_device_errors()
    assert (plain - casc).abs().max().item() < 0.05 * max(1.0, plain.abs().max().item())
