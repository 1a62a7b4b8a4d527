"""The product's front doors on the GPU kernels: a checkpoint directory written to disk is loaded with
``ModelLoader``, served through ``InferencePipeline(device="cuda")`` and through ``python -m unillm_b200 generate
--device cuda``, and its greedy tokens are compared with the fp32 CPU oracle.

The model has head dimension 128 and the prompts share a prefix, so the path under test is the flagship one: tcgen05
prefill attention, the warp-MMA / persistent decode kernels, the shared-prefix cascade and the radix cache -- not the
head-dim-64 fallbacks.  Counterparts in the reference: ``InferencePipeline::generate``
(``crates/runtime/src/inference.rs:159-320``) and ``unillm generate`` (``crates/runtime/src/bin/unillm.rs:73-168``).
"""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _write_checkpoint(path, seed=7):
    """A tiny Llama checkpoint directory (config.json + model.safetensors, HF tensor names), head dimension 128."""
    from unillm_b200.models import configs as C
    from unillm_b200.models.families import LlamaModel
    from unillm_b200.weights.loaders import write_safetensors

    cfg = C.LlamaConfig(vocab_size=512, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                        num_attention_heads=4, num_key_value_heads=2, rms_norm_eps=1e-5, max_position_embeddings=1024)
    m = LlamaModel.new(cfg, init="random", seed=seed)
    m.p = {k: v.to(torch.bfloat16).float() for k, v in m.p.items()}     # the oracle sees what bf16 storage holds
    os.makedirs(path, exist_ok=True)
    hf = m.export_hf()
    write_safetensors(os.path.join(path, "model.safetensors"), {k: v.to(torch.bfloat16) for k, v in hf.tensors.items()})
    d = cfg.to_dict()
    d["architectures"] = ["LlamaForCausalLM"]
    d["model_type"] = "llama"
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(d, f)
    return m


def _oracle_check(model, prompt, got, max_margin=0.05):
    """``got`` must follow the fp32 oracle's greedy choice; where it departs, the oracle's own margin between its
    choice and the token taken has to be a rounding-sized one, and the comparison of that sequence ends there.
    Returns the number of tokens that agreed."""
    ids = list(prompt)
    for k, tok in enumerate(got):
        logits = model.forward_ids(ids) if hasattr(model, "forward_ids") else None
        if logits is None:
            from unillm_b200.model_core import ModelInputs

            logits = model.forward(ModelInputs.text(torch.tensor([ids]))).main_tensor()[0, -1].float()
        best = int(logits.argmax())
        if best != tok:
            margin = float(logits[best] - logits[tok])
            scale = float(logits.abs().max())
            assert margin <= max_margin * max(scale, 1.0), (k, best, tok, margin, scale)
            return k
        ids.append(tok)
    return len(got)


def test_pipeline_and_cli_on_gpu_kernels_match_cpu_oracle(tmp_path):
    from unillm_b200.config import GenerationConfig
    from unillm_b200.ops import cuda_ops
    from unillm_b200.pipeline import InferencePipelineBuilder
    from unillm_b200.weights import ModelLoader

    ckpt = str(tmp_path / "tiny-llama-hd128")
    oracle = _write_checkpoint(ckpt)
    model = ModelLoader().load_model(ckpt, device="cpu")
    assert model.spec.head_dim == 128
    pipe = InferencePipelineBuilder().model(model).device("cuda").engine_options(max_num_seqs=16, max_model_len=512).build()
    assert pipe.engine_note is None and pipe.use_engine
    g = torch.Generator().manual_seed(3)
    shared = torch.randint(0, 512, (80,), generator=g).tolist()          # five whole blocks of shared prefix
    prompts = [shared + torch.randint(0, 512, (n,), generator=g).tolist() for n in (9, 30, 2, 17)]
    cfg = GenerationConfig.greedy(12, eos_token_id=-1)
    agreed = total = 0
    for p in prompts:
        got = pipe.generate_tokens(p, cfg)
        assert len(got) == 12
        agreed += _oracle_check(oracle, p, got)
        total += len(got)
    assert pipe.engine_kind == "gpu-kernels"
    assert cuda_ops.attn_prefill_last_path() == "tcgen05"
    torch.cuda.synchronize()
    cuda_ops.check_device_errors()
    assert pipe._engine.stats.cached_tokens >= 3 * 80               # later prompts reuse the first one's prefix blocks
    assert agreed >= 0.75 * total, (agreed, total)

    # batched: all prompts at once -> 12 decode steps with >= 8... here 4 rows; plus a wider batch for the cascade
    eng = pipe._engine
    from unillm_b200.sampling import SamplingParams

    many = [shared + torch.randint(0, 512, (5 + i,), generator=g).tolist() for i in range(10)]
    outs = eng.generate(many, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    torch.cuda.synchronize()
    cuda_ops.check_device_errors()
    a2 = sum(_oracle_check(oracle, p, o) for p, o in zip(many, outs))
    assert a2 >= 0.75 * 80, a2

    # the CLI takes the same path: its text equals the pipeline's for the same prompt
    text = pipe.generate("the quick brown fox", GenerationConfig.greedy(8, eos_token_id=-1))
    env = dict(os.environ, PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "unillm_b200", "generate", "--device", "cuda", "-m", ckpt, "-p",
                        "the quick brown fox", "--max-tokens", "8", "--temperature", "0"], capture_output=True, text=True,
                       env=env, cwd=ROOT, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "sm_100a kernels" in r.stderr
    assert r.stdout.strip() == text.strip()


def test_pipeline_names_the_reason_when_a_model_stays_off_the_kernel_runner():
    from unillm_b200.engine.factory import why_not_gpu
    from unillm_b200.models import configs as C
    from unillm_b200.models.encoders import BertModel

    m = BertModel.new(C.BertConfig(vocab_size=128, hidden_size=64, num_hidden_layers=1, num_attention_heads=2,
                                   intermediate_size=128))
    assert "not a decoder-only model" in why_not_gpu(m)


def test_block_quantised_weights_serve_like_their_bf16_expansion(tmp_path):
    """Q4_K projection weights kept as blocks on the device: decode rows go through the quantised GEMV kernel, prefill
    rows through dequantise + tensor-core GEMM.  The reference run uses the bf16 expansion of the same blocks, so
    only summation order differs."""
    from unillm_b200.engine.llm_engine import LLMEngine
    from unillm_b200.engine.runner import GpuModelRunner, QWeight, RunnerWeights
    from unillm_b200.models import configs as C
    from unillm_b200.models.families import LlamaModel
    from unillm_b200.ops import cuda_ops
    from unillm_b200.ops import quant as Q
    from unillm_b200.sampling import SamplingParams
    from unillm_b200.weights.gguf import Q4_K, dequantize_blocks, quantize_blocks

    # kernel level: the specialised Q4_K GEMV against the dequantised matrix, every row count it serves
    g = torch.Generator().manual_seed(0)
    N_, Kd = 1000, 1024
    wf = torch.randn(N_, Kd, generator=g) * 0.05
    raw = quantize_blocks(wf, Q4_K)
    wd = dequantize_blocks(raw, Q4_K, (N_, Kd))
    blocks = torch.from_numpy(raw.copy()).cuda()
    for M in (1, 2, 3, 5, 8):
        x = torch.randn(M, Kd, generator=g).to(torch.bfloat16).cuda()
        got = Q.qgemv_cuda(blocks, x, N_, Q4_K).float().cpu()
        ref = x.float().cpu() @ wd.t()
        assert (got - ref).abs().max().item() < 0.02 * max(1.0, ref.abs().max().item()), M

    cfg = C.LlamaConfig(vocab_size=512, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                        num_attention_heads=4, num_key_value_heads=2, rms_norm_eps=1e-5, max_position_embeddings=1024)
    m = LlamaModel.new(cfg, init="random", seed=9)
    wq = RunnerWeights(m.spec, m.p, "cuda").quantize("q4_k")
    assert isinstance(wq.t["layers.0.wqkv"], QWeight) and isinstance(wq.t["lm_head"], QWeight)
    dense_bytes = RunnerWeights(m.spec, m.p, "cuda").nbytes()
    assert wq.nbytes() < 0.5 * dense_bytes
    wref = wq.dequantized_copy()
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (33, 5, 70)]
    outs = {}
    for name, w in (("q", wq), ("ref", wref)):
        runner = GpuModelRunner(m.spec, w, num_blocks=64, max_num_seqs=4, max_num_batched_tokens=256, max_model_len=256,
                                use_cuda_graphs=False)
        eng = LLMEngine(runner, num_blocks=64, max_num_seqs=4, max_num_batched_tokens=256, max_model_len=256)
        outs[name] = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
        torch.cuda.synchronize()
        cuda_ops.check_device_errors()
    total = sum(len(o) for o in outs["ref"])
    same = sum(a == b for x, y in zip(outs["q"], outs["ref"]) for a, b in zip(x, y))
    assert same >= 0.9 * total, (same, total)
