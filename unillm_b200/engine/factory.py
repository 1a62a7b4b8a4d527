"""From a loaded model to a serving engine on the sm_100a kernels.

``build_engine(model, device="cuda")`` is the bridge between the public loading path (``ModelLoader.load_model`` ->
a ``DecoderModel`` with HF-named weights already folded into kernel layout) and the engine that the benchmark
drives: ``RunnerWeights`` (bf16, fused QKV / gate-up, tensor-parallel shards) -> ``GpuModelRunner`` -> ``LLMEngine``.
``why_not_gpu(model)`` names the reason when a model cannot take that path (a family outside the parametric
decoder, a topology the fused runner does not cover); callers then stay on the whole-model path or on the CPU runner.

Reference counterparts: ``InferencePipeline::new`` / ``generate`` (``crates/runtime/src/inference.rs:159-320``) and the
``generate`` sub-command (``crates/runtime/src/bin/unillm.rs:73-168``), which build a LLaMA model and re-run it on
the whole sequence for every token on the CPU.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..types import UnsupportedOperation


def why_not_gpu(model) -> Optional[str]:
    """None when ``model`` can be served by ``GpuModelRunner``; otherwise one sentence saying why not."""
    from ..models.decoder import DecoderModel

    if not torch.cuda.is_available():
        return "no CUDA device is available"
    if not isinstance(model, DecoderModel):
        return f"{type(model).__name__} is not a decoder-only model of the parametric block"
    s = model.spec
    if s.norm not in ("rms", "layer") or s.post_ln or s.embed_proj_dim:
        return "post-LN / projected-embedding topologies run on the whole-model path"
    if getattr(model, "reference_quirks", False):
        return "reference_quirks changes the normalisation; the kernels implement the published architecture"
    if s.hidden_size % 8 or s.head_dim % 8:
        return "hidden size and head size must be multiples of 8 (16-byte rows for the TMA copies)"
    return None


def _auto_num_blocks(spec, weights, block_size: int, device, gpu_memory_fraction: float, max_model_len: int,
                     max_num_seqs: int) -> int:
    """KV blocks that fit in ``gpu_memory_fraction`` of the device after the weights, capped by what the sequence
    limits can ever use."""
    free, total = torch.cuda.mem_get_info(device)
    budget = int(total * gpu_memory_fraction) - (total - free)
    per_block = 2 * spec.num_layers * weights.hkv * block_size * spec.head_dim * 2
    fit = max(budget // max(per_block, 1), 0)
    useful = max_num_seqs * (-(-max_model_len // block_size) + 1) + 64
    n = int(min(fit, useful))
    if n < -(-max_model_len // block_size) + 1:
        raise UnsupportedOperation(f"not enough device memory for one sequence of {max_model_len} tokens "
                                   f"({fit} KV blocks fit)")
    return n


def build_engine(model, *, device="cuda", max_num_seqs: int = 64, max_num_batched_tokens: int = 2048,
                 max_model_len: Optional[int] = None, block_size: int = 16, num_blocks: Optional[int] = None,
                 gpu_memory_fraction: float = 0.9, enable_prefix_caching: bool = True, async_scheduling: bool = False,
                 use_cuda_graphs: bool = True, eos_token_id: Optional[int] = None, rank: int = 0, world: int = 1,
                 tp=None, quantize: Optional[str] = None):
    """An ``LLMEngine`` that runs ``model`` on the hand-written kernels of ``device``.

    ``quantize`` ("q4_k", "q8_0", "q4_0"): keep the projection matrices block-quantised on the device (4.5 - 8.5 bits
    per weight, see ``RunnerWeights.quantize``) instead of bf16.

    Raises ``UnsupportedOperation`` (with the reason) when the model cannot take that path; see ``why_not_gpu``."""
    from .llm_engine import LLMEngine
    from .runner import GpuModelRunner, RunnerWeights

    why = why_not_gpu(model)
    if why is not None:
        raise UnsupportedOperation(why)
    dev = torch.device(device)
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    spec = model.spec
    if max_model_len is None:
        max_model_len = min(spec.max_position_embeddings, 8192)
    weights = RunnerWeights(spec, model.p, dev, rank, world)
    if quantize:
        weights.quantize(quantize)
    if num_blocks is None:
        num_blocks = _auto_num_blocks(spec, weights, block_size, dev, gpu_memory_fraction, max_model_len, max_num_seqs)
    runner = GpuModelRunner(spec, weights, num_blocks=num_blocks, block_size=block_size, max_num_seqs=max_num_seqs,
                            max_num_batched_tokens=max_num_batched_tokens, max_model_len=max_model_len, tp=tp, device=dev,
                            use_cuda_graphs=use_cuda_graphs)
    return LLMEngine(runner, num_blocks=num_blocks, block_size=block_size, max_num_seqs=max_num_seqs,
                     max_num_batched_tokens=max_num_batched_tokens, max_model_len=max_model_len,
                     enable_prefix_caching=enable_prefix_caching, eos_token_id=eos_token_id,
                     async_scheduling=async_scheduling)


def build_cpu_engine(model, *, max_num_seqs: int = 8, max_num_batched_tokens: int = 512, max_model_len: int = 8192,
                     block_size: int = 16, num_blocks: int = 1024, eos_token_id: Optional[int] = None):
    """The same engine over the fp32 CPU runner (the oracle path)."""
    from .cpu_runner import CpuModelRunner
    from .llm_engine import LLMEngine

    runner = CpuModelRunner(model, num_blocks=num_blocks, block_size=block_size, max_model_len=max_model_len)
    return LLMEngine(runner, num_blocks=num_blocks, block_size=block_size, max_num_seqs=max_num_seqs,
                     max_num_batched_tokens=max_num_batched_tokens, max_model_len=max_model_len, eos_token_id=eos_token_id)
