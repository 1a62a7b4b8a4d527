"""``DecoderSpec``: one parametric description of a decoder-only transformer block stack, and
``KeyScheme``: how a family names its tensors on disk.

Thirty-odd of the reference's 47 model files (``crates/runtime/src/models_v2/*.rs``) are the same
pre-norm decoder with small variations; instead of one copy of the code per family, each family
supplies a config -> ``DecoderSpec`` function and a ``KeyScheme``.  The variation axes are exactly the
ones the reference's files differ in: norm kind and bias, rotary variant (full / partial / theta /
linear or Llama-3 scaling / interleaved), ALiBi, learned positions, sliding window, QKV packing,
residual topology (sequential / parallel, shared or separate norms, post-LN), MLP kind (gated /
plain, activation), biases, embedding / logit / residual / attention scalings, tied embeddings, and
mixture-of-experts (experts, top-k, shared experts, dense-parallel MLP, leading dense layers).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass
class MoESpec:
    num_experts: int = 8
    top_k: int = 2
    intermediate_size: int = 14336       # per-expert FFN width
    normalize_topk: bool = True          # softmax over the k selected logits (Mixtral); else softmax over all E
    num_shared_experts: int = 0          # always-on experts (DeepSeek-MoE); width = num_shared * intermediate_size
    dense_parallel: bool = False         # Arctic: dense MLP output + MoE output
    first_k_dense: int = 0               # leading layers that use the dense MLP instead of MoE
    act: str = "silu"
    gated: bool = True


@dataclass
class DecoderSpec:
    vocab_size: int = 32000
    hidden_size: int = 4096
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 32
    head_dim: int = 128
    intermediate_size: int = 11008
    max_position_embeddings: int = 2048
    # norms
    norm: str = "rms"                    # "rms" | "layer"
    norm_eps: float = 1e-6
    norm_bias: bool = False
    norm_weight_offset_one: bool = False  # Gemma: y * (1 + w)
    final_norm: bool = True
    embed_norm: bool = False             # BLOOM word_embeddings_layernorm
    qk_norm: bool = False
    # positions
    pos: str = "rope"                    # "rope" | "learned" | "alibi" | "none"
    rope_theta: float = 10000.0
    rotary_dim: Optional[int] = None     # None = head_dim
    rope_interleaved: bool = False       # GPT-J style adjacent pairs
    rope_pos_scale: float = 1.0          # linear scaling: position * scale
    rope_llama3: Optional[Tuple[float, float, float, float]] = None  # (factor, low, high, original_ctx)
    learned_pos_offset: int = 0          # OPT stores positions shifted by 2
    window: int = 0                      # sliding-window size, 0 = full attention
    # projections
    qkv_bias: bool = False
    o_bias: bool = False
    mlp_bias: bool = False
    lm_head_bias: bool = False
    mlp: str = "gated"                   # "gated" (act(gate) * up) | "plain" (act(fc1))
    act: str = "silu"
    # topology
    parallel_residual: bool = False      # x + attn(n1(x)) + mlp(n2(x))
    parallel_shared_norm: bool = False   # ... with mlp reading n1(x) (GPT-J, Phi, Falcon-7B)
    post_ln: bool = False                # OPT-350m style: norm after the residual add
    # scalings
    embed_scale: float = 1.0
    logit_scale: float = 1.0
    residual_scale: float = 1.0
    attn_scale: Optional[float] = None   # None = 1/sqrt(head_dim)
    tie_embeddings: bool = False
    embed_proj_dim: Optional[int] = None  # OPT word_embed_proj_dim != hidden: project_in / project_out
    moe: Optional[MoESpec] = None
    # behaviour of the reference implementation that differs from the published architecture;
    # applied only when a model is built with reference_quirks=True
    ref_ln_star: bool = False            # uses mean-subtracting layer_norm(x, w, None) where the family has RMSNorm
    ref_layer_eps: Optional[float] = None  # eps hard-coded inside layers (llama.rs:633,642 uses 1e-6)
    initializer_range: float = 0.02

    @property
    def q_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    @property
    def rd(self) -> int:
        return self.head_dim if self.rotary_dim is None else self.rotary_dim

    def layer_is_moe(self, i: int) -> bool:
        return self.moe is not None and i >= self.moe.first_k_dense


@dataclass
class KeyScheme:
    """Tensor names of one family.  Every entry is a tuple of aliases, tried in order; layer-level
    names are relative to ``layer.format(i=...)``.  ``.weight`` / ``.bias`` are appended."""

    embed: Tuple[str, ...] = ("model.embed_tokens",)
    pos_embed: Tuple[str, ...] = ()
    embed_norm: Tuple[str, ...] = ()
    project_in: Tuple[str, ...] = ()
    project_out: Tuple[str, ...] = ()
    layer: Tuple[str, ...] = ("model.layers.{i}.",)
    ln1: Tuple[str, ...] = ("input_layernorm",)
    ln2: Tuple[str, ...] = ("post_attention_layernorm",)
    q: Tuple[str, ...] = ("self_attn.q_proj",)
    k: Tuple[str, ...] = ("self_attn.k_proj",)
    v: Tuple[str, ...] = ("self_attn.v_proj",)
    qkv: Tuple[str, ...] = ()
    qkv_layout: str = "concat"           # "concat" [Q;K;V] | "per_head" [h][q,k,v] | "grouped" [kv group][G q, k, v]
    q_norm: Tuple[str, ...] = ("self_attn.q_norm",)
    k_norm: Tuple[str, ...] = ("self_attn.k_norm",)
    o: Tuple[str, ...] = ("self_attn.o_proj",)
    gate: Tuple[str, ...] = ("mlp.gate_proj",)
    up: Tuple[str, ...] = ("mlp.up_proj",)
    down: Tuple[str, ...] = ("mlp.down_proj",)
    gate_up: Tuple[str, ...] = ()        # packed [gate; up]
    final_norm: Tuple[str, ...] = ("model.norm",)
    lm_head: Tuple[str, ...] = ("lm_head",)
    transposed: bool = False             # GPT-2 Conv1D stores [in, out]
    router: Tuple[str, ...] = ("block_sparse_moe.gate",)
    expert: Tuple[str, ...] = ("block_sparse_moe.experts.{e}.",)
    e_gate: Tuple[str, ...] = ("w1",)
    e_up: Tuple[str, ...] = ("w3",)
    e_down: Tuple[str, ...] = ("w2",)
    shared_gate: Tuple[str, ...] = ("mlp.shared_experts.gate_proj",)
    shared_up: Tuple[str, ...] = ("mlp.shared_experts.up_proj",)
    shared_down: Tuple[str, ...] = ("mlp.shared_experts.down_proj",)
