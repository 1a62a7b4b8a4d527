"""Decoder-only families: config -> ``DecoderSpec`` and on-disk ``KeyScheme`` for each.

Each class corresponds to one file of ``crates/runtime/src/models_v2/`` (cited per class).  The
published architecture is implemented (true RMSNorm where the family has it, per-head packed QKV
for GPT-NeoX / BLOOM, ...); where the reference's implementation deviates, the deviation is
recorded in the spec's ``ref_*`` fields and only applied with ``reference_quirks=True``.
"""
from __future__ import annotations

import math

from . import configs as C
from .decoder import DecoderModel
from .spec import DecoderSpec, KeyScheme, MoESpec


def _base(c, **kw) -> DecoderSpec:
    """Fields shared by the LLaMA-shaped configs."""
    nh = c.num_attention_heads
    d = dict(
        vocab_size=c.vocab_size, hidden_size=c.hidden_size, num_layers=c.num_hidden_layers, num_heads=nh,
        num_kv_heads=getattr(c, "num_key_value_heads", nh) or nh,
        head_dim=getattr(c, "head_dim", None) or c.hidden_size // nh,
        intermediate_size=getattr(c, "intermediate_size", 4 * c.hidden_size),
        max_position_embeddings=getattr(c, "max_position_embeddings", 2048),
        norm_eps=getattr(c, "rms_norm_eps", getattr(c, "layer_norm_eps", 1e-5)),
        rope_theta=getattr(c, "rope_theta", 10000.0), act=_act_name(getattr(c, "hidden_act", "silu")),
        tie_embeddings=getattr(c, "tie_word_embeddings", False),
        initializer_range=getattr(c, "initializer_range", 0.02),
    )
    d.update(kw)
    return DecoderSpec(**d)


def _act_name(a: str) -> str:
    """Normalise HuggingFace activation spellings to the names the kernels know."""
    return {"swiglu": "silu", "swish": "silu", "geglu": "gelu_tanh", "gelu_new": "gelu_tanh",
            "gelu_pytorch_tanh": "gelu_tanh", "gelu_fast": "gelu_tanh"}.get(a, a)


LLAMA_KEYS = KeyScheme()


class LlamaModel(DecoderModel):
    """LLaMA 1/2/3, TinyLlama (``models_v2/llama.rs``).  The reference normalises with a mean-subtracting
    layer norm and a hard-coded eps of 1e-6 inside layers (``llama.rs:633,642``): ``ref_ln_star``."""

    config_class = C.LlamaConfig
    scheme = LLAMA_KEYS

    @classmethod
    def spec_from_config(cls, c):
        return _base(c, qkv_bias=c.attention_bias, o_bias=c.attention_bias, ref_ln_star=True, ref_layer_eps=1e-6)


class QwenModel(DecoderModel):
    """Qwen / Qwen1.5 / Qwen2 (``models_v2/qwen.rs``).  QKV biases are loaded when present (the reference
    does not model them)."""

    config_class = C.QwenConfig
    scheme = LLAMA_KEYS

    @classmethod
    def spec_from_config(cls, c):
        return _base(c, qkv_bias=True, window=c.sliding_window if c.use_sliding_window else 0, ref_ln_star=True)


class GemmaModel(DecoderModel):
    """Gemma 2B / 7B (``models_v2/gemma.rs``): embeddings scaled by sqrt(hidden) (``:174-175``), GeGLU
    (``:604-618``), RMSNorm with (1 + w), tied head."""

    config_class = C.GemmaConfig
    scheme = LLAMA_KEYS

    @classmethod
    def spec_from_config(cls, c):
        act = "gelu_tanh" if c.hidden_act in ("gelu", "gelu_pytorch_tanh", "gelu_tanh") else c.hidden_act
        return _base(c, head_dim=c.head_dim, embed_scale=math.sqrt(c.hidden_size), norm_weight_offset_one=True,
                     act=act, tie_embeddings=True, qkv_bias=c.attention_bias, o_bias=c.attention_bias,
                     ref_ln_star=True)


class PhiModel(DecoderModel):
    """Phi-1 / 1.5 / 2 (``models_v2/phi.rs``): attention and MLP in parallel off one LayerNorm
    (``:335-351``), partial rotary (``:399-465``), fc1 -> GELU -> fc2, biases everywhere."""

    config_class = C.PhiConfig
    scheme = KeyScheme(o=("self_attn.dense", "self_attn.o_proj"), up=("mlp.fc1",), down=("mlp.fc2",),
                       final_norm=("model.final_layernorm",))

    @classmethod
    def spec_from_config(cls, c):
        hd = c.hidden_size // c.num_attention_heads
        rd = int(hd * c.partial_rotary_factor) // 2 * 2
        act = "gelu_tanh" if c.hidden_act in ("gelu_new", "gelu_tanh") else c.hidden_act
        return _base(c, norm="layer", norm_bias=True, rotary_dim=rd, mlp="plain", act=act, qkv_bias=True,
                     o_bias=True, mlp_bias=True, lm_head_bias=True, parallel_residual=True,
                     parallel_shared_norm=True, norm_eps=getattr(c, "layer_norm_eps", c.rms_norm_eps))


class DeepSeekModel(DecoderModel):
    """DeepSeek dense (``models_v2/deepseek.rs``) = LLaMA block."""

    config_class = C.DeepSeekConfig
    scheme = LLAMA_KEYS

    @classmethod
    def spec_from_config(cls, c):
        return _base(c, qkv_bias=c.attention_bias, o_bias=c.attention_bias, ref_ln_star=True)


class MistralModel(DecoderModel):
    """Mistral-7B (``models_v2/mistral.rs``): GQA 32/8 and a 4096-token sliding window."""

    config_class = C.MistralConfig
    scheme = LLAMA_KEYS

    @classmethod
    def spec_from_config(cls, c):
        return _base(c, window=c.sliding_window)


class MixtralModel(DecoderModel):
    """Mixtral 8x7B (``models_v2/mixtral.rs``): 8 experts, top-2, softmax over the two selected logits
    (``:623-630``), SwiGLU experts ``w1 / w3 / w2`` (``:386-404, 692-701``), sliding window (``:557-570``)."""

    config_class = C.MixtralConfig
    scheme = LLAMA_KEYS

    @classmethod
    def spec_from_config(cls, c):
        return _base(c, window=c.sliding_window,
                     moe=MoESpec(num_experts=c.num_experts, top_k=c.num_experts_per_tok,
                                 intermediate_size=c.intermediate_size, normalize_topk=True, act=c.hidden_act))


class CodeLlamaModel(DecoderModel):
    """CodeLlama (``models_v2/codellama.rs``): theta 1e6 and linear position scaling (``:84``)."""

    config_class = C.CodeLlamaConfig
    scheme = LLAMA_KEYS

    @classmethod
    def spec_from_config(cls, c):
        return _base(c, rope_pos_scale=1.0 / c.rope_scaling if c.rope_scaling else 1.0)


class OlmoModel(DecoderModel):
    """OLMo (``models_v2/olmo.rs``): LLaMA block with a weight-only LayerNorm."""

    config_class = C.OlmoConfig
    scheme = LLAMA_KEYS

    @classmethod
    def spec_from_config(cls, c):
        return _base(c, norm="layer", norm_eps=c.layer_norm_eps)


class GraniteModel(DecoderModel):
    """IBM Granite (``models_v2/granite.rs``): residual branches scaled by ``residual_multiplier``
    (``:233-250``) and attention scores by ``attention_multiplier``."""

    config_class = C.GraniteConfig
    scheme = LLAMA_KEYS

    @classmethod
    def spec_from_config(cls, c):
        hd = c.hidden_size // c.num_attention_heads
        scale = None if c.attention_multiplier == 1.0 else c.attention_multiplier / math.sqrt(hd)
        return _base(c, residual_scale=c.residual_multiplier, attn_scale=scale)


class YiModel(DecoderModel):
    """Yi (``models_v2/yi.rs``): LLaMA block, GQA 32/4, theta 5e6."""

    config_class = C.YiConfig
    scheme = LLAMA_KEYS

    @classmethod
    def spec_from_config(cls, c):
        return _base(c, ref_ln_star=True)


class MiniCPMModel(DecoderModel):
    """MiniCPM (``models_v2/minicpm.rs``): embeddings x ``scale_emb`` (``:216``), residual branches x
    ``scale_depth / sqrt(L)`` (``:375``), logits / (hidden / dim_model_base); tied head."""

    config_class = C.MiniCPMConfig
    scheme = LLAMA_KEYS

    @classmethod
    def spec_from_config(cls, c):
        return _base(c, embed_scale=c.scale_emb, residual_scale=c.scale_depth / math.sqrt(c.num_hidden_layers),
                     logit_scale=1.0 / (c.hidden_size / c.dim_model_base), tie_embeddings=True,
                     qkv_bias=c.attention_bias, ref_ln_star=True)


class BaichuanModel(DecoderModel):
    """Baichuan 1/2 (``models_v2/baichuan.rs``): packed ``W_pack`` QKV, ALiBi for the 13B models
    (``:427-520``), rotary otherwise."""

    config_class = C.BaichuanConfig
    scheme = KeyScheme(qkv=("self_attn.W_pack",))

    @classmethod
    def spec_from_config(cls, c):
        return _base(c, pos="alibi" if c.use_alibi else "rope", ref_ln_star=True)


class InternLMModel(DecoderModel):
    """InternLM 1/2 (``models_v2/internlm.rs``): LLaMA block under either naming (``attention.wqkv`` packed
    per KV group + ``feed_forward.w1/w3/w2``, or LLaMA names)."""

    config_class = C.InternLMConfig
    scheme = KeyScheme(embed=("model.tok_embeddings", "model.embed_tokens"),
                       ln1=("attention_norm", "input_layernorm"), ln2=("ffn_norm", "post_attention_layernorm"),
                       qkv=("attention.wqkv",), qkv_layout="grouped",
                       q=("self_attn.q_proj", "attention.wq"), k=("self_attn.k_proj", "attention.wk"),
                       v=("self_attn.v_proj", "attention.wv"), o=("attention.wo", "self_attn.o_proj"),
                       gate=("feed_forward.w1", "mlp.gate_proj"), up=("feed_forward.w3", "mlp.up_proj"),
                       down=("feed_forward.w2", "mlp.down_proj"), lm_head=("output", "lm_head"))

    @classmethod
    def spec_from_config(cls, c):
        return _base(c, qkv_bias=c.bias, o_bias=c.bias, ref_ln_star=True)


def _gelu_name(a: str) -> str:
    return "gelu_tanh" if a in ("gelu_new", "gelu_tanh", "gelu_pytorch_tanh", "gelu_fast") else a


class GPT2Model(DecoderModel):
    """GPT-2 (``models_v2/gpt2.rs``): learned positions, LayerNorm, packed ``c_attn``, Conv1D weights stored
    ``[in, out]``, tied head.  Biases are loaded (the reference ignores them)."""

    config_class = C.GPT2Config
    scheme = KeyScheme(embed=("transformer.wte", "wte"), pos_embed=("transformer.wpe", "wpe"),
                       layer=("transformer.h.{i}.", "h.{i}."), ln1=("ln_1",), ln2=("ln_2",), qkv=("attn.c_attn",),
                       o=("attn.c_proj",), up=("mlp.c_fc",), down=("mlp.c_proj",),
                       final_norm=("transformer.ln_f", "ln_f"), transposed=True)

    @classmethod
    def spec_from_config(cls, c):
        return _base(c, norm="layer", norm_bias=True, norm_eps=c.layer_norm_eps, pos="learned", mlp="plain",
                     act=_gelu_name(c.hidden_act), qkv_bias=True, o_bias=True, mlp_bias=True, tie_embeddings=True)


class GPTJModel(DecoderModel):
    """GPT-J (``models_v2/gptj.rs``): parallel block with one ``ln_1``, interleaved partial rotary
    (``rotary_dim`` 64, ``:270``)."""

    config_class = C.GPTJConfig
    scheme = KeyScheme(embed=("transformer.wte",), layer=("transformer.h.{i}.",), ln1=("ln_1",),
                       q=("attn.q_proj",), k=("attn.k_proj",), v=("attn.v_proj",), o=("attn.out_proj",),
                       up=("mlp.fc_in",), down=("mlp.fc_out",), final_norm=("transformer.ln_f",))

    @classmethod
    def spec_from_config(cls, c):
        return _base(c, norm="layer", norm_bias=True, norm_eps=c.layer_norm_eps, rotary_dim=c.rotary_dim,
                     rope_interleaved=True, mlp="plain", act=_gelu_name(c.hidden_act), mlp_bias=True,
                     lm_head_bias=True, parallel_residual=True, parallel_shared_norm=True)


class GPTNeoXModel(DecoderModel):
    """GPT-NeoX / Pythia (``models_v2/gptneox.rs``): ``use_parallel_residual`` switch (``:184-199``), rotary on
    ``rotary_pct`` of the head (``:268``), per-head packed ``query_key_value`` (the reference splits it as
    [Q|K|V], which does not match published checkpoints)."""

    config_class = C.GPTNeoXConfig
    scheme = KeyScheme(embed=("gpt_neox.embed_in",), layer=("gpt_neox.layers.{i}.",),
                       qkv=("attention.query_key_value",), qkv_layout="per_head", o=("attention.dense",),
                       up=("mlp.dense_h_to_4h",), down=("mlp.dense_4h_to_h",),
                       final_norm=("gpt_neox.final_layer_norm",), lm_head=("embed_out",))

    @classmethod
    def spec_from_config(cls, c):
        hd = c.hidden_size // c.num_attention_heads
        return _base(c, norm="layer", norm_bias=True, norm_eps=c.layer_norm_eps,
                     rotary_dim=int(hd * c.rotary_pct) // 2 * 2, mlp="plain", act=_gelu_name(c.hidden_act),
                     qkv_bias=True, o_bias=True, mlp_bias=True, parallel_residual=c.use_parallel_residual)


class OPTModel(DecoderModel):
    """OPT (``models_v2/opt.rs``): learned positions stored with an offset of 2, ReLU MLP, pre- or post-LN
    (``do_layer_norm_before``), optional ``project_in / project_out`` when the embedding width differs."""

    config_class = C.OPTConfig
    scheme = KeyScheme(embed=("model.decoder.embed_tokens",), pos_embed=("model.decoder.embed_positions",),
                       project_in=("model.decoder.project_in",), project_out=("model.decoder.project_out",),
                       layer=("model.decoder.layers.{i}.",), ln1=("self_attn_layer_norm",), ln2=("final_layer_norm",),
                       o=("self_attn.out_proj",), up=("fc1",), down=("fc2",),
                       final_norm=("model.decoder.final_layer_norm",))

    @classmethod
    def spec_from_config(cls, c):
        proj = c.word_embed_proj_dim if c.word_embed_proj_dim != c.hidden_size else None
        return _base(c, norm="layer", norm_bias=True, norm_eps=c.layer_norm_eps, pos="learned", learned_pos_offset=2,
                     mlp="plain", act=c.hidden_act, qkv_bias=True, o_bias=True, mlp_bias=True, tie_embeddings=True,
                     post_ln=not c.do_layer_norm_before, final_norm=c.do_layer_norm_before, embed_proj_dim=proj)


class BLOOMModel(DecoderModel):
    """BLOOM (``models_v2/bloom.rs``): ALiBi (``:226-252``), LayerNorm on the embeddings, per-head packed QKV."""

    config_class = C.BLOOMConfig
    scheme = KeyScheme(embed=("transformer.word_embeddings", "word_embeddings"),
                       embed_norm=("transformer.word_embeddings_layernorm", "word_embeddings_layernorm"),
                       layer=("transformer.h.{i}.", "h.{i}."), qkv=("self_attention.query_key_value",),
                       qkv_layout="per_head", o=("self_attention.dense",), up=("mlp.dense_h_to_4h",),
                       down=("mlp.dense_4h_to_h",), final_norm=("transformer.ln_f", "ln_f"))

    @classmethod
    def spec_from_config(cls, c):
        return _base(c, norm="layer", norm_bias=True, norm_eps=c.layer_norm_eps, pos="alibi", embed_norm=True,
                     mlp="plain", act=_gelu_name(c.hidden_act), qkv_bias=True, o_bias=True, mlp_bias=True,
                     tie_embeddings=True)


class MPTModel(DecoderModel):
    """MPT (``models_v2/mpt.rs``): ALiBi (``:219``), bias-free LayerNorm / Linear, packed ``Wqkv``."""

    config_class = C.MPTConfig
    scheme = KeyScheme(embed=("transformer.wte",), layer=("transformer.blocks.{i}.",), ln1=("norm_1",),
                       ln2=("norm_2",), qkv=("attn.Wqkv",), o=("attn.out_proj",), up=("ffn.up_proj",),
                       down=("ffn.down_proj",), final_norm=("transformer.norm_f",))

    @classmethod
    def spec_from_config(cls, c):
        b = not c.no_bias
        return _base(c, norm="layer", norm_bias=b, norm_eps=c.layer_norm_eps, pos="alibi" if c.alibi else "learned",
                     mlp="plain", act=_gelu_name(c.hidden_act), qkv_bias=b, o_bias=b, mlp_bias=b, tie_embeddings=True)


class StarCoderModel(DecoderModel):
    """StarCoder (``models_v2/starcoder.rs``): GPT-2 layout with multi-query attention, one KV head packed as
    ``[H*D + 2*D]`` (``:237-262``)."""

    config_class = C.StarCoderConfig
    scheme = KeyScheme(embed=("transformer.wte",), pos_embed=("transformer.wpe",), layer=("transformer.h.{i}.",),
                       ln1=("ln_1",), ln2=("ln_2",), qkv=("attn.c_attn",), o=("attn.c_proj",), up=("mlp.c_fc",),
                       down=("mlp.c_proj",), final_norm=("transformer.ln_f",))

    @classmethod
    def spec_from_config(cls, c):
        return _base(c, num_kv_heads=1, norm="layer", norm_bias=True, norm_eps=c.layer_norm_eps, pos="learned",
                     mlp="plain", act=_gelu_name(c.hidden_act), qkv_bias=True, o_bias=True, mlp_bias=True,
                     tie_embeddings=True)


class FalconModel(DecoderModel):
    """Falcon 7B / 40B / 180B (``models_v2/falcon.rs``): parallel attention + MLP; the 7B shares one LayerNorm,
    the new decoder architecture has ``ln_attn`` / ``ln_mlp`` and QKV packed per KV group; rotary (``:440``)."""

    config_class = C.FalconConfig
    scheme = KeyScheme(embed=("transformer.word_embeddings",), layer=("transformer.h.{i}.",),
                       ln1=("ln_attn", "input_layernorm"), ln2=("ln_mlp", "post_attention_layernorm"),
                       qkv=("self_attention.query_key_value",), qkv_layout="grouped", o=("self_attention.dense",),
                       up=("mlp.dense_h_to_4h",), down=("mlp.dense_4h_to_h",), final_norm=("transformer.ln_f",))

    @classmethod
    def spec_from_config(cls, c):
        return _base(c, norm="layer", norm_bias=True, norm_eps=getattr(c, "layer_norm_epsilon", 1e-5), mlp="plain",
                     act="gelu", qkv_bias=c.bias, o_bias=c.bias, mlp_bias=c.bias, parallel_residual=c.parallel_attn,
                     parallel_shared_norm=c.parallel_attn and not c.new_decoder_architecture)


class ChatGLMModel(DecoderModel):
    """ChatGLM2/3, GLM-4 (``models_v2/chatglm.rs``): multi-query groups, packed QKV with bias (``:521-541``),
    packed SwiGLU ``dense_h_to_4h``, interleaved rotary on half of each head (the reference rotates the
    full head)."""

    config_class = C.ChatGLMConfig
    scheme = KeyScheme(embed=("transformer.embedding.word_embeddings",), layer=("transformer.encoder.layers.{i}.",),
                       qkv=("self_attention.query_key_value",), o=("self_attention.dense",),
                       gate_up=("mlp.dense_h_to_4h",), down=("mlp.dense_4h_to_h",),
                       final_norm=("transformer.encoder.final_layernorm",), lm_head=("transformer.output_layer",))

    @classmethod
    def spec_from_config(cls, c):
        hd = c.kv_channels
        return _base(c, head_dim=hd, rotary_dim=hd // 2, rope_interleaved=True, qkv_bias=c.add_qkv_bias,
                     o_bias=c.add_bias_linear, mlp_bias=False, ref_ln_star=True)


_DS_KEYS = KeyScheme(router=("mlp.gate",), expert=("mlp.experts.{e}.",), e_gate=("gate_proj",), e_up=("up_proj",),
                     e_down=("down_proj",))


class DeepSeekMoEModel(DecoderModel):
    """DeepSeek-MoE 16B (``models_v2/deepseek_moe.rs``): the first ``first_k_dense_replace`` layers are dense,
    the rest have 2 always-on shared experts plus 64 routed experts, top-6 (``:366-431``).  Expert and
    router weights are loaded (the reference never loads them, ``:249-257``)."""

    config_class = C.DeepSeekMoEConfig
    scheme = _DS_KEYS

    @classmethod
    def spec_from_config(cls, c):
        return _base(c, moe=MoESpec(num_experts=c.num_experts, top_k=c.num_experts_per_tok,
                                    intermediate_size=c.moe_intermediate_size, normalize_topk=False,
                                    num_shared_experts=c.num_shared_experts, first_k_dense=c.first_k_dense_replace,
                                    act=c.hidden_act))


class DbrxModel(DecoderModel):
    """DBRX (``models_v2/dbrx.rs``): GQA 48/8 with packed ``Wqkv``, 16 experts top-4."""

    config_class = C.DbrxConfig
    scheme = KeyScheme(embed=("transformer.wte",), layer=("transformer.blocks.{i}.",),
                       ln1=("norm_attn_norm.norm_1",), ln2=("norm_attn_norm.norm_2",),
                       qkv=("norm_attn_norm.attn.Wqkv", "self_attn.Wqkv"),
                       o=("norm_attn_norm.attn.out_proj", "self_attn.out_proj"), router=("ffn.router.layer",),
                       expert=("ffn.experts.{e}.",), e_gate=("w1",), e_up=("v1",), e_down=("w2",),
                       final_norm=("transformer.norm_f",))

    @classmethod
    def spec_from_config(cls, c):
        return _base(c, moe=MoESpec(num_experts=c.num_experts, top_k=c.num_experts_per_tok,
                                    intermediate_size=c.intermediate_size, act=c.hidden_act))


class GrokModel(DecoderModel):
    """Grok-1 (``models_v2/grok.rs``): 8 experts top-2 with GELU-gated experts."""

    config_class = C.GrokConfig
    scheme = KeyScheme(router=("moe_block.gate", "block_sparse_moe.gate"),
                       expert=("moe_block.experts.{e}.", "block_sparse_moe.experts.{e}."),
                       e_gate=("linear", "w1"), e_up=("linear_v", "w3"), e_down=("linear_1", "w2"))

    @classmethod
    def spec_from_config(cls, c):
        act = "gelu" if c.hidden_act not in ("silu", "relu") else c.hidden_act
        return _base(c, moe=MoESpec(num_experts=c.num_experts, top_k=c.num_experts_per_tok,
                                    intermediate_size=c.intermediate_size, act=act), act=act)


class ArcticModel(DecoderModel):
    """Snowflake Arctic (``models_v2/arctic.rs``): every layer adds a dense SwiGLU MLP and a 128-expert
    top-2 MoE (``moe_intermediate_size`` 2816)."""

    config_class = C.ArcticConfig
    scheme = KeyScheme(gate=("residual_mlp.w1", "mlp.gate_proj"), up=("residual_mlp.w3", "mlp.up_proj"),
                       down=("residual_mlp.w2", "mlp.down_proj"))

    @classmethod
    def spec_from_config(cls, c):
        return _base(c, moe=MoESpec(num_experts=c.num_experts, top_k=c.num_experts_per_tok,
                                    intermediate_size=c.moe_intermediate_size, dense_parallel=True, act=c.hidden_act))


DECODER_FAMILIES = {
    "llama": LlamaModel, "qwen": QwenModel, "gemma": GemmaModel, "phi": PhiModel, "deepseek": DeepSeekModel,
    "mistral": MistralModel, "mixtral": MixtralModel, "gpt2": GPT2Model, "gptj": GPTJModel, "gptneox": GPTNeoXModel,
    "opt": OPTModel, "bloom": BLOOMModel, "mpt": MPTModel, "starcoder": StarCoderModel, "codellama": CodeLlamaModel,
    "olmo": OlmoModel, "granite": GraniteModel, "yi": YiModel, "falcon": FalconModel, "baichuan": BaichuanModel,
    "internlm": InternLMModel, "chatglm": ChatGLMModel, "minicpm": MiniCPMModel, "deepseek_moe": DeepSeekMoEModel,
    "dbrx": DbrxModel, "grok": GrokModel, "arctic": ArcticModel,
}
