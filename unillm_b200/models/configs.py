"""Configuration classes of all 47 architectures.

Field names and defaults follow the reference's ``model_config!`` blocks one for one
(``crates/runtime/src/models_v2/<family>.rs``, e.g. ``llama.rs:20-38``, ``mixtral.rs:16-38``), so a
JSON config written for the reference loads here unchanged.  Every class gets ``from_dict / from_json /
from_hf_config / from_gguf_config / validate / architecture`` from :func:`unillm_b200.config.model_config`.
"""
from __future__ import annotations

from typing import Any, List, Optional

from ..config import model_config


@model_config
class ArcticConfig:
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    moe_intermediate_size: int = 2816
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    hidden_act: str = "silu"
    max_position_embeddings: int = 4096
    rms_norm_eps: float = 1e-5
    use_cache: bool = True
    pad_token_id: int = 0
    bos_token_id: int = 1
    eos_token_id: int = 2
    tie_word_embeddings: bool = False
    rope_theta: float = 10000.0
    num_experts: int = 128
    num_experts_per_tok: int = 2


@model_config
class BaichuanConfig:
    vocab_size: int = 64000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 32
    hidden_act: str = "silu"
    max_position_embeddings: int = 4096
    initializer_range: float = 0.02
    rms_norm_eps: float = 1e-6
    use_cache: bool = True
    pad_token_id: int = 0
    bos_token_id: int = 1
    eos_token_id: int = 2
    tie_word_embeddings: bool = False
    use_alibi: bool = True
    model_max_length: int = 4096
    z_loss_weight: float = 0.0


@model_config
class BertConfig:
    vocab_size: int = 30522
    hidden_size: int = 768
    intermediate_size: int = 3072
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    hidden_act: str = "gelu"
    max_position_embeddings: int = 512
    initializer_range: float = 0.02
    layer_norm_eps: float = 1e-12
    pad_token_id: int = 0
    type_vocab_size: int = 2
    rms_norm_eps: float = 1e-12


@model_config
class BLOOMConfig:
    vocab_size: int = 250880
    hidden_size: int = 2048
    intermediate_size: int = 8192
    num_hidden_layers: int = 24
    num_attention_heads: int = 16
    num_key_value_heads: int = 16
    hidden_act: str = "gelu"
    max_position_embeddings: int = 2048
    initializer_range: float = 0.02
    layer_norm_eps: float = 1e-5
    use_cache: bool = True
    pad_token_id: int = 3
    bos_token_id: int = 1
    eos_token_id: int = 2
    tie_word_embeddings: bool = True
    apply_residual_connection_post_layernorm: bool = False


@model_config
class ChatGLMConfig:
    vocab_size: int = 65024
    hidden_size: int = 4096
    intermediate_size: int = 13696
    num_hidden_layers: int = 28
    num_attention_heads: int = 32
    num_key_value_heads: int = 2
    hidden_act: str = "swiglu"
    max_position_embeddings: int = 8192
    initializer_range: float = 0.02
    rms_norm_eps: float = 1e-5
    use_cache: bool = True
    pad_token_id: int = 0
    bos_token_id: int = 1
    eos_token_id: int = 2
    tie_word_embeddings: bool = False
    rope_theta: float = 10000.0
    attention_dropout: float = 0.0
    add_bias_linear: bool = False
    add_qkv_bias: bool = True
    apply_residual_connection_post_layernorm: bool = False
    kv_channels: int = 128
    multi_query_attention: bool = True


@model_config
class CLIPConfig:
    vocab_size: int = 49408
    hidden_size: int = 512
    num_hidden_layers: int = 12
    context_length: int = 77
    transformer_width: int = 512
    transformer_heads: int = 8
    transformer_layers: int = 12
    image_resolution: int = 224
    vision_layers: int = 12
    vision_width: int = 768
    vision_heads: int = 12
    vision_patch_size: int = 32
    embed_dim: int = 512
    projection_dim: int = 512
    layer_norm_eps: float = 1e-5
    attention_dropout: float = 0.0
    initializer_range: float = 0.02


@model_config
class CodeLlamaConfig:
    vocab_size: int = 32016
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 32
    hidden_act: str = "silu"
    max_position_embeddings: int = 16384
    initializer_range: float = 0.02
    rms_norm_eps: float = 1e-5
    use_cache: bool = True
    pad_token_id: int = 0
    bos_token_id: int = 1
    eos_token_id: int = 2
    tie_word_embeddings: bool = False
    rope_theta: float = 1000000.0
    rope_scaling: float = 1.0


@model_config
class CogVLMConfig:
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 32
    vision_hidden_size: int = 1024
    vision_num_hidden_layers: int = 24
    vision_num_attention_heads: int = 16
    vision_patch_size: int = 14
    vision_image_size: int = 224
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    pad_token_id: int = 0
    bos_token_id: int = 1
    eos_token_id: int = 2


@model_config
class DbrxConfig:
    vocab_size: int = 100352
    hidden_size: int = 6144
    intermediate_size: int = 10752
    num_hidden_layers: int = 40
    num_attention_heads: int = 48
    num_key_value_heads: int = 8
    hidden_act: str = "silu"
    max_position_embeddings: int = 32768
    rms_norm_eps: float = 1e-5
    use_cache: bool = True
    pad_token_id: int = 0
    bos_token_id: int = 1
    eos_token_id: int = 2
    tie_word_embeddings: bool = False
    rope_theta: float = 500000.0
    num_experts: int = 16
    num_experts_per_tok: int = 4


@model_config
class DeepSeekConfig:
    vocab_size: int = 102400
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 30
    num_attention_heads: int = 32
    num_key_value_heads: int = 32
    hidden_act: str = "silu"
    max_position_embeddings: int = 4096
    initializer_range: float = 0.02
    rms_norm_eps: float = 1e-6
    use_cache: bool = True
    pad_token_id: int = 0
    bos_token_id: int = 100000
    eos_token_id: int = 100001
    tie_word_embeddings: bool = False
    rope_theta: float = 10000.0
    attention_bias: bool = False
    num_experts: Optional[int] = None
    num_experts_per_tok: Optional[int] = None
    expert_capacity: Optional[int] = None


@model_config
class DeepSeekMoEConfig:
    vocab_size: int = 102400
    hidden_size: int = 2048
    intermediate_size: int = 10944
    moe_intermediate_size: int = 1408
    num_hidden_layers: int = 28
    num_attention_heads: int = 16
    num_key_value_heads: int = 16
    hidden_act: str = "silu"
    max_position_embeddings: int = 4096
    rms_norm_eps: float = 1e-6
    use_cache: bool = True
    pad_token_id: int = 0
    bos_token_id: int = 1
    eos_token_id: int = 2
    tie_word_embeddings: bool = False
    rope_theta: float = 10000.0
    num_experts: int = 64
    num_experts_per_tok: int = 6
    num_shared_experts: int = 2
    first_k_dense_replace: int = 1


@model_config
class EncodecConfig:
    vocab_size: int = 1024
    hidden_size: int = 128
    num_hidden_layers: int = 4
    audio_channels: int = 1
    sample_rate: int = 24000
    num_filters: int = 32
    num_residual_layers: int = 1
    upsampling_ratios: List[int] = [8, 5, 4, 2]
    norm_type: str = "weight_norm"
    codebook_size: int = 1024
    codebook_dim: int = 128
    num_codebooks: int = 32
    use_causal_conv: bool = True
    pad_mode: str = "reflect"
    bandwidth: float = 6.0
    layer_norm_eps: float = 1e-5
    pad_token_id: int = 0
    bos_token_id: int = 1
    eos_token_id: int = 2


@model_config
class FalconConfig:
    vocab_size: int = 65024
    hidden_size: int = 4544
    intermediate_size: int = 18176
    num_hidden_layers: int = 32
    num_attention_heads: int = 71
    num_key_value_heads: int = 1
    hidden_act: str = "gelu"
    max_position_embeddings: int = 2048
    initializer_range: float = 0.02
    rms_norm_eps: float = 1e-5
    use_cache: bool = True
    pad_token_id: int = 11
    bos_token_id: int = 11
    eos_token_id: int = 11
    tie_word_embeddings: bool = False
    rope_theta: float = 10000.0
    parallel_attn: bool = True
    bias: bool = False
    new_decoder_architecture: bool = False


@model_config
class FlorenceConfig:
    vocab_size: int = 51289
    hidden_size: int = 768
    intermediate_size: int = 3072
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    vision_hidden_size: int = 768
    vision_num_hidden_layers: int = 12
    vision_num_attention_heads: int = 12
    vision_patch_size: int = 16
    vision_image_size: int = 384
    layer_norm_eps: float = 1e-6
    pad_token_id: int = 1
    bos_token_id: int = 0
    eos_token_id: int = 2


@model_config
class GemmaConfig:
    vocab_size: int = 256000
    hidden_size: int = 3072
    intermediate_size: int = 24576
    num_hidden_layers: int = 28
    num_attention_heads: int = 16
    num_key_value_heads: int = 16
    hidden_act: str = "gelu"
    max_position_embeddings: int = 8192
    initializer_range: float = 0.02
    rms_norm_eps: float = 1e-6
    use_cache: bool = True
    pad_token_id: int = 0
    bos_token_id: int = 2
    eos_token_id: int = 1
    tie_word_embeddings: bool = True
    rope_theta: float = 10000.0
    attention_bias: bool = False
    head_dim: int = 256


@model_config
class GPT2Config:
    vocab_size: int = 50257
    hidden_size: int = 768
    intermediate_size: int = 3072
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    num_key_value_heads: int = 12
    hidden_act: str = "gelu"
    max_position_embeddings: int = 1024
    initializer_range: float = 0.02
    layer_norm_eps: float = 1e-5
    use_cache: bool = True
    pad_token_id: int = 50256
    bos_token_id: int = 50256
    eos_token_id: int = 50256
    tie_word_embeddings: bool = True
    attention_dropout: float = 0.1
    residual_dropout: float = 0.1


@model_config
class GPTJConfig:
    vocab_size: int = 50400
    hidden_size: int = 4096
    intermediate_size: int = 16384
    num_hidden_layers: int = 28
    num_attention_heads: int = 16
    num_key_value_heads: int = 16
    hidden_act: str = "gelu"
    max_position_embeddings: int = 2048
    initializer_range: float = 0.02
    layer_norm_eps: float = 1e-5
    use_cache: bool = True
    pad_token_id: int = 50256
    bos_token_id: int = 50256
    eos_token_id: int = 50256
    tie_word_embeddings: bool = True
    rope_theta: float = 10000.0
    rotary_dim: int = 64


@model_config
class GPTNeoXConfig:
    vocab_size: int = 50432
    hidden_size: int = 6144
    intermediate_size: int = 24576
    num_hidden_layers: int = 44
    num_attention_heads: int = 64
    num_key_value_heads: int = 64
    hidden_act: str = "gelu"
    max_position_embeddings: int = 2048
    initializer_range: float = 0.02
    layer_norm_eps: float = 1e-5
    use_cache: bool = True
    pad_token_id: int = 0
    bos_token_id: int = 0
    eos_token_id: int = 0
    tie_word_embeddings: bool = False
    rope_theta: float = 10000.0
    rotary_pct: float = 0.25
    use_parallel_residual: bool = True


@model_config
class GraniteConfig:
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    hidden_act: str = "silu"
    max_position_embeddings: int = 8192
    initializer_range: float = 0.02
    rms_norm_eps: float = 1e-5
    use_cache: bool = True
    pad_token_id: int = 0
    bos_token_id: int = 1
    eos_token_id: int = 2
    tie_word_embeddings: bool = False
    rope_theta: float = 10000.0
    attention_multiplier: float = 1.0
    residual_multiplier: float = 1.0


@model_config
class GrokConfig:
    vocab_size: int = 131072
    hidden_size: int = 6144
    intermediate_size: int = 32768
    num_hidden_layers: int = 64
    num_attention_heads: int = 48
    num_key_value_heads: int = 8
    hidden_act: str = "gelu"
    max_position_embeddings: int = 8192
    rms_norm_eps: float = 1e-5
    use_cache: bool = True
    pad_token_id: int = 0
    bos_token_id: int = 1
    eos_token_id: int = 2
    tie_word_embeddings: bool = False
    rope_theta: float = 10000.0
    num_experts: int = 8
    num_experts_per_tok: int = 2


@model_config
class HuBERTConfig:
    vocab_size: int = 100
    hidden_size: int = 768
    intermediate_size: int = 3072
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    conv_dim: List[int] = [512, 512, 512, 512, 512, 512, 512]
    conv_kernel: List[int] = [10, 3, 3, 3, 3, 2, 2]
    conv_stride: List[int] = [5, 2, 2, 2, 2, 2, 2]
    layer_norm_eps: float = 1e-5
    hidden_dropout: float = 0.1
    pad_token_id: int = 0
    bos_token_id: int = 1
    eos_token_id: int = 2


@model_config
class IdeficsConfig:
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    vision_hidden_size: int = 1024
    vision_num_hidden_layers: int = 24
    vision_num_attention_heads: int = 16
    vision_patch_size: int = 14
    vision_image_size: int = 224
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    cross_attention_frequency: int = 4
    pad_token_id: int = 0
    bos_token_id: int = 1
    eos_token_id: int = 2


@model_config
class InternLMConfig:
    vocab_size: int = 103168
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    hidden_act: str = "silu"
    max_position_embeddings: int = 2048
    initializer_range: float = 0.02
    rms_norm_eps: float = 1e-6
    use_cache: bool = True
    pad_token_id: int = 0
    bos_token_id: int = 1
    eos_token_id: int = 2
    tie_word_embeddings: bool = False
    rope_theta: float = 10000.0
    attention_dropout: float = 0.0
    bias: bool = False


@model_config
class InternVLConfig:
    vocab_size: int = 92544
    hidden_size: int = 4096
    intermediate_size: int = 14336
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    max_position_embeddings: int = 8192
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    vision_hidden_size: int = 3200
    vision_intermediate_size: int = 12800
    vision_num_hidden_layers: int = 48
    vision_num_attention_heads: int = 25
    vision_patch_size: int = 14
    vision_image_size: int = 448
    pad_token_id: int = 0
    bos_token_id: int = 1
    eos_token_id: int = 2


@model_config
class JambaConfig:
    vocab_size: int = 65536
    hidden_size: int = 4096
    intermediate_size: int = 14336
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    hidden_act: str = "silu"
    max_position_embeddings: int = 262144
    initializer_range: float = 0.02
    rms_norm_eps: float = 1e-6
    use_cache: bool = True
    pad_token_id: int = 0
    bos_token_id: int = 1
    eos_token_id: int = 2
    tie_word_embeddings: bool = False
    rope_theta: float = 10000.0
    attention_dropout: float = 0.0
    d_state: int = 16
    d_conv: int = 4
    expand: int = 2
    num_experts: int = 16
    num_experts_per_tok: int = 2
    attn_layer_period: int = 8
    attn_layer_offset: int = 4
    use_mamba_preprocessing: bool = True
    mamba_d_inner: int = 0
    mamba_dt_rank: int = 0


@model_config
class LlamaConfig:
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 32
    hidden_act: str = "silu"
    max_position_embeddings: int = 2048
    initializer_range: float = 0.02
    rms_norm_eps: float = 1e-6
    use_cache: bool = True
    pad_token_id: int = 0
    bos_token_id: int = 1
    eos_token_id: int = 2
    tie_word_embeddings: bool = False
    rope_theta: float = 10000.0
    attention_bias: bool = False


@model_config
class LLaVAConfig:
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 32
    hidden_act: str = "silu"
    max_position_embeddings: int = 4096
    initializer_range: float = 0.02
    rms_norm_eps: float = 1e-5
    use_cache: bool = True
    pad_token_id: int = 0
    bos_token_id: int = 1
    eos_token_id: int = 2
    tie_word_embeddings: bool = False
    rope_theta: float = 10000.0
    attention_bias: bool = False
    attention_dropout: float = 0.0
    vision_hidden_size: int = 1024
    vision_intermediate_size: int = 4096
    vision_num_hidden_layers: int = 24
    vision_num_attention_heads: int = 16
    vision_num_channels: int = 3
    vision_patch_size: int = 14
    vision_image_size: int = 336
    vision_layer_norm_eps: float = 1e-5
    mm_projector_type: str = "mlp2x_gelu"
    mm_hidden_size: int = 1024
    mm_vision_select_layer: int = -2
    mm_vision_select_feature: str = "patch"
    image_token_len: int = 576
    im_patch_token: int = 32000
    im_start_token: int = 32001
    im_end_token: int = 32002


@model_config
class MambaConfig:
    vocab_size: int = 50280
    hidden_size: int = 768
    num_hidden_layers: int = 24
    d_state: int = 16
    d_conv: int = 4
    expand: int = 2
    dt_rank: int = 0
    d_inner: int = 0
    dt_scale: float = 1.0
    dt_min: float = 0.001
    dt_max: float = 0.1
    dt_init_floor: float = 1e-4
    conv_bias: bool = True
    bias: bool = False
    layer_norm_epsilon: float = 1e-5
    rms_norm: bool = True
    initializer_range: float = 0.02
    tie_embeddings: bool = True
    pad_token_id: int = 0
    bos_token_id: int = 0
    eos_token_id: int = 0


@model_config
class MiniCPMConfig:
    vocab_size: int = 122753
    hidden_size: int = 2304
    intermediate_size: int = 5760
    num_hidden_layers: int = 40
    num_attention_heads: int = 36
    num_key_value_heads: int = 36
    hidden_act: str = "silu"
    max_position_embeddings: int = 4096
    initializer_range: float = 0.02
    rms_norm_eps: float = 1e-5
    use_cache: bool = True
    pad_token_id: int = 0
    bos_token_id: int = 1
    eos_token_id: int = 2
    tie_word_embeddings: bool = True
    rope_theta: float = 10000.0
    rope_scaling: Optional[str] = None
    attention_bias: bool = False
    attention_dropout: float = 0.0
    scale_emb: float = 12.0
    scale_depth: float = 1.4
    dim_model_base: int = 256
    scale_width: float = 2.0


@model_config
class MistralConfig:
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 14336
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    hidden_act: str = "silu"
    max_position_embeddings: int = 32768
    initializer_range: float = 0.02
    rms_norm_eps: float = 1e-5
    use_cache: bool = True
    pad_token_id: int = 0
    bos_token_id: int = 1
    eos_token_id: int = 2
    tie_word_embeddings: bool = False
    rope_theta: float = 10000.0
    sliding_window: int = 4096
    attention_dropout: float = 0.0


@model_config
class MixtralConfig:
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 14336
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    hidden_act: str = "silu"
    max_position_embeddings: int = 32768
    initializer_range: float = 0.02
    rms_norm_eps: float = 1e-5
    use_cache: bool = True
    pad_token_id: int = 0
    bos_token_id: int = 1
    eos_token_id: int = 2
    tie_word_embeddings: bool = False
    rope_theta: float = 1000000.0
    sliding_window: int = 4096
    attention_dropout: float = 0.0
    num_experts: int = 8
    num_experts_per_tok: int = 2
    router_aux_loss_coef: float = 0.02


@model_config
class MPTConfig:
    vocab_size: int = 50432
    hidden_size: int = 4096
    intermediate_size: int = 16384
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 32
    hidden_act: str = "gelu"
    max_position_embeddings: int = 2048
    initializer_range: float = 0.02
    layer_norm_eps: float = 1e-5
    use_cache: bool = True
    pad_token_id: int = 0
    bos_token_id: int = 0
    eos_token_id: int = 0
    tie_word_embeddings: bool = True
    alibi: bool = True
    no_bias: bool = True


@model_config
class MusicGenConfig:
    vocab_size: int = 2048
    hidden_size: int = 1024
    intermediate_size: int = 4096
    num_hidden_layers: int = 24
    num_attention_heads: int = 16
    num_key_value_heads: int = 16
    max_position_embeddings: int = 2048
    num_codebooks: int = 4
    audio_channels: int = 1
    sampling_rate: int = 32000
    frame_rate: int = 50
    layer_norm_eps: float = 1e-5
    hidden_dropout: float = 0.0
    pad_token_id: int = 2048
    bos_token_id: int = 2048
    eos_token_id: int = 2048


@model_config
class OlmoConfig:
    vocab_size: int = 50304
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 32
    hidden_act: str = "silu"
    max_position_embeddings: int = 2048
    initializer_range: float = 0.02
    layer_norm_eps: float = 1e-5
    use_cache: bool = True
    pad_token_id: int = 1
    bos_token_id: int = 0
    eos_token_id: int = 0
    tie_word_embeddings: bool = False
    rope_theta: float = 10000.0


@model_config
class OPTConfig:
    vocab_size: int = 50272
    hidden_size: int = 768
    intermediate_size: int = 3072
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    num_key_value_heads: int = 12
    hidden_act: str = "relu"
    max_position_embeddings: int = 2048
    initializer_range: float = 0.02
    layer_norm_eps: float = 1e-5
    use_cache: bool = True
    pad_token_id: int = 1
    bos_token_id: int = 2
    eos_token_id: int = 2
    tie_word_embeddings: bool = False
    word_embed_proj_dim: int = 768
    do_layer_norm_before: bool = True


@model_config
class PhiConfig:
    vocab_size: int = 51200
    hidden_size: int = 2560
    intermediate_size: int = 10240
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 32
    hidden_act: str = "gelu_new"
    max_position_embeddings: int = 2048
    initializer_range: float = 0.02
    rms_norm_eps: float = 1e-5
    use_cache: bool = True
    pad_token_id: int = 0
    bos_token_id: int = 1
    eos_token_id: int = 2
    tie_word_embeddings: bool = False
    rope_theta: float = 10000.0
    attention_dropout: float = 0.0
    partial_rotary_factor: float = 0.5


@model_config
class Phi3VisionConfig:
    vocab_size: int = 32064
    hidden_size: int = 3072
    intermediate_size: int = 8192
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 32
    max_position_embeddings: int = 131072
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    vision_hidden_size: int = 1024
    vision_intermediate_size: int = 4096
    vision_num_hidden_layers: int = 24
    vision_num_attention_heads: int = 16
    vision_patch_size: int = 14
    vision_image_size: int = 336
    pad_token_id: int = 32000
    bos_token_id: int = 1
    eos_token_id: int = 32000
    image_token_id: int = 32044


@model_config
class QwenConfig:
    vocab_size: int = 151936
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 32
    hidden_act: str = "silu"
    max_position_embeddings: int = 32768
    initializer_range: float = 0.02
    rms_norm_eps: float = 1e-6
    use_cache: bool = True
    pad_token_id: int = 151643
    bos_token_id: int = 151643
    eos_token_id: int = 151643
    tie_word_embeddings: bool = False
    rope_theta: float = 1000000.0
    use_sliding_window: bool = False
    sliding_window: int = 4096
    attention_dropout: float = 0.0


@model_config
class Qwen2VLConfig:
    vocab_size: int = 151936
    hidden_size: int = 3584
    intermediate_size: int = 18944
    num_hidden_layers: int = 28
    num_attention_heads: int = 28
    num_key_value_heads: int = 4
    max_position_embeddings: int = 32768
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1000000.0
    tie_word_embeddings: bool = False
    vision_hidden_size: int = 1280
    vision_intermediate_size: int = 5120
    vision_num_hidden_layers: int = 32
    vision_num_attention_heads: int = 16
    vision_patch_size: int = 14
    vision_image_size: int = 448
    vision_temporal_patch_size: int = 2
    projector_hidden_size: int = 0
    pad_token_id: int = 151643
    bos_token_id: int = 151643
    eos_token_id: int = 151645
    image_token_id: int = 151655
    video_token_id: int = 151656


@model_config
class RecurrentGemmaConfig:
    vocab_size: int = 256000
    hidden_size: int = 2560
    num_hidden_layers: int = 26
    intermediate_size: int = 7680
    num_attention_heads: int = 10
    num_key_value_heads: int = 1
    head_dim: int = 256
    max_position_embeddings: int = 8192
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    attention_window_size: int = 2048
    lru_width: int = 0
    recurrent_block_ratio: int = 2
    tie_word_embeddings: bool = True
    pad_token_id: int = 0
    bos_token_id: int = 2
    eos_token_id: int = 1


@model_config
class Rwkv4Config:
    vocab_size: int = 50277
    hidden_size: int = 768
    num_hidden_layers: int = 12
    intermediate_size: int = 0
    layer_norm_epsilon: float = 1e-5
    rescale_every: int = 6
    tie_word_embeddings: bool = False
    pad_token_id: int = 0
    bos_token_id: int = 0
    eos_token_id: int = 0


@model_config
class Rwkv6Config:
    vocab_size: int = 65536
    hidden_size: int = 2048
    num_hidden_layers: int = 24
    intermediate_size: int = 0
    head_size: int = 64
    num_heads: int = 0
    layer_norm_epsilon: float = 1e-5
    rescale_every: int = 6
    tie_word_embeddings: bool = False
    pad_token_id: int = 0
    bos_token_id: int = 1
    eos_token_id: int = 2


@model_config
class StarCoderConfig:
    vocab_size: int = 49152
    hidden_size: int = 6144
    intermediate_size: int = 24576
    num_hidden_layers: int = 40
    num_attention_heads: int = 48
    num_key_value_heads: int = 1
    hidden_act: str = "gelu_new"
    max_position_embeddings: int = 8192
    initializer_range: float = 0.02
    layer_norm_eps: float = 1e-5
    use_cache: bool = True
    pad_token_id: int = 49152
    bos_token_id: int = 49152
    eos_token_id: int = 0
    tie_word_embeddings: bool = True


@model_config
class T5Config:
    vocab_size: int = 32128
    d_model: int = 512
    d_kv: int = 64
    d_ff: int = 2048
    num_layers: int = 6
    num_decoder_layers: int = 6
    num_heads: int = 8
    relative_attention_num_buckets: int = 32
    relative_attention_max_distance: int = 128
    dropout_rate: float = 0.1
    layer_norm_epsilon: float = 1e-6
    initializer_factor: float = 1.0
    feed_forward_proj: str = "relu"
    is_encoder_decoder: bool = True
    use_cache: bool = True
    pad_token_id: int = 0
    eos_token_id: int = 1
    decoder_start_token_id: int = 0
    tie_word_embeddings: bool = True
    is_gated_act: bool = False
    hidden_size: int = 512
    num_hidden_layers: int = 6


@model_config
class Wav2Vec2Config:
    vocab_size: int = 32
    hidden_size: int = 768
    intermediate_size: int = 3072
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    conv_dim: List[int] = [512, 512, 512, 512, 512, 512, 512]
    conv_kernel: List[int] = [10, 3, 3, 3, 3, 2, 2]
    conv_stride: List[int] = [5, 2, 2, 2, 2, 2, 2]
    feat_extract_norm: str = "group"
    layer_norm_eps: float = 1e-5
    hidden_dropout: float = 0.1
    attention_dropout: float = 0.1
    final_dropout: float = 0.1
    pad_token_id: int = 0
    bos_token_id: int = 1
    eos_token_id: int = 2


@model_config
class WhisperConfig:
    vocab_size: int = 51865
    d_model: int = 512
    encoder_layers: int = 6
    decoder_layers: int = 6
    encoder_attention_heads: int = 8
    decoder_attention_heads: int = 8
    encoder_ffn_dim: int = 2048
    decoder_ffn_dim: int = 2048
    dropout: float = 0.0
    attention_dropout: float = 0.0
    activation_dropout: float = 0.0
    activation_function: str = "gelu"
    init_std: float = 0.02
    layer_norm_eps: float = 1e-5
    scale_embedding: bool = False
    use_cache: bool = True
    is_encoder_decoder: bool = True
    pad_token_id: int = 50257
    bos_token_id: int = 50258
    eos_token_id: int = 50257
    decoder_start_token_id: int = 50258
    max_source_positions: int = 1500
    max_target_positions: int = 448
    num_mel_bins: int = 80
    num_hidden_layers: int = 6
    hidden_size: int = 512


@model_config
class YiConfig:
    vocab_size: int = 64000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 4
    hidden_act: str = "silu"
    max_position_embeddings: int = 4096
    initializer_range: float = 0.02
    rms_norm_eps: float = 1e-5
    use_cache: bool = True
    pad_token_id: int = 0
    bos_token_id: int = 1
    eos_token_id: int = 2
    tie_word_embeddings: bool = False
    rope_theta: float = 5000000.0
    attention_dropout: float = 0.0


