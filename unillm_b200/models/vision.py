"""Vision and vision-language families: CLIP, LLaVA, Qwen2-VL, Phi-3-Vision, InternVL, CogVLM, Idefics, Florence.

CLIP (``models_v2/clip.rs``): causal text transformer + ViT (patch embedding, class token, learned positions, pre/post
LayerNorm), quick-GELU MLPs, projections into a shared space, ``logit_scale``; ``encode_text`` / ``encode_image`` /
``compute_similarity`` (``:355-373``).  The patch embedding uses stride = patch and no padding (the reference passes
padding = patch size, ``:658-664``) and the text feature is pooled at the highest token id (EOS), as published, not at
the last position (``:403-421``).

The vision-language models share one composition: vision tower -> projector -> language model, image features
spliced into the token embeddings at the image-token positions (``llava.rs:1356-1405``, ``qwen2_vl.rs:333``).  LLaVA
and Qwen2-VL implement that in the reference; Phi-3-Vision, InternVL, CogVLM, Idefics and Florence are text-only
skeletons there (``phi3_vision.rs:131-146`` etc.) and run the same multimodal path here.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config import GenerationConfig
from ..model_core import Model, ModelInputs, ModelOutputs, ModelWeights
from ..tensor_core import ops_fn
from ..types import InvalidInput
from . import configs as C
from .decoder import DecoderModel
from .families import LLAMA_KEYS, _base
from .spec import KeyScheme
from .simple import ParamModel, _f, mha


# ------------------------------------------------------------------------------------------------
# ViT tower over a parameter dict
# ------------------------------------------------------------------------------------------------
class VisionTower:
    """CLIP-style ViT whose parameters live in the owner's ``p`` under ``prefix``."""

    def __init__(self, prefix: str, hidden: int, layers: int, heads: int, inter: int, patch: int, image: int,
                 channels: int = 3, eps: float = 1e-5, act: str = "quick_gelu", temporal: int = 1, cls_token: bool = True):
        self.pre, self.H, self.L, self.nh, self.I = prefix, hidden, layers, heads, inter
        self.patch, self.image, self.ch, self.eps, self.act, self.temporal, self.cls = patch, image, channels, eps, act, temporal, cls_token
        self.num_patches = (image // patch) ** 2

    def shapes(self) -> Dict[str, tuple]:
        P, H = self.pre, self.H
        s = {P + "embeddings.patch_embedding.weight": (H, self.ch * self.temporal * self.patch * self.patch),
             P + "embeddings.position_embedding.weight": (self.num_patches + (1 if self.cls else 0), H),
             P + "pre_layrnorm.weight": (H,), P + "pre_layrnorm.bias": (H,),
             P + "post_layernorm.weight": (H,), P + "post_layernorm.bias": (H,)}
        if self.cls:
            s[P + "embeddings.class_embedding"] = (H,)
        for i in range(self.L):
            L = f"{P}encoder.layers.{i}."
            for n in ("q_proj", "k_proj", "v_proj", "out_proj"):
                s[L + f"self_attn.{n}.weight"], s[L + f"self_attn.{n}.bias"] = (H, H), (H,)
            for n in ("layer_norm1", "layer_norm2"):
                s[L + n + ".weight"], s[L + n + ".bias"] = (H,), (H,)
            s[L + "mlp.fc1.weight"], s[L + "mlp.fc1.bias"] = (self.I, H), (self.I,)
            s[L + "mlp.fc2.weight"], s[L + "mlp.fc2.bias"] = (H, self.I), (H,)
        return s

    def patchify(self, pixels: torch.Tensor) -> torch.Tensor:
        """[B, C, H, W] (or [B, C, T, H, W] with temporal patches) -> [B, patches, C*T*p*p]."""
        p = self.patch
        if pixels.dim() == 5:
            B, Cc, T, Hh, Ww = pixels.shape
            x = pixels.reshape(B, Cc, T // self.temporal, self.temporal, Hh // p, p, Ww // p, p)
            return x.permute(0, 2, 4, 6, 1, 3, 5, 7).reshape(B, -1, Cc * self.temporal * p * p)
        if self.temporal > 1:
            pixels = pixels[:, :, None].expand(-1, -1, self.temporal, -1, -1)
            return self.patchify(pixels)
        B, Cc, Hh, Ww = pixels.shape
        if Hh % p or Ww % p:
            raise InvalidInput(f"image size {Hh}x{Ww} is not a multiple of the patch size {p}")
        x = pixels.reshape(B, Cc, Hh // p, p, Ww // p, p)
        return x.permute(0, 2, 4, 1, 3, 5).reshape(B, -1, Cc * p * p)

    def forward(self, p: Dict[str, torch.Tensor], pixels: torch.Tensor, select_layer: Optional[int] = None,
                apply_post_ln: bool = True) -> torch.Tensor:
        """Hidden states after ``select_layer`` (negative counts from the end, -1 = last); all tokens incl. class."""
        P = self.pre
        w = p[P + "embeddings.patch_embedding.weight"]
        x = ops_fn.linear(self.patchify(pixels.to(w.dtype)), w.reshape(self.H, -1))
        if self.cls:
            cls = p[P + "embeddings.class_embedding"].to(x.dtype)[None, None].expand(x.shape[0], 1, -1)
            x = torch.cat([cls, x], 1)
        pos = p[P + "embeddings.position_embedding.weight"]
        if x.shape[1] > pos.shape[0]:
            raise InvalidInput(f"{x.shape[1]} vision tokens exceed the position table ({pos.shape[0]})")
        x = x + pos[:x.shape[1]][None].to(x.dtype)
        x = ops_fn.layer_norm(x, p[P + "pre_layrnorm.weight"], p[P + "pre_layrnorm.bias"], self.eps)
        n_run = self.L if select_layer is None else (self.L + 1 + select_layer if select_layer < 0 else select_layer)
        for i in range(n_run):
            L = f"{P}encoder.layers.{i}."
            h = ops_fn.layer_norm(x, p[L + "layer_norm1.weight"], p[L + "layer_norm1.bias"], self.eps)
            A = L + "self_attn."
            x = x + mha(h, h, p[A + "q_proj.weight"], p[A + "q_proj.bias"], p[A + "k_proj.weight"], p[A + "k_proj.bias"],
                        p[A + "v_proj.weight"], p[A + "v_proj.bias"], p[A + "out_proj.weight"], p[A + "out_proj.bias"], self.nh)
            h = ops_fn.layer_norm(x, p[L + "layer_norm2.weight"], p[L + "layer_norm2.bias"], self.eps)
            h = ops_fn.linear(h, p[L + "mlp.fc1.weight"], p[L + "mlp.fc1.bias"], act=self.act)
            x = x + ops_fn.linear(h, p[L + "mlp.fc2.weight"], p[L + "mlp.fc2.bias"])
        if apply_post_ln and n_run == self.L:
            x = ops_fn.layer_norm(x, p[P + "post_layernorm.weight"], p[P + "post_layernorm.bias"], self.eps)
        return x


# ------------------------------------------------------------------------------------------------
# CLIP
# ------------------------------------------------------------------------------------------------
class ClipModel(ParamModel):
    config_class = C.CLIPConfig

    def __init__(self, config):
        super().__init__(config)
        c = config
        self.vit = VisionTower("vision_model.", c.vision_width, c.vision_layers, c.vision_heads, 4 * c.vision_width,
                               c.vision_patch_size, c.image_resolution, eps=c.layer_norm_eps)

    def param_shapes(self) -> Dict[str, tuple]:
        c = self._config
        W = c.transformer_width
        s = {"text_model.embeddings.token_embedding.weight": (c.vocab_size, W),
             "text_model.embeddings.position_embedding.weight": (c.context_length, W)}
        for i in range(c.transformer_layers):
            L = f"text_model.encoder.layers.{i}."
            for n in ("q_proj", "k_proj", "v_proj", "out_proj"):
                s[L + f"self_attn.{n}.weight"], s[L + f"self_attn.{n}.bias"] = (W, W), (W,)
            for n in ("layer_norm1", "layer_norm2"):
                s[L + n + ".weight"], s[L + n + ".bias"] = (W,), (W,)
            s[L + "mlp.fc1.weight"], s[L + "mlp.fc1.bias"] = (4 * W, W), (4 * W,)
            s[L + "mlp.fc2.weight"], s[L + "mlp.fc2.bias"] = (W, 4 * W), (W,)
        s["text_model.final_layer_norm.weight"], s["text_model.final_layer_norm.bias"] = (W,), (W,)
        s.update(self.vit.shapes())
        s["text_projection.weight"] = (c.projection_dim, W)
        s["visual_projection.weight"] = (c.projection_dim, c.vision_width)
        s["logit_scale"] = ()
        return s

    def aliases(self, name):
        if name.endswith("_projection.weight"):
            return (name, name[:-len(".weight")])
        if "pre_layrnorm" in name:
            return (name, name.replace("pre_layrnorm", "pre_layernorm"))
        return (name,)

    def special_init(self, name, shape, g):
        if name == "logit_scale":
            return torch.tensor(2.6592)
        return None

    def encode_text(self, ids: torch.Tensor) -> torch.Tensor:
        c, p = self._config, self.p
        B, T = ids.shape
        if T > c.context_length:
            raise InvalidInput(f"text length {T} exceeds context_length {c.context_length}")
        x = ops_fn.embedding(ids, p["text_model.embeddings.token_embedding.weight"]) + \
            p["text_model.embeddings.position_embedding.weight"][:T][None]
        for i in range(c.transformer_layers):
            L = f"text_model.encoder.layers.{i}."
            A = L + "self_attn."
            h = self.ln(x, L + "layer_norm1", c.layer_norm_eps)
            x = x + mha(h, h, p[A + "q_proj.weight"], p[A + "q_proj.bias"], p[A + "k_proj.weight"], p[A + "k_proj.bias"],
                        p[A + "v_proj.weight"], p[A + "v_proj.bias"], p[A + "out_proj.weight"], p[A + "out_proj.bias"],
                        c.transformer_heads, causal=True)
            h = self.ln(x, L + "layer_norm2", c.layer_norm_eps)
            x = x + self.lin(self.lin(h, L + "mlp.fc1", act="quick_gelu"), L + "mlp.fc2")
        x = self.ln(x, "text_model.final_layer_norm", c.layer_norm_eps)
        pooled = x[torch.arange(B, device=x.device), ids.argmax(-1)]
        return ops_fn.normalize(ops_fn.linear(pooled, p["text_projection.weight"]))

    def encode_image(self, pixels: torch.Tensor) -> torch.Tensor:
        x = self.vit.forward(self.p, pixels)
        return ops_fn.normalize(ops_fn.linear(x[:, 0], self.p["visual_projection.weight"]))

    def compute_similarity(self, text_embeds: torch.Tensor, image_embeds: torch.Tensor) -> torch.Tensor:
        """``logits_per_text`` [num_texts, num_images]."""
        return torch.exp(_f(self.p["logit_scale"])) * (_f(text_embeds) @ _f(image_embeds).t())

    def forward(self, inputs: ModelInputs) -> ModelOutputs:
        if inputs.kind == "text" or inputs.pixel_values is None:
            return ModelOutputs.embeddings(self.encode_text(inputs.input_ids))
        if inputs.input_ids is None:
            return ModelOutputs.embeddings(self.encode_image(inputs.pixel_values))
        t, im = self.encode_text(inputs.input_ids), self.encode_image(inputs.pixel_values)
        lpt = self.compute_similarity(t, im)
        return ModelOutputs.clip(lpt, lpt.t(), t, im)


# ------------------------------------------------------------------------------------------------
# Vision-language composition
# ------------------------------------------------------------------------------------------------
class _LM(DecoderModel):
    """Language model of a VLM: a LLaMA-shaped decoder stack described by the VLM's own config."""

    scheme = LLAMA_KEYS
    spec_extra: dict = {}

    @classmethod
    def spec_from_config(cls, c):
        return _base(c, **cls.spec_extra)


def _lm_class(name: str, scheme: KeyScheme = LLAMA_KEYS, **extra):
    return type(name, (_LM,), {"spec_extra": extra, "scheme": scheme})


class VisionLanguageModel(Model):
    """vision tower -> projector -> language model.  Parameters: ``<vision_prefix>*``, ``<projector_prefix>*`` and the
    language model's tensors under ``<lm_prefix>``."""

    lm_cls = _lm_class("LlamaLM")
    lm_prefix = "language_model."
    vision_prefix = "vision_tower.vision_model."
    projector_prefix = "mm_projector."
    projector = "mlp2x_gelu"           # "linear" | "mlp2x_gelu" | "merger"
    select_layer = -2
    drop_cls = True
    strict_vision = False              # the reference's skeleton families ship no vision weights

    def __init__(self, config):
        super().__init__(config)
        c = config
        self.lm = self.lm_cls(c)
        self.vit = self.make_tower(c)
        self.p: Dict[str, torch.Tensor] = {}

    def make_tower(self, c) -> VisionTower:
        return VisionTower(self.vision_prefix, c.vision_hidden_size, c.vision_num_hidden_layers, c.vision_num_attention_heads,
                           getattr(c, "vision_intermediate_size", 4 * c.vision_hidden_size), c.vision_patch_size,
                           c.vision_image_size, eps=getattr(c, "vision_layer_norm_eps", 1e-5))

    def image_token_id(self) -> int:
        c = self._config
        return getattr(c, "image_token_id", getattr(c, "im_patch_token", c.vocab_size - 1))

    # -- parameters --
    def projector_shapes(self) -> Dict[str, tuple]:
        c, P = self._config, self.projector_prefix
        Hv, H = c.vision_hidden_size, c.hidden_size
        if self.projector == "linear":
            return {P + "0.weight": (H, Hv), P + "0.bias": (H,)}
        if self.projector == "merger":
            Hm = 4 * Hv
            return {P + "ln_q.weight": (Hv,), P + "ln_q.bias": (Hv,), P + "mlp.0.weight": (Hm, Hm), P + "mlp.0.bias": (Hm,),
                    P + "mlp.2.weight": (H, Hm), P + "mlp.2.bias": (H,)}
        return {P + "0.weight": (H, Hv), P + "0.bias": (H,), P + "2.weight": (H, H), P + "2.bias": (H,)}

    def own_shapes(self) -> Dict[str, tuple]:
        s = self.vit.shapes()
        s.update(self.projector_shapes())
        return s

    def _init_params(self, init="zeros", seed=0, dtype=torch.float32, device=torch.device("cpu")):
        self.lm._init_params(init=init, seed=seed, dtype=dtype, device=device)
        g = torch.Generator().manual_seed(seed + 1)
        self.p = {}
        for name, shape in self.own_shapes().items():
            if init == "zeros":
                t = torch.zeros(shape)
            elif ParamModel.is_norm_scale(name, shape):
                t = torch.ones(shape)
            elif name.endswith(".bias"):
                t = torch.zeros(shape)
            else:
                t = torch.randn(shape, generator=g) * 0.02
            self.p[name] = t.to(dtype).to(device)
        self.device, self.dtype = device, dtype

    def _load(self, weights: ModelWeights, dtype=None, device=None):
        dtype = dtype or torch.float32
        dev = torch.device(device) if device is not None else torch.device("cpu")
        sub = ModelWeights({k[len(self.lm_prefix):]: v for k, v in weights.tensors.items() if k.startswith(self.lm_prefix)})
        self.lm._load(sub if len(sub) else weights, dtype=dtype, device=dev)
        self.p = {}
        for name, shape in self.own_shapes().items():
            t = weights.get(name)
            if t is None:
                if self.strict_vision:
                    from ..types import LoadingError

                    raise LoadingError(f"{type(self).__name__}: missing tensor {name}")
                t = torch.ones(shape) if ParamModel.is_norm_scale(name, shape) else torch.zeros(shape)
            self.p[name] = t.reshape(shape).to(dtype).to(dev)
        self.device, self.dtype = dev, dtype

    def export_hf(self) -> ModelWeights:
        out = {self.lm_prefix + k: v for k, v in self.lm.export_hf().tensors.items()}
        out.update({k: v.detach().clone() for k, v in self.p.items()})
        return ModelWeights(out)

    def parameters(self):
        d = {self.lm_prefix + k: v for k, v in self.lm.parameters().items()}
        d.update(self.p)
        return d

    def _move(self, dev, dtype):
        self.lm.to_device(dev, dtype)
        self.p = {k: v.to(device=dev, dtype=dtype or v.dtype) for k, v in self.p.items()}

    # -- forward --
    def encode_images(self, pixels: torch.Tensor) -> torch.Tensor:
        """[B, C, H, W] -> image features in the language model's hidden size, [B, tokens, hidden]."""
        x = self.vit.forward(self.p, pixels, select_layer=self.select_layer, apply_post_ln=False)
        if self.drop_cls and self.vit.cls:
            x = x[:, 1:]
        P, p = self.projector_prefix, self.p
        if self.projector == "linear":
            return ops_fn.linear(x, p[P + "0.weight"], p[P + "0.bias"])
        if self.projector == "merger":
            x = ops_fn.layer_norm(x, p[P + "ln_q.weight"], p[P + "ln_q.bias"], 1e-6)
            B, N, Hv = x.shape
            side = int(N ** 0.5)
            x = x.reshape(B, side // 2, 2, side // 2, 2, Hv).permute(0, 1, 3, 2, 4, 5).reshape(B, N // 4, 4 * Hv)
            x = ops_fn.linear(x, p[P + "mlp.0.weight"], p[P + "mlp.0.bias"], act="gelu")
            return ops_fn.linear(x, p[P + "mlp.2.weight"], p[P + "mlp.2.bias"])
        x = ops_fn.linear(x, p[P + "0.weight"], p[P + "0.bias"], act="gelu")
        return ops_fn.linear(x, p[P + "2.weight"], p[P + "2.bias"])

    def merge_multimodal_inputs(self, input_ids: torch.Tensor, image_features: torch.Tensor) -> torch.Tensor:
        """Token embeddings with image features spliced in.  A run of image tokens is overwritten one feature per
        token; a single image token is expanded to all features of the image; with no image token the features are
        put in front of the text."""
        lm = self.lm
        tok = self.image_token_id()
        safe = input_ids.clamp_max(lm.spec.vocab_size - 1)
        emb = ops_fn.embedding(safe, lm.p["embed"])
        if lm.spec.embed_scale != 1.0:
            emb = (_f(emb) * lm.spec.embed_scale).to(emb.dtype)
        rows = []
        for b in range(input_ids.shape[0]):
            feats = image_features[min(b, image_features.shape[0] - 1)].to(emb.dtype)
            pos = (input_ids[b] == tok).nonzero().flatten()
            e = emb[b]
            if pos.numel() == 0:
                rows.append(torch.cat([feats, e], 0))
            elif pos.numel() == 1:
                i = int(pos[0])
                rows.append(torch.cat([e[:i], feats, e[i + 1:]], 0))
            else:
                n = min(pos.numel(), feats.shape[0])
                e = e.clone()
                e[pos[:n]] = feats[:n]
                rows.append(e)
        L = max(r.shape[0] for r in rows)
        if any(r.shape[0] != L for r in rows):
            raise InvalidInput("sequences of a batch expand to different lengths; pad the image tokens explicitly")
        return torch.stack(rows, 0)

    def forward(self, inputs: ModelInputs) -> ModelOutputs:
        if inputs.input_ids is None:
            raise InvalidInput(f"{type(self).__name__} needs input_ids")
        if inputs.pixel_values is None:
            x = self.lm.hidden_states(inputs.input_ids)
        else:
            x = self.lm.hidden_states(None, inputs_embeds=self.merge_multimodal_inputs(inputs.input_ids, self.encode_images(inputs.pixel_values)))
        return ModelOutputs.from_logits(self.lm.lm_logits(x), hidden_states=x)

    def new_cache(self, max_seq_len: Optional[int] = None):
        return self.lm.new_cache(max_seq_len)

    def forward_with_cache(self, input_ids: torch.Tensor, cache=None, pixel_values: Optional[torch.Tensor] = None) -> torch.Tensor:
        if input_ids.dim() == 1:
            input_ids = input_ids[None]
        if pixel_values is None:
            return self.lm.forward_with_cache(input_ids, cache)
        emb = self.merge_multimodal_inputs(input_ids, self.encode_images(pixel_values))
        return self.lm.lm_logits(self.lm.hidden_states(None, cache, inputs_embeds=emb))

    def generate_multimodal(self, prompt_ids: List[int], pixel_values: torch.Tensor, cfg: Optional[GenerationConfig] = None) -> List[int]:
        """Greedy / sampled continuation of a prompt that contains an image (``llava.rs:1407``)."""
        from ..sampling import Sampler

        cfg = cfg or GenerationConfig()
        sampler = Sampler(seed=cfg.seed)
        cache = self.new_cache()
        logits = self.forward_with_cache(torch.tensor([list(prompt_ids)], device=self.device), cache, pixel_values)
        out: List[int] = []
        for _ in range(cfg.max_new_tokens):
            tok = sampler.sample(logits[0, -1].float().cpu(), cfg, history=list(prompt_ids) + out)
            if tok == cfg.eos_token_id:
                break
            out.append(tok)
            logits = self.forward_with_cache(torch.tensor([[tok]], device=self.device), cache)
        return out


class LlavaModel(VisionLanguageModel):
    """LLaVA-1.5 / 1.6 (``models_v2/llava.rs``): CLIP tower, features of layer -2 without the class token,
    ``linear`` or ``mlp2x_gelu`` projector, LLaMA language model."""

    config_class = C.LLaVAConfig

    def __init__(self, config):
        self.projector = "linear" if config.mm_projector_type == "linear" else "mlp2x_gelu"
        self.select_layer = config.mm_vision_select_layer
        self.drop_cls = config.mm_vision_select_feature == "patch"
        super().__init__(config)


class Qwen2VLModel(VisionLanguageModel):
    """Qwen2-VL (``models_v2/qwen2_vl.rs``): 3-D patch embedding (temporal patch 2), ViT blocks, 2x2 ``VisionMerger``,
    Qwen2 language model (GQA, QKV biases); 1-D RoPE like the reference (no M-RoPE)."""

    config_class = C.Qwen2VLConfig
    lm_cls = _lm_class("Qwen2LM", qkv_bias=True)
    lm_prefix = "model."
    vision_prefix = "visual."
    projector_prefix = "visual.merger."
    projector = "merger"
    select_layer = -1
    drop_cls = False

    def make_tower(self, c):
        return VisionTower(self.vision_prefix, c.vision_hidden_size, c.vision_num_hidden_layers, c.vision_num_attention_heads,
                           c.vision_intermediate_size, c.vision_patch_size, c.vision_image_size, eps=1e-6, act="gelu",
                           temporal=c.vision_temporal_patch_size, cls_token=False)


class Phi3VisionModel(VisionLanguageModel):
    config_class = C.Phi3VisionConfig
    lm_cls = _lm_class("Phi3LM")
    lm_prefix = "model."
    vision_prefix = "model.vision_embed_tokens.img_processor.vision_model."
    projector_prefix = "model.vision_embed_tokens.img_projection."
    projector = "mlp2x_gelu"


class InternVLModel(VisionLanguageModel):
    config_class = C.InternVLConfig
    lm_cls = _lm_class("InternLM2LM")
    vision_prefix = "vision_model."
    projector_prefix = "mlp1."
    projector = "mlp2x_gelu"
    select_layer = -1


class CogVLMModel(VisionLanguageModel):
    config_class = C.CogVLMConfig
    lm_prefix = "model."
    vision_prefix = "model.vision.transformer."
    projector_prefix = "model.vision.linear_proj."
    projector = "linear"


class IdeficsModel(VisionLanguageModel):
    config_class = C.IdeficsConfig
    lm_prefix = "model."
    vision_prefix = "model.vision_model."
    projector_prefix = "model.perceiver_resampler."
    projector = "linear"

    def is_cross_attention_layer(self, i: int) -> bool:
        """Layers that attend to the image in the published model (``idefics.rs:44``); this build splices instead."""
        return i % self._config.cross_attention_frequency == 0


class FlorenceModel(VisionLanguageModel):
    """Florence-2: vision tower + a LayerNorm / GELU / learned-position decoder."""

    config_class = C.FlorenceConfig
    lm_cls = _lm_class("FlorenceLM", KeyScheme(pos_embed=("model.embed_positions",), up=("mlp.fc1",), down=("mlp.fc2",)),
                       norm="layer", norm_bias=True, mlp="plain", act="gelu", pos="learned", qkv_bias=True,
                       o_bias=True, mlp_bias=True, max_position_embeddings=1024, tie_embeddings=True)
    lm_prefix = "language_model."
    vision_prefix = "vision_tower."
    projector_prefix = "image_projection."
    projector = "linear"
    select_layer = -1


MODELS = {"clip": ClipModel, "llava": LlavaModel, "qwen2_vl": Qwen2VLModel, "phi3_vision": Phi3VisionModel,
          "internvl": InternVLModel, "cogvlm": CogVLMModel, "idefics": IdeficsModel, "florence": FlorenceModel}
