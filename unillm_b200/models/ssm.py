"""State-space families: Mamba and the Jamba hybrid (Mamba + attention + MoE).

Mamba (``models_v2/mamba.rs:541-572``): norm -> in_proj -> split (x, z) -> causal depthwise conv (d_conv 4) -> SiLU ->
selective scan -> * SiLU(z) -> out_proj -> residual.  Jamba (``models_v2/jamba.rs:68-70,380-404``): layer i is an
attention layer iff ``(i + offset) % period == 0`` with the reference's offsets (4, 8), otherwise a Mamba block; every
layer's feed-forward is a 16-expert top-2 MoE.  Unlike the reference (``mamba.rs:584-590``) prefill leaves the
recurrent state behind, so ``forward_with_cache`` over a prompt followed by single-token steps equals ``forward``.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F

from ..model_core import ModelInputs, ModelOutputs
from ..ops import recurrent as R
from ..tensor_core import ops_fn
from ..types import InvalidInput
from . import configs as C
from .simple import ParamModel, _f, mha, rope_tables


class RecurrentCache:
    """Per-layer recurrent state (conv window + SSM state, or attention K/V for hybrid layers)."""

    def __init__(self, num_layers: int):
        self.layers: List[dict] = [dict() for _ in range(num_layers)]
        self.seq_len = 0

    def reset(self) -> None:
        for l in self.layers:
            l.clear()
        self.seq_len = 0


class _MambaMixin:
    """The Mamba mixer over parameters named ``<prefix>.{in_proj,conv1d,x_proj,dt_proj,A_log,D,out_proj}``."""

    def mixer_shapes(self, pre: str, H: int, d_inner: int, d_state: int, d_conv: int, dt_rank: int, conv_bias=True, bias=False):
        s = {pre + ".in_proj.weight": (2 * d_inner, H), pre + ".conv1d.weight": (d_inner, 1, d_conv),
             pre + ".x_proj.weight": (dt_rank + 2 * d_state, d_inner), pre + ".dt_proj.weight": (d_inner, dt_rank),
             pre + ".dt_proj.bias": (d_inner,), pre + ".A_log": (d_inner, d_state), pre + ".D": (d_inner,),
             pre + ".out_proj.weight": (H, d_inner)}
        if conv_bias:
            s[pre + ".conv1d.bias"] = (d_inner,)
        if bias:
            s[pre + ".in_proj.bias"] = (2 * d_inner,)
            s[pre + ".out_proj.bias"] = (H,)
        return s

    def mixer_special_init(self, name: str, shape: tuple, g) -> Optional[torch.Tensor]:
        if name.endswith(".A_log"):
            return torch.log(torch.arange(1, shape[1] + 1, dtype=torch.float32)).expand(shape).clone()
        if name.endswith(".D"):
            return torch.ones(shape)
        if name.endswith("dt_proj.bias"):
            dt = torch.exp(torch.rand(shape, generator=g) * (math.log(0.1) - math.log(0.001)) + math.log(0.001)).clamp_min(1e-4)
            return dt + torch.log(-torch.expm1(-dt))          # inverse softplus
        return None

    def mixer(self, h: torch.Tensor, pre: str, d_inner: int, d_state: int, dt_rank: int, state: Optional[dict]) -> torch.Tensor:
        p = self.p
        B, L, _ = h.shape
        xz = ops_fn.linear(h, p[pre + ".in_proj.weight"], p.get(pre + ".in_proj.bias"))
        x_in, z = xz[..., :d_inner].contiguous(), xz[..., d_inner:].contiguous()
        Kw = p[pre + ".conv1d.weight"].shape[-1]
        conv_state = ssm_state = None
        if state is not None:
            if "conv" not in state:
                state["conv"] = torch.zeros(B, Kw - 1, d_inner, dtype=h.dtype, device=h.device)
                state["ssm"] = torch.zeros(B, d_inner, d_state, dtype=torch.float32, device=h.device)
            conv_state, ssm_state = state["conv"], state["ssm"]
        xc = R.causal_dwconv1d(x_in, p[pre + ".conv1d.weight"].reshape(d_inner, Kw), p.get(pre + ".conv1d.bias"), conv_state,
                               act_silu=True)
        dbl = ops_fn.linear(xc, p[pre + ".x_proj.weight"])
        dt, Bm, Cm = dbl[..., :dt_rank], dbl[..., dt_rank:dt_rank + d_state], dbl[..., dt_rank + d_state:]
        dt = ops_fn.linear(dt.contiguous(), p[pre + ".dt_proj.weight"], p[pre + ".dt_proj.bias"])
        A = -torch.exp(_f(p[pre + ".A_log"]))
        y = R.selective_scan(xc, dt, A, Bm.contiguous(), Cm.contiguous(), _f(p[pre + ".D"]), z, ssm_state, delta_softplus=True)
        return ops_fn.linear(y, p[pre + ".out_proj.weight"], p.get(pre + ".out_proj.bias"))


class MambaModel(ParamModel, _MambaMixin):
    config_class = C.MambaConfig

    def _dims(self):
        c = self._config
        d_inner = c.d_inner or c.expand * c.hidden_size
        dt_rank = c.dt_rank or math.ceil(c.hidden_size / 16)
        return d_inner, dt_rank

    def param_shapes(self) -> Dict[str, tuple]:
        c = self._config
        d_inner, dt_rank = self._dims()
        s = {"backbone.embeddings.weight": (c.vocab_size, c.hidden_size)}
        for i in range(c.num_hidden_layers):
            s[f"backbone.layers.{i}.norm.weight"] = (c.hidden_size,)
            s.update(self.mixer_shapes(f"backbone.layers.{i}.mixer", c.hidden_size, d_inner, c.d_state, c.d_conv, dt_rank,
                                       c.conv_bias, c.bias))
        s["backbone.norm_f.weight"] = (c.hidden_size,)
        if not c.tie_embeddings:
            s["lm_head.weight"] = (c.vocab_size, c.hidden_size)
        return s

    def aliases(self, name):
        return (name, name.replace("backbone.embeddings", "backbone.embedding"))

    def special_init(self, name, shape, g):
        return self.mixer_special_init(name, shape, g)

    def new_cache(self, max_seq_len: Optional[int] = None) -> RecurrentCache:
        return RecurrentCache(self._config.num_hidden_layers)

    def hidden_states(self, ids: torch.Tensor, cache: Optional[RecurrentCache] = None) -> torch.Tensor:
        c = self._config
        d_inner, dt_rank = self._dims()
        x = ops_fn.embedding(ids, self.p["backbone.embeddings.weight"])
        for i in range(c.num_hidden_layers):
            h = self.rms(x, f"backbone.layers.{i}.norm", c.layer_norm_epsilon)
            x = x + self.mixer(h, f"backbone.layers.{i}.mixer", d_inner, c.d_state, dt_rank,
                               cache.layers[i] if cache is not None else None)
        if cache is not None:
            cache.seq_len += ids.shape[1]
        return self.rms(x, "backbone.norm_f", c.layer_norm_epsilon)

    def lm_logits(self, x):
        w = self.p["backbone.embeddings.weight"] if self._config.tie_embeddings else self.p["lm_head.weight"]
        return ops_fn.linear(x, w)

    def forward(self, inputs: ModelInputs) -> ModelOutputs:
        if inputs.input_ids is None:
            raise InvalidInput("MambaModel takes text inputs")
        ids = inputs.input_ids if inputs.input_ids.dim() == 2 else inputs.input_ids[None]
        x = self.hidden_states(ids)
        return ModelOutputs.from_logits(self.lm_logits(x), hidden_states=x)

    def forward_with_cache(self, ids: torch.Tensor, cache: Optional[RecurrentCache] = None) -> torch.Tensor:
        if ids.dim() == 1:
            ids = ids[None]
        return self.lm_logits(self.hidden_states(ids, cache))


class JambaModel(ParamModel, _MambaMixin):
    config_class = C.JambaConfig

    def _dims(self):
        c = self._config
        return (c.mamba_d_inner or c.expand * c.hidden_size), (c.mamba_dt_rank or math.ceil(c.hidden_size / 16))

    def is_attention_layer(self, i: int) -> bool:
        c = self._config
        return (i + c.attn_layer_offset) % c.attn_layer_period == 0

    def param_shapes(self):
        c = self._config
        H, I = c.hidden_size, c.intermediate_size
        d_inner, dt_rank = self._dims()
        D = H // c.num_attention_heads
        s = {"model.embed_tokens.weight": (c.vocab_size, H)}
        for i in range(c.num_hidden_layers):
            L = f"model.layers.{i}"
            s[L + ".input_layernorm.weight"] = (H,)
            s[L + ".post_attention_layernorm.weight"] = (H,)
            if self.is_attention_layer(i):
                s[L + ".self_attn.q_proj.weight"] = (c.num_attention_heads * D, H)
                s[L + ".self_attn.k_proj.weight"] = (c.num_key_value_heads * D, H)
                s[L + ".self_attn.v_proj.weight"] = (c.num_key_value_heads * D, H)
                s[L + ".self_attn.o_proj.weight"] = (H, c.num_attention_heads * D)
            else:
                s.update(self.mixer_shapes(L + ".mamba", H, d_inner, c.d_state, c.d_conv, dt_rank))
            s[L + ".block_sparse_moe.gate.weight"] = (c.num_experts, H)
            for e in range(c.num_experts):
                E = f"{L}.block_sparse_moe.experts.{e}"
                s[E + ".w1.weight"], s[E + ".w3.weight"], s[E + ".w2.weight"] = (I, H), (I, H), (H, I)
        s["model.norm.weight"] = (H,)
        if not c.tie_word_embeddings:
            s["lm_head.weight"] = (c.vocab_size, H)
        return s

    def special_init(self, name, shape, g):
        return self.mixer_special_init(name, shape, g)

    def new_cache(self, max_seq_len: Optional[int] = None) -> RecurrentCache:
        return RecurrentCache(self._config.num_hidden_layers)

    def _moe(self, x: torch.Tensor, L: str) -> torch.Tensor:
        c, p = self._config, self.p
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        logits = F.linear(_f(x2), _f(p[L + ".block_sparse_moe.gate.weight"]))
        v, idx = torch.topk(logits, c.num_experts_per_tok, dim=-1)
        w = torch.softmax(v, -1)
        out = torch.zeros(x2.shape, dtype=torch.float32, device=x.device)
        for e in range(c.num_experts):
            tok, slot = (idx == e).nonzero(as_tuple=True)
            if tok.numel() == 0:
                continue
            E = f"{L}.block_sparse_moe.experts.{e}"
            xe = x2[tok]
            hdn = (F.silu(_f(ops_fn.linear(xe, p[E + ".w1.weight"]))) * _f(ops_fn.linear(xe, p[E + ".w3.weight"]))).to(x.dtype)
            out.index_add_(0, tok, _f(ops_fn.linear(hdn, p[E + ".w2.weight"])) * w[tok, slot, None])
        return out.to(x.dtype).reshape(shape)

    def hidden_states(self, ids, cache: Optional[RecurrentCache] = None):
        c, p = self._config, self.p
        d_inner, dt_rank = self._dims()
        D = c.hidden_size // c.num_attention_heads
        if getattr(self, "_rope", None) is None or self._rope[0].device != ids.device:
            self._rope = rope_tables(min(c.max_position_embeddings, 8192), D, c.rope_theta, ids.device)
        x = ops_fn.embedding(ids, p["model.embed_tokens.weight"])
        for i in range(c.num_hidden_layers):
            L = f"model.layers.{i}"
            st = cache.layers[i] if cache is not None else None
            h = self.rms(x, L + ".input_layernorm", c.rms_norm_eps)
            if self.is_attention_layer(i):
                A = L + ".self_attn."
                x = x + mha(h, h, p[A + "q_proj.weight"], None, p[A + "k_proj.weight"], None, p[A + "v_proj.weight"], None,
                            p[A + "o_proj.weight"], None, c.num_attention_heads, causal=True,
                            num_kv_heads=c.num_key_value_heads, cache=st, rope=self._rope)
            else:
                x = x + self.mixer(h, L + ".mamba", d_inner, c.d_state, dt_rank, st)
            x = x + self._moe(self.rms(x, L + ".post_attention_layernorm", c.rms_norm_eps), L)
        if cache is not None:
            cache.seq_len += ids.shape[1]
        return self.rms(x, "model.norm", c.rms_norm_eps)

    def lm_logits(self, x):
        w = self.p["model.embed_tokens.weight"] if self._config.tie_word_embeddings else self.p["lm_head.weight"]
        return ops_fn.linear(x, w)

    def forward(self, inputs: ModelInputs) -> ModelOutputs:
        if inputs.input_ids is None:
            raise InvalidInput("JambaModel takes text inputs")
        ids = inputs.input_ids if inputs.input_ids.dim() == 2 else inputs.input_ids[None]
        x = self.hidden_states(ids)
        return ModelOutputs.from_logits(self.lm_logits(x), hidden_states=x)

    def forward_with_cache(self, ids, cache=None):
        if ids.dim() == 1:
            ids = ids[None]
        return self.lm_logits(self.hidden_states(ids, cache))


MODELS = {"mamba": MambaModel, "jamba": JambaModel}
