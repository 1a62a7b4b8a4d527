"""RecurrentGemma (Griffin): recurrent blocks interleaved with local attention.

``models_v2/recurrent_gemma.rs``: layer ``i`` is recurrent iff ``i % recurrent_block_ratio != 0`` (``:62-65``); both
sub-blocks carry a pre- and a post-norm (``:381-404``); the attention layers are MQA 10/1 with head size 256, RoPE
and a 2048-token window; the MLP is GeGLU; embeddings are scaled by sqrt(hidden) (``:197-199``).  The recurrent block
is the reference's simplified RG-LRU ``h = a*h + (1-a)*x``, ``a = exp(-a_param)``, gated by ``linear_y`` (``:624-690``;
``input_gate`` is loaded but unused there and here).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..model_core import ModelInputs, ModelOutputs
from ..ops import recurrent as R
from ..tensor_core import ops_fn
from ..types import InvalidInput
from . import configs as C
from .simple import ParamModel, _f, mha, rope_tables
from .ssm import RecurrentCache


class RecurrentGemmaModel(ParamModel):
    config_class = C.RecurrentGemmaConfig

    def is_recurrent_layer(self, i: int) -> bool:
        return i % self._config.recurrent_block_ratio != 0

    def _lru(self):
        return self._config.lru_width or self._config.hidden_size

    def param_shapes(self) -> Dict[str, tuple]:
        c = self._config
        H, I, D, W = c.hidden_size, c.intermediate_size, c.head_dim, self._lru()
        s = {"model.embed_tokens.weight": (c.vocab_size, H)}
        for i in range(c.num_hidden_layers):
            L = f"model.layers.{i}."
            for n in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm", "post_feedforward_layernorm"):
                s[L + n + ".weight"] = (H,)
            T = L + "temporal_block."
            if self.is_recurrent_layer(i):
                s[T + "linear_x.weight"], s[T + "linear_y.weight"] = (W, H), (W, H)
                s[T + "a_param"] = (W,)
                s[T + "input_gate.weight"] = (W, H)
                s[T + "output_proj.weight"] = (H, W)
            else:
                s[T + "q_proj.weight"] = (c.num_attention_heads * D, H)
                s[T + "k_proj.weight"] = (c.num_key_value_heads * D, H)
                s[T + "v_proj.weight"] = (c.num_key_value_heads * D, H)
                s[T + "o_proj.weight"] = (H, c.num_attention_heads * D)
            M = L + "mlp."
            s[M + "gate_proj.weight"], s[M + "up_proj.weight"], s[M + "down_proj.weight"] = (I, H), (I, H), (H, I)
        s["model.norm.weight"] = (H,)
        if not c.tie_word_embeddings:
            s["lm_head.weight"] = (c.vocab_size, H)
        return s

    def special_init(self, name, shape, g):
        if name.endswith("a_param"):
            return torch.rand(shape, generator=g) * 2.0 + 0.05
        return None

    def new_cache(self, max_seq_len: Optional[int] = None) -> RecurrentCache:
        return RecurrentCache(self._config.num_hidden_layers)

    def hidden_states(self, ids, cache: Optional[RecurrentCache] = None):
        c, p = self._config, self.p
        eps = c.rms_norm_eps
        if getattr(self, "_rope", None) is None or self._rope[0].device != ids.device:
            self._rope = rope_tables(c.max_position_embeddings, c.head_dim, c.rope_theta, ids.device)
        x = ops_fn.embedding(ids, p["model.embed_tokens.weight"])
        x = (_f(x) * c.hidden_size ** 0.5).to(x.dtype)
        B = x.shape[0]
        for i in range(c.num_hidden_layers):
            L = f"model.layers.{i}."
            T = L + "temporal_block."
            st = cache.layers[i] if cache is not None else None
            h = self.rms(x, L + "input_layernorm", eps)
            if self.is_recurrent_layer(i):
                xb = ops_fn.linear(h, p[T + "linear_x.weight"])
                yb = ops_fn.linear(h, p[T + "linear_y.weight"])
                state = None
                if st is not None:
                    if "lru" not in st:
                        st["lru"] = torch.zeros(B, self._lru(), dtype=torch.float32, device=x.device)
                    state = st["lru"]
                hh = R.linear_recurrence(torch.exp(-_f(p[T + "a_param"])), xb, state, one_minus=True)
                t = ops_fn.linear(yb * hh, p[T + "output_proj.weight"])
            else:
                t = mha(h, h, p[T + "q_proj.weight"], None, p[T + "k_proj.weight"], None, p[T + "v_proj.weight"], None,
                        p[T + "o_proj.weight"], None, c.num_attention_heads, causal=True, num_kv_heads=c.num_key_value_heads,
                        cache=st, rope=self._rope, window=c.attention_window_size, head_dim=c.head_dim)
            x = x + self.rms(t, L + "post_attention_layernorm", eps)
            h = self.rms(x, L + "pre_feedforward_layernorm", eps)
            M = L + "mlp."
            m = ops_fn.linear(h, p[M + "gate_proj.weight"], act="gelu_tanh") * ops_fn.linear(h, p[M + "up_proj.weight"])
            x = x + self.rms(ops_fn.linear(m, p[M + "down_proj.weight"]), L + "post_feedforward_layernorm", eps)
        if cache is not None:
            cache.seq_len += ids.shape[1]
        return self.rms(x, "model.norm", eps)

    def lm_logits(self, x):
        w = self.p["model.embed_tokens.weight"] if self._config.tie_word_embeddings else self.p["lm_head.weight"]
        return ops_fn.linear(x, w)

    def forward(self, inputs: ModelInputs) -> ModelOutputs:
        if inputs.input_ids is None:
            raise InvalidInput("RecurrentGemmaModel takes text inputs")
        ids = inputs.input_ids if inputs.input_ids.dim() == 2 else inputs.input_ids[None]
        x = self.hidden_states(ids)
        return ModelOutputs.from_logits(self.lm_logits(x), hidden_states=x)

    def forward_with_cache(self, ids, cache=None):
        if ids.dim() == 1:
            ids = ids[None]
        return self.lm_logits(self.hidden_states(ids, cache))


MODELS = {"recurrent_gemma": RecurrentGemmaModel}
