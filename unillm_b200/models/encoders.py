"""Encoder-only family: BERT / RoBERTa.

``models_v2/bert.rs``: word + position + token-type embeddings -> LayerNorm -> post-LN encoder layers with biased
bidirectional attention and GELU -> optional pooler (dense + tanh on [CLS]).  Output kind ``embeddings`` with ``pooled``;
``generate`` is rejected (``:183``).  Checkpoints are accepted with or without the ``bert.`` prefix and with the legacy
``gamma`` / ``beta`` names (``:575-576,659-660``).
"""
from __future__ import annotations

from typing import Dict

import torch

from ..model_core import ModelInputs, ModelOutputs
from ..tensor_core import ops_fn
from ..types import InvalidInput, UnsupportedOperation
from . import configs as C
from .simple import ParamModel, _f, mha


class BertModel(ParamModel):
    config_class = C.BertConfig

    def param_shapes(self) -> Dict[str, tuple]:
        c = self._config
        H, I = c.hidden_size, c.intermediate_size
        s = {"embeddings.word_embeddings.weight": (c.vocab_size, H),
             "embeddings.position_embeddings.weight": (c.max_position_embeddings, H),
             "embeddings.token_type_embeddings.weight": (c.type_vocab_size, H),
             "embeddings.LayerNorm.weight": (H,), "embeddings.LayerNorm.bias": (H,)}
        for i in range(c.num_hidden_layers):
            L = f"encoder.layer.{i}."
            for n in ("attention.self.query", "attention.self.key", "attention.self.value", "attention.output.dense"):
                s[L + n + ".weight"], s[L + n + ".bias"] = (H, H), (H,)
            s[L + "attention.output.LayerNorm.weight"], s[L + "attention.output.LayerNorm.bias"] = (H,), (H,)
            s[L + "intermediate.dense.weight"], s[L + "intermediate.dense.bias"] = (I, H), (I,)
            s[L + "output.dense.weight"], s[L + "output.dense.bias"] = (H, I), (H,)
            s[L + "output.LayerNorm.weight"], s[L + "output.LayerNorm.bias"] = (H,), (H,)
        s["pooler.dense.weight"], s["pooler.dense.bias"] = (H, H), (H,)
        return s

    def aliases(self, name):
        legacy = name.replace("LayerNorm.weight", "LayerNorm.gamma").replace("LayerNorm.bias", "LayerNorm.beta")
        return (name, "bert." + name, "roberta." + name, legacy, "bert." + legacy)

    def forward(self, inputs: ModelInputs) -> ModelOutputs:
        if inputs.input_ids is None:
            raise InvalidInput("BertModel takes text inputs")
        c, p = self._config, self.p
        ids = inputs.input_ids
        B, T = ids.shape
        if T > c.max_position_embeddings:
            raise InvalidInput(f"sequence length {T} exceeds max_position_embeddings {c.max_position_embeddings}")
        pos = torch.arange(T, device=ids.device)
        tt = torch.zeros_like(ids)          # token types: a single segment
        x = (ops_fn.embedding(ids, p["embeddings.word_embeddings.weight"]) +
             ops_fn.embedding(pos, p["embeddings.position_embeddings.weight"])[None] +
             ops_fn.embedding(tt, p["embeddings.token_type_embeddings.weight"]))
        x = self.ln(x, "embeddings.LayerNorm", c.layer_norm_eps)
        bias = None
        if inputs.attention_mask is not None:
            bias = (1.0 - _f(inputs.attention_mask))[:, None, None, :] * -1e9
        for i in range(c.num_hidden_layers):
            L = f"encoder.layer.{i}."
            A = L + "attention.self."
            a = mha(x, x, p[A + "query.weight"], p[A + "query.bias"], p[A + "key.weight"], p[A + "key.bias"],
                    p[A + "value.weight"], p[A + "value.bias"], p[L + "attention.output.dense.weight"],
                    p[L + "attention.output.dense.bias"], c.num_attention_heads, bias=bias)
            x = self.ln(x + a, L + "attention.output.LayerNorm", c.layer_norm_eps)
            m = self.lin(self.lin(x, L + "intermediate.dense", act=c.hidden_act), L + "output.dense")
            x = self.ln(x + m, L + "output.LayerNorm", c.layer_norm_eps)
        pooled = torch.tanh(_f(self.lin(x[:, 0], "pooler.dense"))).to(x.dtype)
        return ModelOutputs.embeddings(x, pooled)

    def generate(self, prompt, config=None):
        raise UnsupportedOperation("BERT is an encoder; it does not generate text")

    def generate_ids(self, *a, **k):
        raise UnsupportedOperation("BERT is an encoder; it does not generate text")


MODELS = {"bert": BertModel}
