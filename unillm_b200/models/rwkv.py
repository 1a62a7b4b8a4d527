"""RWKV-4 and RWKV-6: linear-attention language models with O(1) state per layer.

RWKV-4 (``models_v2/rwkv4.rs:419-529,595-666``): LN -> time mixing (token shift, WKV with per-channel decay and bonus)
-> LN -> channel mixing ``sigmoid(r) * (relu(k)^2 W_v)``, hidden state halved every ``rescale_every`` layers
(``:340-344``).  The WKV core runs in the running-maximum form, which equals the reference's plain (num, den) form
wherever that one does not overflow.

RWKV-6 (``models_v2/rwkv6.rs:483-553``): the same skeleton with a matrix-valued state per 64-wide head, a
data-dependent decay ``exp(-exp(time_decay + tanh(x W1) W2))``, per-projection token-shift mixes ``time_maa_*``, a SiLU
gate and a per-head group norm ``ln_x``.  The reference collapses the five mixes into ``time_maa_x`` and replaces the
group norm by a scale; this implementation uses all the tensors the checkpoint format defines.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.nn.functional as F

from ..model_core import ModelInputs, ModelOutputs
from ..ops import recurrent as R
from ..tensor_core import ops_fn
from ..types import InvalidInput
from . import configs as C
from .simple import ParamModel, _f
from .ssm import RecurrentCache


def token_shift(h: torch.Tensor, st: Optional[dict], key: str) -> torch.Tensor:
    """Previous token's features for every position; the last position is remembered in ``st[key]``."""
    B, L, H = h.shape
    first = st[key] if (st is not None and key in st) else torch.zeros(B, H, dtype=h.dtype, device=h.device)
    prev = torch.cat([first[:, None], h[:, :-1]], 1)
    if st is not None:
        st[key] = h[:, -1].clone()
    return prev


def _mix(h, prev, m):
    m = m.to(h.dtype)
    return h * m + prev * (1 - m)


class _RwkvBase(ParamModel):
    def new_cache(self, max_seq_len: Optional[int] = None) -> RecurrentCache:
        return RecurrentCache(self._config.num_hidden_layers)

    def aliases(self, name):
        alt = name.replace("emb.weight", "rwkv.embeddings.weight").replace("ln_out.", "rwkv.ln_out.")
        return (name, alt) if alt != name else (name,)

    def special_init(self, name, shape, g):
        if name.endswith(("time_mix_k", "time_mix_v", "time_mix_r")) or "time_maa_" in name:
            return torch.rand(shape, generator=g)
        if name.endswith("time_decay"):
            return torch.randn(shape, generator=g) * 0.5 - 1.0
        if name.endswith("time_first"):
            return torch.randn(shape, generator=g) * 0.3
        return None

    def lm_logits(self, x):
        w = self.p["emb.weight"] if self._config.tie_word_embeddings else self.p["head.weight"]
        return ops_fn.linear(x, w)

    def forward(self, inputs: ModelInputs) -> ModelOutputs:
        if inputs.input_ids is None:
            raise InvalidInput(f"{type(self).__name__} takes text inputs")
        ids = inputs.input_ids if inputs.input_ids.dim() == 2 else inputs.input_ids[None]
        x = self.hidden_states(ids)
        return ModelOutputs.from_logits(self.lm_logits(x), hidden_states=x)

    def forward_with_cache(self, ids, cache=None):
        if ids.dim() == 1:
            ids = ids[None]
        return self.lm_logits(self.hidden_states(ids, cache))

    def _channel_mix(self, h, st, pre, mk, mr):
        p = self.p
        prev = token_shift(h, st, "cm")
        k = ops_fn.linear(_mix(h, prev, p[pre + mk]), p[pre + "key.weight"], act="relu2")
        r = ops_fn.sigmoid(ops_fn.linear(_mix(h, prev, p[pre + mr]), p[pre + "receptance.weight"]))
        return r * ops_fn.linear(k, p[pre + "value.weight"])


class Rwkv4Model(_RwkvBase):
    config_class = C.Rwkv4Config

    def _inter(self):
        c = self._config
        return c.intermediate_size or 4 * c.hidden_size

    def param_shapes(self) -> Dict[str, tuple]:
        c = self._config
        H, I = c.hidden_size, self._inter()
        s = {"emb.weight": (c.vocab_size, H), "blocks.0.ln0.weight": (H,), "blocks.0.ln0.bias": (H,)}
        for i in range(c.num_hidden_layers):
            b = f"blocks.{i}."
            for ln in ("ln1", "ln2"):
                s[b + ln + ".weight"], s[b + ln + ".bias"] = (H,), (H,)
            for t in ("time_decay", "time_first", "time_mix_k", "time_mix_v", "time_mix_r"):
                s[b + "att." + t] = (H,)
            for w in ("key", "value", "receptance", "output"):
                s[b + f"att.{w}.weight"] = (H, H)
            s[b + "ffn.time_mix_k"], s[b + "ffn.time_mix_r"] = (H,), (H,)
            s[b + "ffn.key.weight"], s[b + "ffn.value.weight"], s[b + "ffn.receptance.weight"] = (I, H), (H, I), (H, H)
        s["ln_out.weight"], s["ln_out.bias"] = (H,), (H,)
        if not c.tie_word_embeddings:
            s["head.weight"] = (c.vocab_size, H)
        return s

    def hidden_states(self, ids, cache: Optional[RecurrentCache] = None):
        c, p = self._config, self.p
        eps = c.layer_norm_epsilon
        x = self.ln(ops_fn.embedding(ids, p["emb.weight"]), "blocks.0.ln0", eps)
        B = x.shape[0]
        for i in range(c.num_hidden_layers):
            b = f"blocks.{i}."
            st = cache.layers[i] if cache is not None else None
            h = self.ln(x, b + "ln1", eps)
            prev = token_shift(h, st, "tm")
            a = b + "att."
            k = ops_fn.linear(_mix(h, prev, p[a + "time_mix_k"]), p[a + "key.weight"])
            v = ops_fn.linear(_mix(h, prev, p[a + "time_mix_v"]), p[a + "value.weight"])
            r = ops_fn.sigmoid(ops_fn.linear(_mix(h, prev, p[a + "time_mix_r"]), p[a + "receptance.weight"]))
            wkv_state = None
            if st is not None:
                if "wkv" not in st:
                    st["wkv"] = R.wkv4_new_state(B, c.hidden_size, x.device)
                wkv_state = st["wkv"]
            wkv = R.wkv4(k, v, -torch.exp(_f(p[a + "time_decay"])), _f(p[a + "time_first"]), wkv_state)
            x = x + ops_fn.linear(r * wkv, p[a + "output.weight"])
            x = x + self._channel_mix(self.ln(x, b + "ln2", eps), st, b + "ffn.", "time_mix_k", "time_mix_r")
            if c.rescale_every > 0 and (i + 1) % c.rescale_every == 0:
                x = x * 0.5
        if cache is not None:
            cache.seq_len += ids.shape[1]
        return self.ln(x, "ln_out", eps)


class Rwkv6Model(_RwkvBase):
    config_class = C.Rwkv6Config
    DECAY_RANK = 64

    def _dims(self):
        c = self._config
        heads = c.num_heads or c.hidden_size // c.head_size
        inter = c.intermediate_size or int(c.hidden_size * 3.5) // 32 * 32
        return heads, inter

    def param_shapes(self) -> Dict[str, tuple]:
        c = self._config
        H = c.hidden_size
        _, I = self._dims()
        s = {"emb.weight": (c.vocab_size, H), "blocks.0.ln0.weight": (H,), "blocks.0.ln0.bias": (H,)}
        for i in range(c.num_hidden_layers):
            b = f"blocks.{i}."
            for ln in ("ln1", "ln2"):
                s[b + ln + ".weight"], s[b + ln + ".bias"] = (H,), (H,)
            for t in ("time_maa_x", "time_maa_w", "time_maa_k", "time_maa_v", "time_maa_r", "time_maa_g", "time_decay", "time_first"):
                s[b + "att." + t] = (H,)
            s[b + "att.time_decay_w1"], s[b + "att.time_decay_w2"] = (H, self.DECAY_RANK), (self.DECAY_RANK, H)
            for w in ("receptance", "key", "value", "output", "gate"):
                s[b + f"att.{w}.weight"] = (H, H)
            s[b + "att.ln_x.weight"], s[b + "att.ln_x.bias"] = (H,), (H,)
            s[b + "ffn.time_maa_k"], s[b + "ffn.time_maa_r"] = (H,), (H,)
            s[b + "ffn.key.weight"], s[b + "ffn.value.weight"], s[b + "ffn.receptance.weight"] = (I, H), (H, I), (H, H)
        s["ln_out.weight"], s["ln_out.bias"] = (H,), (H,)
        if not c.tie_word_embeddings:
            s["head.weight"] = (c.vocab_size, H)
        return s

    def hidden_states(self, ids, cache: Optional[RecurrentCache] = None):
        c, p = self._config, self.p
        eps = c.layer_norm_epsilon
        heads, _ = self._dims()
        Dh = c.hidden_size // heads
        x = self.ln(ops_fn.embedding(ids, p["emb.weight"]), "blocks.0.ln0", eps)
        B, L, H = x.shape
        for i in range(c.num_hidden_layers):
            b = f"blocks.{i}."
            a = b + "att."
            st = cache.layers[i] if cache is not None else None
            h = self.ln(x, b + "ln1", eps)
            prev = token_shift(h, st, "tm")
            # token-shift interpolation toward the previous token, one mix per projection (time_maa_x feeds the
            # data-dependent mixing LoRA of full Finch checkpoints, whose tensors this format does not carry)
            dx = prev - h
            xw, xk, xv, xr, xg = (h + dx * p[a + "time_maa_" + n].to(h.dtype) for n in ("w", "k", "v", "r", "g"))
            r = ops_fn.linear(xr, p[a + "receptance.weight"])
            k = ops_fn.linear(xk, p[a + "key.weight"])
            v = ops_fn.linear(xv, p[a + "value.weight"])
            g = ops_fn.silu(ops_fn.linear(xg, p[a + "gate.weight"]))
            lora = torch.tanh(_f(xw) @ _f(p[a + "time_decay_w1"])) @ _f(p[a + "time_decay_w2"])
            ww = _f(p[a + "time_decay"]) + lora                                        # decay = exp(-exp(ww))
            wkv_state = None
            if st is not None:
                if "wkv" not in st:
                    st["wkv"] = torch.zeros(B, heads, Dh, Dh, dtype=torch.float32, device=x.device)
                wkv_state = st["wkv"]
            y = R.wkv6(r, k, v, ww.contiguous(), _f(p[a + "time_first"]), heads, wkv_state)
            y = F.group_norm(_f(y).reshape(B * L, H), heads, _f(p[a + "ln_x.weight"]), _f(p[a + "ln_x.bias"]), eps=64e-5)
            y = y.reshape(B, L, H).to(x.dtype) * g
            x = x + ops_fn.linear(y, p[a + "output.weight"])
            x = x + self._channel_mix(self.ln(x, b + "ln2", eps), st, b + "ffn.", "time_maa_k", "time_maa_r")
            if c.rescale_every > 0 and (i + 1) % c.rescale_every == 0:
                x = x * 0.5
        if cache is not None:
            cache.seq_len += ids.shape[1]
        return self.ln(x, "ln_out", eps)


MODELS = {"rwkv4": Rwkv4Model, "rwkv6": Rwkv6Model}
