"""Encoder-decoder families: T5 (text) and Whisper (audio).

T5 (``models_v2/t5.rs``): RMS-style layer norm without bias, unscaled attention ``q k^T`` with a learned relative
position bias shared by all layers of a stack, ReLU or gated-GELU feed-forward, cross-attention in the decoder.  The
reference's ``compute_position_bias`` returns zeros and its bucket function is dead code (``:401-409,872-903``); here
the bias is computed (bidirectional buckets in the encoder, causal buckets in the decoder).

Whisper (``models_v2/whisper.rs``): two GELU conv1d stems (k3 s1 p1; k3 s2 p1) -> + sinusoidal positions -> pre-LN
bidirectional encoder -> pre-LN causal decoder with cross-attention and learned positions -> ``proj_out`` tied to the
token embedding; ``transcribe`` decodes greedily (``:284-343``).  Unlike the reference the decoder keeps self- and
cross-attention K/V caches.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from ..model_core import ModelInputs, ModelOutputs
from ..tensor_core import ops_fn
from ..types import InvalidInput
from . import configs as C
from .simple import ParamModel, _f, conv1d, mha


def t5_relative_bucket(rel: torch.Tensor, bidirectional: bool, num_buckets: int, max_distance: int) -> torch.Tensor:
    """Bucket index of ``rel = key_pos - query_pos`` (T5's log-spaced buckets)."""
    ret = torch.zeros_like(rel)
    n = num_buckets
    if bidirectional:
        n //= 2
        ret = ret + (rel > 0).long() * n
        rel = rel.abs()
    else:
        rel = (-rel).clamp_min(0)
    max_exact = n // 2
    is_small = rel < max_exact
    large = max_exact + (torch.log(rel.float().clamp_min(1) / max_exact) / math.log(max_distance / max_exact) *
                         (n - max_exact)).long()
    large = large.clamp_max(n - 1)
    return ret + torch.where(is_small, rel, large)


class T5Model(ParamModel):
    config_class = C.T5Config

    def _gated(self):
        c = self._config
        return c.is_gated_act or c.feed_forward_proj.startswith("gated")

    def _act(self):
        f = self._config.feed_forward_proj
        return "gelu_tanh" if "gelu" in f else "relu"

    def param_shapes(self) -> Dict[str, tuple]:
        c = self._config
        H, inner, F_ = c.d_model, c.num_heads * c.d_kv, c.d_ff
        s = {"shared.weight": (c.vocab_size, H)}

        def attn(pre, rel):
            for n, shp in (("q", (inner, H)), ("k", (inner, H)), ("v", (inner, H)), ("o", (H, inner))):
                s[f"{pre}.{n}.weight"] = shp
            if rel:
                s[pre + ".relative_attention_bias.weight"] = (c.relative_attention_num_buckets, c.num_heads)

        def ff(pre):
            s[pre + ".layer_norm.weight"] = (H,)
            if self._gated():
                s[pre + ".DenseReluDense.wi_0.weight"], s[pre + ".DenseReluDense.wi_1.weight"] = (F_, H), (F_, H)
            else:
                s[pre + ".DenseReluDense.wi.weight"] = (F_, H)
            s[pre + ".DenseReluDense.wo.weight"] = (H, F_)

        for i in range(c.num_layers):
            b = f"encoder.block.{i}"
            s[b + ".layer.0.layer_norm.weight"] = (H,)
            attn(b + ".layer.0.SelfAttention", i == 0)
            ff(b + ".layer.1")
        s["encoder.final_layer_norm.weight"] = (H,)
        for i in range(c.num_decoder_layers):
            b = f"decoder.block.{i}"
            s[b + ".layer.0.layer_norm.weight"] = (H,)
            attn(b + ".layer.0.SelfAttention", i == 0)
            s[b + ".layer.1.layer_norm.weight"] = (H,)
            attn(b + ".layer.1.EncDecAttention", False)
            ff(b + ".layer.2")
        s["decoder.final_layer_norm.weight"] = (H,)
        if not c.tie_word_embeddings:
            s["lm_head.weight"] = (c.vocab_size, H)
        return s

    def aliases(self, name):
        if name == "shared.weight":
            return (name, "encoder.embed_tokens.weight", "decoder.embed_tokens.weight")
        return (name,)

    def _bias(self, stack: str, Tq: int, Tk: int, device, bidirectional: bool) -> torch.Tensor:
        c = self._config
        q = torch.arange(Tk - Tq, Tk, device=device)[:, None]
        k = torch.arange(Tk, device=device)[None, :]
        b = t5_relative_bucket(k - q, bidirectional, c.relative_attention_num_buckets, c.relative_attention_max_distance)
        w = self.p[f"{stack}.block.0.layer.0.SelfAttention.relative_attention_bias.weight"]
        return _f(w)[b].permute(2, 0, 1)[None]                     # [1, heads, Tq, Tk]

    def _attn(self, pre, xq, xkv, bias=None, causal=False, cache=None):
        p, c = self.p, self._config
        return mha(xq, xkv, p[pre + ".q.weight"], None, p[pre + ".k.weight"], None, p[pre + ".v.weight"], None,
                   p[pre + ".o.weight"], None, c.num_heads, causal=causal, bias=bias, scale=1.0, cache=cache, head_dim=c.d_kv)

    def _ff(self, pre, x):
        p = self.p
        h = self.rms(x, pre + ".layer_norm", self._config.layer_norm_epsilon)
        if self._gated():
            m = ops_fn.linear(h, p[pre + ".DenseReluDense.wi_0.weight"], act=self._act()) * \
                ops_fn.linear(h, p[pre + ".DenseReluDense.wi_1.weight"])
        else:
            m = ops_fn.linear(h, p[pre + ".DenseReluDense.wi.weight"], act=self._act())
        return x + ops_fn.linear(m, p[pre + ".DenseReluDense.wo.weight"])

    def encode(self, ids: torch.Tensor, attention_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        c = self._config
        x = ops_fn.embedding(ids, self.p["shared.weight"])
        T = ids.shape[1]
        bias = self._bias("encoder", T, T, ids.device, True)
        if attention_mask is not None:
            bias = bias + (1.0 - _f(attention_mask))[:, None, None, :] * -1e9
        for i in range(c.num_layers):
            b = f"encoder.block.{i}"
            h = self.rms(x, b + ".layer.0.layer_norm", c.layer_norm_epsilon)
            x = x + self._attn(b + ".layer.0.SelfAttention", h, h, bias)
            x = self._ff(b + ".layer.1", x)
        return self.rms(x, "encoder.final_layer_norm", c.layer_norm_epsilon)

    def decode(self, dec_ids: torch.Tensor, enc: torch.Tensor, cache: Optional[List[dict]] = None) -> torch.Tensor:
        c = self._config
        x = ops_fn.embedding(dec_ids, self.p["shared.weight"])
        Tq = dec_ids.shape[1]
        past = cache[0]["self"]["k"].shape[2] if (cache and cache[0].get("self", {}).get("k") is not None) else 0
        bias = self._bias("decoder", Tq, past + Tq, dec_ids.device, False)
        for i in range(c.num_decoder_layers):
            b = f"decoder.block.{i}"
            st = cache[i] if cache is not None else None
            h = self.rms(x, b + ".layer.0.layer_norm", c.layer_norm_epsilon)
            x = x + self._attn(b + ".layer.0.SelfAttention", h, h, bias, causal=True,
                               cache=st.setdefault("self", {}) if st is not None else None)
            h = self.rms(x, b + ".layer.1.layer_norm", c.layer_norm_epsilon)
            x = x + self._cross(b + ".layer.1.EncDecAttention", h, enc, st)
            x = self._ff(b + ".layer.2", x)
        x = self.rms(x, "decoder.final_layer_norm", c.layer_norm_epsilon)
        if c.tie_word_embeddings:
            return ops_fn.linear((_f(x) * c.d_model ** -0.5).to(x.dtype), self.p["shared.weight"])
        return ops_fn.linear(x, self.p["lm_head.weight"])

    def _cross(self, pre, h, enc, st):
        """Cross-attention; the encoder's K/V projections are computed once per sequence and kept in ``st``."""
        p, c = self.p, self._config
        B, Tq, _ = h.shape
        D, nh = c.d_kv, c.num_heads
        if st is not None and "cross_k" in st:
            k, v = st["cross_k"], st["cross_v"]
        else:
            k = ops_fn.linear(enc, p[pre + ".k.weight"]).view(B, -1, nh, D).transpose(1, 2)
            v = ops_fn.linear(enc, p[pre + ".v.weight"]).view(B, -1, nh, D).transpose(1, 2)
            if st is not None:
                st["cross_k"], st["cross_v"] = k, v
        q = ops_fn.linear(h, p[pre + ".q.weight"]).view(B, Tq, nh, D).transpose(1, 2)
        a = torch.softmax(torch.matmul(_f(q), _f(k).transpose(-1, -2)), -1)
        o = torch.matmul(a, _f(v)).to(h.dtype).transpose(1, 2).reshape(B, Tq, nh * D)
        return ops_fn.linear(o, p[pre + ".o.weight"])

    def forward(self, inputs: ModelInputs) -> ModelOutputs:
        if inputs.input_ids is None:
            raise InvalidInput("T5Model takes text inputs")
        c = self._config
        enc = self.encode(inputs.input_ids, inputs.attention_mask)
        dec_ids = inputs.decoder_input_ids
        if dec_ids is None:
            dec_ids = torch.full((inputs.input_ids.shape[0], 1), c.decoder_start_token_id, dtype=torch.long,
                                 device=inputs.input_ids.device)
        logits = self.decode(dec_ids, enc)
        return ModelOutputs.sequence(logits, encoder_hidden_states=enc)

    def generate_ids(self, prompt_ids, cfg, on_token=None):
        from ..sampling import Sampler

        c = self._config
        sampler = Sampler(seed=cfg.seed)
        enc = self.encode(torch.tensor([list(prompt_ids)], device=self.device))
        cache = [dict() for _ in range(c.num_decoder_layers)]
        tok, out = c.decoder_start_token_id, []
        for _ in range(cfg.max_new_tokens):
            logits = self.decode(torch.tensor([[tok]], device=self.device), enc, cache)
            tok = sampler.sample(logits[0, -1].float().cpu(), cfg, history=out)
            if tok == cfg.eos_token_id:
                break
            out.append(tok)
            if on_token is not None:
                on_token(tok)
        return out


def sinusoids(length: int, channels: int) -> torch.Tensor:
    inc = math.log(10000.0) / (channels // 2 - 1)
    inv = torch.exp(-inc * torch.arange(channels // 2, dtype=torch.float32))
    t = torch.arange(length, dtype=torch.float32)[:, None] * inv[None]
    return torch.cat([t.sin(), t.cos()], 1)


class WhisperModel(ParamModel):
    config_class = C.WhisperConfig

    def param_shapes(self) -> Dict[str, tuple]:
        c = self._config
        H = c.d_model
        s = {"model.encoder.conv1.weight": (H, c.num_mel_bins, 3), "model.encoder.conv1.bias": (H,),
             "model.encoder.conv2.weight": (H, H, 3), "model.encoder.conv2.bias": (H,),
             "model.encoder.embed_positions.weight": (c.max_source_positions, H)}

        def attn(pre):
            for n in ("q_proj", "v_proj", "out_proj"):
                s[f"{pre}.{n}.weight"], s[f"{pre}.{n}.bias"] = (H, H), (H,)
            s[pre + ".k_proj.weight"] = (H, H)

        def block(pre, F_, cross):
            s[pre + ".self_attn_layer_norm.weight"], s[pre + ".self_attn_layer_norm.bias"] = (H,), (H,)
            attn(pre + ".self_attn")
            if cross:
                s[pre + ".encoder_attn_layer_norm.weight"], s[pre + ".encoder_attn_layer_norm.bias"] = (H,), (H,)
                attn(pre + ".encoder_attn")
            s[pre + ".final_layer_norm.weight"], s[pre + ".final_layer_norm.bias"] = (H,), (H,)
            s[pre + ".fc1.weight"], s[pre + ".fc1.bias"] = (F_, H), (F_,)
            s[pre + ".fc2.weight"], s[pre + ".fc2.bias"] = (H, F_), (H,)

        for i in range(c.encoder_layers):
            block(f"model.encoder.layers.{i}", c.encoder_ffn_dim, False)
        s["model.encoder.layer_norm.weight"], s["model.encoder.layer_norm.bias"] = (H,), (H,)
        s["model.decoder.embed_tokens.weight"] = (c.vocab_size, H)
        s["model.decoder.embed_positions.weight"] = (c.max_target_positions, H)
        for i in range(c.decoder_layers):
            block(f"model.decoder.layers.{i}", c.decoder_ffn_dim, True)
        s["model.decoder.layer_norm.weight"], s["model.decoder.layer_norm.bias"] = (H,), (H,)
        return s

    def special_init(self, name, shape, g):
        if name == "model.encoder.embed_positions.weight":
            return sinusoids(shape[0], shape[1])
        return None

    def _attn(self, pre, xq, xkv, heads, causal=False, cache=None):
        p = self.p
        return mha(xq, xkv, p[pre + ".q_proj.weight"], p[pre + ".q_proj.bias"], p[pre + ".k_proj.weight"], None,
                   p[pre + ".v_proj.weight"], p[pre + ".v_proj.bias"], p[pre + ".out_proj.weight"], p[pre + ".out_proj.bias"],
                   heads, causal=causal, cache=cache)

    def encode(self, mel: torch.Tensor) -> torch.Tensor:
        """``mel`` [B, num_mel_bins, frames] -> [B, frames/2, d_model]."""
        c, p = self._config, self.p
        if mel.dim() == 2:
            mel = mel[None]
        x = ops_fn.gelu(conv1d(mel.to(self.dtype), p["model.encoder.conv1.weight"], p["model.encoder.conv1.bias"], padding=1))
        x = ops_fn.gelu(conv1d(x, p["model.encoder.conv2.weight"], p["model.encoder.conv2.bias"], stride=2, padding=1))
        x = x.transpose(1, 2).contiguous()
        T = x.shape[1]
        if T > c.max_source_positions:
            raise InvalidInput(f"{T} encoder positions exceed max_source_positions {c.max_source_positions}")
        x = x + p["model.encoder.embed_positions.weight"][:T][None].to(x.dtype)
        eps = c.layer_norm_eps
        for i in range(c.encoder_layers):
            L = f"model.encoder.layers.{i}"
            x = x + self._self(L, x, c.encoder_attention_heads, eps, False, None)
            x = x + self.lin(self.lin(self.ln(x, L + ".final_layer_norm", eps), L + ".fc1", act="gelu"), L + ".fc2")
        return self.ln(x, "model.encoder.layer_norm", eps)

    def _self(self, L, x, heads, eps, causal, cache):
        h = self.ln(x, L + ".self_attn_layer_norm", eps)
        return self._attn(L + ".self_attn", h, h, heads, causal, cache)

    def decode(self, ids: torch.Tensor, enc: torch.Tensor, cache: Optional[List[dict]] = None) -> torch.Tensor:
        c, p = self._config, self.p
        eps = c.layer_norm_eps
        past = cache[0]["self"]["k"].shape[2] if (cache and cache[0].get("self", {}).get("k") is not None) else 0
        T = ids.shape[1]
        if past + T > c.max_target_positions:
            raise InvalidInput(f"{past + T} decoder positions exceed max_target_positions {c.max_target_positions}")
        x = ops_fn.embedding(ids, p["model.decoder.embed_tokens.weight"])
        if c.scale_embedding:
            x = (_f(x) * c.d_model ** 0.5).to(x.dtype)
        x = x + p["model.decoder.embed_positions.weight"][past:past + T][None].to(x.dtype)
        for i in range(c.decoder_layers):
            L = f"model.decoder.layers.{i}"
            st = cache[i] if cache is not None else None
            x = x + self._self(L, x, c.decoder_attention_heads, eps, True, st.setdefault("self", {}) if st is not None else None)
            h = self.ln(x, L + ".encoder_attn_layer_norm", eps)
            x = x + self._cross(L + ".encoder_attn", h, enc, st)
            x = x + self.lin(self.lin(self.ln(x, L + ".final_layer_norm", eps), L + ".fc1", act="gelu"), L + ".fc2")
        x = self.ln(x, "model.decoder.layer_norm", eps)
        return ops_fn.linear(x, p["model.decoder.embed_tokens.weight"])

    def _cross(self, pre, h, enc, st):
        p, c = self.p, self._config
        B, Tq, H = h.shape
        nh = c.decoder_attention_heads
        D = H // nh
        if st is not None and "cross_k" in st:
            k, v = st["cross_k"], st["cross_v"]
        else:
            k = ops_fn.linear(enc, p[pre + ".k_proj.weight"]).view(B, -1, nh, D).transpose(1, 2)
            v = ops_fn.linear(enc, p[pre + ".v_proj.weight"], p[pre + ".v_proj.bias"]).view(B, -1, nh, D).transpose(1, 2)
            if st is not None:
                st["cross_k"], st["cross_v"] = k, v
        q = ops_fn.linear(h, p[pre + ".q_proj.weight"], p[pre + ".q_proj.bias"]).view(B, Tq, nh, D).transpose(1, 2)
        a = torch.softmax(torch.matmul(_f(q), _f(k).transpose(-1, -2)) * D ** -0.5, -1)
        o = torch.matmul(a, _f(v)).to(h.dtype).transpose(1, 2).reshape(B, Tq, H)
        return ops_fn.linear(o, p[pre + ".out_proj.weight"], p[pre + ".out_proj.bias"])

    def forward(self, inputs: ModelInputs) -> ModelOutputs:
        if inputs.input_features is None:
            raise InvalidInput("WhisperModel takes audio inputs (log-mel features)")
        c = self._config
        enc = self.encode(inputs.input_features)
        dec = inputs.decoder_input_ids
        if dec is None:
            dec = torch.full((enc.shape[0], 1), c.decoder_start_token_id, dtype=torch.long, device=enc.device)
        return ModelOutputs.sequence(self.decode(dec, enc), encoder_hidden_states=enc)

    def transcribe(self, mel: torch.Tensor, max_new_tokens: int = 64, prompt_ids: Optional[List[int]] = None) -> List[int]:
        """Greedy decoding of one utterance; returns token ids without the start tokens and without EOS."""
        c = self._config
        enc = self.encode(mel)
        cache = [dict() for _ in range(c.decoder_layers)]
        feed = list(prompt_ids) if prompt_ids else [c.decoder_start_token_id]
        out: List[int] = []
        for _ in range(min(max_new_tokens, c.max_target_positions - len(feed))):
            logits = self.decode(torch.tensor([feed], device=enc.device), enc, cache)
            tok = int(logits[0, -1].argmax())
            if tok == c.eos_token_id:
                break
            out.append(tok)
            feed = [tok]
        return out

    def generate(self, prompt, config=None):
        return f"[Whisper: use transcribe() with audio input; max tokens {(config.max_new_tokens if config else 448)}]"


MODELS = {"t5": T5Model, "whisper": WhisperModel}
