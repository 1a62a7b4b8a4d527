"""Audio families: Wav2Vec2, HuBERT (speech encoders with a CTC head), MusicGen (codebook language model) and
EnCodec (neural codec).

Wav2Vec2 (``models_v2/wav2vec2.rs:184-215``): a 7-layer conv1d feature extractor (kernels 10,3,3,3,3,2,2, strides
5,2,2,2,2,2,2, GELU; group norm on the first layer) -> LayerNorm + projection -> convolutional position embedding
-> post-LN transformer encoder -> ``lm_head``.  HuBERT shares the architecture (the reference runs only its
transformer, ``hubert.rs``); both take ``ModelInputs.audio`` with raw waveforms ``[B, samples]``.

MusicGen (``models_v2/musicgen.rs:108-126``): a decoder over 4 codebooks; the input embedding is the sum of the
per-codebook embeddings and there is one head per codebook (the reference uses codebook 0 only).  Inputs are
``[B, K, T]`` codes (or ``[B, T]`` for codebook 0); the output logits are ``[B, K, T, vocab]`` (``[B, T, vocab]``).

EnCodec (``models_v2/encodec.rs:108-217``): SEANet encoder (conv_in, 4 down blocks with ratios 8,5,4,2 and ELU
residual units, conv_out) -> 2-layer LSTM with skip -> residual vector quantiser (32 codebooks of 1024 x 128) ->
mirrored decoder with transposed convolutions.  ``encode`` / ``decode`` / ``forward`` (reconstruction) work from
loaded or random weights; the reference loads none (``:131-135``).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn.functional as F

from ..model_core import ModelInputs, ModelOutputs
from ..tensor_core import ops_fn
from ..types import InvalidInput, UnsupportedOperation
from . import configs as C
from .simple import ParamModel, _f, conv1d, conv_transpose1d, mha


class Wav2Vec2Model(ParamModel):
    config_class = C.Wav2Vec2Config
    root = "wav2vec2."
    POS_KERNEL, POS_GROUPS = 128, 16

    def param_shapes(self) -> Dict[str, tuple]:
        c, R = self._config, self.root
        H, I = c.hidden_size, c.intermediate_size
        s: Dict[str, tuple] = {}
        cin = 1
        for i, (d, k) in enumerate(zip(c.conv_dim, c.conv_kernel)):
            s[f"{R}feature_extractor.conv_layers.{i}.conv.weight"] = (d, cin, k)
            if i == 0:
                s[f"{R}feature_extractor.conv_layers.0.layer_norm.weight"] = (d,)
                s[f"{R}feature_extractor.conv_layers.0.layer_norm.bias"] = (d,)
            cin = d
        s[R + "feature_projection.layer_norm.weight"], s[R + "feature_projection.layer_norm.bias"] = (cin,), (cin,)
        s[R + "feature_projection.projection.weight"], s[R + "feature_projection.projection.bias"] = (H, cin), (H,)
        pk = min(self.POS_KERNEL, 2 * (H // 8) or 2)
        pg = self.POS_GROUPS if H % self.POS_GROUPS == 0 else 1
        s[R + "encoder.pos_conv_embed.conv.weight"], s[R + "encoder.pos_conv_embed.conv.bias"] = (H, H // pg, pk), (H,)
        s[R + "encoder.layer_norm.weight"], s[R + "encoder.layer_norm.bias"] = (H,), (H,)
        for i in range(c.num_hidden_layers):
            L = f"{R}encoder.layers.{i}."
            for n in ("q_proj", "k_proj", "v_proj", "out_proj"):
                s[L + f"attention.{n}.weight"], s[L + f"attention.{n}.bias"] = (H, H), (H,)
            s[L + "layer_norm.weight"], s[L + "layer_norm.bias"] = (H,), (H,)
            s[L + "feed_forward.intermediate_dense.weight"], s[L + "feed_forward.intermediate_dense.bias"] = (I, H), (I,)
            s[L + "feed_forward.output_dense.weight"], s[L + "feed_forward.output_dense.bias"] = (H, I), (H,)
            s[L + "final_layer_norm.weight"], s[L + "final_layer_norm.bias"] = (H,), (H,)
        s["lm_head.weight"], s["lm_head.bias"] = (c.vocab_size, H), (c.vocab_size,)
        return s

    def aliases(self, name):
        return (name, name[len(self.root):]) if name.startswith(self.root) else (name,)

    def extract_features(self, wav: torch.Tensor) -> torch.Tensor:
        """[B, samples] -> [B, frames, conv_dim[-1]]."""
        c, p, R = self._config, self.p, self.root
        x = wav[:, None].to(self.dtype)
        for i, st in enumerate(c.conv_stride):
            if x.shape[-1] < c.conv_kernel[i]:
                raise InvalidInput("audio too short for the feature extractor")
            x = conv1d(x, p[f"{R}feature_extractor.conv_layers.{i}.conv.weight"], None, stride=st)
            if i == 0:
                d = x.shape[1]
                x = F.group_norm(_f(x), d, _f(p[f"{R}feature_extractor.conv_layers.0.layer_norm.weight"]),
                                 _f(p[f"{R}feature_extractor.conv_layers.0.layer_norm.bias"]), 1e-5).to(x.dtype)
            x = ops_fn.gelu(x)
        return x.transpose(1, 2).contiguous()

    def num_frames(self, samples: int) -> int:
        c = self._config
        for k, s in zip(c.conv_kernel, c.conv_stride):
            samples = (samples - k) // s + 1
        return samples

    def encode(self, wav: torch.Tensor) -> torch.Tensor:
        c, p, R = self._config, self.p, self.root
        eps = c.layer_norm_eps
        x = self.extract_features(wav)
        x = self.lin(self.ln(x, R + "feature_projection.layer_norm", eps), R + "feature_projection.projection")
        w = p[R + "encoder.pos_conv_embed.conv.weight"]
        k = w.shape[-1]
        pos = conv1d(x.transpose(1, 2), w, p[R + "encoder.pos_conv_embed.conv.bias"], padding=k // 2, groups=x.shape[-1] // w.shape[1])
        if k % 2 == 0:
            pos = pos[..., :-1]
        x = x + ops_fn.gelu(pos).transpose(1, 2)
        x = self.ln(x, R + "encoder.layer_norm", eps)
        for i in range(c.num_hidden_layers):
            L = f"{R}encoder.layers.{i}."
            A = L + "attention."
            a = mha(x, x, p[A + "q_proj.weight"], p[A + "q_proj.bias"], p[A + "k_proj.weight"], p[A + "k_proj.bias"],
                    p[A + "v_proj.weight"], p[A + "v_proj.bias"], p[A + "out_proj.weight"], p[A + "out_proj.bias"], c.num_attention_heads)
            x = self.ln(x + a, L + "layer_norm", eps)
            m = self.lin(self.lin(x, L + "feed_forward.intermediate_dense", act="gelu"), L + "feed_forward.output_dense")
            x = self.ln(x + m, L + "final_layer_norm", eps)
        return x

    def forward(self, inputs: ModelInputs) -> ModelOutputs:
        if inputs.input_features is None:
            raise InvalidInput(f"{type(self).__name__} takes audio inputs (raw waveform [B, samples])")
        wav = inputs.input_features
        if wav.dim() == 1:
            wav = wav[None]
        x = self.encode(wav)
        return ModelOutputs.from_logits(self.lin(x, "lm_head"), hidden_states=x)

    def ctc_decode(self, wav: torch.Tensor, blank: int = 0) -> List[List[int]]:
        """Greedy CTC: argmax per frame, collapse repeats, drop blanks."""
        ids = self.forward(ModelInputs.audio(wav)).logits.argmax(-1)
        out = []
        for row in ids.tolist():
            seq, prev = [], None
            for t in row:
                if t != prev and t != blank:
                    seq.append(t)
                prev = t
            out.append(seq)
        return out

    def generate(self, prompt, config=None):
        raise UnsupportedOperation("speech encoders do not generate text from text; use ctc_decode(waveform)")


class HubertModel(Wav2Vec2Model):
    config_class = C.HuBERTConfig
    root = "hubert."


class MusicGenModel(ParamModel):
    config_class = C.MusicGenConfig

    def param_shapes(self) -> Dict[str, tuple]:
        c = self._config
        H, I = c.hidden_size, c.intermediate_size
        s: Dict[str, tuple] = {}
        for k in range(c.num_codebooks):
            s[f"model.decoder.embed_tokens.{k}.weight"] = (c.vocab_size + 1, H)
            s[f"lm_heads.{k}.weight"] = (c.vocab_size, H)
        for i in range(c.num_hidden_layers):
            L = f"model.decoder.layers.{i}."
            for n in ("q_proj", "k_proj", "v_proj", "out_proj"):
                s[L + f"self_attn.{n}.weight"] = (H, H)
            s[L + "self_attn_layer_norm.weight"], s[L + "self_attn_layer_norm.bias"] = (H,), (H,)
            s[L + "fc1.weight"], s[L + "fc2.weight"] = (I, H), (H, I)
            s[L + "final_layer_norm.weight"], s[L + "final_layer_norm.bias"] = (H,), (H,)
        s["model.decoder.final_layer_norm.weight"], s["model.decoder.final_layer_norm.bias"] = (H,), (H,)
        return s

    def _positions(self, T: int, past: int, device) -> torch.Tensor:
        H = self._config.hidden_size
        half = H // 2
        inv = torch.exp(torch.arange(half, dtype=torch.float32, device=device) * -(math.log(10000.0) / max(half - 1, 1)))
        ang = torch.arange(past, past + T, dtype=torch.float32, device=device)[:, None] * inv[None]
        return torch.cat([ang.cos(), ang.sin()], 1)

    def hidden_states(self, codes: torch.Tensor, cache: Optional[List[dict]] = None) -> torch.Tensor:
        c, p = self._config, self.p
        if codes.dim() == 2:
            codes = codes[:, None]
        B, Kc, T = codes.shape
        if Kc > c.num_codebooks:
            raise InvalidInput(f"{Kc} codebooks given, model has {c.num_codebooks}")
        x = sum(ops_fn.embedding(codes[:, k], p[f"model.decoder.embed_tokens.{k}.weight"]) for k in range(Kc))
        past = cache[0]["k"].shape[2] if (cache and cache[0].get("k") is not None) else 0
        x = x + self._positions(T, past, x.device)[None].to(x.dtype)
        for i in range(c.num_hidden_layers):
            L = f"model.decoder.layers.{i}."
            A = L + "self_attn."
            h = self.ln(x, L + "self_attn_layer_norm", c.layer_norm_eps)
            x = x + mha(h, h, p[A + "q_proj.weight"], None, p[A + "k_proj.weight"], None, p[A + "v_proj.weight"], None,
                        p[A + "out_proj.weight"], None, c.num_attention_heads, causal=True,
                        cache=cache[i] if cache is not None else None)
            h = self.ln(x, L + "final_layer_norm", c.layer_norm_eps)
            x = x + ops_fn.linear(ops_fn.linear(h, p[L + "fc1.weight"], act="gelu"), p[L + "fc2.weight"])
        return self.ln(x, "model.decoder.final_layer_norm", c.layer_norm_eps)

    def heads(self, x: torch.Tensor, num: int) -> torch.Tensor:
        return torch.stack([ops_fn.linear(x, self.p[f"lm_heads.{k}.weight"]) for k in range(num)], 1)

    def forward(self, inputs: ModelInputs) -> ModelOutputs:
        if inputs.input_ids is None:
            raise InvalidInput("MusicGenModel takes codebook ids ([B, T] for codebook 0 or [B, K, T])")
        codes = inputs.input_ids
        x = self.hidden_states(codes)
        if codes.dim() == 2:
            return ModelOutputs.from_logits(ops_fn.linear(x, self.p["lm_heads.0.weight"]), hidden_states=x)
        return ModelOutputs.from_logits(self.heads(x, codes.shape[1]), hidden_states=x)

    def new_cache(self, max_seq_len=None):
        return [dict() for _ in range(self._config.num_hidden_layers)]

    def forward_with_cache(self, ids: torch.Tensor, cache=None) -> torch.Tensor:
        if ids.dim() == 1:
            ids = ids[None]
        return ops_fn.linear(self.hidden_states(ids, cache), self.p["lm_heads.0.weight"])

    def generate_codes(self, steps: int, batch: int = 1, seed: int = 0, temperature: float = 1.0, top_k: int = 250) -> torch.Tensor:
        """Samples ``[B, K, steps]`` codes with the delay pattern (codebook k lags k steps behind codebook 0)."""
        c = self._config
        Kc, pad = c.num_codebooks, c.vocab_size
        g = torch.Generator().manual_seed(seed)
        total = steps + Kc - 1
        seq = torch.full((batch, Kc, total + 1), pad, dtype=torch.long)
        cache = self.new_cache()
        for t in range(total):
            x = self.hidden_states(seq[:, :, t:t + 1].to(self.device), cache)
            logits = self.heads(x, Kc)[:, :, 0].float().cpu() / max(temperature, 1e-5)
            if top_k:
                kth = torch.topk(logits, min(top_k, logits.shape[-1]), -1).values[..., -1:]
                logits = logits.masked_fill(logits < kth, float("-inf"))
            nxt = torch.multinomial(torch.softmax(logits, -1).reshape(-1, logits.shape[-1]), 1, generator=g).reshape(batch, Kc)
            for k in range(Kc):
                if k <= t < k + steps:
                    seq[:, k, t + 1] = nxt[:, k]
        return torch.stack([seq[:, k, 1 + k:1 + k + steps] for k in range(Kc)], 1)


class EncodecModel(ParamModel):
    config_class = C.EncodecConfig

    def _plan(self) -> List[Tuple[str, tuple]]:
        """(name, shape) of every convolution, encoder first."""
        c = self._config
        nf, D = c.num_filters, c.hidden_size
        s: List[Tuple[str, tuple]] = [("encoder.conv_in", (nf, c.audio_channels, 7))]
        ch = nf
        for i, r in enumerate(reversed(c.upsampling_ratios)):
            for j in range(c.num_residual_layers):
                s.append((f"encoder.blocks.{i}.res.{j}.conv1", (ch // 2, ch, 3)))
                s.append((f"encoder.blocks.{i}.res.{j}.conv2", (ch, ch // 2, 1)))
            s.append((f"encoder.blocks.{i}.down", (ch * 2, ch, 2 * r)))
            ch *= 2
        s.append(("encoder.conv_out", (D, ch, 7)))
        s.append(("decoder.conv_in", (ch, D, 7)))
        for i, r in enumerate(c.upsampling_ratios):
            s.append((f"decoder.blocks.{i}.up", (ch, ch // 2, 2 * r)))       # ConvTranspose1d: [in, out, k]
            ch //= 2
            for j in range(c.num_residual_layers):
                s.append((f"decoder.blocks.{i}.res.{j}.conv1", (ch // 2, ch, 3)))
                s.append((f"decoder.blocks.{i}.res.{j}.conv2", (ch, ch // 2, 1)))
        s.append(("decoder.conv_out", (c.audio_channels, ch, 7)))
        return s

    def param_shapes(self) -> Dict[str, tuple]:
        c = self._config
        D = c.hidden_size
        s: Dict[str, tuple] = {}
        for name, shape in self._plan():
            s[name + ".weight"] = shape
            s[name + ".bias"] = (shape[1] if name.endswith(".up") else shape[0],)
        for side in ("encoder", "decoder"):
            for l in range(2):
                s[f"{side}.lstm.weight_ih_l{l}"], s[f"{side}.lstm.weight_hh_l{l}"] = (4 * D, D), (4 * D, D)
                s[f"{side}.lstm.bias_ih_l{l}"], s[f"{side}.lstm.bias_hh_l{l}"] = (4 * D,), (4 * D,)
        for q in range(c.num_codebooks):
            s[f"quantizer.layers.{q}.codebook.embed"] = (c.codebook_size, c.codebook_dim)
        return s

    def special_init(self, name, shape, g):
        if name.endswith(".weight") and len(shape) == 3:
            fan = shape[1] * shape[2]
            return torch.randn(shape, generator=g) * (1.0 / fan) ** 0.5
        if name.endswith("codebook.embed"):
            return torch.randn(shape, generator=g)
        if "lstm.weight" in name:
            return torch.randn(shape, generator=g) * shape[1] ** -0.5
        return None

    # causal convolution: all padding on the left
    def _conv(self, x, name, stride=1, dilation=1):
        w = self.p[name + ".weight"]
        pad = (w.shape[-1] - 1) * dilation - (stride - 1)
        x = F.pad(_f(x), (max(pad, 0), 0), mode="reflect" if (self._config.pad_mode == "reflect" and x.shape[-1] > pad) else "constant")
        return conv1d(x, w, self.p[name + ".bias"], stride=stride, dilation=dilation)

    def _convT(self, x, name, stride):
        w = self.p[name + ".weight"]
        y = conv_transpose1d(x, w, self.p[name + ".bias"], stride=stride)
        return y[..., :y.shape[-1] - (w.shape[-1] - stride)]                   # trim the right: causal

    def _res(self, x, pre):
        h = self._conv(F.elu(x), pre + ".conv1")
        return x + self._conv(F.elu(h), pre + ".conv2")

    def _lstm(self, x, side):
        """2-layer LSTM over [B, D, T] with a skip connection."""
        p = self.p
        y = _f(x).transpose(1, 2)
        B, T, D = y.shape
        inp = y
        for l in range(2):
            wi, wh = _f(p[f"{side}.lstm.weight_ih_l{l}"]), _f(p[f"{side}.lstm.weight_hh_l{l}"])
            b = _f(p[f"{side}.lstm.bias_ih_l{l}"]) + _f(p[f"{side}.lstm.bias_hh_l{l}"])
            h = torch.zeros(B, D, device=y.device)
            cst = torch.zeros(B, D, device=y.device)
            pre = inp @ wi.t() + b
            outs = []
            for t in range(T):
                gates = pre[:, t] + h @ wh.t()
                i_, f_, g_, o_ = gates.chunk(4, -1)
                cst = torch.sigmoid(f_) * cst + torch.sigmoid(i_) * torch.tanh(g_)
                h = torch.sigmoid(o_) * torch.tanh(cst)
                outs.append(h)
            inp = torch.stack(outs, 1)
        return (inp + y).transpose(1, 2)

    def hop_length(self) -> int:
        return math.prod(self._config.upsampling_ratios)

    def encode_latent(self, wav: torch.Tensor) -> torch.Tensor:
        """[B, channels, samples] -> continuous latents [B, D, frames]."""
        c = self._config
        if wav.dim() == 2:
            wav = wav[:, None]
        x = self._conv(wav.to(self.dtype), "encoder.conv_in")
        for i, r in enumerate(reversed(c.upsampling_ratios)):
            for j in range(c.num_residual_layers):
                x = self._res(x, f"encoder.blocks.{i}.res.{j}")
            x = self._conv(F.elu(x), f"encoder.blocks.{i}.down", stride=r)
        x = self._lstm(x, "encoder")
        return self._conv(F.elu(x), "encoder.conv_out")

    def num_quantizers(self, bandwidth: Optional[float] = None) -> int:
        c = self._config
        bw = c.bandwidth if bandwidth is None else bandwidth
        frame_rate = c.sample_rate / self.hop_length()
        per_q = math.log2(c.codebook_size) * frame_rate / 1000.0           # kbps per codebook
        return max(1, min(c.num_codebooks, int(bw // per_q) if per_q > 0 else c.num_codebooks))

    def quantize(self, z: torch.Tensor, num_q: Optional[int] = None) -> torch.Tensor:
        """Residual VQ of latents [B, D, T] -> codes [B, Q, T]."""
        nq = num_q or self.num_quantizers()
        r = _f(z).transpose(1, 2)
        codes = []
        for q in range(nq):
            e = _f(self.p[f"quantizer.layers.{q}.codebook.embed"])
            d = (r * r).sum(-1, keepdim=True) - 2 * r @ e.t() + (e * e).sum(-1)[None, None]
            idx = d.argmin(-1)
            codes.append(idx)
            r = r - e[idx]
        return torch.stack(codes, 1)

    def dequantize(self, codes: torch.Tensor) -> torch.Tensor:
        z = sum(_f(self.p[f"quantizer.layers.{q}.codebook.embed"])[codes[:, q]] for q in range(codes.shape[1]))
        return z.transpose(1, 2)

    def encode(self, wav: torch.Tensor, bandwidth: Optional[float] = None) -> torch.Tensor:
        return self.quantize(self.encode_latent(wav), self.num_quantizers(bandwidth))

    def decode(self, codes: torch.Tensor) -> torch.Tensor:
        c = self._config
        x = self._conv(self.dequantize(codes), "decoder.conv_in")
        x = self._lstm(x, "decoder")
        for i, r in enumerate(c.upsampling_ratios):
            x = self._convT(F.elu(x), f"decoder.blocks.{i}.up", r)
            for j in range(c.num_residual_layers):
                x = self._res(x, f"decoder.blocks.{i}.res.{j}")
        return self._conv(F.elu(x), "decoder.conv_out").to(self.dtype)

    def forward(self, inputs: ModelInputs) -> ModelOutputs:
        if inputs.input_features is None:
            raise InvalidInput("EncodecModel takes audio inputs (waveform [B, channels, samples])")
        codes = self.encode(inputs.input_features)
        return ModelOutputs.embeddings(self.decode(codes), pooled=codes)

    def generate(self, prompt, config=None):
        raise UnsupportedOperation("EnCodec is an audio codec; use encode() / decode()")


MODELS = {"wav2vec2": Wav2Vec2Model, "hubert": HubertModel, "musicgen": MusicGenModel, "encodec": EncodecModel}
