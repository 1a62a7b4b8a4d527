"""GGUF container: reader, (test) writer, block dequantisation, metadata extraction and the GGUF -> HF
tensor-name map.

Reference behaviour (``crates/runtime/src/weight_loader_core.rs``): metadata -> ``GGUFModelConfig`` with
``{arch}.*`` keys falling back to ``llama.*`` and to defaults (``:19-98``), ``tokenizer.ggml.*`` ->
``GGUFTokenizer`` (``:102-160``), ``*_proj.weight`` and ``lm_head.weight`` stay quantised while everything
else is dequantised to f32 (``:554-584``), names rewritten by ``gguf_to_hf_name`` (``:760-798``).
The reference delegates parsing and dequantisation to Candle; here the container is parsed directly
and the block formats are implemented to the ggml definitions (Q4_0, Q4_1, Q5_0, Q8_0, Q4_K, Q6_K, F16,
BF16, F32) in vectorised torch (host) -- the device kernels in ``csrc/quant`` and the C++ scalar oracle
in ``csrc/quant/quant_ref.cpp`` implement the same formats and are tested against this module.
Q4_0 uses ggml's nibble order (low nibbles = elements 0..15, high = 16..31), not the even/odd order of
the reference's own SIMD block type (``simd/quant/block.rs:27-61``), which would mis-read real files.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field
from typing import Any, BinaryIO, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..types import LoadingError

GGUF_MAGIC = 0x46554747
# ggml tensor types
F32, F16, Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q4_K, Q6_K, BF16 = 0, 1, 2, 3, 6, 7, 8, 12, 14, 30
TYPE_NAMES = {F32: "F32", F16: "F16", Q4_0: "Q4_0", Q4_1: "Q4_1", Q5_0: "Q5_0", Q8_0: "Q8_0", Q4_K: "Q4_K",
              Q6_K: "Q6_K", BF16: "BF16"}
# (elements per block, bytes per block)
BLOCK = {F32: (1, 4), F16: (1, 2), BF16: (1, 2), Q4_0: (32, 18), Q4_1: (32, 20), Q5_0: (32, 22), Q8_0: (32, 34),
         Q4_K: (256, 144), Q6_K: (256, 210)}

_VT_U8, _VT_I8, _VT_U16, _VT_I16, _VT_U32, _VT_I32, _VT_F32, _VT_BOOL, _VT_STR, _VT_ARR, _VT_U64, _VT_I64, _VT_F64 = range(13)
_SCALAR = {_VT_U8: "<B", _VT_I8: "<b", _VT_U16: "<H", _VT_I16: "<h", _VT_U32: "<I", _VT_I32: "<i", _VT_F32: "<f",
           _VT_BOOL: "<?", _VT_U64: "<Q", _VT_I64: "<q", _VT_F64: "<d"}


@dataclass
class GGUFTensorInfo:
    name: str
    shape: Tuple[int, ...]       # logical shape, outermost first (ggml stores innermost first)
    qtype: int
    offset: int                  # from the start of the data section


@dataclass
class GGUFFile:
    metadata: Dict[str, Any]
    tensors: Dict[str, GGUFTensorInfo]
    data_offset: int
    path: str

    def raw(self, name: str) -> np.ndarray:
        """Raw bytes of one tensor (memory-mapped)."""
        ti = self.tensors[name]
        n = int(np.prod(ti.shape))
        epb, bpb = BLOCK[ti.qtype]
        nbytes = n // epb * bpb
        mm = np.memmap(self.path, dtype=np.uint8, mode="r", offset=self.data_offset + ti.offset, shape=(nbytes,))
        return mm


def _read_str(f: BinaryIO) -> str:
    (n,) = struct.unpack("<Q", f.read(8))
    return f.read(n).decode("utf-8", errors="replace")


def _read_value(f: BinaryIO, vt: int):
    if vt in _SCALAR:
        fmt = _SCALAR[vt]
        return struct.unpack(fmt, f.read(struct.calcsize(fmt)))[0]
    if vt == _VT_STR:
        return _read_str(f)
    if vt == _VT_ARR:
        (et,) = struct.unpack("<I", f.read(4))
        (n,) = struct.unpack("<Q", f.read(8))
        if et in _SCALAR and et != _VT_BOOL:
            fmt = _SCALAR[et]
            sz = struct.calcsize(fmt)
            return np.frombuffer(f.read(sz * n), dtype=np.dtype(fmt)).tolist()
        return [_read_value(f, et) for _ in range(n)]
    raise LoadingError(f"unknown GGUF value type {vt}")


def read_gguf(path: str) -> GGUFFile:
    with open(path, "rb") as f:
        magic, version = struct.unpack("<II", f.read(8))
        if magic != GGUF_MAGIC:
            raise LoadingError(f"{path}: not a GGUF file")
        if version < 2:
            raise LoadingError(f"{path}: GGUF version {version} is not supported")
        n_tensors, n_kv = struct.unpack("<QQ", f.read(16))
        meta: Dict[str, Any] = {}
        for _ in range(n_kv):
            key = _read_str(f)
            (vt,) = struct.unpack("<I", f.read(4))
            meta[key] = _read_value(f, vt)
        infos: Dict[str, GGUFTensorInfo] = {}
        for _ in range(n_tensors):
            name = _read_str(f)
            (nd,) = struct.unpack("<I", f.read(4))
            dims = struct.unpack("<" + "Q" * nd, f.read(8 * nd))
            qtype, off = struct.unpack("<IQ", f.read(12))
            if qtype not in BLOCK:
                raise LoadingError(f"{path}: tensor {name} has unsupported ggml type {qtype}")
            infos[name] = GGUFTensorInfo(name, tuple(reversed(dims)), qtype, off)
        align = int(meta.get("general.alignment", 32))
        pos = f.tell()
        data_offset = (pos + align - 1) // align * align
    return GGUFFile(meta, infos, data_offset, path)


# ------------------------------------------------------------------------------------------------
# block formats
# ------------------------------------------------------------------------------------------------
def _f16(b: np.ndarray) -> np.ndarray:
    return b.view(np.float16).astype(np.float32)


def dequantize_blocks(data, qtype: int, shape: Sequence[int]) -> torch.Tensor:
    """Raw block bytes -> float32 tensor of ``shape``."""
    raw = data.cpu().numpy() if isinstance(data, torch.Tensor) else np.asarray(data)
    raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
    n = int(np.prod(shape))
    if qtype == F32:
        return torch.from_numpy(raw.view(np.float32)[:n].copy()).reshape(*shape)
    if qtype == F16:
        return torch.from_numpy(raw.view(np.float16)[:n].astype(np.float32)).reshape(*shape)
    if qtype == BF16:
        return torch.from_numpy(raw.view(np.int16)[:n].copy()).view(torch.bfloat16).float().reshape(*shape)
    epb, bpb = BLOCK[qtype]
    nb = n // epb
    blk = raw[: nb * bpb].reshape(nb, bpb)
    if qtype == Q4_0:
        d = _f16(blk[:, 0:2].copy()).reshape(nb, 1)
        qs = blk[:, 2:18]
        lo, hi = (qs & 0x0F).astype(np.int8) - 8, (qs >> 4).astype(np.int8) - 8
        out = np.concatenate([lo, hi], axis=1).astype(np.float32) * d
    elif qtype == Q4_1:
        d = _f16(blk[:, 0:2].copy()).reshape(nb, 1)
        m = _f16(blk[:, 2:4].copy()).reshape(nb, 1)
        qs = blk[:, 4:20]
        out = np.concatenate([qs & 0x0F, qs >> 4], axis=1).astype(np.float32) * d + m
    elif qtype == Q5_0:
        d = _f16(blk[:, 0:2].copy()).reshape(nb, 1)
        qh = blk[:, 2:6].copy().view(np.uint32).reshape(nb, 1)
        qs = blk[:, 6:22]
        j = np.arange(16, dtype=np.uint32)[None]
        xh0 = ((qh >> j) & 1).astype(np.uint8) << 4
        xh1 = ((qh >> (j + 16)) & 1).astype(np.uint8) << 4
        lo = ((qs & 0x0F) | xh0).astype(np.int16) - 16
        hi = ((qs >> 4) | xh1).astype(np.int16) - 16
        out = np.concatenate([lo, hi], axis=1).astype(np.float32) * d
    elif qtype == Q8_0:
        d = _f16(blk[:, 0:2].copy()).reshape(nb, 1)
        out = blk[:, 2:34].view(np.int8).astype(np.float32) * d
    elif qtype == Q4_K:
        d = _f16(blk[:, 0:2].copy()).reshape(nb, 1)
        dmin = _f16(blk[:, 2:4].copy()).reshape(nb, 1)
        sc = blk[:, 4:16].astype(np.uint8)
        qs = blk[:, 16:144]
        scales = np.empty((nb, 8), dtype=np.float32)
        mins = np.empty((nb, 8), dtype=np.float32)
        for j in range(8):
            if j < 4:
                s, m = sc[:, j] & 63, sc[:, j + 4] & 63
            else:
                s = (sc[:, j + 4] & 0x0F) | ((sc[:, j - 4] >> 6) << 4)
                m = (sc[:, j + 4] >> 4) | ((sc[:, j] >> 6) << 4)
            scales[:, j], mins[:, j] = s, m
        out = np.empty((nb, 256), dtype=np.float32)
        for g in range(4):                      # 64 values per group: low nibbles then high nibbles of 32 bytes
            q = qs[:, g * 32:(g + 1) * 32]
            out[:, g * 64:g * 64 + 32] = d * scales[:, 2 * g:2 * g + 1] * (q & 0x0F) - dmin * mins[:, 2 * g:2 * g + 1]
            out[:, g * 64 + 32:g * 64 + 64] = d * scales[:, 2 * g + 1:2 * g + 2] * (q >> 4) - dmin * mins[:, 2 * g + 1:2 * g + 2]
    elif qtype == Q6_K:
        ql, qh = blk[:, 0:128], blk[:, 128:192]
        sc = blk[:, 192:208].view(np.int8).astype(np.float32)
        d = _f16(blk[:, 208:210].copy()).reshape(nb, 1)
        out = np.empty((nb, 256), dtype=np.float32)
        for half in range(2):
            l_ = ql[:, half * 64:(half + 1) * 64]
            h_ = qh[:, half * 32:(half + 1) * 32]
            s_ = sc[:, half * 8:(half + 1) * 8]
            q1 = ((l_[:, :32] & 0x0F) | ((h_ & 3) << 4)).astype(np.int8) - 32
            q2 = ((l_[:, 32:] & 0x0F) | (((h_ >> 2) & 3) << 4)).astype(np.int8) - 32
            q3 = ((l_[:, :32] >> 4) | (((h_ >> 4) & 3) << 4)).astype(np.int8) - 32
            q4 = ((l_[:, 32:] >> 4) | (((h_ >> 6) & 3) << 4)).astype(np.int8) - 32
            idx = np.arange(32) // 16
            base = half * 128
            out[:, base + 0:base + 32] = d * s_[:, idx + 0] * q1
            out[:, base + 32:base + 64] = d * s_[:, idx + 2] * q2
            out[:, base + 64:base + 96] = d * s_[:, idx + 4] * q3
            out[:, base + 96:base + 128] = d * s_[:, idx + 6] * q4
    else:
        raise LoadingError(f"dequantisation of ggml type {qtype} is not implemented")
    return torch.from_numpy(out.reshape(-1)[:n].copy()).reshape(*shape)


def quantize_blocks(x: torch.Tensor, qtype: int) -> np.ndarray:
    """float tensor -> raw block bytes (Q4_0, Q8_0, Q4_K, F16, F32, BF16): used to write test files and to quantise
    weights for the block-quantised serving mode."""
    a = x.detach().float().cpu().numpy().reshape(-1)
    if qtype == F32:
        return a.astype(np.float32).view(np.uint8)
    if qtype == F16:
        return a.astype(np.float16).view(np.uint8)
    if qtype == BF16:
        return x.detach().to(torch.bfloat16).cpu().view(torch.int16).numpy().reshape(-1).view(np.uint8)
    nb = a.size // 32
    b = a[: nb * 32].reshape(nb, 32)
    if qtype == Q8_0:
        amax = np.abs(b).max(axis=1, keepdims=True)
        d = amax / 127.0
        inv = np.where(d > 0, 1.0 / np.maximum(d, 1e-30), 0.0)
        q = np.clip(np.rint(b * inv), -127, 127).astype(np.int8)
        out = np.empty((nb, 34), dtype=np.uint8)
        out[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(nb, 2)
        out[:, 2:] = q.view(np.uint8)
        return out.reshape(-1)
    if qtype == Q4_0:
        idx = np.abs(b).argmax(axis=1)
        mx = b[np.arange(nb), idx].reshape(nb, 1)
        d = mx / -8.0
        inv = np.where(d != 0, 1.0 / np.where(d == 0, 1, d), 0.0)
        q = np.clip(np.floor(b * inv + 8.5), 0, 15).astype(np.uint8)
        out = np.empty((nb, 18), dtype=np.uint8)
        out[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(nb, 2)
        out[:, 2:] = q[:, :16] | (q[:, 16:] << 4)
        return out.reshape(-1)
    if qtype == Q4_K:
        if a.size % 256:
            raise LoadingError("Q4_K quantisation needs a multiple of 256 elements")
        nb = a.size // 256
        b = a.reshape(nb, 8, 32)
        # per 32-value sub-block: value = scale * q - min with q in 0..15 (min >= 0 as ggml stores it)
        lo = np.minimum(b.min(axis=2), 0.0)
        hi = b.max(axis=2)
        sub_scale = (hi - lo) / 15.0
        sub_min = -lo
        d = sub_scale.max(axis=1, keepdims=True) / 63.0
        dmin = sub_min.max(axis=1, keepdims=True) / 63.0
        d16, dmin16 = d.astype(np.float16), dmin.astype(np.float16)
        df, dminf = d16.astype(np.float32), dmin16.astype(np.float32)
        sc = np.where(df > 0, np.rint(sub_scale / np.where(df > 0, df, 1)), 0).clip(0, 63).astype(np.uint8)
        mn = np.where(dminf > 0, np.rint(sub_min / np.where(dminf > 0, dminf, 1)), 0).clip(0, 63).astype(np.uint8)
        eff_s = df * sc.astype(np.float32)
        eff_m = dminf * mn.astype(np.float32)
        q = np.where(eff_s[..., None] > 0, np.rint((b + eff_m[..., None]) / np.where(eff_s[..., None] > 0, eff_s[..., None], 1)), 0)
        q = q.clip(0, 15).astype(np.uint8)
        out = np.zeros((nb, 144), dtype=np.uint8)
        out[:, 0:2] = d16.view(np.uint8).reshape(nb, 2)
        out[:, 2:4] = dmin16.view(np.uint8).reshape(nb, 2)
        for j in range(4):                       # 6-bit scales / mins packed as ggml's get_scale_min_k4 reads them
            out[:, 4 + j] = (sc[:, j] & 63) | ((sc[:, j + 4] >> 4) << 6)
            out[:, 8 + j] = (mn[:, j] & 63) | ((mn[:, j + 4] >> 4) << 6)
            out[:, 12 + j] = (sc[:, j + 4] & 0x0F) | ((mn[:, j + 4] & 0x0F) << 4)
        for g in range(4):                       # 64 values per group: low nibbles = first 32, high nibbles = next 32
            out[:, 16 + g * 32:16 + (g + 1) * 32] = q[:, 2 * g] | (q[:, 2 * g + 1] << 4)
        return out.reshape(-1)
    raise LoadingError(f"quantisation to ggml type {qtype} is not implemented")


def write_gguf(path: str, metadata: Dict[str, Any], tensors: Dict[str, Tuple[torch.Tensor, int]], alignment: int = 32):
    """Minimal GGUF v3 writer (tests, export).  ``tensors``: name -> (float tensor, ggml type)."""
    def w_str(f, s):
        b = s.encode("utf-8")
        f.write(struct.pack("<Q", len(b)))
        f.write(b)

    def w_val(f, v):
        if isinstance(v, bool):
            f.write(struct.pack("<I?", _VT_BOOL, v))
        elif isinstance(v, int):
            f.write(struct.pack("<II", _VT_U32, v) if 0 <= v < 2 ** 32 else struct.pack("<Iq", _VT_I64, v))
        elif isinstance(v, float):
            f.write(struct.pack("<If", _VT_F32, v))
        elif isinstance(v, str):
            f.write(struct.pack("<I", _VT_STR))
            w_str(f, v)
        elif isinstance(v, (list, tuple)):
            f.write(struct.pack("<I", _VT_ARR))
            if v and isinstance(v[0], str):
                f.write(struct.pack("<IQ", _VT_STR, len(v)))
                for s in v:
                    w_str(f, s)
            elif v and isinstance(v[0], float):
                f.write(struct.pack("<IQ", _VT_F32, len(v)))
                f.write(np.asarray(v, dtype=np.float32).tobytes())
            else:
                f.write(struct.pack("<IQ", _VT_I32, len(v)))
                f.write(np.asarray(v, dtype=np.int32).tobytes())
        else:
            raise LoadingError(f"cannot write GGUF value {type(v)}")

    blobs, infos, off = [], [], 0
    for name, (t, qt) in tensors.items():
        raw = quantize_blocks(t, qt)
        infos.append((name, tuple(t.shape), qt, off))
        blobs.append(raw)
        off = (off + raw.size + alignment - 1) // alignment * alignment
    with open(path, "wb") as f:
        f.write(struct.pack("<IIQQ", GGUF_MAGIC, 3, len(tensors), len(metadata)))
        for k, v in metadata.items():
            w_str(f, k)
            w_val(f, v)
        for name, shape, qt, o in infos:
            w_str(f, name)
            f.write(struct.pack("<I", len(shape)))
            f.write(struct.pack("<" + "Q" * len(shape), *reversed(shape)))
            f.write(struct.pack("<IQ", qt, o))
        pos = f.tell()
        f.write(b"\0" * ((pos + alignment - 1) // alignment * alignment - pos))
        base = f.tell()
        for (name, shape, qt, o), raw in zip(infos, blobs):
            f.seek(base + o)
            f.write(raw.tobytes())


# ------------------------------------------------------------------------------------------------
# metadata -> config / tokenizer; name map
# ------------------------------------------------------------------------------------------------
@dataclass
class GGUFModelConfig:
    architecture: str = "llama"
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 32
    head_dim: int = 128
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    max_position_embeddings: int = 2048

    @staticmethod
    def from_gguf_metadata(md: Dict[str, Any]) -> "GGUFModelConfig":
        arch = md.get("general.architecture", "llama")

        def get(key, default):
            v = md.get(f"{arch}.{key}", md.get(f"llama.{key}"))
            return default if v is None else v

        vocab = md.get(f"{arch}.vocab_size", md.get("llama.vocab_size"))
        if vocab is None:
            vocab = len(md["tokenizer.ggml.tokens"]) if "tokenizer.ggml.tokens" in md else 32000
        hidden = int(get("embedding_length", 4096))
        heads = int(get("attention.head_count", 32))
        return GGUFModelConfig(
            architecture=arch, vocab_size=int(vocab), hidden_size=hidden,
            intermediate_size=int(get("feed_forward_length", 11008)), num_hidden_layers=int(get("block_count", 32)),
            num_attention_heads=heads, num_key_value_heads=int(get("attention.head_count_kv", heads)),
            head_dim=hidden // heads, rms_norm_eps=float(get("attention.layer_norm_rms_epsilon", 1e-5)),
            rope_theta=float(get("rope.freq_base", 10000.0)), max_position_embeddings=int(get("context_length", 2048)))


@dataclass
class GGUFTokenizer:
    tokens: List[str]
    token_types: Optional[List[int]] = None
    scores: Optional[List[float]] = None
    model_type: str = "llama"
    bos_token_id: int = 1
    eos_token_id: int = 2
    unknown_token_id: int = 0
    padding_token_id: Optional[int] = None

    @staticmethod
    def from_gguf_metadata(md: Dict[str, Any]) -> Optional["GGUFTokenizer"]:
        toks = md.get("tokenizer.ggml.tokens")
        if not toks:
            return None
        return GGUFTokenizer(
            tokens=list(toks), token_types=md.get("tokenizer.ggml.token_type"), scores=md.get("tokenizer.ggml.scores"),
            model_type=md.get("tokenizer.ggml.model", "llama"), bos_token_id=int(md.get("tokenizer.ggml.bos_token_id", 1)),
            eos_token_id=int(md.get("tokenizer.ggml.eos_token_id", 2)),
            unknown_token_id=int(md.get("tokenizer.ggml.unknown_token_id", 0)),
            padding_token_id=md.get("tokenizer.ggml.padding_token_id"))

    def vocab_size(self) -> int:
        return len(self.tokens)


_RENAMES = (
    ("token_embd.weight", "model.embed_tokens.weight"), ("blk.", "model.layers."),
    (".attn_output.weight", ".self_attn.o_proj.weight"), (".attn_q.weight", ".self_attn.q_proj.weight"),
    (".attn_k.weight", ".self_attn.k_proj.weight"), (".attn_v.weight", ".self_attn.v_proj.weight"),
    (".attn_output.bias", ".self_attn.o_proj.bias"), (".attn_q.bias", ".self_attn.q_proj.bias"),
    (".attn_k.bias", ".self_attn.k_proj.bias"), (".attn_v.bias", ".self_attn.v_proj.bias"),
    ("output_norm.weight", "model.norm.weight"), ("output.weight", "lm_head.weight"),
    (".ffn_gate_inp.weight", ".block_sparse_moe.gate.weight"),
    (".ffn_gate.weight", ".mlp.gate_proj.weight"), (".ffn_up.weight", ".mlp.up_proj.weight"),
    (".ffn_down.weight", ".mlp.down_proj.weight"), (".ffn_gate.bias", ".mlp.gate_proj.bias"),
    (".ffn_up.bias", ".mlp.up_proj.bias"), (".ffn_down.bias", ".mlp.down_proj.bias"),
    (".attn_norm.weight", ".input_layernorm.weight"), (".ffn_norm.weight", ".post_attention_layernorm.weight"),
    (".attn_norm.bias", ".input_layernorm.bias"), (".ffn_norm.bias", ".post_attention_layernorm.bias"),
)


def gguf_to_hf_name(name: str) -> str:
    """Same ordered replacement table as the reference (more specific patterns first)."""
    for a, b in _RENAMES:
        name = name.replace(a, b)
    return name


def unpermute_rope_rows(w: torch.Tensor, n_heads: int) -> torch.Tensor:
    """llama.cpp stores q/k projection rows in interleaved-rotary order; HF (and this framework) use the
    half-split order.  Inverse of the conversion script's permutation."""
    rows, cols = w.shape
    hd = rows // n_heads
    return w.reshape(n_heads, hd // 2, 2, cols).transpose(1, 2).reshape(rows, cols)
