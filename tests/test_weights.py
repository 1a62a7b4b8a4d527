"""Loaders on synthetic files: SafeTensors / PyTorch / GGUF round trips, name map, config discovery."""
import json
import os

import pytest
import torch

from unillm_b200.model_core import ModelInputs
from unillm_b200.models import configs as C
from unillm_b200.models.families import LlamaModel
from unillm_b200.weights import (ConfigLoader, ModelLoader, UnifiedWeightLoader, dequantize_blocks, gguf_to_hf_name,
                                 quantize_blocks, read_gguf, read_safetensors, write_gguf, write_safetensors)
from unillm_b200.weights import gguf as G


def _tiny():
    cfg = C.LlamaConfig(vocab_size=64, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                        num_attention_heads=4, num_key_value_heads=2)
    return cfg, LlamaModel.new(cfg, init="random", seed=3)


def test_safetensors_roundtrip_and_model_load(tmp_path):
    cfg, m = _tiny()
    w = m.export_hf()
    d = tmp_path / "model"
    d.mkdir()
    names = w.tensor_names()
    write_safetensors(str(d / "model-00001-of-00002.safetensors"), {n: w.tensors[n] for n in names[::2]}, {"architecture": "LlamaConfig"})
    write_safetensors(str(d / "model-00002-of-00002.safetensors"), {n: w.tensors[n].to(torch.bfloat16) for n in names[1::2]})
    (d / "config.json").write_text(json.dumps({"architectures": ["LlamaForCausalLM"], **cfg.to_dict()}))
    t, meta = read_safetensors(str(d / "model-00001-of-00002.safetensors"))
    assert meta["architecture"] == "LlamaConfig" and torch.equal(t[names[0]], w.tensors[names[0]])
    u = UnifiedWeightLoader()
    assert u.detect_format(str(d)) == "SafeTensors" and u.supported_formats() == ["SafeTensors", "PyTorch", "GGUF"]
    m2 = ModelLoader().load_model(str(d))
    ids = torch.randint(0, 64, (1, 9))
    a, b = m.forward(ModelInputs.text(ids)).main_tensor(), m2.forward(ModelInputs.text(ids)).main_tensor()
    assert (a - b).abs().max() < 0.05      # half of the tensors went through bf16
    assert ConfigLoader.get_architecture(ConfigLoader.load_config(str(d))) == "LlamaForCausalLM"


def test_pytorch_checkpoint_load(tmp_path):
    cfg, m = _tiny()
    p = tmp_path / "pytorch_model.bin"
    torch.save({"state_dict": dict(m.export_hf().tensors)}, str(p))
    w = UnifiedWeightLoader().load_weights(str(p))
    assert w.metadata.format == "PyTorch" and len(w) == len(m.export_hf())
    m2 = LlamaModel.from_weights(cfg, w)
    ids = torch.randint(0, 64, (2, 5))
    assert torch.allclose(m.forward(ModelInputs.text(ids)).main_tensor(), m2.forward(ModelInputs.text(ids)).main_tensor())


@pytest.mark.parametrize("qt,tol", [(G.F16, 1e-3), (G.Q8_0, 0.02), (G.Q4_0, 0.2), (G.BF16, 1e-2)])
def test_block_quant_roundtrip(qt, tol):
    x = torch.randn(4, 64)
    y = dequantize_blocks(quantize_blocks(x, qt), qt, x.shape)
    assert (x - y).abs().max() < tol * x.abs().max()


def test_q4k_q6k_dequant_against_scalar_definition():
    import numpy as np

    rng = np.random.default_rng(0)
    # Q4_K: one block, compare with a literal scalar transcription of the format definition
    blk = rng.integers(0, 256, size=144, dtype=np.uint8)
    blk[0:2] = np.float16(0.01).view(np.uint8) if False else np.frombuffer(np.float16(0.01).tobytes(), dtype=np.uint8)
    blk[2:4] = np.frombuffer(np.float16(0.02).tobytes(), dtype=np.uint8)
    got = dequantize_blocks(blk, G.Q4_K, (256,)).numpy()
    d, dmin, sc, qs = 0.01, 0.02, blk[4:16], blk[16:]
    d, dmin = float(np.float16(d)), float(np.float16(dmin))
    ref = np.zeros(256, dtype=np.float32)
    for j in range(8):
        if j < 4:
            s, m = sc[j] & 63, sc[j + 4] & 63
        else:
            s = (sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4)
            m = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4)
        g, hi = j // 2, j % 2
        for l in range(32):
            q = (qs[g * 32 + l] >> 4) if hi else (qs[g * 32 + l] & 0xF)
            ref[g * 64 + hi * 32 + l] = d * s * q - dmin * m
    assert np.allclose(got, ref, atol=1e-6)
    blk6 = rng.integers(0, 256, size=210, dtype=np.uint8)
    blk6[208:210] = np.frombuffer(np.float16(0.05).tobytes(), dtype=np.uint8)
    got6 = dequantize_blocks(blk6, G.Q6_K, (256,)).numpy()
    ql, qh, sc6, d6 = blk6[:128], blk6[128:192], blk6[192:208].view(np.int8), float(np.float16(0.05))
    ref6 = np.zeros(256, dtype=np.float32)
    for half in range(2):
        for l in range(32):
            i_s = l // 16
            L, Hh, S = ql[half * 64:], qh[half * 32:], sc6[half * 8:]
            q1 = int((L[l] & 0xF) | ((Hh[l] & 3) << 4)) - 32
            q2 = int((L[l + 32] & 0xF) | (((Hh[l] >> 2) & 3) << 4)) - 32
            q3 = int((L[l] >> 4) | (((Hh[l] >> 4) & 3) << 4)) - 32
            q4 = int((L[l + 32] >> 4) | (((Hh[l] >> 6) & 3) << 4)) - 32
            b = half * 128
            ref6[b + l] = d6 * S[i_s] * q1
            ref6[b + 32 + l] = d6 * S[i_s + 2] * q2
            ref6[b + 64 + l] = d6 * S[i_s + 4] * q3
            ref6[b + 96 + l] = d6 * S[i_s + 6] * q4
    assert np.allclose(got6, ref6, atol=1e-6)


def test_gguf_file_roundtrip_name_map_and_model(tmp_path):
    cfg, m = _tiny()
    w = m.export_hf().tensors
    inv = {"model.embed_tokens.weight": "token_embd.weight", "model.norm.weight": "output_norm.weight",
           "lm_head.weight": "output.weight"}
    per = {"self_attn.q_proj": "attn_q", "self_attn.k_proj": "attn_k", "self_attn.v_proj": "attn_v",
           "self_attn.o_proj": "attn_output", "mlp.gate_proj": "ffn_gate", "mlp.up_proj": "ffn_up",
           "mlp.down_proj": "ffn_down", "input_layernorm": "attn_norm", "post_attention_layernorm": "ffn_norm"}
    tensors = {}
    for name, t in w.items():
        if name in inv:
            g = inv[name]
        else:
            parts = name.split(".")
            g = f"blk.{parts[2]}.{per['.'.join(parts[3:-1])]}.weight"
        if ".attn_q." in g or ".attn_k." in g:        # store in llama.cpp's rotary row order
            nh = 4 if ".attn_q." in g else 2
            hd = t.shape[0] // nh
            t = t.reshape(nh, 2, hd // 2, -1).transpose(1, 2).reshape(t.shape)
        tensors[g] = (t, G.Q8_0 if t.dim() == 2 and "norm" not in g else G.F32)
    md = {"general.architecture": "llama", "llama.embedding_length": 64, "llama.feed_forward_length": 128,
          "llama.block_count": 2, "llama.attention.head_count": 4, "llama.attention.head_count_kv": 2,
          "llama.attention.layer_norm_rms_epsilon": 1e-6, "llama.rope.freq_base": 10000.0, "llama.context_length": 128,
          "tokenizer.ggml.tokens": [f"<t{i}>" for i in range(64)], "tokenizer.ggml.scores": [0.0] * 64,
          "tokenizer.ggml.bos_token_id": 1, "tokenizer.ggml.eos_token_id": 2}
    p = str(tmp_path / "tiny.gguf")
    write_gguf(p, md, tensors)
    gf = read_gguf(p)
    assert gf.metadata["llama.block_count"] == 2 and len(gf.tensors) == len(tensors)
    assert gguf_to_hf_name("blk.3.attn_output.weight") == "model.layers.3.self_attn.o_proj.weight"
    assert gguf_to_hf_name("output.weight") == "lm_head.weight"
    mw = UnifiedWeightLoader().load_weights(p)
    assert mw.metadata.format == "GGUF" and mw.gguf_config.num_key_value_heads == 2 and mw.gguf_tokenizer.vocab_size() == 64
    assert mw.has_quantized("model.layers.0.mlp.down_proj.weight")
    m2 = ModelLoader().load_model(p)
    ids = torch.randint(0, 64, (1, 7))
    a, b = m.forward(ModelInputs.text(ids)).main_tensor(), m2.forward(ModelInputs.text(ids)).main_tensor()
    assert (a - b).abs().max() < 0.05
    assert m2.tokenizer().vocab_size() == 64
