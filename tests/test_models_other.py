"""State-space, RWKV, Griffin, encoder, encoder-decoder, vision and audio families: shapes, incremental == full,
weight round trip, registry completeness; recurrence oracles against naive definitions."""
import dataclasses

import pytest
import torch

from unillm_b200.config import GenerationConfig
from unillm_b200.model_core import ModelInputs, registry
from unillm_b200.models import ALL_MODELS, configs as C
from unillm_b200.ops import recurrent as R

REFERENCE_ARCHITECTURES = [
    "llama", "qwen", "gemma", "phi", "deepseek", "mistral", "mixtral", "gpt2", "gptj", "gptneox", "opt", "bloom", "mpt",
    "starcoder", "codellama", "olmo", "granite", "yi", "falcon", "baichuan", "internlm", "chatglm", "bert", "t5", "whisper",
    "clip", "llava", "mamba", "minicpm", "deepseek_moe", "dbrx", "grok", "arctic", "jamba", "rwkv4", "rwkv6",
    "recurrent_gemma", "qwen2_vl", "phi3_vision", "internvl", "cogvlm", "idefics", "florence", "wav2vec2", "hubert",
    "musicgen", "encodec",
]


def test_all_47_architectures_registered():
    assert len(REFERENCE_ARCHITECTURES) == 47
    for a in REFERENCE_ARCHITECTURES:
        assert a in ALL_MODELS, a
        assert registry().supports(a)


STATEFUL = {
    "mamba": C.MambaConfig(vocab_size=97, hidden_size=32, num_hidden_layers=2),
    "jamba": C.JambaConfig(vocab_size=97, hidden_size=32, intermediate_size=48, num_hidden_layers=8, num_attention_heads=4,
                           num_key_value_heads=2, num_experts=4),
    "rwkv4": C.Rwkv4Config(vocab_size=97, hidden_size=32, num_hidden_layers=3, rescale_every=2),
    "rwkv6": C.Rwkv6Config(vocab_size=97, hidden_size=64, num_hidden_layers=2, head_size=32),
    "recurrent_gemma": C.RecurrentGemmaConfig(vocab_size=97, hidden_size=32, num_hidden_layers=4, intermediate_size=48,
                                              num_attention_heads=4, num_key_value_heads=1, head_dim=8, attention_window_size=6,
                                              max_position_embeddings=64),
}


@pytest.mark.parametrize("name", sorted(STATEFUL))
def test_stateful_models_incremental_equals_full(name):
    cls, cfg = ALL_MODELS[name], STATEFUL[name]
    m = cls.new(cfg, init="random", seed=1)
    ids = torch.randint(0, 97, (2, 11), generator=torch.Generator().manual_seed(0))
    y = m.forward(ModelInputs.text(ids)).main_tensor()
    assert y.shape == (2, 11, 97) and torch.isfinite(y).all() and y.std() > 1e-3
    cache = m.new_cache()
    parts = [m.forward_with_cache(ids[:, :6], cache)] + [m.forward_with_cache(ids[:, i:i + 1], cache) for i in range(6, 11)]
    assert (torch.cat(parts, 1) - y).abs().max() < 1e-4
    m2 = cls.from_weights(cfg, m.export_hf())
    assert (m2.forward(ModelInputs.text(ids)).main_tensor() - y).abs().max() == 0
    assert len(m.generate_ids([1, 2, 3], GenerationConfig.greedy(4, eos_token_id=-1))) == 4
    z = cls.new(cfg)
    assert float(z.forward(ModelInputs.text(ids)).main_tensor().abs().max()) == 0.0


def test_jamba_layer_pattern():
    m = ALL_MODELS["jamba"].new(STATEFUL["jamba"])
    assert [m.is_attention_layer(i) for i in range(8)] == [False, False, False, False, True, False, False, False]
    g = ALL_MODELS["recurrent_gemma"].new(STATEFUL["recurrent_gemma"])
    assert [g.is_recurrent_layer(i) for i in range(4)] == [False, True, False, True]


def test_bert_embeddings_and_no_generate():
    from unillm_b200.types import UnsupportedOperation

    cfg = C.BertConfig(vocab_size=97, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                       max_position_embeddings=32)
    m = ALL_MODELS["bert"].new(cfg, init="random", seed=1)
    ids = torch.randint(0, 97, (2, 9))
    o = m.forward(ModelInputs.text(ids))
    assert o.kind == "embeddings" and o.embeddings_.shape == (2, 9, 32) and o.pooled.shape == (2, 32)
    mask = torch.ones(2, 9)
    mask[:, 6:] = 0
    om = m.forward(ModelInputs.text_with_mask(ids, mask))
    short = m.forward(ModelInputs.text(ids[:, :6]))
    assert (om.embeddings_[:, :6] - short.embeddings_).abs().max() < 1e-4
    with pytest.raises(UnsupportedOperation):
        m.generate("x")
    w = m.export_hf()
    legacy = {("bert." + k).replace("LayerNorm.weight", "LayerNorm.gamma").replace("LayerNorm.bias", "LayerNorm.beta"): v
              for k, v in w.tensors.items()}
    from unillm_b200.model_core import ModelWeights

    m2 = ALL_MODELS["bert"].from_weights(cfg, ModelWeights(legacy))
    assert (m2.forward(ModelInputs.text(ids)).embeddings_ - o.embeddings_).abs().max() == 0


def test_t5_cached_decoding_and_buckets():
    from unillm_b200.models.encdec import t5_relative_bucket

    cfg = C.T5Config(vocab_size=97, d_model=32, d_kv=8, d_ff=64, num_layers=2, num_decoder_layers=2, num_heads=4, hidden_size=32)
    m = ALL_MODELS["t5"].new(cfg, init="random", seed=1)
    ids, dec = torch.randint(0, 97, (2, 9)), torch.randint(0, 97, (2, 5))
    inp = ModelInputs.text(ids)
    inp.decoder_input_ids = dec
    o = m.forward(inp)
    assert o.kind == "sequence" and o.logits.shape == (2, 5, 97) and o.encoder_hidden_states.shape == (2, 9, 32)
    enc = m.encode(ids)
    cache = [dict() for _ in range(2)]
    inc = torch.cat([m.decode(dec[:, i:i + 1], enc, cache) for i in range(5)], 1)
    assert (o.logits - inc).abs().max() < 1e-5
    rel = torch.arange(-200, 201)
    b = t5_relative_bucket(rel, True, 32, 128)
    assert b.min() == 0 and b.max() == 31 and b[200] == 0 and b[201] == 17 and b[199] == 1
    bc = t5_relative_bucket(rel, False, 32, 128)
    assert bc[201:].eq(0).all() and bc[0] == 31
    g = cfg.replace(feed_forward_proj="gated-gelu", is_gated_act=True, tie_word_embeddings=False)
    mg = ALL_MODELS["t5"].new(g, init="random", seed=1)
    assert "encoder.block.0.layer.1.DenseReluDense.wi_0.weight" in mg.p and "lm_head.weight" in mg.p
    assert mg.forward(inp).logits.shape == (2, 5, 97)


def test_whisper_transcribe_and_cache():
    cfg = C.WhisperConfig(vocab_size=97, d_model=32, encoder_layers=2, decoder_layers=2, encoder_attention_heads=4,
                          decoder_attention_heads=4, encoder_ffn_dim=64, decoder_ffn_dim=64, max_source_positions=20,
                          max_target_positions=16, num_mel_bins=8, eos_token_id=96, decoder_start_token_id=1, hidden_size=32)
    m = ALL_MODELS["whisper"].new(cfg, init="random", seed=2)
    mel = torch.randn(1, 8, 40)
    o = m.forward(ModelInputs.audio(mel, decoder_input_ids=torch.tensor([[1, 5, 7]])))
    assert o.logits.shape == (1, 3, 97) and o.encoder_hidden_states.shape == (1, 20, 32)
    enc = m.encode(mel)
    cache = [dict() for _ in range(2)]
    inc = torch.cat([m.decode(torch.tensor([[t]]), enc, cache) for t in (1, 5, 7)], 1)
    assert (o.logits - inc).abs().max() < 1e-5
    toks = m.transcribe(mel, 5)
    assert len(toks) <= 5 and all(0 <= t < 97 for t in toks)
    from unillm_b200.types import InvalidInput

    with pytest.raises(InvalidInput):
        m.encode(torch.randn(1, 8, 100))


def test_clip_similarity():
    cfg = C.CLIPConfig(vocab_size=97, hidden_size=32, context_length=12, transformer_width=32, transformer_heads=4,
                       transformer_layers=2, image_resolution=16, vision_layers=2, vision_width=48, vision_heads=4,
                       vision_patch_size=8, projection_dim=24)
    m = ALL_MODELS["clip"].new(cfg, init="random", seed=1)
    o = m.forward(ModelInputs.multimodal(torch.randint(0, 97, (3, 7)), torch.randn(2, 3, 16, 16)))
    assert o.kind == "clip" and o.logits_per_text.shape == (3, 2) and o.logits_per_image.shape == (2, 3)
    assert torch.allclose(o.text_embeds.norm(dim=-1), torch.ones(3), atol=1e-5)
    assert torch.allclose(o.logits_per_text, m.compute_similarity(o.text_embeds, o.image_embeds))
    assert m.vit.patchify(torch.randn(1, 3, 16, 16)).shape == (1, 4, 3 * 64)


VLMS = ["llava", "qwen2_vl", "phi3_vision", "internvl", "cogvlm", "idefics", "florence"]


@pytest.mark.parametrize("name", VLMS)
def test_vlm_multimodal_forward(name):
    cls = ALL_MODELS[name]
    c = cls.config_class()
    names = {f.name for f in dataclasses.fields(c)}
    kw = dict(vocab_size=97, hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, vision_hidden_size=24, vision_intermediate_size=32, vision_num_hidden_layers=2,
              vision_num_attention_heads=4, vision_patch_size=4, vision_image_size=16, im_patch_token=90, image_token_id=90,
              max_position_embeddings=128)
    c = c.replace(**{k: v for k, v in kw.items() if k in names})
    m = cls.new(c, init="random", seed=3)
    tok = m.image_token_id()
    ids = torch.tensor([[1, 2, tok, 4, 5]])
    px = torch.randn(1, 3, 16, 16)
    feats = m.encode_images(px)
    n_img = feats.shape[1]
    assert feats.shape[2] == 32 and n_img == (4 if name == "qwen2_vl" else 16)
    y = m.forward(ModelInputs.multimodal(ids, px)).main_tensor()
    assert y.shape == (1, 4 + n_img, 97) and torch.isfinite(y).all()
    assert m.forward(ModelInputs.text(ids.clamp_max(96))).main_tensor().shape == (1, 5, 97)
    # a run of image tokens is overwritten in place
    run = torch.tensor([[1] + [tok] * n_img + [7]])
    assert m.forward(ModelInputs.multimodal(run, px)).main_tensor().shape == (1, n_img + 2, 97)
    m2 = cls.from_weights(c, m.export_hf())
    assert (m2.forward(ModelInputs.multimodal(ids, px)).main_tensor() - y).abs().max() == 0
    out = m.generate_multimodal([1, 2, tok, 4], px, GenerationConfig.greedy(3, eos_token_id=-1))
    assert len(out) == 3


def test_audio_encoders_and_ctc():
    for name in ("wav2vec2", "hubert"):
        cls = ALL_MODELS[name]
        c = cls.config_class().replace(vocab_size=20, hidden_size=32, intermediate_size=48, num_hidden_layers=2,
                                       num_attention_heads=4, conv_dim=[8, 8, 16], conv_kernel=[10, 3, 2], conv_stride=[5, 2, 2])
        m = cls.new(c, init="random", seed=1)
        wav = torch.randn(2, 400)
        o = m.forward(ModelInputs.audio(wav))
        assert o.logits.shape == (2, m.num_frames(400), 20)
        dec = m.ctc_decode(wav)
        assert len(dec) == 2 and all(t != 0 for t in dec[0])
    full = ALL_MODELS["wav2vec2"].config_class()
    assert ALL_MODELS["wav2vec2"](full).num_frames(16000) == 49


def test_musicgen_and_encodec():
    mg = ALL_MODELS["musicgen"].new(C.MusicGenConfig(vocab_size=50, hidden_size=32, intermediate_size=48, num_hidden_layers=2,
                                                     num_attention_heads=4, num_key_value_heads=4, num_codebooks=3),
                                    init="random", seed=1)
    codes = torch.randint(0, 50, (2, 3, 7))
    y = mg.forward(ModelInputs.text(codes)).logits
    assert y.shape == (2, 3, 7, 50)
    cache = mg.new_cache()
    yi = torch.cat([mg.heads(mg.hidden_states(codes[:, :, t:t + 1], cache), 3) for t in range(7)], 2)
    assert (y - yi).abs().max() < 1e-5
    assert mg.forward(ModelInputs.text(codes[:, 0])).logits.shape == (2, 7, 50)
    g = mg.generate_codes(5, seed=3)
    assert g.shape == (1, 3, 5) and int(g.max()) < 50
    ec = ALL_MODELS["encodec"].new(C.EncodecConfig(hidden_size=16, num_filters=4, upsampling_ratios=[4, 2], codebook_size=32,
                                                   codebook_dim=16, num_codebooks=4, sample_rate=8000, bandwidth=20.0),
                                   init="random", seed=1)
    wav = torch.randn(1, 1, 160)
    codes = ec.encode(wav)
    assert codes.shape == (1, ec.num_quantizers(), 160 // ec.hop_length()) and ec.num_quantizers() == 4
    rec = ec.decode(codes)
    assert rec.shape == wav.shape and torch.isfinite(rec).all()
    # residual VQ: the codes of a lower bandwidth are a prefix of the codes of a higher one, and every stage
    # picks the nearest code of its residual
    z = ec.encode_latent(wav)
    assert torch.equal(ec.quantize(z, 4)[:, :2], ec.quantize(z, 2))
    e0 = ec.p["quantizer.layers.0.codebook.embed"]
    d = torch.cdist(z.transpose(1, 2), e0[None])
    assert torch.equal(d.argmin(-1), ec.quantize(z, 1)[:, 0])


# ---- recurrence oracles against the textbook definitions ----
def test_selective_scan_matches_naive_loop():
    torch.manual_seed(0)
    B, L, D, N = 2, 7, 5, 4
    u, dt, z = torch.randn(B, L, D), torch.randn(B, L, D), torch.randn(B, L, D)
    A, Bm, Cm, Dv = -torch.rand(D, N), torch.randn(B, L, N), torch.randn(B, L, N), torch.randn(D)
    st = torch.zeros(B, D, N)
    y = R.selective_scan(u, dt, A, Bm, Cm, Dv, z, st)
    ref = torch.zeros(B, L, D)
    for b in range(B):
        h = torch.zeros(D, N)
        for l in range(L):
            d = torch.nn.functional.softplus(dt[b, l])
            h = torch.exp(d[:, None] * A) * h + d[:, None] * Bm[b, l][None] * u[b, l][:, None]
            ref[b, l] = ((h * Cm[b, l][None]).sum(-1) + Dv * u[b, l]) * torch.nn.functional.silu(z[b, l])
        assert torch.allclose(st[b], h, atol=1e-5)
    assert torch.allclose(y, ref, atol=1e-5)


def test_conv_wkv_lru_chunking_invariance():
    torch.manual_seed(1)
    B, L, Cn = 2, 9, 8
    x, w, b = torch.randn(B, L, Cn), torch.randn(Cn, 4), torch.randn(Cn)
    st = torch.zeros(B, 3, Cn)
    full = R.causal_dwconv1d(x, w, b, None, True)
    parts = torch.cat([R.causal_dwconv1d(x[:, :5], w, b, st, True), R.causal_dwconv1d(x[:, 5:6], w, b, st, True),
                       R.causal_dwconv1d(x[:, 6:], w, b, st, True)], 1)
    assert torch.allclose(full, parts, atol=1e-6)
    k, v, wd, u = torch.randn(B, L, Cn), torch.randn(B, L, Cn), -torch.exp(torch.randn(Cn)), torch.randn(Cn)
    y = R.wkv4(k, v, wd, u)
    num, den, ys = torch.zeros(B, Cn), torch.zeros(B, Cn), []
    for l in range(L):
        ek, eu = torch.exp(k[:, l]), torch.exp(u + k[:, l])
        ys.append((num + eu * v[:, l]) / (den + eu))
        num, den = torch.exp(wd) * num + ek * v[:, l], torch.exp(wd) * den + ek
    assert torch.allclose(y, torch.stack(ys, 1), atol=1e-5)
    s4 = R.wkv4_new_state(B, Cn, "cpu")
    y2 = torch.cat([R.wkv4(k[:, :4], v[:, :4], wd, u, s4), R.wkv4(k[:, 4:], v[:, 4:], wd, u, s4)], 1)
    assert torch.allclose(y, y2, atol=1e-5)
    H, Dh = 2, 4
    r6, k6, v6, w6 = (torch.randn(B, L, H * Dh) for _ in range(4))
    u6 = torch.randn(H * Dh)
    s6 = torch.zeros(B, H, Dh, Dh)
    y6 = R.wkv6(r6, k6, v6, w6, u6, H)
    y6b = torch.cat([R.wkv6(r6[:, :4], k6[:, :4], v6[:, :4], w6[:, :4], u6, H, s6),
                     R.wkv6(r6[:, 4:], k6[:, 4:], v6[:, 4:], w6[:, 4:], u6, H, s6)], 1)
    assert torch.allclose(y6, y6b, atol=1e-5)
    a = torch.rand(Cn)
    h = R.linear_recurrence(a, x, None, one_minus=True)
    ref, hh = [], torch.zeros(B, Cn)
    for l in range(L):
        hh = a * hh + (1 - a) * x[:, l]
        ref.append(hh)
    assert torch.allclose(h, torch.stack(ref, 1), atol=1e-6)
