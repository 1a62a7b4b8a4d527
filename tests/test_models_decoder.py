"""Every decoder family: forward shape, finite logits, cached == uncached, HF-name export/import round trip."""
import dataclasses

import pytest
import torch

from unillm_b200.model_core import ModelInputs
from unillm_b200.models.families import DECODER_FAMILIES

MHA_ONLY = ("gpt2", "gptj", "gptneox", "opt", "bloom", "mpt", "phi", "olmo", "baichuan")


def tiny_config(name, cls):
    c = cls.config_class()
    kw = dict(vocab_size=97, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=96,
              max_position_embeddings=64)
    names = {f.name for f in dataclasses.fields(c)}
    if "num_key_value_heads" in names:
        kw["num_key_value_heads"] = 4 if name in MHA_ONLY else 2
    extra = dict(head_dim=16, kv_channels=16, rotary_dim=8, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32,
                 word_embed_proj_dim=64, sliding_window=8, num_shared_experts=1)
    for k, v in extra.items():
        if k in names:
            kw[k] = v
    if name == "deepseek":
        kw.pop("num_experts", None)
        kw.pop("num_experts_per_tok", None)
    return c.replace(**{k: v for k, v in kw.items() if k in names})


@pytest.mark.parametrize("name", sorted(DECODER_FAMILIES))
def test_family_forward_cache_roundtrip(name):
    cls = DECODER_FAMILIES[name]
    c = tiny_config(name, cls)
    torch.manual_seed(0)
    m = cls.new(c, init="random", seed=1)
    ids = torch.randint(0, 97, (2, 12))
    y = m.forward(ModelInputs.text(ids)).main_tensor()
    assert y.shape == (2, 12, 97)
    assert torch.isfinite(y).all()
    cache = m.new_cache(64)
    y1 = m.forward_with_cache(ids[:, :7], cache)
    y2 = m.forward_with_cache(ids[:, 7:], cache)
    assert (torch.cat([y1, y2], 1) - y).abs().max().item() < 1e-4
    w = m.export_hf()
    m2 = cls.from_weights(c, w)
    y3 = m2.forward(ModelInputs.text(ids)).main_tensor()
    assert (y3 - y).abs().max().item() < 1e-5


def test_zero_weight_model_gives_zero_logits():
    cls = DECODER_FAMILIES["llama"]
    m = cls.new(tiny_config("llama", cls))
    y = m.forward(ModelInputs.text(torch.zeros(1, 4, dtype=torch.long))).main_tensor()
    assert y.shape == (1, 4, 97) and float(y.abs().max()) == 0.0


def test_registry_lists_all_architectures():
    from unillm_b200 import models  # noqa: F401
    from unillm_b200.model_core import registry

    archs = set(registry().supported_architectures())
    for n in DECODER_FAMILIES:
        assert n in archs
    m = registry().create_model("llama", '{"vocab_size": 50, "hidden_size": 32, "num_hidden_layers": 1, '
                                '"num_attention_heads": 2, "num_key_value_heads": 2, "intermediate_size": 48}')
    assert m.config().vocab_size == 50
