"""Model zoo.  Importing this package fills the global registry (``unillm_b200.model_core.registry()``)
with every architecture; names follow the reference's module names (``crates/runtime/src/models_v2/mod.rs:10-83``)
and each class is also exported under the reference's ``<Family>ModelV2`` alias."""
from __future__ import annotations

from ..model_core import ModelFactory, registry
from . import configs
from .decoder import DecoderModel
from .families import DECODER_FAMILIES
from .spec import DecoderSpec, KeyScheme, MoESpec

ALL_MODELS = dict(DECODER_FAMILIES)


def _register_all() -> None:
    reg = registry()
    for name, cls in ALL_MODELS.items():
        archs = [name, cls.config_class.__name__, cls.__name__, cls.config_class.__name__.replace("Config", "ForCausalLM")]
        f = ModelFactory(cls, archs)
        for a in archs:
            reg.register(a, f)


def _late_imports() -> None:
    """Non-decoder families live in their own modules; import them if present."""
    import importlib

    for mod in ("ssm", "rwkv", "griffin", "encoders", "encdec", "vision", "audio"):
        try:
            m = importlib.import_module(f"{__name__}.{mod}")
        except ModuleNotFoundError as e:
            if e.name != f"{__name__}.{mod}":
                raise
            continue
        ALL_MODELS.update(getattr(m, "MODELS", {}))


_late_imports()
_register_all()


def get_model_class(name: str):
    f = registry().get(name)
    if f is None:
        raise KeyError(f"unknown architecture {name!r}; known: {sorted(ALL_MODELS)}")
    return f.model_cls


globals().update({cls.__name__: cls for cls in ALL_MODELS.values()})
globals().update({cls.__name__ + "V2": cls for cls in ALL_MODELS.values()})
