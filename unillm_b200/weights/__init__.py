"""Weight containers and loaders (SafeTensors, PyTorch, GGUF)."""
from .gguf import GGUFModelConfig, GGUFTokenizer, dequantize_blocks, gguf_to_hf_name, quantize_blocks, read_gguf, write_gguf
from .loaders import (ConfigLoader, GGUFWeightLoader, ModelLoader, PyTorchWeightLoader, SafeTensorsWeightLoader,
                      UnifiedWeightLoader, WeightLoader, loader, read_safetensors, save_sharded_for_tp, write_safetensors)
