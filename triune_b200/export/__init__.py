"""Export: safetensors, Hugging Face bundle, LoRA adapters."""

from .exporter import export_gguf, export_lora_safetensors, export_model, export_onnx, export_safetensors
from .hf_compat import export_to_huggingface, extract_triune_hf_config, load_from_huggingface
from .safetensors_io import load_file, save_file

__all__ = ["export_gguf", "export_lora_safetensors", "export_model", "export_onnx", "export_safetensors",
           "export_to_huggingface", "extract_triune_hf_config", "load_from_huggingface", "load_file", "save_file"]
