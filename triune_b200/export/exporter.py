"""Model export: safetensors, LoRA-only safetensors, Hugging Face bundle, ONNX; GGUF is refused explicitly.

Parity: ``triune/export/exporter.py:28-146`` (``export_safetensors``, ``export_lora_safetensors``, ``export_onnx``,
``export_gguf`` raising ``NotImplementedError``, ``export_model`` dispatcher).
"""

from __future__ import annotations

from pathlib import Path

import torch

from .safetensors_io import save_file


def _dedup(sd):
    seen, out = set(), {}
    for k, v in sd.items():
        key = (v.data_ptr(), tuple(v.shape))
        out[k] = v.clone() if key in seen and v.numel() else v
        seen.add(key)
    return out


def export_safetensors(model: torch.nn.Module, output_path) -> Path:
    p = Path(output_path)
    p.parent.mkdir(parents=True, exist_ok=True)
    save_file(_dedup(model.state_dict()), str(p), metadata={"format": "pt"})
    return p


def export_lora_safetensors(model: torch.nn.Module, output_path) -> Path:
    ad = {n: t.detach().cpu().contiguous() for n, t in model.named_parameters() if n.endswith(("lora_A", "lora_B"))}
    if not ad:
        raise ValueError("No attached LoRA adapter matrices were found; no file was written.")
    p = Path(output_path)
    p.parent.mkdir(parents=True, exist_ok=True)
    save_file(ad, str(p), metadata={"format": "pt"})
    return p


def export_gguf(model: torch.nn.Module, output_path, quantization: str = "q4_k_m") -> Path:
    raise NotImplementedError("GGUF export is not implemented for GLA layers, hierarchical exits and routed experts; "
                              "the model was not exported.")


def export_onnx(model: torch.nn.Module, output_path, seq_len: int = 128) -> Path:
    p = Path(output_path)
    p.parent.mkdir(parents=True, exist_ok=True)
    model.eval()
    vocab = int(getattr(model, "vocab_size", 1000))
    torch.onnx.export(model, torch.randint(0, vocab, (1, seq_len)), str(p), input_names=["input_ids"],
                      output_names=["logits", "router_logits"], dynamic_axes={"input_ids": {0: "batch_size", 1: "seq_len"}},
                      opset_version=17)
    return p


def export_model(model: torch.nn.Module, output_path, fmt: str = "safetensors", **kw) -> Path:
    f = fmt.lower()
    if f == "gguf":
        return export_gguf(model, output_path)
    if f == "onnx":
        return export_onnx(model, output_path, **kw)
    if f in ("hf", "huggingface"):
        from .hf_compat import export_to_huggingface

        return export_to_huggingface(model, output_path, **kw)
    if f == "lora":
        return export_lora_safetensors(model, output_path)
    if f in ("pt", "torch"):
        p = Path(output_path)
        p.parent.mkdir(parents=True, exist_ok=True)
        torch.save({"model_state": model.state_dict()}, p)
        return p
    if f == "safetensors":
        return export_safetensors(model, output_path)
    raise ValueError(f"unknown export format {fmt!r}")
