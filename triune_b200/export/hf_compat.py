"""Hugging Face bundle: ``TriuneConfig`` / ``TriuneForCausalLM`` and ``export_to_huggingface``.

Parity (``triune/export/hf_compat.py:18-292``): the bundle holds ``config.json`` (with an ``auto_map`` to the two
generated Python files), ``generation_config.json``, ``configuration_triune.py``, ``modeling_triune.py``,
``model.safetensors`` with keys prefixed ``transformer.`` (tied tensors stored twice so every key is present) and the
tokenizer file. State-dict keys are the reference's per-projection / per-expert names, so bundles are interchangeable.

Here the two classes are real importable classes of this package and the generated files only re-export them; the
config also carries the fields the reference hard-codes (top-k, expert / dense hidden sizes, shared expert).
"""

from __future__ import annotations

import json
import shutil
from pathlib import Path
from typing import Any, Dict, Optional

import torch
import torch.nn as nn

from ..config import ModelConfig

_CFG_FIELDS = ("vocab_size", "hidden_dim", "num_layers", "num_heads", "head_dim", "num_experts", "router_prefix_layers",
               "reflex_exit_layer", "limbic_exit_layer", "use_fp4", "use_fp8", "top_k", "expert_hidden", "dense_hidden",
               "shared_expert")

CONFIGURATION_FILE = '''"""Triune model configuration (generated; the implementation lives in the triune_b200 package)."""
from triune_b200.export.hf_compat import TriuneConfig  # noqa: F401
'''
MODELING_FILE = '''"""Triune causal LM for Hugging Face Transformers (generated; the implementation lives in the triune_b200 package)."""
from triune_b200.export.hf_compat import TriuneForCausalLM, TriunePreTrainedModel  # noqa: F401
'''

try:
    from transformers.configuration_utils import PretrainedConfig
    from transformers.modeling_outputs import CausalLMOutputWithPast
    from transformers.modeling_utils import PreTrainedModel

    _HAVE_HF = True
except Exception:  # transformers missing: export still works, the wrapper classes do not exist
    _HAVE_HF = False


def _model_config(cfg) -> ModelConfig:
    kw = {k: getattr(cfg, k) for k in _CFG_FIELDS if getattr(cfg, k, None) is not None}
    return ModelConfig(**kw)


if _HAVE_HF:

    class TriuneConfig(PretrainedConfig):
        model_type = "triune"
        keys_to_ignore_at_inference = ["past_key_values"]

        def __init__(self, vocab_size=2048, hidden_dim=256, num_layers=6, num_heads=4, head_dim=64, num_experts=4,
                     router_prefix_layers=1, reflex_exit_layer=2, limbic_exit_layer=4, use_fp4=False, use_fp8=False, top_k=1,
                     expert_hidden=None, dense_hidden=None, shared_expert=True, pad_token_id=0, bos_token_id=1,
                     eos_token_id=2, tie_word_embeddings=False, **kwargs):
            super().__init__(pad_token_id=pad_token_id, bos_token_id=bos_token_id, eos_token_id=eos_token_id,
                             tie_word_embeddings=tie_word_embeddings, **kwargs)
            self.vocab_size, self.hidden_dim, self.num_layers = vocab_size, hidden_dim, num_layers
            self.num_heads, self.head_dim, self.num_experts = num_heads, head_dim, num_experts
            self.router_prefix_layers, self.reflex_exit_layer = router_prefix_layers, reflex_exit_layer
            self.limbic_exit_layer, self.use_fp4, self.use_fp8 = limbic_exit_layer, use_fp4, use_fp8
            self.top_k, self.expert_hidden, self.dense_hidden, self.shared_expert = top_k, expert_hidden, dense_hidden, shared_expert
            self.hidden_size, self.num_hidden_layers, self.num_attention_heads = hidden_dim, num_layers, num_heads

    class TriunePreTrainedModel(PreTrainedModel):
        config_class = TriuneConfig
        base_model_prefix = "transformer"
        supports_gradient_checkpointing = True
        _no_split_modules = ["TransformerBlock", "VectorisedGLA", "MoE_FFN"]

        def _init_weights(self, module):
            if isinstance(module, (nn.Linear, nn.Embedding)):
                module.weight.data.normal_(mean=0.0, std=0.02)
                if getattr(module, "bias", None) is not None:
                    module.bias.data.zero_()

    class TriuneForCausalLM(TriunePreTrainedModel):
        _tied_weights_keys = {}

        def __init__(self, config: "TriuneConfig"):
            super().__init__(config)
            from ..models.transformer import TriuneTransformer

            self.transformer = TriuneTransformer.from_config(_model_config(config))
            self.post_init()

        @classmethod
        def from_pretrained(cls, pretrained_model_name_or_path, *model_args, config=None, torch_dtype=None, dtype=None,
                            **kwargs):
            """Load a local bundle. The checkpoint uses per-projection / per-expert keys while the module stores fused
            and stacked parameters, so the weights go through ``load_state_dict`` (whose hooks do the regrouping) rather
            than through the key-by-key loader of ``transformers``."""
            from .safetensors_io import load_file

            d = Path(pretrained_model_name_or_path)
            if not (d / "model.safetensors").is_file():
                raise FileNotFoundError(f"{d} is not a local Triune bundle (model.safetensors missing)")
            cfg = config if isinstance(config, TriuneConfig) else TriuneConfig.from_pretrained(str(d))
            model = cls(cfg)
            missing, unexpected = model.load_state_dict(load_file(str(d / "model.safetensors")), strict=False)
            if unexpected:
                raise RuntimeError(f"unexpected keys in the bundle: {unexpected[:5]}")
            want = dtype or torch_dtype
            if isinstance(want, str) and want != "auto":
                want = getattr(torch, want)
            if isinstance(want, torch.dtype):
                model = model.to(want)
            return model.eval()

        def get_input_embeddings(self):
            return self.transformer.token_embed

        def set_input_embeddings(self, value):
            self.transformer.token_embed = value

        def get_output_embeddings(self):
            return self.transformer.final_head

        def set_output_embeddings(self, value):
            self.transformer.final_head = value

        def forward(self, input_ids=None, attention_mask=None, position_ids=None, past_key_values=None, inputs_embeds=None,
                    labels=None, use_cache=None, output_attentions=None, output_hidden_states=None, return_dict=None,
                    force_depth: Optional[int] = None, **kwargs):
            return_dict = getattr(self.config, "return_dict", True) if return_dict is None else return_dict
            if input_ids is None and inputs_embeds is None:
                raise ValueError("You must specify either input_ids or inputs_embeds")
            cache = past_key_values
            if use_cache and cache is None:
                cache = self.transformer.init_cache(input_ids.shape[0] if input_ids is not None else inputs_embeds.shape[0])
            res = self.transformer(input_ids, force_depth=2 if force_depth is None and labels is not None else force_depth,
                                   cache=cache, inputs_embeds=inputs_embeds)
            logits, new_cache = (res[0], res[1]) if cache is not None else (res[0], None)
            loss = None
            if labels is not None:
                loss = nn.functional.cross_entropy(logits[..., :-1, :].reshape(-1, logits.size(-1)).float(),
                                                   labels[..., 1:].reshape(-1), ignore_index=-100)
            if not return_dict:
                out = (logits,) + ((new_cache,) if new_cache is not None else ())
                return ((loss,) + out) if loss is not None else out
            return CausalLMOutputWithPast(loss=loss, logits=logits, past_key_values=new_cache)

        def prepare_inputs_for_generation(self, input_ids, past_key_values=None, attention_mask=None, **kw):
            if past_key_values is not None:
                input_ids = input_ids[:, -1:]  # the recurrent state already holds the prefix
            return {"input_ids": input_ids, "past_key_values": past_key_values, "force_depth": kw.get("force_depth"),
                    "use_cache": kw.get("use_cache", True)}


def extract_triune_hf_config(model: nn.Module) -> Dict[str, Any]:
    core = getattr(model, "transformer", model)
    moe = next((l.ffn for l in core.layers if hasattr(l.ffn, "w1")), None)
    dense = next((l.ffn for l in core.layers if not hasattr(l.ffn, "w1")), None)
    cfg = {"architectures": ["TriuneForCausalLM"], "model_type": "triune",
           "auto_map": {"AutoConfig": "configuration_triune.TriuneConfig",
                        "AutoModelForCausalLM": "modeling_triune.TriuneForCausalLM"},
           "torch_dtype": str(next(core.parameters()).dtype).split(".")[-1], "transformers_version": "4.49.0"}
    for k, default in (("vocab_size", 2048), ("hidden_dim", 256), ("num_layers", 6), ("num_heads", 4), ("head_dim", 64),
                       ("num_experts", 4), ("router_prefix_layers", 1), ("reflex_exit_layer", 2), ("limbic_exit_layer", 4),
                       ("use_fp4", False), ("use_fp8", False)):
        cfg[k] = getattr(core, k, default)
    if moe is not None:
        cfg.update(top_k=int(moe.top_k), expert_hidden=int(moe.expert_hidden), shared_expert=moe.shared is not None)
    if dense is not None:
        cfg["dense_hidden"] = int(dense[0].out_features)
    return cfg


def prefixed_state_dict(model: nn.Module, prefix: str = "transformer.") -> Dict[str, torch.Tensor]:
    """State dict with ``prefix`` on every key; tensors that share storage are cloned so each key owns its bytes."""
    core = getattr(model, "transformer", model)
    seen, out = set(), {}
    for k, v in core.state_dict().items():
        ptr = (v.data_ptr(), tuple(v.shape))
        out[prefix + k] = v.clone() if ptr in seen else v
        seen.add(ptr)
    return out


def export_to_huggingface(model: nn.Module, save_directory, tokenizer: Any = None, tokenizer_path=None) -> Path:
    from .safetensors_io import save_file

    d = Path(save_directory)
    d.mkdir(parents=True, exist_ok=True)
    (d / "config.json").write_text(json.dumps(extract_triune_hf_config(model), indent=2), encoding="utf-8")
    gen = {"_from_model_config": True, "bos_token_id": 1, "eos_token_id": 2, "pad_token_id": 0, "transformers_version": "4.49.0",
           "temperature": 0.7, "top_k": 50, "top_p": 0.95, "repetition_penalty": 1.1}
    (d / "generation_config.json").write_text(json.dumps(gen, indent=2), encoding="utf-8")
    (d / "configuration_triune.py").write_text(CONFIGURATION_FILE, encoding="utf-8")
    (d / "modeling_triune.py").write_text(MODELING_FILE, encoding="utf-8")
    save_file(prefixed_state_dict(model), str(d / "model.safetensors"), metadata={"format": "pt"})
    if tokenizer_path is not None and Path(tokenizer_path).exists():
        shutil.copy(str(tokenizer_path), str(d / "tokenizer.json"))
    elif tokenizer is not None and hasattr(tokenizer, "save"):
        tokenizer.save(str(d / "tokenizer.json"))
    return d


def load_from_huggingface(directory, device="cpu", dtype: Optional[torch.dtype] = None):
    """Load a bundle written by :func:`export_to_huggingface` (or by the reference) into a native TriuneTransformer."""
    from ..models.transformer import TriuneTransformer
    from .safetensors_io import load_file

    d = Path(directory)
    raw = json.loads((d / "config.json").read_text(encoding="utf-8"))
    cfg = ModelConfig(**{k: raw[k] for k in _CFG_FIELDS if raw.get(k) is not None})
    sd = {k.removeprefix("transformer."): v for k, v in load_file(str(d / "model.safetensors")).items()}
    if "expert_hidden" not in raw:  # bundles of the reference do not record these; read them off the tensors
        for k, v in sd.items():
            if k.endswith("ffn.experts.0.0.weight"):
                cfg.expert_hidden = int(v.shape[0])
            elif k.endswith("ffn.0.weight"):
                cfg.dense_hidden = int(v.shape[0])
    model = TriuneTransformer.from_config(cfg)
    model.load_state_dict(sd, strict=False)
    model = model.to(device=device, dtype=dtype) if dtype is not None else model.to(device)
    return model.eval()
