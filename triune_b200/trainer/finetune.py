"""LoRA / QLoRA fine-tuning.

Parity (``triune/trainer/finetune.py:49-958``): ``LoRALayer`` over ``nn.Linear`` / ``NVFP4Linear`` with optional NVFP4
quantisation of the frozen base (QLoRA), ``LoRAConfig`` (PEFT field aliases), ``TriuneFineTuner`` (attach / detach /
merge, PEFT-format ``adapter_config.json`` + ``adapter_model.safetensors``, SFT with prompt masking and a cosine
schedule), ``list_adapters``, ``export_adapter``, ``merge_adapter_checkpoint``.

The native model keeps Q, K, V and the decay gate in ONE fused ``[4*H*D, d]`` weight; ``FusedProjectionLoRA`` adapts
row blocks of it (targets ``q_proj`` / ``k_proj`` / ``v_proj`` / ``g_proj``) with a single rank-r pair whose B factor
is zero outside the targeted blocks. On the GPU both adapters run ``ops.lora_linear``: the base GEMM on tensor cores
with the low-rank product accumulated into its output by the reduce-add epilogue.
"""

from __future__ import annotations

import json
import math
import time
from pathlib import Path
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..models.quant_linear import NVFP4Linear

DEFAULT_TARGETS = ["q_proj", "k_proj", "v_proj", "g_proj", "o_proj", "out_proj", "gate_proj", "up_proj", "down_proj",
                   "qkv_proj", "gate_up_proj", "0", "2"]
_SKIP_ATTRS = ("original_layer", "lm_head", "final_head", "exit_head", "router")
_QKVG = ("q_proj", "k_proj", "v_proj", "g_proj")


def _dev_dtype(mod: nn.Module, fallback: Optional[torch.device] = None):
    for p in list(mod.parameters()) + list(mod.buffers()):
        if p.device.type != "meta" and p.dtype.is_floating_point and p.dtype not in (torch.float8_e4m3fn,):
            return p.device, p.dtype
    for p in list(mod.parameters()) + list(mod.buffers()):
        if p.device.type != "meta":
            return p.device, torch.bfloat16
    return fallback or torch.device("cpu"), torch.bfloat16


class LoRALayer(nn.Module):
    def __init__(self, original_layer: nn.Module, rank: int = 16, alpha: float = 32.0, dropout: float = 0.05,
                 adapter_device: Optional[torch.device] = None):
        super().__init__()
        self.original_layer = original_layer
        self.rank, self.alpha, self.scaling = rank, alpha, alpha / rank
        dev, dt = _dev_dtype(original_layer, adapter_device)
        dev = adapter_device or dev
        self.lora_A = nn.Parameter(torch.empty(rank, original_layer.in_features, device=dev, dtype=dt))
        self.lora_B = nn.Parameter(torch.zeros(original_layer.out_features, rank, device=dev, dtype=dt))
        nn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))
        self.dropout = nn.Dropout(dropout) if dropout > 0 else nn.Identity()
        for p in original_layer.parameters():
            p.requires_grad = False

    @property
    def in_features(self):
        return self.original_layer.in_features

    @property
    def out_features(self):
        return self.original_layer.out_features

    @property
    def weight(self):
        return getattr(self.original_layer, "weight", None)

    @property
    def bias(self):
        return getattr(self.original_layer, "bias", None)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        base = self.original_layer
        no_drop = isinstance(self.dropout, nn.Identity) or not self.training
        if type(base) is nn.Linear and no_drop and x.dtype == base.weight.dtype == self.lora_A.dtype:
            return ops.lora_linear(x, base.weight, base.bias, self.lora_A, self.lora_B, self.scaling)
        y = base(x)
        xd = self.dropout(x).to(device=self.lora_A.device, dtype=self.lora_A.dtype)
        return y + (F.linear(F.linear(xd, self.lora_A), self.lora_B) * self.scaling).to(device=y.device, dtype=y.dtype)

    @torch.no_grad()
    def delta(self) -> torch.Tensor:
        return (self.lora_B.float() @ self.lora_A.float()) * self.scaling

    @torch.no_grad()
    def merge(self) -> None:
        base = self.original_layer
        if isinstance(base, NVFP4Linear):
            w = base.dequantized(torch.float32)
            if base.hadamard:
                w = ops.ref.fwht16(w)  # the rotation is an involution: back to the unrotated weight
            base.load_weight(w + self.delta().to(w.device))
        else:
            base.weight.add_(self.delta().to(device=base.weight.device, dtype=base.weight.dtype))
        self.lora_B.zero_()


class FusedProjectionLoRA(nn.Module):
    """Adapter for ``VectorisedGLA.qkvg_weight``; ``blocks`` selects which of q, k, v, g receive an update."""

    def __init__(self, gla: nn.Module, blocks: Sequence[int], rank: int = 16, alpha: float = 32.0, dropout: float = 0.05):
        super().__init__()
        object.__setattr__(self, "gla", gla)
        self.blocks = tuple(sorted(set(blocks)))
        self.rank, self.alpha, self.scaling = rank, alpha, alpha / rank
        w = gla.qkvg_weight
        self.lora_A = nn.Parameter(torch.empty(rank, w.shape[1], device=w.device, dtype=w.dtype))
        self.lora_B = nn.Parameter(torch.zeros(w.shape[0], rank, device=w.device, dtype=w.dtype))
        nn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))
        mask = torch.zeros(w.shape[0], 1, device=w.device, dtype=w.dtype)
        hd = gla.hidden_dim
        for b in self.blocks:
            mask[b * hd : (b + 1) * hd] = 1
        self.register_buffer("row_mask", mask, persistent=False)
        self.dropout = nn.Dropout(dropout) if dropout > 0 else nn.Identity()
        w.requires_grad = False

    def forward(self, x2: torch.Tensor) -> torch.Tensor:
        B = self.lora_B * self.row_mask if len(self.blocks) < 4 else self.lora_B
        if isinstance(self.dropout, nn.Identity) or not self.training:
            return ops.lora_linear(x2, self.gla.qkvg_weight, None, self.lora_A, B, self.scaling)
        return F.linear(x2, self.gla.qkvg_weight) + F.linear(F.linear(self.dropout(x2), self.lora_A), B) * self.scaling

    @torch.no_grad()
    def merge(self) -> None:
        d = ((self.lora_B * self.row_mask).float() @ self.lora_A.float()) * self.scaling
        self.gla.qkvg_weight.add_(d.to(self.gla.qkvg_weight.dtype))
        self.lora_B.zero_()


class LoRAConfig:
    def __init__(self, rank: int = 16, r: Optional[int] = None, alpha: float = 32.0, lora_alpha: Optional[float] = None,
                 dropout: float = 0.05, target_modules: Optional[List[str]] = None, use_qlora: bool = False,
                 quantization: Optional[str] = None, quantize_base: Optional[bool] = None, hadamard: bool = True):
        self.rank = r if r is not None else rank
        self.alpha = lora_alpha if lora_alpha is not None else alpha
        self.dropout = dropout
        self.target_modules = list(target_modules) if target_modules else list(DEFAULT_TARGETS)
        self.quantization = quantization or ("4-bit NVFP4" if use_qlora else "FP16")
        q = self.quantization.lower()
        self.use_qlora = bool(use_qlora or any(t in q for t in ("4-bit", "nf4", "nvfp4")))
        self.quantize_base = bool(quantize_base if quantize_base is not None else "nvfp4" in q)
        self.hadamard = bool(hadamard)

    @classmethod
    def from_pretrained(cls, adapter_dir) -> "LoRAConfig":
        p = Path(adapter_dir)
        f = (p.parent if p.is_file() else p) / "adapter_config.json"
        if not f.is_file():
            return cls()
        d = json.loads(f.read_text(encoding="utf-8"))
        return cls(rank=int(d.get("r", d.get("rank", 16))), alpha=float(d.get("lora_alpha", d.get("alpha", 32.0))),
                   dropout=float(d.get("lora_dropout", d.get("dropout", 0.05))), target_modules=d.get("target_modules"),
                   quantization=d.get("quantization"), quantize_base=d.get("quantize_base"))

    def to_dict(self, base_name: str = "triune-base", trainable: int = 0) -> Dict[str, Any]:
        return {"peft_type": "LORA", "auto_mapping": None, "base_model_name_or_path": base_name, "r": self.rank,
                "lora_alpha": self.alpha, "lora_dropout": self.dropout, "target_modules": self.target_modules, "bias": "none",
                "task_type": "CAUSAL_LM", "rank": self.rank, "alpha": self.alpha, "dropout": self.dropout,
                "quantization": self.quantization, "quantize_base": self.quantize_base, "trainable_params": trainable}


def _save_tensors(sd: Dict[str, torch.Tensor], path: Path) -> Path:
    from ..export.safetensors_io import save_file

    save_file(sd, str(path))
    return path


def _load_tensors(path: Path) -> Dict[str, torch.Tensor]:
    if path.suffix == ".safetensors":
        from ..export.safetensors_io import load_file

        return load_file(str(path))
    from .checkpoint import safe_torch_load

    return safe_torch_load(path)


class TriuneFineTuner:
    def __init__(self, model: nn.Module, lora_config: Optional[LoRAConfig] = None, *, tokenizer: Any = None,
                 model_name_or_path: Optional[str] = None, adapter_device=None):
        self.model = model
        self.lora_config = lora_config or LoRAConfig()
        self.tokenizer = getattr(tokenizer, "hf", tokenizer) if tokenizer is not None else None
        self.model_name_or_path = (model_name_or_path or getattr(model, "name_or_path", None)
                                   or getattr(getattr(model, "config", None), "_name_or_path", None))
        self._adapter_device = torch.device(adapter_device) if adapter_device is not None else None
        self.applied_adapters: Dict[str, nn.Module] = {}
        self.history: List[Dict[str, float]] = []
        self.attach_lora()

    # ------------------------------------------------------------------ adapters
    def _matches(self, name: str) -> bool:
        return any(t == name or t in name for t in self.lora_config.target_modules)

    def attach_lora(self) -> None:
        if self.applied_adapters:
            return
        cfg = self.lora_config
        for p in self.model.parameters():
            p.requires_grad = False
        mods = dict(self.model.named_modules())
        for name, mod in list(mods.items()):
            if isinstance(mod, (LoRALayer, FusedProjectionLoRA)):
                continue
            if hasattr(mod, "qkvg_weight") and isinstance(getattr(mod, "qkvg_weight"), nn.Parameter):
                blocks = [i for i, t in enumerate(_QKVG) if t in cfg.target_modules or "qkv_proj" in cfg.target_modules and i < 3]
                if blocks:
                    ad = FusedProjectionLoRA(mod, blocks, cfg.rank, cfg.alpha, cfg.dropout)
                    ad.train(mod.training)  # an adapter on an eval-mode model must not drop activations
                    mod.qkvg_lora = ad
                    self.applied_adapters[f"{name}.qkvg" if name else "qkvg"] = ad
                continue
            if not isinstance(mod, (nn.Linear, NVFP4Linear)) or not self._matches(name):
                continue
            parent_name, _, attr = name.rpartition(".")
            if attr in _SKIP_ATTRS or any(s in name for s in ("exit_head", "router")):
                continue
            parent = mods.get(parent_name, self.model) if parent_name else self.model
            if isinstance(parent, LoRALayer):
                continue
            base = mod
            if (cfg.quantize_base and type(mod) is nn.Linear and mod.in_features % 16 == 0 and mod.weight.device.type != "meta"
                    and mod.weight.numel() > 0):
                base = NVFP4Linear.from_linear(mod, hadamard=cfg.hadamard)
            ad = LoRALayer(base, cfg.rank, cfg.alpha, cfg.dropout, self._adapter_device)
            ad.train(mod.training)
            if isinstance(parent, (nn.Sequential, nn.ModuleList)) and attr.isdigit():
                parent[int(attr)] = ad
            else:
                setattr(parent, attr, ad)
            self.applied_adapters[name] = ad

    def detach_lora(self) -> None:
        mods = dict(self.model.named_modules())
        for name, ad in list(self.applied_adapters.items()):
            if isinstance(ad, FusedProjectionLoRA):
                ad.gla.qkvg_lora = None
                continue
            parent_name, _, attr = name.rpartition(".")
            parent = mods.get(parent_name, self.model) if parent_name else self.model
            if isinstance(parent, (nn.Sequential, nn.ModuleList)) and attr.isdigit():
                parent[int(attr)] = ad.original_layer
            else:
                setattr(parent, attr, ad.original_layer)
        self.applied_adapters.clear()
        for p in self.model.parameters():
            p.requires_grad = True

    def merge_and_unload(self) -> None:
        for ad in self.applied_adapters.values():
            ad.merge()
        self.detach_lora()

    def get_trainable_parameters(self) -> List[nn.Parameter]:
        return [p for ad in self.applied_adapters.values() for p in (ad.lora_A, ad.lora_B)]

    def count_trainable_parameters(self) -> int:
        return sum(p.numel() for p in self.get_trainable_parameters())

    def get_optimizer(self, lr: float = 2e-4, weight_decay: float = 0.0):
        fused = any(p.is_cuda for p in self.get_trainable_parameters())
        return torch.optim.AdamW(self.get_trainable_parameters(), lr=lr, weight_decay=weight_decay, fused=fused)

    # ------------------------------------------------------------------ persistence (PEFT layout)
    def save_adapter(self, save_dir) -> Path:
        p = Path(save_dir)
        p.mkdir(parents=True, exist_ok=True)
        sd = {}
        for name, ad in self.applied_adapters.items():
            a, b = ad.lora_A.detach().cpu().contiguous(), ad.lora_B.detach().cpu().contiguous()
            if isinstance(ad, FusedProjectionLoRA):
                b = (b * ad.row_mask.cpu()).contiguous()
            sd[f"{name}.lora_A"], sd[f"{name}.lora_B"] = a, b
            sd[f"base_model.model.{name}.lora_A.weight"], sd[f"base_model.model.{name}.lora_B.weight"] = a.clone(), b.clone()
        base = self.model_name_or_path or getattr(self.model, "active_model_id", None) or "triune-base"
        (p / "adapter_config.json").write_text(
            json.dumps(self.lora_config.to_dict(str(base), self.count_trainable_parameters()), indent=2), encoding="utf-8")
        _save_tensors(sd, p / "adapter_model.safetensors")
        if self.tokenizer is not None and hasattr(self.tokenizer, "save_pretrained"):
            try:
                self.tokenizer.save_pretrained(str(p))
            except Exception:
                pass
        return p

    def load_adapter(self, load_dir) -> None:
        p = Path(load_dir)
        f = p if p.is_file() else next((p / n for n in ("adapter_model.safetensors", "adapter_model.pt") if (p / n).is_file()), None)
        if f is None or not f.is_file():
            raise FileNotFoundError(f"adapter weights not found at {load_dir}")
        sd = _load_tensors(f)
        self.attach_lora()
        for name, ad in self.applied_adapters.items():
            for which, param in (("lora_A", ad.lora_A), ("lora_B", ad.lora_B)):
                for k in (f"{name}.{which}", f"{name}.{which}.weight", f"base_model.model.{name}.{which}.weight",
                          f"base_model.model.{name}.{which}"):
                    if k in sd:
                        param.data.copy_(sd[k].to(device=param.device, dtype=param.dtype))
                        break

    # ------------------------------------------------------------------ data
    @staticmethod
    def _encode_ids(tokenizer, text: str) -> List[int]:
        out = tokenizer.encode(text)
        return list(getattr(out, "ids", out))

    @staticmethod
    def parse_records(records: Iterable[Any]) -> List[Tuple[str, str]]:
        """Accepts {'prompt','completion'}, {'instruction','input','output'}, {'messages':[...]}, {'text'} or strings;
        returns (prompt, completion) pairs (prompt may be empty)."""
        pairs = []
        for r in records:
            if isinstance(r, str):
                pairs.append(("", r))
            elif "messages" in r:
                msgs = r["messages"]
                last = max((i for i, m in enumerate(msgs) if m.get("role") == "assistant"), default=None)
                if last is None:
                    continue
                prompt = "".join(f"{m.get('role', 'user').capitalize()}: {m.get('content', '')}\n" for m in msgs[:last])
                pairs.append((prompt + "Assistant:", " " + str(msgs[last].get("content", ""))))
            elif "prompt" in r and ("completion" in r or "response" in r):
                pairs.append((str(r["prompt"]), str(r.get("completion", r.get("response")))))
            elif "instruction" in r:
                inp = f"\n{r['input']}" if r.get("input") else ""
                pairs.append((f"User: {r['instruction']}{inp}\nAssistant:", " " + str(r.get("output", ""))))
            elif "text" in r:
                pairs.append(("", str(r["text"])))
        return pairs

    def build_examples(self, records: Iterable[Any], tokenizer=None, max_seq_len: int = 512, mask_prompt: bool = True):
        """-> list of (input_ids, labels) 1-D tensors; prompt positions carry label -100 when ``mask_prompt``."""
        tok = tokenizer or self.tokenizer
        if tok is None:
            raise ValueError("a tokenizer is required to build training examples")
        out = []
        for prompt, completion in self.parse_records(records):
            p_ids = self._encode_ids(tok, prompt) if prompt else []
            c_ids = self._encode_ids(tok, completion)
            ids = (p_ids + c_ids)[: max_seq_len + 1]
            if len(ids) < 2:
                continue
            x = torch.tensor(ids[:-1], dtype=torch.long)
            y = torch.tensor(ids[1:], dtype=torch.long)
            if mask_prompt and p_ids:
                y[: max(0, min(len(p_ids) - 1, y.numel()))] = -100
            if (y != -100).any():
                out.append((x, y))
        return out

    # ------------------------------------------------------------------ training
    def _logits(self, input_ids: torch.Tensor) -> torch.Tensor:
        m = self.model
        if hasattr(m, "forward_all_exits") or hasattr(m, "reflex_exit_layer") and hasattr(m, "layers"):
            out = m(input_ids, force_depth=2)
        else:
            out = m(input_ids)
        return out.logits if hasattr(out, "logits") else (out[0] if isinstance(out, tuple) else out)

    def fit(self, dataset: Iterable[Any], *, tokenizer=None, epochs: int = 1, batch_size: int = 4, lr: float = 2e-4,
            max_seq_len: int = 512, warmup_ratio: float = 0.05, weight_decay: float = 0.0, grad_clip: float = 1.0,
            mask_prompt: bool = True, max_steps: Optional[int] = None, log_every: int = 10, callback=None,
            pad_token_id: int = 0) -> Dict[str, Any]:
        examples = dataset if (isinstance(dataset, list) and dataset and isinstance(dataset[0], tuple)
                               and torch.is_tensor(dataset[0][0])) else self.build_examples(dataset, tokenizer, max_seq_len, mask_prompt)
        if not examples:
            raise ValueError("no usable training examples")
        dev = next((p.device for p in self.model.parameters() if p.device.type != "meta"), torch.device("cpu"))
        opt = self.get_optimizer(lr, weight_decay)
        steps_per_epoch = math.ceil(len(examples) / batch_size)
        total = min(max_steps, steps_per_epoch * epochs) if max_steps else steps_per_epoch * epochs
        warm = max(1, int(total * warmup_ratio))
        self.model.train()
        step, t0, tokens = 0, time.perf_counter(), 0
        losses: List[torch.Tensor] = []
        g = torch.Generator().manual_seed(0)
        done = False
        for _ in range(epochs):
            order = torch.randperm(len(examples), generator=g).tolist()
            for s in range(0, len(order), batch_size):
                batch = [examples[i] for i in order[s : s + batch_size]]
                T = max(x.numel() for x, _ in batch)
                X = torch.full((len(batch), T), pad_token_id, dtype=torch.long)
                Y = torch.full((len(batch), T), -100, dtype=torch.long)
                for i, (x, y) in enumerate(batch):
                    X[i, : x.numel()], Y[i, : y.numel()] = x, y
                X, Y = X.to(dev, non_blocking=True), Y.to(dev, non_blocking=True)
                cur_lr = lr * (step + 1) / warm if step < warm else lr * 0.5 * (1 + math.cos(math.pi * (step - warm) / max(1, total - warm)))
                for gp in opt.param_groups:
                    gp["lr"] = cur_lr
                logits = self._logits(X)
                loss = F.cross_entropy(logits.reshape(-1, logits.size(-1)).float(), Y.reshape(-1), ignore_index=-100)
                opt.zero_grad(set_to_none=True)
                loss.backward()
                if grad_clip:
                    torch.nn.utils.clip_grad_norm_(self.get_trainable_parameters(), grad_clip)
                opt.step()
                losses.append(loss.detach())
                tokens += int(X.numel())
                step += 1
                if step % log_every == 0 or step == total:
                    rec = {"step": step, "loss": float(torch.stack(losses[-log_every:]).mean()), "lr": cur_lr,
                           "tok_s": tokens / max(1e-9, time.perf_counter() - t0)}
                    self.history.append(rec)
                    if callback is not None:
                        callback(rec)
                if step >= total:
                    done = True
                    break
            if done:
                break
        self.model.eval()
        all_l = torch.stack(losses).float()
        return {"steps": step, "first_loss": float(all_l[0]), "final_loss": float(all_l[-1]), "mean_loss": float(all_l.mean()),
                "trainable_params": self.count_trainable_parameters(), "history": self.history}


def list_adapters(scan_dirs: Optional[List[str]] = None) -> List[Dict[str, Any]]:
    out = []
    for d in scan_dirs or ["adapters", "checkpoints", "outputs"]:
        root = Path(d)
        if not root.is_dir():
            continue
        for cfg in root.rglob("adapter_config.json"):
            try:
                meta = json.loads(cfg.read_text(encoding="utf-8"))
            except Exception:
                continue
            w = next((cfg.parent / n for n in ("adapter_model.safetensors", "adapter_model.pt") if (cfg.parent / n).is_file()), None)
            out.append({"name": cfg.parent.name, "path": str(cfg.parent), "base_model": meta.get("base_model_name_or_path"),
                        "rank": meta.get("r", meta.get("rank")), "alpha": meta.get("lora_alpha"),
                        "size_bytes": w.stat().st_size if w else 0, "has_weights": w is not None})
    return out


def export_adapter(adapter_path, output_path=None, fmt: str = "safetensors") -> Path:
    src = Path(adapter_path)
    f = src if src.is_file() else next((src / n for n in ("adapter_model.safetensors", "adapter_model.pt") if (src / n).is_file()), None)
    if f is None:
        raise FileNotFoundError(f"no adapter weights under {adapter_path}")
    sd = _load_tensors(f)
    out = Path(output_path) if output_path else f.with_name(f"adapter_export.{'safetensors' if fmt == 'safetensors' else 'pt'}")
    out.parent.mkdir(parents=True, exist_ok=True)
    if fmt == "safetensors":
        _save_tensors({k: v.contiguous() for k, v in sd.items()}, out)
    else:
        torch.save(sd, out)
    return out


def merge_adapter_checkpoint(model: nn.Module, adapter_dir, output_path=None) -> nn.Module:
    """Attach the adapter stored in ``adapter_dir``, fold it into the base weights, optionally save the merged model."""
    ft = TriuneFineTuner(model, LoRAConfig.from_pretrained(adapter_dir))
    ft.load_adapter(adapter_dir)
    ft.merge_and_unload()
    if output_path:
        torch.save({"model_state": model.state_dict()}, output_path)
    return model
