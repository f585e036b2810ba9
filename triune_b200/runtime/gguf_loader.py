"""GGUF reader and GGML de-quantisation.

Parity (``triune/runtime/gguf_loader.py:56-1321``): a dependency-free GGUF v2/v3 parser (metadata key/values, tensor
directory, alignment), de-quantisers for F32 / F16 / BF16 / Q4_0 / Q4_1 / Q5_0 / Q8_0 / Q4_K / Q5_K / Q6_K, the Ollama blob
resolver, the llama-family tensor-name map to Hugging Face names (including the Q/K row un-permutation), and tokenizer
reconstruction from the metadata arrays.

On the GPU the raw blocks are uploaded as bytes and decoded by the ``ggml_dequant`` kernel to bf16, or by
``ggml_to_nvfp4`` straight into packed NVFP4 (with the optional 16-point Hadamard rotation) without a bf16 copy of the
tensor ever existing; the vectorised PyTorch decoders below are the CPU path and the oracle for those kernels.
``write_gguf`` / ``quantize_ggml`` produce files in the same format (Q8_0, Q4_0, F16, F32), used by the tests and for
exporting small models.
"""

from __future__ import annotations

import json
import mmap
import os
import struct
from pathlib import Path
from typing import Any, BinaryIO, Dict, Iterator, List, Optional, Tuple

import numpy as np
import torch

GGUF_MAGIC = b"GGUF"
GGML_F32, GGML_F16, GGML_Q4_0, GGML_Q4_1, GGML_Q5_0, GGML_Q5_1, GGML_Q8_0 = 0, 1, 2, 3, 6, 7, 8
GGML_Q4_K, GGML_Q5_K, GGML_Q6_K, GGML_BF16 = 12, 13, 14, 30
BLOCK = {GGML_F32: (1, 4), GGML_F16: (1, 2), GGML_BF16: (1, 2), GGML_Q4_0: (32, 18), GGML_Q4_1: (32, 20), GGML_Q5_0: (32, 22),
         GGML_Q8_0: (32, 34), GGML_Q4_K: (256, 144), GGML_Q5_K: (256, 176), GGML_Q6_K: (256, 210)}
TYPE_NAMES = {GGML_F32: "F32", GGML_F16: "F16", GGML_BF16: "BF16", GGML_Q4_0: "Q4_0", GGML_Q4_1: "Q4_1", GGML_Q5_0: "Q5_0",
              GGML_Q8_0: "Q8_0", GGML_Q4_K: "Q4_K", GGML_Q5_K: "Q5_K", GGML_Q6_K: "Q6_K"}
_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
_T_STRING, _T_ARRAY = 8, 9


def is_gguf_file(path) -> bool:
    try:
        with open(path, "rb") as f:
            return f.read(4) == GGUF_MAGIC
    except OSError:
        return False


def resolve_ollama_gguf_blob(ollama_ref: str, models_dir: Optional[str] = None) -> Optional[Path]:
    """``ollama:family:tag`` -> path of the GGUF blob in the local Ollama store (manifest -> model layer digest)."""
    ref = ollama_ref[7:] if ollama_ref.lower().startswith("ollama:") else ollama_ref
    name, _, tag = ref.partition(":")
    tag = tag or "latest"
    roots = [Path(models_dir)] if models_dir else [Path(os.environ.get("OLLAMA_MODELS", "")), Path.home() / ".ollama" / "models",
                                                   Path("/usr/share/ollama/.ollama/models")]
    for root in roots:
        if not str(root) or not root.is_dir():
            continue
        ns, _, short = name.rpartition("/")
        manifest = root / "manifests" / "registry.ollama.ai" / (ns or "library") / short / tag
        if not manifest.is_file():
            continue
        try:
            layers = json.loads(manifest.read_text()).get("layers", [])
        except (OSError, ValueError):
            continue
        for layer in layers:
            if layer.get("mediaType", "").endswith("image.model"):
                blob = root / "blobs" / layer["digest"].replace(":", "-")
                if blob.is_file():
                    return blob
    return None


# ---------------------------------------------------------------------------------------------------- parsing
def _read_str(f: BinaryIO) -> str:
    (n,) = struct.unpack("<Q", f.read(8))
    return f.read(n).decode("utf-8", errors="replace")


def _read_value(f: BinaryIO, t: int, load_arrays: bool, max_array: int = 1 << 22):
    if t in _SCALARS:
        fmt = _SCALARS[t]
        return struct.unpack(fmt, f.read(struct.calcsize(fmt)))[0]
    if t == _T_STRING:
        return _read_str(f)
    if t == _T_ARRAY:
        (et,) = struct.unpack("<I", f.read(4))
        (n,) = struct.unpack("<Q", f.read(8))
        if et in _SCALARS:
            fmt = _SCALARS[et]
            size = struct.calcsize(fmt)
            raw = f.read(size * n)
            if not load_arrays or n > max_array:
                return None
            return list(np.frombuffer(raw, dtype=np.dtype(fmt[1]).newbyteorder("<")).tolist())
        out = [_read_value(f, et, load_arrays) for _ in range(n)]
        return out if load_arrays else None
    raise ValueError(f"unknown GGUF value type {t}")


def read_gguf_directory(gguf_path, *, load_tokenizer_arrays: bool = True) -> Dict[str, Any]:
    """-> {"version", "metadata": {...}, "tensors": {name: {"shape" (row-major, outermost first), "type", "offset",
    "nbytes"}}, "data_offset", "alignment"}."""
    with open(gguf_path, "rb") as f:
        if f.read(4) != GGUF_MAGIC:
            raise ValueError(f"{gguf_path} is not a GGUF file")
        (version,) = struct.unpack("<I", f.read(4))
        if version < 2:
            raise ValueError(f"GGUF version {version} is not supported")
        n_tensors, n_kv = struct.unpack("<QQ", f.read(16))
        meta: Dict[str, Any] = {}
        for _ in range(n_kv):
            key = _read_str(f)
            (t,) = struct.unpack("<I", f.read(4))
            meta[key] = _read_value(f, t, load_tokenizer_arrays or not key.startswith("tokenizer."))
        tensors: Dict[str, Dict[str, Any]] = {}
        for _ in range(n_tensors):
            name = _read_str(f)
            (nd,) = struct.unpack("<I", f.read(4))
            dims = struct.unpack(f"<{nd}Q", f.read(8 * nd))
            gtype, offset = struct.unpack("<IQ", f.read(12))
            numel = int(np.prod(dims)) if dims else 1
            be, bb = BLOCK.get(gtype, (0, 0))
            tensors[name] = {"shape": tuple(reversed(dims)), "type": gtype, "offset": offset, "numel": numel,
                             "nbytes": numel // be * bb if be else 0}
        align = int(meta.get("general.alignment", 32))
        pos = f.tell()
        data_offset = (pos + align - 1) // align * align
    return {"version": version, "metadata": meta, "tensors": tensors, "data_offset": data_offset, "alignment": align}


# ---------------------------------------------------------------------------------------------------- decoding (PyTorch)
def _f16(b: torch.Tensor) -> torch.Tensor:
    """[..., 2] uint8 -> float32 via fp16."""
    return b.contiguous().view(torch.float16).float().squeeze(-1)


def _k4_scales(s: torch.Tensor):
    """[nb, 12] uint8 -> (scales [nb, 8], mins [nb, 8]) as float."""
    s = s.to(torch.int32)
    sc = torch.empty(s.shape[0], 8, dtype=torch.int32, device=s.device)
    mn = torch.empty_like(sc)
    sc[:, :4], mn[:, :4] = s[:, 0:4] & 63, s[:, 4:8] & 63
    sc[:, 4:] = (s[:, 8:12] & 0xF) | ((s[:, 0:4] >> 6) << 4)
    mn[:, 4:] = (s[:, 8:12] >> 4) | ((s[:, 4:8] >> 6) << 4)
    return sc.float(), mn.float()


def dequantize_ggml(raw: torch.Tensor, ggml_type: int, numel: int, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Vectorised PyTorch decoder (any device). ``raw`` is a flat uint8 tensor."""
    if ggml_type == GGML_F32:
        return raw.view(torch.float32)[:numel].to(dtype)
    if ggml_type == GGML_F16:
        return raw.view(torch.float16)[:numel].to(dtype)
    if ggml_type == GGML_BF16:
        return raw.view(torch.bfloat16)[:numel].to(dtype)
    be, bb = BLOCK[ggml_type]
    b = raw[: numel // be * bb].view(-1, bb)
    i32 = torch.int32
    if ggml_type in (GGML_Q4_0, GGML_Q4_1):
        hdr = 2 if ggml_type == GGML_Q4_0 else 4
        d = _f16(b[:, 0:2]).unsqueeze(1)
        qs = b[:, hdr:].to(i32)
        q = torch.cat((qs & 0xF, qs >> 4), dim=1).float()
        out = (q - 8.0) * d if ggml_type == GGML_Q4_0 else q * d + _f16(b[:, 2:4]).unsqueeze(1)
    elif ggml_type == GGML_Q5_0:
        d = _f16(b[:, 0:2]).unsqueeze(1)
        qh = b[:, 2:6].contiguous().view(torch.int32)  # [nb, 1]
        bits = (qh >> torch.arange(32, device=raw.device, dtype=i32).view(1, 32)) & 1
        qs = b[:, 6:].to(i32)
        q = torch.cat((qs & 0xF, qs >> 4), dim=1) | (bits << 4)
        out = (q.float() - 16.0) * d
    elif ggml_type == GGML_Q8_0:
        out = b[:, 2:].contiguous().view(torch.int8).float() * _f16(b[:, 0:2]).unsqueeze(1)
    elif ggml_type in (GGML_Q4_K, GGML_Q5_K):
        d, dmin = _f16(b[:, 0:2]).view(-1, 1, 1), _f16(b[:, 2:4]).view(-1, 1, 1)
        sc, mn = _k4_scales(b[:, 4:16])
        if ggml_type == GGML_Q4_K:
            qs = b[:, 16:144].to(i32).view(-1, 4, 32)
            q = torch.stack((qs & 0xF, qs >> 4), dim=2)  # [nb, 4 groups, 2 halves, 32]
        else:
            qh = b[:, 16:48].to(i32).view(-1, 1, 1, 32)
            qs = b[:, 48:176].to(i32).view(-1, 4, 32)
            shifts = torch.arange(8, device=raw.device, dtype=i32).view(1, 4, 2, 1)
            q = torch.stack((qs & 0xF, qs >> 4), dim=2) + (((qh >> shifts) & 1) << 4)
        out = d.unsqueeze(-1) * sc.view(-1, 4, 2, 1) * q.float() - dmin.unsqueeze(-1) * mn.view(-1, 4, 2, 1)
    elif ggml_type == GGML_Q6_K:
        ql = b[:, 0:128].to(i32).view(-1, 2, 64)
        qh = b[:, 128:192].to(i32).view(-1, 2, 32)
        sc = b[:, 192:208].contiguous().view(torch.int8).float().view(-1, 2, 8)
        d = _f16(b[:, 208:210]).view(-1, 1, 1, 1)
        lo = torch.stack((ql[:, :, :32] & 0xF, ql[:, :, 32:] & 0xF, ql[:, :, :32] >> 4, ql[:, :, 32:] >> 4), dim=2)  # [nb,2,4,32]
        hi = torch.stack([(qh >> s) & 3 for s in (0, 2, 4, 6)], dim=2)
        q = (lo | (hi << 4)).float() - 32.0
        idx = (torch.arange(32, device=raw.device) // 16).view(1, 1, 1, 32) + 2 * torch.arange(4, device=raw.device).view(1, 1, 4, 1)
        scale = torch.gather(sc.unsqueeze(2).expand(-1, -1, 4, -1), 3, idx.expand(sc.shape[0], 2, 4, 32))
        out = d * scale * q
    else:
        raise NotImplementedError(f"GGML type {ggml_type} ({TYPE_NAMES.get(ggml_type, '?')}) is not supported")
    return out.reshape(-1)[:numel].to(dtype)


def dequantize_ggml_tensor(raw, ggml_type: int, shape: Tuple[int, ...], device="cpu", dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Bytes of one tensor -> dense tensor of ``shape``. On a GPU the decode kernel runs on the uploaded bytes."""
    numel = int(np.prod(shape)) if shape else 1
    t = raw if torch.is_tensor(raw) else torch.frombuffer(bytearray(raw), dtype=torch.uint8)
    dev = torch.device(device)
    if dev.type == "cuda":
        from .. import _ext

        t = t.to(dev, non_blocking=True)
        if _ext.ext_available() and ggml_type in BLOCK:
            return _ext.ext().ggml_dequant(t.contiguous(), int(ggml_type), numel).view(shape).to(dtype)
    return dequantize_ggml(t.to(dev), ggml_type, numel, dtype).view(shape)


def ggml_to_nvfp4(raw, ggml_type: int, rows: int, K: int, device, hadamard: bool = False):
    """GGML bytes -> (packed E2M1 [rows, K/2], E4M3 scales [rows, K/16], fp32 tensor scale), decoded and re-quantised in
    one pass over the bytes on the GPU; falls back to decode + quantise elsewhere."""
    from .. import _ext, ops

    t = raw if torch.is_tensor(raw) else torch.frombuffer(bytearray(raw), dtype=torch.uint8)
    dev = torch.device(device)
    if dev.type == "cuda" and _ext.ext_available():
        return tuple(_ext.ext().ggml_to_nvfp4(t.to(dev).contiguous(), int(ggml_type), rows, K, bool(hadamard)))
    w = dequantize_ggml(t.to(dev), ggml_type, rows * K, torch.float32).view(rows, K)
    return ops.nvfp4_quantize(w, hadamard=hadamard)


class GGUFFile:
    """Memory-mapped access to the tensors of a GGUF file."""

    def __init__(self, path):
        self.path = Path(path)
        self.directory = read_gguf_directory(self.path)
        self.metadata, self.tensors = self.directory["metadata"], self.directory["tensors"]
        self._f = open(self.path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)

    def close(self):
        self._mm.close()
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def raw(self, name: str) -> torch.Tensor:
        info = self.tensors[name]
        start = self.directory["data_offset"] + info["offset"]
        return torch.frombuffer(bytearray(self._mm[start : start + info["nbytes"]]), dtype=torch.uint8)

    def tensor(self, name: str, device="cpu", dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        info = self.tensors[name]
        return dequantize_ggml_tensor(self.raw(name), info["type"], info["shape"], device, dtype)

    def items(self, device="cpu", dtype: torch.dtype = torch.bfloat16) -> Iterator[Tuple[str, torch.Tensor]]:
        for name in self.tensors:
            yield name, self.tensor(name, device, dtype)


# ---------------------------------------------------------------------------------------------------- HF mapping
_LAYER_MAP = {"attn_norm": "input_layernorm", "ffn_norm": "post_attention_layernorm", "attn_q": "self_attn.q_proj",
              "attn_k": "self_attn.k_proj", "attn_v": "self_attn.v_proj", "attn_output": "self_attn.o_proj", "ffn_gate": "mlp.gate_proj",
              "ffn_up": "mlp.up_proj", "ffn_down": "mlp.down_proj", "attn_q_norm": "self_attn.q_norm", "attn_k_norm": "self_attn.k_norm"}
_ROOT_MAP = {"token_embd": "model.embed_tokens", "output_norm": "model.norm", "output": "lm_head"}


def gguf_to_hf_name(name: str) -> Optional[str]:
    base, _, suffix = name.rpartition(".")
    if base in _ROOT_MAP:
        return f"{_ROOT_MAP[base]}.{suffix}"
    parts = base.split(".")
    if len(parts) == 3 and parts[0] == "blk" and parts[2] in _LAYER_MAP:
        return f"model.layers.{parts[1]}.{_LAYER_MAP[parts[2]]}.{suffix}"
    return None


def unpermute_llama_qk(w: torch.Tensor, n_heads: int) -> torch.Tensor:
    """llama.cpp stores Q/K rows with the two rotary halves interleaved per head; HF expects them split."""
    rows = w.shape[0]
    hd = rows // n_heads
    return w.view(n_heads, hd // 2, 2, *w.shape[1:]).transpose(1, 2).reshape(w.shape)


def hf_config_from_gguf(meta: Dict[str, Any]) -> Dict[str, Any]:
    arch = meta.get("general.architecture", "llama")
    g = lambda k, d=None: meta.get(f"{arch}.{k}", d)  # noqa: E731
    heads = int(g("attention.head_count", 32))
    hidden = int(g("embedding_length", 4096))
    vocab = g("vocab_size") or (len(meta["tokenizer.ggml.tokens"]) if meta.get("tokenizer.ggml.tokens") else 32000)
    return {"architecture": arch, "hidden_size": hidden, "num_hidden_layers": int(g("block_count", 32)), "num_attention_heads": heads,
            "num_key_value_heads": int(g("attention.head_count_kv", heads)), "intermediate_size": int(g("feed_forward_length", 4 * hidden)),
            "rms_norm_eps": float(g("attention.layer_norm_rms_epsilon", 1e-5)), "rope_theta": float(g("rope.freq_base", 10000.0)),
            "max_position_embeddings": int(g("context_length", 4096)), "vocab_size": int(vocab),
            "head_dim": int(g("attention.key_length", hidden // heads)), "bos_token_id": meta.get("tokenizer.ggml.bos_token_id"),
            "eos_token_id": meta.get("tokenizer.ggml.eos_token_id")}


def load_gguf_state_dict(path, device="cpu", dtype: torch.dtype = torch.bfloat16) -> Tuple[Dict[str, torch.Tensor], Dict[str, Any]]:
    """-> (state dict with Hugging Face llama-style names, HF-style config dict)."""
    with GGUFFile(path) as gf:
        cfg = hf_config_from_gguf(gf.metadata)
        sd: Dict[str, torch.Tensor] = {}
        for name, t in gf.items(device, dtype):
            hf = gguf_to_hf_name(name)
            if hf is None:
                continue
            if cfg["architecture"] == "llama" and hf.endswith("q_proj.weight"):
                t = unpermute_llama_qk(t, cfg["num_attention_heads"])
            elif cfg["architecture"] == "llama" and hf.endswith("k_proj.weight"):
                t = unpermute_llama_qk(t, cfg["num_key_value_heads"])
            sd[hf] = t
        if "lm_head.weight" not in sd and "model.embed_tokens.weight" in sd:
            sd["lm_head.weight"] = sd["model.embed_tokens.weight"]
    return sd, cfg


def load_gguf_hf_model(path, device="cpu", dtype: torch.dtype = torch.bfloat16):
    """Instantiate a Hugging Face ``LlamaForCausalLM`` from a llama-family GGUF file."""
    from transformers import LlamaConfig, LlamaForCausalLM

    sd, cfg = load_gguf_state_dict(path, device, dtype)
    keep = ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "intermediate_size", "rms_norm_eps",
            "rope_theta", "max_position_embeddings", "vocab_size", "head_dim")
    hf_cfg = LlamaConfig(**{k: cfg[k] for k in keep}, tie_word_embeddings=False)
    with torch.device(device):
        model = LlamaForCausalLM(hf_cfg).to(dtype)
    missing, unexpected = model.load_state_dict(sd, strict=False)
    real_missing = [m for m in missing if "rotary_emb" not in m]
    if real_missing:
        raise RuntimeError(f"GGUF file lacks tensors for: {real_missing[:5]}")
    return model.eval(), cfg


def tokenizer_vocab_from_gguf(meta: Dict[str, Any]) -> Dict[str, Any]:
    """Token list, scores / merges and special ids as stored in the metadata (enough to rebuild a tokenizer)."""
    return {"model": meta.get("tokenizer.ggml.model"), "tokens": meta.get("tokenizer.ggml.tokens") or [],
            "scores": meta.get("tokenizer.ggml.scores"), "merges": meta.get("tokenizer.ggml.merges"),
            "token_type": meta.get("tokenizer.ggml.token_type"), "bos_token_id": meta.get("tokenizer.ggml.bos_token_id"),
            "eos_token_id": meta.get("tokenizer.ggml.eos_token_id"), "pad_token_id": meta.get("tokenizer.ggml.padding_token_id"),
            "chat_template": meta.get("tokenizer.chat_template")}


def build_hf_tokenizer_from_gguf(meta: Dict[str, Any]):
    """A ``PreTrainedTokenizerFast`` rebuilt from the vocabulary a GGUF file carries, token ids preserved: byte-pair
    encoding when the file stores merges (SentencePiece-style pieces with the U+2581 space marker, or GPT-2 byte-level
    pieces), a unigram model over the stored scores otherwise. Control tokens (type 3) and the usual chat markers become
    special tokens; the chat template travels along (``triune/runtime/gguf_loader.py:544-620`` of the reference)."""
    from tokenizers import AddedToken, Tokenizer, decoders, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast

    v = tokenizer_vocab_from_gguf(meta)
    tokens = [str(t) for t in v["tokens"]]
    if not tokens:
        raise ValueError("GGUF metadata contains no tokenizer vocabulary.")
    ids = {t: i for i, t in enumerate(tokens)}

    def named(key: str, default_id: int, fallback: str) -> str:
        i = meta.get(key)
        i = default_id if i is None else int(i)
        return tokens[i] if 0 <= i < len(tokens) else fallback

    bos, eos = named("tokenizer.ggml.bos_token_id", 1, "<s>"), named("tokenizer.ggml.eos_token_id", 2, "</s>")
    unk = named("tokenizer.ggml.unknown_token_id", 0, "<unk>")
    pad_id = meta.get("tokenizer.ggml.padding_token_id")
    pad = tokens[int(pad_id)] if pad_id is not None and 0 <= int(pad_id) < len(tokens) else eos
    sentencepiece = any(t.startswith("\u2581") for t in tokens[:1000])
    if v["merges"]:
        pairs = [tuple(p) for p in (str(m).split(" ") for m in v["merges"]) if len(p) == 2 and p[0] in ids and p[1] in ids]
        tk = Tokenizer(models.BPE(vocab=ids, merges=pairs, unk_token=unk, ignore_merges=True))
        if sentencepiece:
            tk.pre_tokenizer = pre_tokenizers.Metaspace(replacement="\u2581", prepend_scheme="never")
            tk.decoder = decoders.Sequence([decoders.Replace("\u2581", " "), decoders.ByteFallback()])
        else:
            tk.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
            tk.decoder = decoders.ByteLevel()
    else:
        scores = list(v["scores"] or [])
        table = [(t, float(scores[i]) if i < len(scores) else -10.0) for i, t in enumerate(tokens)]
        tk = Tokenizer(models.Unigram(table, unk_id=ids.get(unk, 0)))
        tk.pre_tokenizer = pre_tokenizers.Metaspace(replacement="\u2581", prepend_scheme="never")
        tk.decoder = decoders.Metaspace(replacement="\u2581")
    types = list(v["token_type"] or [])
    special = [tokens[i] for i, tt in enumerate(types) if tt == 3 and i < len(tokens)]
    special += [t for t in ("<start_of_turn>", "<end_of_turn>", "<|eot_id|>", "<|im_start|>", "<|im_end|>") if t in ids and t not in special]
    tk.add_special_tokens([AddedToken(t, special=True, normalized=False) for t in special])
    fast = PreTrainedTokenizerFast(tokenizer_object=tk, bos_token=bos, eos_token=eos, unk_token=unk, pad_token=pad)
    if v["chat_template"]:
        fast.chat_template = str(v["chat_template"])
    return fast


# ---------------------------------------------------------------------------------------------------- writing
def quantize_ggml(w: torch.Tensor, ggml_type: int) -> bytes:
    """Encode a tensor as F32 / F16 / BF16 / Q8_0 / Q4_0 blocks."""
    flat = w.detach().float().reshape(-1).cpu()
    if ggml_type == GGML_F32:
        return flat.numpy().tobytes()
    if ggml_type == GGML_F16:
        return flat.half().numpy().tobytes()
    if ggml_type == GGML_BF16:
        return flat.bfloat16().view(torch.int16).numpy().tobytes()
    blocks = flat.view(-1, 32)
    amax = blocks.abs().amax(1, keepdim=True)
    if ggml_type == GGML_Q8_0:
        d = (amax / 127.0).half()
        q = torch.where(d.float() > 0, (blocks / d.float().clamp_min(1e-30)).round(), torch.zeros_like(blocks)).clamp(-127, 127).to(torch.int8)
        out = np.empty((blocks.shape[0], 34), dtype=np.uint8)
        out[:, :2] = d.view(torch.int16).numpy().view(np.uint8).reshape(-1, 2)
        out[:, 2:] = q.numpy().view(np.uint8)
        return out.tobytes()
    if ggml_type == GGML_Q4_0:
        idx = blocks.abs().argmax(1, keepdim=True)
        mx = blocks.gather(1, idx)
        d = (mx / -8.0).half()
        q = torch.where(d.float() != 0, blocks / d.float().where(d.float() != 0, torch.ones_like(d.float())), torch.zeros_like(blocks))
        q = (q + 8.5).floor().clamp(0, 15).to(torch.uint8)
        out = np.empty((blocks.shape[0], 18), dtype=np.uint8)
        out[:, :2] = d.view(torch.int16).numpy().view(np.uint8).reshape(-1, 2)
        out[:, 2:] = (q[:, :16] | (q[:, 16:] << 4)).numpy()
        return out.tobytes()
    raise NotImplementedError(f"encoding GGML type {ggml_type} is not supported")


def _w_str(f, s: str):
    b = s.encode("utf-8")
    f.write(struct.pack("<Q", len(b)))
    f.write(b)


def _w_value(f, v):
    if isinstance(v, bool):
        f.write(struct.pack("<I?", 7, v))
    elif isinstance(v, int):
        f.write(struct.pack("<Iq", 11, v) if v < 0 else struct.pack("<II", 4, v) if v < 2**32 else struct.pack("<IQ", 10, v))
    elif isinstance(v, float):
        f.write(struct.pack("<If", 6, v))
    elif isinstance(v, str):
        f.write(struct.pack("<I", _T_STRING))
        _w_str(f, v)
    elif isinstance(v, (list, tuple)):
        f.write(struct.pack("<I", _T_ARRAY))
        if v and isinstance(v[0], str):
            f.write(struct.pack("<IQ", _T_STRING, len(v)))
            for s in v:
                _w_str(f, s)
        elif v and isinstance(v[0], float):
            f.write(struct.pack("<IQ", 6, len(v)))
            f.write(np.asarray(v, dtype="<f4").tobytes())
        else:
            f.write(struct.pack("<IQ", 5, len(v)))
            f.write(np.asarray(v, dtype="<i4").tobytes())
    else:
        raise TypeError(f"cannot store {type(v)} in GGUF metadata")


def write_gguf(path, tensors: Dict[str, Tuple[torch.Tensor, int]], metadata: Optional[Dict[str, Any]] = None, alignment: int = 32) -> Path:
    """``tensors``: name -> (tensor, ggml type). Quantised types need a last dimension that is a multiple of 32."""
    meta = dict(metadata or {})
    meta.setdefault("general.alignment", alignment)
    blobs, infos, off = [], [], 0
    for name, (t, gtype) in tensors.items():
        data = quantize_ggml(t, gtype)
        infos.append((name, tuple(reversed(t.shape)), gtype, off))
        blobs.append(data)
        off = (off + len(data) + alignment - 1) // alignment * alignment
    with open(path, "wb") as f:
        f.write(GGUF_MAGIC)
        f.write(struct.pack("<IQQ", 3, len(infos), len(meta)))
        for k, v in meta.items():
            _w_str(f, k)
            _w_value(f, v)
        for name, dims, gtype, o in infos:
            _w_str(f, name)
            f.write(struct.pack("<I", len(dims)))
            f.write(struct.pack(f"<{len(dims)}Q", *dims))
            f.write(struct.pack("<IQ", gtype, o))
        pos = f.tell()
        f.write(b"\0" * ((pos + alignment - 1) // alignment * alignment - pos))
        for data in blobs:
            f.write(data)
            f.write(b"\0" * ((len(data) + alignment - 1) // alignment * alignment - len(data)))
    return Path(path)
