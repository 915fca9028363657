"""Minimal safetensors reader/writer and the HF GPT-2 ↔ flat-parameter mapping.

Parity: ``llmm/safetensors.mojo:287-474`` (JSON header parse, dtype map, transpose-on-read,
``read_hf_gpt2_config``), ``train_gpt2.mojo:2162-2321`` (HF names; Conv1D weights are stored
``[in, out]`` so the four linear weights are transposed), ``scripts/export_to_hf.py`` (export;
done natively here because the upstream converter is not vendored).
"""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, Optional, Tuple

import numpy as np
import torch

from ..config import GPT2Config, PARAM_NAMES

_DTYPES = {"F32": (torch.float32, np.float32, 4), "BF16": (torch.bfloat16, np.int16, 2),
           "F16": (torch.float16, np.float16, 2), "I32": (torch.int32, np.int32, 4),
           "I64": (torch.int64, np.int64, 8), "U8": (torch.uint8, np.uint8, 1)}
_REV = {torch.float32: "F32", torch.bfloat16: "BF16", torch.float16: "F16",
        torch.int32: "I32", torch.int64: "I64", torch.uint8: "U8"}


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        with open(path, "rb") as f:
            (n,) = struct.unpack("<Q", f.read(8))
            if n > 100 * 1024 * 1024:
                raise ValueError("safetensors error: header too large")
            self.header = json.loads(f.read(n).decode("utf-8"))
        self.data_start = 8 + n
        self.metadata = self.header.pop("__metadata__", {})

    def keys(self):
        return self.header.keys()

    def has(self, name: str) -> bool:
        return name in self.header

    def read_tensor(self, name: str, transpose: bool = False) -> torch.Tensor:
        if name not in self.header:
            raise KeyError(f"safetensors error: tensor {name!r} not found")
        e = self.header[name]
        tdt, ndt, esz = _DTYPES[e["dtype"]]
        b, end = e["data_offsets"]
        count = (end - b) // esz
        arr = np.fromfile(self.path, dtype=ndt, count=count, offset=self.data_start + b)
        t = torch.from_numpy(arr)
        if tdt == torch.bfloat16:
            t = t.view(torch.bfloat16)
        t = t.reshape(e["shape"])
        if transpose:
            t = t.t().contiguous()
        return t


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Optional[Dict[str, str]] = None) -> None:
    header, off, blobs = {}, 0, []
    if metadata:
        header["__metadata__"] = metadata
    for name, t in tensors.items():
        t = t.detach().contiguous().cpu()
        raw = t.view(torch.int16).numpy().tobytes() if t.dtype == torch.bfloat16 else t.numpy().tobytes()
        header[name] = {"dtype": _REV[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def read_hf_gpt2_config(config_json_path: str) -> GPT2Config:
    with open(config_json_path) as f:
        c = json.load(f)
    V = c["vocab_size"]
    Vp = (V + 127) // 128 * 128
    return GPT2Config(c.get("n_positions", c.get("n_ctx", 1024)), V, c["n_layer"], c["n_head"], c["n_embd"], Vp)


def _hf_name(sf: SafetensorsFile, name: str) -> str:
    return name if sf.has(name) else "transformer." + name


# flat tensor name → (HF per-layer suffix, transpose)
_LAYER_MAP = {
    "ln1w": ("ln_1.weight", False), "ln1b": ("ln_1.bias", False),
    "qkvw": ("attn.c_attn.weight", True), "qkvb": ("attn.c_attn.bias", False),
    "attprojw": ("attn.c_proj.weight", True), "attprojb": ("attn.c_proj.bias", False),
    "ln2w": ("ln_2.weight", False), "ln2b": ("ln_2.bias", False),
    "fcw": ("mlp.c_fc.weight", True), "fcb": ("mlp.c_fc.bias", False),
    "fcprojw": ("mlp.c_proj.weight", True), "fcprojb": ("mlp.c_proj.bias", False),
}


def load_hf_gpt2(path: str, config: Optional[GPT2Config] = None) -> Tuple[GPT2Config, torch.Tensor]:
    """Read an HF GPT-2 ``model.safetensors`` into the flat fp32 parameter vector."""
    sf = SafetensorsFile(path)
    if config is None:
        cj = os.path.join(os.path.dirname(path), "config.json")
        if os.path.exists(cj):
            config = read_hf_gpt2_config(cj)
        else:
            wte = sf.read_tensor(_hf_name(sf, "wte.weight"))
            wpe = sf.read_tensor(_hf_name(sf, "wpe.weight"))
            L = 0
            while sf.has(_hf_name(sf, f"h.{L}.ln_1.weight")):
                L += 1
            C = wte.shape[1]
            config = GPT2Config(wpe.shape[0], wte.shape[0], L, C // 64, C, (wte.shape[0] + 127) // 128 * 128)
    flat = torch.zeros(config.num_parameters(), dtype=torch.float32)
    shapes, sizes = config.param_shapes(), config.param_sizes()
    off = 0
    for name, shape, size in zip(PARAM_NAMES, shapes, sizes):
        view = flat[off:off + size].view(shape)
        if name == "wte":
            view[:config.vocab_size] = sf.read_tensor(_hf_name(sf, "wte.weight")).float()
        elif name == "wpe":
            view.copy_(sf.read_tensor(_hf_name(sf, "wpe.weight")).float())
        elif name in ("lnfw", "lnfb"):
            view.copy_(sf.read_tensor(_hf_name(sf, "ln_f.weight" if name == "lnfw" else "ln_f.bias")).float())
        else:
            suffix, tr = _LAYER_MAP[name]
            for l in range(config.num_layer):
                view[l].copy_(sf.read_tensor(_hf_name(sf, f"h.{l}.{suffix}"), transpose=tr).float())
        off += size
    return config, flat


def export_hf_gpt2(out_dir: str, config: GPT2Config, params_flat: torch.Tensor,
                   dtype: torch.dtype = torch.float32) -> None:
    """Write ``model.safetensors`` + ``config.json`` loadable by ``transformers.GPT2LMHeadModel``."""
    os.makedirs(out_dir, exist_ok=True)
    flat = params_flat.detach().float().cpu()
    shapes, sizes = config.param_shapes(), config.param_sizes()
    out: Dict[str, torch.Tensor] = {}
    off = 0
    for name, shape, size in zip(PARAM_NAMES, shapes, sizes):
        view = flat[off:off + size].view(shape)
        if name == "wte":
            out["wte.weight"] = view[:config.vocab_size].to(dtype)
        elif name == "wpe":
            out["wpe.weight"] = view.to(dtype)
        elif name in ("lnfw", "lnfb"):
            out["ln_f.weight" if name == "lnfw" else "ln_f.bias"] = view.to(dtype)
        else:
            suffix, tr = _LAYER_MAP[name]
            for l in range(config.num_layer):
                t = view[l].t() if tr else view[l]
                out[f"h.{l}.{suffix}"] = t.contiguous().to(dtype)
        off += size
    for k, t in out.items():
        if not torch.isfinite(t.float()).all():
            raise ValueError(f"export error: non-finite values in {k}")
    write_safetensors(os.path.join(out_dir, "model.safetensors"), out, {"format": "pt"})
    cfg = {"architectures": ["GPT2LMHeadModel"], "model_type": "gpt2", "vocab_size": config.vocab_size,
           "n_positions": config.max_seq_len, "n_ctx": config.max_seq_len, "n_embd": config.channels,
           "n_layer": config.num_layer, "n_head": config.num_heads, "activation_function": "gelu_new",
           "layer_norm_epsilon": 1e-5, "resid_pdrop": 0.0, "embd_pdrop": 0.0, "attn_pdrop": 0.0,
           "bos_token_id": 50256, "eos_token_id": 50256, "tie_word_embeddings": True}
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg, f, indent=2)


def fetch_hf_checkpoint(repo_id: str) -> str:
    """Download a Hub repo and return the local ``model.safetensors`` (``llmm/hf_download.mojo:20``)."""
    try:
        from huggingface_hub import snapshot_download
    except ImportError as e:  # pragma: no cover - optional dependency
        raise RuntimeError("huggingface_hub is required for --hf downloads") from e
    d = snapshot_download(repo_id, allow_patterns=["*.safetensors", "config.json"])
    return os.path.join(d, "model.safetensors")
