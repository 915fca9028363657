"""Model configuration, model descriptors and the precision axis.

Parity: ``train_gpt2.mojo:807-813`` (GPT2Config), ``:997-1089`` (descriptor ladders),
``:240-303`` (precision → storage / master dtype).  In the reference the precision is a
compile-time define; here every kernel is pre-built so it is a runtime value.
"""
from __future__ import annotations

import os

from dataclasses import dataclass, field
from typing import Dict, List, Tuple

import torch

MODEL_MAGIC = 20240520          # train_gpt2.mojo:320
LEGACY_MODEL_MAGIC = 20240326
LN_EPS = 1e-5
INIT_RNG_SEED = 42
INIT_WEIGHT_STD = 0.02
SCRATCH_VOCAB_SIZE = 50257
SCRATCH_PADDED_VOCAB_SIZE = 50304

# The 16 parameter tensors in llm.c order (train_gpt2.mojo:447-463).
PARAM_NAMES: Tuple[str, ...] = (
    "wte", "wpe", "ln1w", "ln1b", "qkvw", "qkvb", "attprojw", "attprojb",
    "ln2w", "ln2b", "fcw", "fcb", "fcprojw", "fcprojb", "lnfw", "lnfb",
)
NUM_PARAMETER_TENSORS = len(PARAM_NAMES)

_GPT2_LADDER: Dict[int, Tuple[int, int]] = {
    6: (384, 6), 12: (768, 12), 24: (1024, 16), 36: (1280, 20), 48: (1600, 25),
    60: (1920, 30), 72: (2880, 30), 84: (3456, 36),
}
_GPT3_LADDER: Dict[int, Tuple[int, int]] = {
    384: (6, 64), 768: (12, 64), 1024: (24, 64), 1536: (24, 96), 2048: (24, 128),
    2560: (32, 80), 4096: (32, 128), 5140: (40, 128), 12288: (96, 128),
}


@dataclass
class GPT2Config:
    max_seq_len: int = 1024
    vocab_size: int = SCRATCH_VOCAB_SIZE
    num_layer: int = 12
    num_heads: int = 12
    channels: int = 768
    padded_vocab_size: int = SCRATCH_PADDED_VOCAB_SIZE

    @property
    def head_size(self) -> int:
        return self.channels // self.num_heads

    def param_shapes(self) -> List[Tuple[int, ...]]:
        """Shapes of the 16 tensors, llm.c order (llmm/checkpointing.mojo:60-90)."""
        L, C, Vp, maxT = self.num_layer, self.channels, self.padded_vocab_size, self.max_seq_len
        return [
            (Vp, C), (maxT, C), (L, C), (L, C), (L, 3 * C, C), (L, 3 * C), (L, C, C), (L, C),
            (L, C), (L, C), (L, 4 * C, C), (L, 4 * C), (L, C, 4 * C), (L, C), (C,), (C,),
        ]

    def param_sizes(self) -> List[int]:
        out = []
        for s in self.param_shapes():
            n = 1
            for d in s:
                n *= d
            out.append(n)
        return out

    def num_parameters(self) -> int:
        return sum(self.param_sizes())

    def header(self, version: int) -> List[int]:
        h = [0] * 256
        h[0], h[1] = MODEL_MAGIC, version
        h[2:8] = [self.max_seq_len, self.vocab_size, self.num_layer, self.num_heads,
                  self.channels, self.padded_vocab_size]
        return h


def parse_model_descriptor(desc: str) -> GPT2Config:
    """``dX`` / ``gpt2:dX`` / ``gpt3:cX`` → config (train_gpt2.mojo:1041-1089)."""
    try:
        if desc.startswith("gpt2:d"):
            depth = int(desc[6:])
            C, NH = _GPT2_LADDER[depth]
            L, maxT = depth, 1024
        elif desc.startswith("gpt3:c"):
            C = int(desc[6:])
            L, hs = _GPT3_LADDER[C]
            if C % hs:
                raise ValueError("GPT-3 channels not divisible by head size")
            NH, maxT = C // hs, 2048
        elif desc.startswith("d"):
            depth = int(desc[1:])
            C, NH = _GPT2_LADDER[depth]
            L, maxT = depth, 1024
        else:
            raise KeyError(desc)
    except KeyError:
        raise ValueError(f"Unsupported model descriptor: {desc}") from None
    return GPT2Config(maxT, SCRATCH_VOCAB_SIZE, L, NH, C, SCRATCH_PADDED_VOCAB_SIZE)


def is_model_descriptor(s: str) -> bool:
    return (s.startswith("d") and s[1:].isdigit()) or s.startswith("gpt2:d") or s.startswith("gpt3:c")


@dataclass
class Precision:
    """Runtime precision axis: fp32 | tf32 | bf16 | fp8 | fp4 (train_gpt2.mojo:240-303).

    ``storage`` is the dtype of parameters/activations, ``master`` the dtype of the AdamW
    master copy (None = parameters are their own master).  Gradients are always
    accumulated in fp32 locally and cast to bf16 only on the wire.
    """
    name: str = "bf16"
    fp8_sites: Tuple[str, ...] = ("qkv", "attproj", "fc", "fcproj")
    fp8_block_scales: bool = False    # per-tensor delayed scaling when False
    fp4_first: int = 2                # first layer whose MLP runs NVFP4 (train_gpt2.mojo:318)
    fp4_last_offset: int = 2          # layers [first, L - offset) run NVFP4
    fp4_rht: bool = True
    fp4_sr: bool = True
    fp32_storage: bool = False        # low-precision GEMM numerics over fp32 tensors (the emulation that runs on a CPU)

    def __post_init__(self):
        alias = {"float32": "fp32", "bfloat16": "bf16", "nvfp4": "fp4", "float8": "fp8"}
        self.name = alias.get(self.name, self.name)
        if self.name in ("fp8b", "fp8_block"):          # fp8 with per-128 block scales instead of per-tensor delayed scaling
            self.name, self.fp8_block_scales = "fp8", True
        if self.name not in ("fp32", "tf32", "bf16", "fp8", "fp4"):
            raise ValueError(f"unknown precision {self.name!r}")
        if self.name == "fp8" and os.environ.get("LLMM_FP8_BLOCK", "") not in ("", "0"):
            self.fp8_block_scales = True

    @property
    def storage(self) -> torch.dtype:
        return torch.float32 if self.name in ("fp32", "tf32") or self.fp32_storage else torch.bfloat16

    @property
    def use_master(self) -> bool:
        return self.storage != torch.float32

    @property
    def lowp(self) -> bool:
        return self.name in ("fp8", "fp4")

    @property
    def checkpoint_version(self) -> int:
        return 3 if self.storage == torch.float32 else 5

    def layer_in_fp4_range(self, layer: int, num_layer: int) -> bool:
        return self.name == "fp4" and self.fp4_first <= layer < num_layer - self.fp4_last_offset
