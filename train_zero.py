#!/usr/bin/env python
"""train_zero — launch a ZeRO run from a ``zero/zeroN.json`` config (``scripts/train_zero.py:25-76``
in the reference): reads {zero_stage, world_size, precision, train_flags}, then starts one
``train_gpt2.py`` process per GPU under torchrun with ``-z <stage>`` and the listed flags."""
from __future__ import annotations

import json
import os
import subprocess
import sys


def build_command(config_path: str, extra):
    with open(config_path) as f:
        cfg = json.load(f)
    world = int(cfg.get("world_size", 1))
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1", "--nnodes=1",
           f"--nproc-per-node={world}", os.path.join(here, "train_gpt2.py"), "-z", str(cfg.get("zero_stage", 0)),
           "--precision", cfg.get("precision", "bf16")]
    for k, v in cfg.get("train_flags", {}).items():
        cmd += ["-" + k if not k.startswith("-") else k, str(v)]
    return cmd + list(extra), world


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if not argv:
        print("usage: train_zero.py zero/zeroN.json [extra train_gpt2 flags]")
        return 2
    cmd, _ = build_command(argv[0], argv[1:])
    print(" ".join(cmd), flush=True)
    return subprocess.call(cmd)


if __name__ == "__main__":
    sys.exit(main())
