#!/usr/bin/env python
"""train_gpt2 — llm.c-style command line of the trainer (one process per GPU).

Same flags as the reference binary (``train_gpt2.mojo:6649-6777``): -i -j -e -o -n -y -b -t -d -l
-k -u -q -c -v -m -s -g -a -x -z -pn -pr, and the environment variables RANK, WORLD_SIZE,
ZERO_STAGE, LLMM_OUTPUT_DIR, LLMM_SAVE_EVERY, LLMM_USE_CPU, LLMM_RECOMPUTE, LLMM_MEM_REPORT,
LLMM_TRACE.  Axes that are compile-time defines in the reference are runtime options here:
``--precision fp32|tf32|bf16|fp8|fp8b|fp4``, ``--synthetic``, ``--comm p2p|nccl|gloo``.

Multi-GPU: ``torchrun --nproc-per-node N train_gpt2.py -z 1 ...`` (rank/world from the env), or
``-pn N`` on a single command line, which re-launches this script under torchrun.
"""
from __future__ import annotations

import os
import subprocess
import sys

USAGE = """Usage: python train_gpt2.py [options]
Options (mirroring Karpathy's train_gpt2.cu):
  -h, --help  print this help message and exit
  -i <string> train data filename pattern (glob ok)
  -j <string> val data filename pattern (glob ok)
  -e <string> input .bin / .safetensors filename OR model descriptor (dX / gpt2:dX / gpt3:cX) to train from scratch
  -o <string> output log/checkpoint dir (default = none)
  -n <int>    write a checkpoint every N steps (default 0)
  -y <int>    resume from latest checkpoint in -o? (0/1)
  -b <int>    (micro) batch size B (default = 4)
  -t <int>    sequence length T (default = 1024)
  -d <int>    total desired batch size (default = B*T*num_processes)
  -l <float>  learning rate (default = 3e-4)
  -k <string> learning rate scheduler cosine|linear|constant|wsd (default = cosine)
  -u <int>    learning rate warmup iterations (default = 0)
  -q <float>  final learning rate fraction (default = 1.0)
  -c <float>  weight decay (default = 0.0)
  -v <int>    val_loss_every (default = 20)
  -m <int>    val_max_steps (default = 20)
  -s <int>    sample_every (default = 20)
  -g <int>    genT, tokens of inference to generate (default = 64)
  -a <int>    overfit a single batch? 0/1 (default = 0)
  -x <int>    max_steps (-1 = one epoch, default)
  -z <int>    zero_stage, ZeRO optimization stage 0/1/2/3 (default 0)
  -pn <int>   num_processes / world_size (default = 1)
  -pr <int>   process_rank (default = 0)
  --precision <fp32|tf32|bf16|fp8|fp8b|fp4>   (default bf16 on GPU, fp32 on CPU; fp8b = fp8 with per-128 block scales)
  --fp8-static-scales <json>  with --precision fp8: fixed scales from calibrate_fp8_scales.py instead of delayed scaling
  --synthetic 1     train on uniform random tokens (no data files needed)
  --comm <auto|p2p|nccl|gloo>  collective backend (default auto: peer-memory kernels on GPUs)
  --config <zero json>  read {zero_stage, world_size, precision, train_flags} from a zero/zeroN.json
"""

_FLAGS = {
    "-i": ("train_data_pattern", str), "-j": ("val_data_pattern", str), "-e": ("load_filename", str),
    "-o": ("output_log_dir", str), "-n": ("checkpoint_every", int), "-y": ("resume", int),
    "-b": ("batch_size", int), "-t": ("seq_len", int), "-d": ("total_batch_size", int),
    "-l": ("learning_rate", float), "-k": ("lr_scheduler_type", str), "-u": ("warmup_iterations", int),
    "-q": ("final_learning_rate_frac", float), "-c": ("weight_decay", float), "-v": ("val_loss_every", int),
    "-m": ("val_max_steps", int), "-s": ("sample_every", int), "-g": ("gen_tokens", int),
    "-a": ("overfit_single_batch", int), "-x": ("max_steps", int), "-z": ("zero_stage", int),
    "--precision": ("precision", str), "--synthetic": ("synthetic", lambda v: bool(int(v))),
    "--comm": ("comm_backend", str), "--grad-clip": ("grad_clip", float), "--beta2": ("beta2", float),
    "--recompute": ("recompute", lambda v: bool(int(v))), "--fp8-static-scales": ("fp8_static_scales", str),
}


class UsageError(Exception):
    pass


def parse_train_args(argv, env=os.environ):
    """Returns (TrainArgs, rank, world_size) or None when help was requested."""
    from llm_mojo_b200.trainer import TrainArgs
    args = TrainArgs()
    rank = int(env["RANK"]) if env.get("RANK") else 0
    world = int(env["WORLD_SIZE"]) if env.get("WORLD_SIZE") else 1
    if env.get("ZERO_STAGE"):
        args.zero_stage = int(env["ZERO_STAGE"])
    if env.get("LLMM_OUTPUT_DIR"):
        args.output_log_dir = env["LLMM_OUTPUT_DIR"]
    if env.get("LLMM_SAVE_EVERY"):
        args.checkpoint_every = int(env["LLMM_SAVE_EVERY"])
    if env.get("LLMM_RECOMPUTE", "") not in ("", "0"):
        args.recompute = True
    explicit_pn = None
    i = 0
    while i < len(argv):
        flag = argv[i]
        if flag in ("-h", "--help"):
            print(USAGE)
            return None
        if i + 1 >= len(argv) or not flag.startswith("-") or len(flag) < 2:
            raise UsageError(f"invalid command-line usage near {flag!r}")
        val = argv[i + 1]
        if flag == "-pn":
            explicit_pn = int(val)
        elif flag == "-pr":
            rank = int(val)
        elif flag == "--config":
            import json
            with open(val) as f:
                cfg = json.load(f)
            args.zero_stage = int(cfg.get("zero_stage", args.zero_stage))
            if "precision" in cfg:
                args.precision = cfg["precision"]
            if "world_size" in cfg and explicit_pn is None and not env.get("WORLD_SIZE"):
                explicit_pn = int(cfg["world_size"])
            for k, v in cfg.get("train_flags", {}).items():
                key = "-" + k if not k.startswith("-") else k
                if key in _FLAGS:
                    name, conv = _FLAGS[key]
                    setattr(args, name, conv(v))
        elif flag in _FLAGS:
            name, conv = _FLAGS[flag]
            try:
                setattr(args, name, conv(val))
            except ValueError:
                raise UsageError(f"bad value {val!r} for {flag}") from None
        else:
            raise UsageError(f"Unknown flag: {flag}")
        i += 2
    if explicit_pn is not None and not env.get("WORLD_SIZE"):
        world = explicit_pn
    return args, rank, world, explicit_pn


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    try:
        parsed = parse_train_args(argv)
    except UsageError as e:
        print(e)
        print(USAGE)
        return 2
    if parsed is None:
        return 0
    args, rank, world, explicit_pn = parsed
    if explicit_pn and explicit_pn > 1 and not os.environ.get("WORLD_SIZE"):
        # -pn N on a plain command line: become the launcher (one process per GPU)
        cmd = [sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1",
               "--nnodes=1", f"--nproc-per-node={explicit_pn}", os.path.abspath(__file__)] + \
              [a for j, a in enumerate(argv) if not (a == "-pn" or (j > 0 and argv[j - 1] == "-pn"))]
        return subprocess.call(cmd)
    from llm_mojo_b200.parallel.runtime import init_distributed, shutdown_distributed
    from llm_mojo_b200.trainer import Trainer
    ctx = init_distributed(rank, world) if world > 1 else None
    try:
        trainer = Trainer(args, rank, world, dist_ctx=ctx)
        trainer.train()
    except BaseException:
        if ctx is not None:
            ctx.abort()          # peers waiting on this rank fail fast instead of hanging
        raise
    finally:
        if ctx is not None:
            shutdown_distributed(ctx)
    return 0


if __name__ == "__main__":
    sys.exit(main())
