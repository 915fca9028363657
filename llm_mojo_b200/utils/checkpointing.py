"""llm.c-compatible model and optimizer-state checkpoints.

Parity: ``llmm/checkpointing.mojo:25-37`` (magics/versions), ``:148-184`` (model file:
256×int32 header ``[0]`` 20240520 ``[1]`` 3=fp32 / 5=bf16 ``[2]`` maxT ``[3]`` V ``[4]`` L
``[5]`` NH ``[6]`` C ``[7]`` Vp, then the 16 tensors in llm.c order), ``:266-305`` (state file:
magic 20240527 v1, ``[2]`` nproc ``[3]`` rank ``[4]`` use_master ``[5]`` shuffle ``[10]`` step,
u64 slots 10/11/15/16 = sampler RNG, shuffle draws, shard idx, sample idx; then the rank's
m and v shards as fp32 — no master copy, it is re-seeded from the parameters on load).
"""
from __future__ import annotations

import os
import re
import struct
from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np
import torch

from ..config import GPT2Config, MODEL_MAGIC

CHECKPOINT_HEADER_SIZE = 256
VERSION_FP32 = 3
VERSION_BF16 = 5
STATE_MAGIC = 20240527
STATE_VERSION = 1


@dataclass
class TrainingState:
    step: int = 0
    num_processes: int = 1
    process_rank: int = 0
    use_master_weights: int = 0
    should_shuffle: int = 0
    sampler_rng_state: int = 0
    shuffle_rng_state: int = 0
    current_shard_idx: int = 0
    current_sample_idx: int = 0


def _tensor_bytes(t: torch.Tensor) -> bytes:
    t = t.detach().contiguous().cpu()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().tobytes()
    return t.numpy().tobytes()


def write_model_checkpoint(path: str, config: GPT2Config, params_flat: torch.Tensor,
                           version: Optional[int] = None) -> None:
    """Write header + flat parameters. ``version`` defaults from the dtype (3 fp32, 5 bf16)."""
    if version is None:
        version = VERSION_BF16 if params_flat.dtype in (torch.bfloat16, torch.float16) else VERSION_FP32
    want = torch.float32 if version == VERSION_FP32 else torch.bfloat16
    n = config.num_parameters()
    if params_flat.numel() < n:
        raise ValueError(f"Checkpoint error: params buffer too small (need {n}, got {params_flat.numel()})")
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<256i", *config.header(version)))
        flat = params_flat[:n]
        chunk = 1 << 26
        for i in range(0, n, chunk):
            f.write(_tensor_bytes(flat[i:i + chunk].to(want)))
    os.replace(tmp, path)


def read_model_header(path: str) -> Tuple[GPT2Config, int]:
    with open(path, "rb") as f:
        raw = f.read(1024)
    if len(raw) < 1024:
        raise ValueError("Checkpoint error: header is too short")
    h = struct.unpack("<256i", raw)
    if h[0] != MODEL_MAGIC:
        raise ValueError(f"Checkpoint error: bad model magic number in header: {h[0]}")
    if h[1] not in (VERSION_FP32, VERSION_BF16):
        raise ValueError(f"Checkpoint error: unsupported model version in header: {h[1]}")
    return GPT2Config(h[2], h[3], h[4], h[5], h[6], h[7]), h[1]


def read_model_checkpoint(path: str, dtype: Optional[torch.dtype] = None,
                          offset: int = 0, count: Optional[int] = None) -> Tuple[GPT2Config, int, torch.Tensor]:
    """Read (a slice ``[offset, offset+count)`` of) the flat parameter vector.

    The slice form lets a ZeRO-3 rank load only the range it owns
    (``train_gpt2.mojo:5719-5738``)."""
    config, version = read_model_header(path)
    n = config.num_parameters()
    count = n - offset if count is None else count
    if offset < 0 or offset + count > n:
        raise ValueError("Checkpoint error: slice outside the parameter vector")
    esz = 4 if version == VERSION_FP32 else 2
    npdt = np.float32 if version == VERSION_FP32 else np.int16
    arr = np.fromfile(path, dtype=npdt, count=count, offset=1024 + offset * esz)
    if arr.size < count:
        raise ValueError("Checkpoint error: truncated parameter payload")
    t = torch.from_numpy(arr)
    if version == VERSION_BF16:
        t = t.view(torch.bfloat16)
    if dtype is not None:
        t = t.to(dtype)
    return config, version, t


def write_state_checkpoint(path: str, state: TrainingState, m: torch.Tensor, v: torch.Tensor) -> None:
    header = [0] * 256
    header[0], header[1] = STATE_MAGIC, STATE_VERSION
    header[2], header[3] = state.num_processes, state.process_rank
    header[4], header[5] = state.use_master_weights, state.should_shuffle
    header[10] = state.step
    raw = bytearray(struct.pack("<256i", *header))
    struct.pack_into("<Q", raw, 10 * 8, state.sampler_rng_state & (2 ** 64 - 1))
    struct.pack_into("<Q", raw, 11 * 8, state.shuffle_rng_state & (2 ** 64 - 1))
    struct.pack_into("<Q", raw, 15 * 8, state.current_shard_idx)
    struct.pack_into("<Q", raw, 16 * 8, state.current_sample_idx)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(raw)
        f.write(_tensor_bytes(m.float()))
        f.write(_tensor_bytes(v.float()))
    os.replace(tmp, path)


def read_state_header(path: str) -> TrainingState:
    with open(path, "rb") as f:
        raw = f.read(1024)
    if len(raw) < 1024:
        raise ValueError("Checkpoint error: state header is too short")
    h = struct.unpack("<256i", raw)
    if h[0] != STATE_MAGIC:
        raise ValueError(f"Checkpoint error: bad state magic number in header: {h[0]}")
    if h[1] != STATE_VERSION:
        raise ValueError(f"Checkpoint error: unsupported state version in header: {h[1]}")
    u = struct.unpack("<128Q", raw)
    return TrainingState(step=h[10], num_processes=h[2], process_rank=h[3], use_master_weights=h[4],
                         should_shuffle=h[5], sampler_rng_state=u[10], shuffle_rng_state=u[11],
                         current_shard_idx=u[15], current_sample_idx=u[16])


def read_state_checkpoint(path: str, shard_num_parameters: int) -> Tuple[TrainingState, torch.Tensor, torch.Tensor]:
    state = read_state_header(path)
    arr = np.fromfile(path, dtype=np.float32, count=2 * shard_num_parameters, offset=1024)
    if arr.size < 2 * shard_num_parameters:
        raise ValueError("Checkpoint error: truncated optimizer state payload")
    t = torch.from_numpy(arr)
    return state, t[:shard_num_parameters], t[shard_num_parameters:]


def find_max_step(output_dir: str) -> int:
    """Highest N with ``model_N.bin`` present, −1 if none (``train_gpt2.mojo:6130-6147``)."""
    best = -1
    if not output_dir or not os.path.isdir(output_dir):
        return best
    for name in os.listdir(output_dir):
        m = re.fullmatch(r"model_(\d+)\.bin", name)
        if m:
            best = max(best, int(m.group(1)))
    return best


def model_path(output_dir: str, step: int) -> str:
    return os.path.join(output_dir, f"model_{step}.bin")


def state_path(output_dir: str, step: int, rank: int) -> str:
    return os.path.join(output_dir, f"state_{step}_{rank}.bin")
