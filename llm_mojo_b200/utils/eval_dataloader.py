"""Multiple-choice eval loader (HellaSwag format) and the accuracy statistic.

Parity: ``llmm/eval_dataloader.mojo:30-323`` and ``data/utils.py:101-165``: header magic
20240522 v1, ``[2]`` = examples, ``[3]`` = longest example bytes; per example a uint16 stream
``<65535><bytes><index><label><ncompl><nctx><ctx…>(<n><completion…>)×4``.  A batch holds
``B // 4`` examples, 4 rows each; ``mask`` marks the completion positions of ``targets``.
"""
from __future__ import annotations

import struct
from typing import Sequence

import numpy as np
import torch

EVAL_MAGIC = 20240522
EVAL_VERSION = 1
ASSUMED_NUM_COMPLETIONS = 4
START_EXAMPLE_DELIM = 65535


def write_evalfile(filename: str, datum: Sequence[dict]) -> None:
    header = np.zeros(256, dtype=np.int32)
    header[0], header[1], header[2] = EVAL_MAGIC, EVAL_VERSION, len(datum)
    assert len(datum) < 2 ** 16, "Too many examples"
    full, longest = [], 0
    for idx, d in enumerate(datum):
        s = [START_EXAMPLE_DELIM, 0, idx, d["label"], len(d["ending_tokens"]), len(d["ctx_tokens"])]
        assert len(d["ending_tokens"]) == ASSUMED_NUM_COMPLETIONS
        s.extend(d["ctx_tokens"])
        for e in d["ending_tokens"]:
            s.append(len(e))
            s.extend(e)
        nbytes = len(s) * 2
        assert nbytes < 2 ** 16, "Example too long"
        s[1] = nbytes
        longest = max(longest, nbytes)
        full.extend(s)
    header[3] = longest
    with open(filename, "wb") as f:
        f.write(header.tobytes())
        f.write(np.asarray(full, dtype=np.uint16).tobytes())


class EvalDataLoader:
    def __init__(self, filename: str, batch_size: int, seq_len: int,
                 process_rank: int = 0, num_processes: int = 1):
        self.process_rank, self.num_processes = process_rank, num_processes
        self.batch_size, self.seq_len = batch_size, seq_len
        if batch_size // ASSUMED_NUM_COMPLETIONS == 0:
            raise ValueError(f"EvalDataLoader error: batch size {batch_size} is < "
                             f"{ASSUMED_NUM_COMPLETIONS} (HINT: increase batch size, e.g. -b 16)")
        self.can_fit_examples = batch_size // ASSUMED_NUM_COMPLETIONS
        self.f = open(filename, "rb")
        raw = self.f.read(1024)
        if len(raw) < 1024:
            raise ValueError(f"EvalDataLoader error: header is too short in file {filename}")
        header = struct.unpack("<256i", raw)
        if header[0] != EVAL_MAGIC:
            raise ValueError(f"EvalDataLoader error: bad magic number in {filename}")
        if header[1] != EVAL_VERSION:
            raise ValueError(f"EvalDataLoader error: bad version in {filename}")
        self.num_examples, self.longest_example_bytes = header[2], header[3]
        if self.num_examples < num_processes:
            raise ValueError(f"EvalDataLoader error: fewer examples ({self.num_examples}) than "
                             f"processes ({num_processes})")
        n = batch_size * seq_len
        self.inputs = torch.zeros(n, dtype=torch.int32)
        self.targets = torch.zeros(n, dtype=torch.int32)
        self.mask = torch.zeros(n, dtype=torch.uint8)
        self.label = torch.zeros(self.can_fit_examples, dtype=torch.int32)
        self.reset()

    def reset(self) -> None:
        per = (self.num_examples + self.num_processes - 1) // self.num_processes
        self.num_batches = (per + self.can_fit_examples - 1) // self.can_fit_examples
        self.start_example_index = per * self.process_rank
        self.end_example_index = min(per * (self.process_rank + 1), self.num_examples)
        self.f.seek(1024)
        for i in range(self.start_example_index):
            self._read_example_payload(i)
        self.current_example_index = self.start_example_index

    def _read_example_payload(self, expected_index: int) -> np.ndarray:
        sub = self.f.read(6)
        if len(sub) < 6:
            raise ValueError("EvalDataLoader error: truncated example sub-header")
        delim, nbytes, index = struct.unpack("<3H", sub)
        if delim != START_EXAMPLE_DELIM:
            raise ValueError("EvalDataLoader error: bad <START_EXAMPLE> delimiter")
        if index != expected_index:
            raise ValueError(f"EvalDataLoader error: <EXAMPLE_INDEX> mismatch (expected "
                             f"{expected_index}, got {index})")
        payload = nbytes - 6
        if payload <= 0:
            raise ValueError("EvalDataLoader error: non-positive example payload size")
        raw = self.f.read(payload)
        if len(raw) < payload:
            raise ValueError("EvalDataLoader error: truncated example payload")
        return np.frombuffer(raw, dtype=np.uint16).astype(np.int64)

    def _next_example(self, slot: int) -> None:
        T = self.seq_len
        base = slot * ASSUMED_NUM_COMPLETIONS
        buf = self._read_example_payload(self.current_example_index)
        label = int(buf[0])
        if not 0 <= label < ASSUMED_NUM_COMPLETIONS:
            raise ValueError("EvalDataLoader error: label out of range")
        self.label[slot] = label
        if int(buf[1]) != ASSUMED_NUM_COMPLETIONS:
            raise ValueError(f"EvalDataLoader error: expected {ASSUMED_NUM_COMPLETIONS} "
                             f"completions, got {int(buf[1])}")
        ctx_len = int(buf[2])
        if ctx_len <= 0 or ctx_len >= T:
            raise ValueError(f"EvalDataLoader error: context_length out of range (T={T})")
        inp, tgt, msk = self.inputs.numpy(), self.targets.numpy(), self.mask.numpy()
        ctx = buf[3:3 + ctx_len]
        cursor = 3 + ctx_len
        for c in range(ASSUMED_NUM_COMPLETIONS):
            row = (base + c) * T
            inp[row:row + ctx_len] = ctx
            n = int(buf[cursor])
            if n <= 0 or ctx_len + n > T:
                raise ValueError(f"EvalDataLoader error: completion doesn't fit in T={T}")
            comp = buf[cursor + 1:cursor + 1 + n]
            inp[row + ctx_len:row + ctx_len + n] = comp
            tgt[row + ctx_len - 1:row + ctx_len - 1 + n] = comp
            msk[row + ctx_len - 1:row + ctx_len - 1 + n] = 1
            cursor += 1 + n
        self.current_example_index += 1

    def next_batch(self) -> None:
        self.mask.zero_()
        for i in range(self.can_fit_examples):
            if self.current_example_index >= self.end_example_index:
                break
            self._next_example(i)

    def close(self) -> None:
        self.f.close()


def eval_stat_correct(loader: EvalDataLoader, losses: torch.Tensor) -> int:
    """Examples of the current batch whose lowest masked-mean-loss completion is the label
    (``llmm/eval_dataloader.mojo:290``)."""
    B, T = loader.batch_size, loader.seq_len
    losses = losses.detach().float().cpu().reshape(B, T)
    mask = loader.mask.reshape(B, T).float()
    tot = (losses * mask).sum(1)
    cnt = mask.sum(1)
    avg = torch.where(cnt > 0, tot / cnt.clamp(min=1), torch.zeros_like(tot))
    correct = 0
    for i in range(loader.can_fit_examples):
        rows = slice(i * ASSUMED_NUM_COMPLETIONS, (i + 1) * ASSUMED_NUM_COMPLETIONS)
        if cnt[rows].sum() == 0:
            continue
        if int(torch.argmin(avg[rows])) == int(loader.label[i]):
            correct += 1
    return correct
