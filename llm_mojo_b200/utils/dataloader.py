"""Token-shard data loader (llm.c ``.bin`` shards) with per-rank strided batches.

Parity: ``llmm/dataloader.mojo:13-19`` (header: 256×int32, magic 20240520 → uint16 tokens,
20240801 → uint32; ``[2]`` = token count), ``:65-390`` (batch = B·T+1 tokens starting at
``header + idx·W·B·T + rank·B·T``; optional shard permutation + intra-shard permutation drawn
from MT19937 seeded ``42 + rank``; draw counting for exact resume).

B200-first additions: batches are produced into *pinned* host tensors so the trainer can
issue an asynchronous H2D copy, and ``prefetch()`` reads the next batch on a worker thread
while the GPU runs the current micro-step.  A pinned buffer is only rewritten once the
host-to-device copies that read it have run: the consumer calls ``mark_consumed()`` right after
it has enqueued those copies, which records a CUDA event for the buffer, and the producer
waits for that event (on the worker thread, so the training thread is not blocked) before it
writes into the buffer again.  ``state()`` may be called while a batch is prefetched: it then
reports the position from which that batch was produced, so a resumed run reads it again.
"""
from __future__ import annotations

import glob
import os
import struct
import threading
from typing import List, Optional, Sequence

import numpy as np
import torch

from .rand import MT19937, random_permutation

HEADER_SIZE = 256
GPT2_MAGIC = 20240520
LLAMA3_MAGIC = 20240801
RNG_SEED = 42


def resolve_data_files(pattern: str) -> List[str]:
    """Sorted glob expansion (``llmm/dataloader.mojo:27-57``)."""
    files = sorted(glob.glob(pattern))
    if not files:
        raise FileNotFoundError(f"DataLoader error: no files match pattern {pattern}")
    return files


def write_datafile(filename: str, tokens: Sequence[int] | np.ndarray, model_desc: str = "gpt-2") -> None:
    """Write a token shard (``data/utils.py:72-98``)."""
    magic, version, dt = {"gpt-2": (GPT2_MAGIC, 1, np.uint16),
                          "llama-3": (LLAMA3_MAGIC, 7, np.uint32)}[model_desc]
    assert len(tokens) < 2 ** 31, "Too many tokens"
    header = np.zeros(HEADER_SIZE, dtype=np.int32)
    header[0], header[1], header[2] = magic, version, len(tokens)
    with open(filename, "wb") as f:
        f.write(header.tobytes())
        f.write(np.asarray(tokens, dtype=dt).tobytes())


class DataLoader:
    def __init__(self, files: str | Sequence[str], batch_size: int, seq_len: int,
                 process_rank: int = 0, num_processes: int = 1, should_shuffle: bool = False,
                 pin_memory: Optional[bool] = None):
        if isinstance(files, str):
            files = resolve_data_files(files)
        self.files = list(files)
        if not self.files:
            raise ValueError("DataLoader error: empty file list")
        self.process_rank, self.num_processes = process_rank, num_processes
        self.batch_size, self.seq_len = batch_size, seq_len
        self.should_shuffle = should_shuffle
        self.shuffle_rng = MT19937(RNG_SEED + process_rank)
        self.shuffle_draws = 0
        self.shard_indices = list(range(len(self.files)))
        self.intra_shard_indices: List[int] = []
        self.current_shard_idx = 0
        self.current_sample_idx = 0
        self.header_bytes = HEADER_SIZE * 4
        self._fd: Optional[int] = None
        pin = torch.cuda.is_available() if pin_memory is None else pin_memory
        n = batch_size * seq_len
        self._bufs = [(torch.empty(n, dtype=torch.int32, pin_memory=pin),
                       torch.empty(n, dtype=torch.int32, pin_memory=pin)) for _ in range(2)]
        self._cur = 0
        self._prefetch_thread: Optional[threading.Thread] = None
        self._prefetched = False
        self._pre_state: Optional[dict] = None          # position before the prefetched batch was produced
        self._copy_events = [None, None]                # per buffer: CUDA event after the H2D copies that read it
        self._copy_pending = [False, False]
        self.inputs, self.targets = self._bufs[0]

        self._open(self.files[0])
        self.total_batch_size_bytes = num_processes * n * self.token_size
        self.local_batch_offset_bytes = process_rank * n * self.token_size
        num_tokens = 0
        for i in range(len(self.files)):
            ntok = self._load_shard(i)
            need = num_processes * n + 1
            if ntok < need:
                raise ValueError(f"DataLoader error: Shard is too small for batch size (need {need} tokens, got {ntok})")
            num_tokens += ntok
        self.num_tokens = num_tokens
        self.reset()

    # -- shard handling --------------------------------------------------------------
    def _open(self, filename: str) -> None:
        if self._fd is not None:
            os.close(self._fd)
        self._fd = os.open(filename, os.O_RDONLY)
        raw = os.pread(self._fd, self.header_bytes, 0)
        if len(raw) < self.header_bytes:
            raise ValueError(f"DataLoader error: Header is too short in file {filename}")
        header = struct.unpack("<256i", raw)
        self.magic, self.version = header[0], header[1]
        if self.magic == GPT2_MAGIC:
            self.token_size, self._np_dtype = 2, np.uint16
        elif self.magic == LLAMA3_MAGIC:
            self.token_size, self._np_dtype = 4, np.uint32
        else:
            raise ValueError(f"DataLoader error: Invalid magic number in header: {self.magic}")
        self.current_shard_tokens = header[2]

    def _load_shard(self, shard_index: int) -> int:
        actual = self.shard_indices[shard_index] if self.should_shuffle else shard_index
        self._open(self.files[actual])
        self.file_size_bytes = self.header_bytes + self.current_shard_tokens * self.token_size
        self.shard_num_samples = (self.current_shard_tokens * self.token_size - self.token_size) \
            // self.total_batch_size_bytes
        return self.current_shard_tokens

    def _prepare_intra_shard_indices(self) -> None:
        self.intra_shard_indices = list(range(self.shard_num_samples))
        random_permutation(self.intra_shard_indices, self.shuffle_rng)
        if len(self.intra_shard_indices) > 1:
            self.shuffle_draws += len(self.intra_shard_indices) - 1

    def reset(self) -> None:
        self._join_prefetch(discard=True)
        self.current_shard_idx = 0
        self.current_sample_idx = 0
        if self.should_shuffle:
            random_permutation(self.shard_indices, self.shuffle_rng)
            if len(self.shard_indices) > 1:
                self.shuffle_draws += len(self.shard_indices) - 1
        self._load_shard(self.current_shard_idx)
        if self.should_shuffle:
            self._prepare_intra_shard_indices()

    def _advance(self) -> None:
        if self.current_shard_idx == len(self.files) - 1:
            self.reset()
            return
        self.current_shard_idx = (self.current_shard_idx + 1) % len(self.files)
        self.current_sample_idx = 0
        self._load_shard(self.current_shard_idx)
        if self.should_shuffle:
            self._prepare_intra_shard_indices()

    # -- batches ---------------------------------------------------------------------
    def _load_batch_into(self, inputs: torch.Tensor, targets: torch.Tensor) -> None:
        idx = self.intra_shard_indices[self.current_sample_idx] if self.should_shuffle \
            else self.current_sample_idx
        off = self.header_bytes + idx * self.total_batch_size_bytes + self.local_batch_offset_bytes
        n = self.batch_size * self.seq_len
        nbytes = (n + 1) * self.token_size
        raw = os.pread(self._fd, nbytes, off)
        if len(raw) < nbytes:
            raise ValueError("DataLoader error: Failed to read enough bytes from file")
        toks = np.frombuffer(raw, dtype=self._np_dtype).astype(np.int32)
        inputs.numpy()[:] = toks[:-1]
        targets.numpy()[:] = toks[1:]

    def _produce(self, slot: int) -> None:
        if self.current_sample_idx >= self.shard_num_samples:
            self._advance()
        if self._copy_pending[slot]:                    # the device may not have read the old contents yet
            self._copy_events[slot].synchronize()
            self._copy_pending[slot] = False
        self._load_batch_into(*self._bufs[slot])
        self.current_sample_idx += 1

    def mark_consumed(self) -> None:
        """Call right after enqueuing the asynchronous host-to-device copies of the current batch (on the
        stream that carries them): the buffer is not rewritten before those copies have run.  The events
        are created once per buffer and reused, so steady-state steps allocate nothing."""
        if not (torch.cuda.is_available() and self._bufs[self._cur][0].is_pinned()):
            return
        if self._copy_events[self._cur] is None:
            self._copy_events[self._cur] = torch.cuda.Event()
        self._copy_events[self._cur].record()
        self._copy_pending[self._cur] = True

    def _snapshot(self) -> dict:
        return {"should_shuffle": int(self.should_shuffle), "shuffle_draws": self.shuffle_draws,
                "current_shard_idx": self.current_shard_idx, "current_sample_idx": self.current_sample_idx}

    def _join_prefetch(self, discard: bool = False) -> None:
        if self._prefetch_thread is not None:
            self._prefetch_thread.join()
            self._prefetch_thread = None
        if discard:
            self._prefetched = False

    def prefetch(self) -> None:
        """Read the next batch into the idle buffer on a worker thread."""
        if self._prefetched or self._prefetch_thread is not None:
            return
        slot = 1 - self._cur
        self._pre_state = self._snapshot()
        self._prefetch_thread = threading.Thread(target=self._produce, args=(slot,), daemon=True)
        self._prefetch_thread.start()
        self._prefetched = True

    def next_batch(self):
        """Advance; afterwards ``inputs``/``targets`` (host int32 ``[B·T]``) hold the batch."""
        if self._prefetched:
            self._join_prefetch()
            self._prefetched = False
            self._cur = 1 - self._cur
        else:
            self._produce(self._cur)
        self.inputs, self.targets = self._bufs[self._cur]
        return self.inputs, self.targets

    # -- resume ----------------------------------------------------------------------
    def state(self) -> dict:
        """Position of the next batch ``next_batch()`` will return.  With a batch already prefetched that is the
        position the prefetch started from (a shard change it triggered is replayed by ``restore`` + the next read)."""
        self._join_prefetch()
        if self._prefetched:
            return dict(self._pre_state)
        return self._snapshot()

    def restore(self, should_shuffle: int, shuffle_draws: int, current_shard_idx: int,
                current_sample_idx: int) -> None:
        """Reposition so that the next batch equals the one the saved run would produce
        (``llmm/checkpointing.mojo:392-423``): reseed, replay the draws that preceded the
        current shard's intra permutation, regenerate that permutation."""
        self._join_prefetch(discard=True)
        if self.should_shuffle and should_shuffle == 1:
            # the shard permutation is part of the replayed stream: rebuild it first
            self.shuffle_rng = MT19937(RNG_SEED + self.process_rank)
            self.shard_indices = list(range(len(self.files)))
            self.current_shard_idx = current_shard_idx
            self._load_shard_after_replay(shuffle_draws, current_shard_idx)
        else:
            self.current_shard_idx = current_shard_idx
            self._load_shard(current_shard_idx)
            if self.should_shuffle:
                self._prepare_intra_shard_indices()
        self.current_sample_idx = current_sample_idx

    def _load_shard_after_replay(self, shuffle_draws: int, shard_idx: int) -> None:
        # Replay the stream structurally: (shard perm, intra perm)* until the draw count of
        # the state *before* the current intra permutation is reached.
        nshards = len(self.files)
        draws = 0
        while True:
            pass_start = draws
            random_permutation(self.shard_indices, self.shuffle_rng)
            draws += max(nshards - 1, 0)
            for s in range(nshards):
                self.current_shard_idx = s
                self._load_shard(s)
                intra = max(self.shard_num_samples - 1, 0)
                if draws + intra == shuffle_draws and s == shard_idx:
                    self.shuffle_draws = draws
                    self._prepare_intra_shard_indices()
                    return
                for _ in range(intra):
                    self.shuffle_rng.randint32()
                draws += intra
                if draws > shuffle_draws:
                    raise ValueError("DataLoader error: shuffle state does not match these shards")
            if draws == pass_start:
                raise ValueError("DataLoader error: shuffle state does not match these shards")

    def close(self) -> None:
        self._join_prefetch()
        if self._fd is not None:
            os.close(self._fd)
            self._fd = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
