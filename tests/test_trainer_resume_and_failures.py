"""Trainer paths around checkpoints and failures, all on the host:

* checkpoint + resume over real token shards while the loader has a batch prefetched (the resumed run must read the
  batch the uninterrupted run read and reproduce its loss);
* a Gloo rank that fails between steps: its peers' next step raises ``PeerAborted`` within seconds instead of
  hanging (after the reference's abort-flag liveness tests, ``tests/test_zero.mojo:254-314``).
"""
import multiprocessing as mp
import os
import socket
import sys
import time

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from llm_mojo_b200.trainer import TrainArgs, Trainer
from llm_mojo_b200.utils.dataloader import DataLoader, write_datafile


def _shards(tmp_path, n=3, ntok=2000):
    rng = np.random.default_rng(7)
    for i in range(n):
        write_datafile(str(tmp_path / f"train_{i:03d}.bin"), rng.integers(0, 50257, size=ntok, dtype=np.uint16))
    return str(tmp_path / "train_*.bin")


def test_loader_state_is_valid_while_a_batch_is_prefetched(tmp_path):
    pattern = _shards(tmp_path)
    a = DataLoader(pattern, 2, 32, should_shuffle=True, pin_memory=False)
    seq = []
    for _ in range(5):
        a.next_batch()
        a.prefetch()
    st = a.state()                                     # a prefetch is pending: must not raise
    for _ in range(40):                                # crosses shard boundaries and a full reshuffle
        x, _ = a.next_batch()
        a.prefetch()
        seq.append(x.clone())
    b = DataLoader(pattern, 2, 32, should_shuffle=True, pin_memory=False)
    b.restore(st["should_shuffle"], st["shuffle_draws"], st["current_shard_idx"], st["current_sample_idx"])
    for want in seq:
        x, _ = b.next_batch()
        b.prefetch()
        assert torch.equal(x, want)


def test_trainer_checkpoint_and_resume_over_shards(tmp_path):
    pattern = _shards(tmp_path)
    out = tmp_path / "log"

    def make(resume):
        return Trainer(TrainArgs(train_data_pattern=pattern, val_data_pattern="", load_filename="d6", batch_size=2,
                                 seq_len=32, total_batch_size=128, max_steps=6, learning_rate=1e-3, device="cpu",
                                 precision="fp32", val_loss_every=0, sample_every=0, checkpoint_every=1,
                                 output_log_dir=str(out), resume=resume))

    a = make(0)
    for _ in range(2):
        a.train_step()
    a.save(2)                                          # the loader has prefetched the next batch at this point
    want_x = None
    r3 = a.train_step()
    b = make(1)
    assert b.step == 2
    x, _ = b.train_loader.next_batch()
    a2 = DataLoader(pattern, 2, 32, should_shuffle=True, pin_memory=False)
    for _ in range(2 * 2 + 1):                         # two steps of grad_accum 2, then the first batch of step 3
        want_x, _ = a2.next_batch()
    assert torch.equal(x, want_x)
    c = make(1)
    r3b = c.train_step()
    assert abs(r3b["loss"] - r3["loss"]) < 1e-5, (r3b["loss"], r3["loss"])


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _failing_rank_worker(rank, W, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), LLMM_USE_CPU="1")
    from llm_mojo_b200.parallel.runtime import PeerAborted, init_distributed, shutdown_distributed
    ctx = init_distributed(rank, W, backend="gloo", timeout_s=30)
    try:
        tr = Trainer(TrainArgs(load_filename="d6", batch_size=1, seq_len=16, total_batch_size=16 * W, max_steps=10,
                               device="cpu", precision="fp32", synthetic=True, val_loss_every=0, sample_every=0),
                     rank, W, dist_ctx=ctx)
        tr.train_step()
        if rank == 1:
            try:
                raise RuntimeError("injected failure between steps")
            except RuntimeError as e:
                tr.abort(str(e))
                q.put((rank, "raised", 0.0))
                return
        time.sleep(1.0)                                # let the abort key land; the poll at step start then sees it
        t0 = time.monotonic()
        try:
            tr.train_step()
            q.put((rank, "stepped", time.monotonic() - t0))
        except PeerAborted:
            q.put((rank, "aborted", time.monotonic() - t0))
    finally:
        shutdown_distributed(ctx)


def test_failed_rank_stops_its_peers_at_their_next_step():
    W = 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_failing_rank_worker, args=(r, W, port, q)) for r in range(W)]
    for p in procs:
        p.start()
    seen = [q.get(timeout=240) for _ in range(W)]
    for p in procs:
        p.join(timeout=60)
        assert not p.is_alive()
    got = {r: (what, dt) for r, what, dt in seen}
    assert got[1][0] == "raised"
    for r in (0, 2):
        assert got[r][0] == "aborted" and got[r][1] < 5.0, got
