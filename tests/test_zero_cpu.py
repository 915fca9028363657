"""ZeRO / DDP numerical equivalence and liveness on CPU ranks (Gloo).

After the reference's tests/test_zero_equivalence.mojo (stages 1/2/3 must reproduce the W=1
parameters after an optimizer step) and tests/test_zero.mojo:254-314 (a rank that raises must abort
its peers instead of hanging them) — here with real processes instead of simulated ranks."""
import os
import socket
import sys
import traceback

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from llm_mojo_b200.config import GPT2Config
from llm_mojo_b200.models import GPT2

CFG = GPT2Config(max_seq_len=16, vocab_size=60, num_layer=2, num_heads=2, channels=16, padded_vocab_size=64)


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _batch(B, T, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randint(0, CFG.vocab_size, (B, T + 1), generator=g, dtype=torch.int32)
    return x[:, :-1].contiguous(), x[:, 1:].contiguous()


def _train(model, xs, ys, steps, accum):
    """xs/ys: [steps*accum micro-batches]."""
    i = 0
    losses = []
    for step in range(1, steps + 1):
        for micro in range(accum):
            model.forward(xs[i], ys[i], accum)
            model.backward(accum, micro)
            i += 1
        norm = model.calculate_grad_norm()
        model.update(step, lr=1e-2, weight_decay=0.01, dev_scale=model.clip_scale_from_norm(norm, 1.0))
        losses.append(model.read_loss())
    return losses


def _baseline(W, steps, accum, Bp=2, T=8):
    """Single process on the concatenated batch of all ranks."""
    model = GPT2(CFG, "fp32", "cpu")
    xs, ys = [], []
    for i in range(steps * accum):
        parts = [_batch(Bp, T, seed=100 * r + i) for r in range(W)]
        xs.append(torch.cat([p[0] for p in parts]))
        ys.append(torch.cat([p[1] for p in parts]))
    losses = _train(model, xs, ys, steps, accum)
    return model.params.clone(), losses


def _worker(rank, W, port, stage, steps, accum, q, vocab_parallel=False):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=W)
        from llm_mojo_b200.parallel.zero import ZeroEngine
        eng = ZeroEngine(stage, rank, W, torch.device("cpu"), backend="gloo")
        model = GPT2(CFG, "fp32", "cpu", zero=eng, vocab_parallel=vocab_parallel)
        assert model.vocab_parallel == vocab_parallel
        xs, ys = zip(*[_batch(2, 8, seed=100 * rank + i) for i in range(steps * accum)])
        losses = _train(model, list(xs), list(ys), steps, accum)
        losses = [eng.mean_scalar(l) for l in losses]
        full = model.full_params().clone()
        if rank == 0:
            q.put(("ok", full, losses, model.memory_report()))
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        q.put(("err", traceback.format_exc(), None, None))
        raise


def _run(W, stage, steps=2, accum=2, vocab_parallel=False):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, W, port, stage, steps, accum, q, vocab_parallel)) for r in range(W)]
    for p in procs:
        p.start()
    tag, full, losses, rep = q.get(timeout=180)
    for p in procs:
        p.join(timeout=60)
    assert tag == "ok", full
    return full, losses, rep


@pytest.mark.parametrize("stage", [0, 1, 2, 3])
def test_zero_stage_matches_single_process(stage):
    W = 2
    ref_params, ref_losses = _baseline(W, 2, 2)
    full, losses, rep = _run(W, stage)
    assert torch.allclose(full[:ref_params.numel()], ref_params, atol=1e-5, rtol=1e-4), \
        (full[:ref_params.numel()] - ref_params).abs().max()
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 1e-5
    if stage >= 1:
        assert rep["m_bytes"] < ref_params.numel() * 4 * 0.6        # optimizer state is sharded
    if stage >= 2:
        assert rep["grads_bytes"] == 0 and rep["grad_pool_bytes"] > 0
    if stage == 3:
        assert rep["params_bytes"] == 0 and rep["param_shard_bytes"] > 0


@pytest.mark.parametrize("W,stage", [(2, 0), (4, 1), (3, 2)])
def test_vocab_parallel_lm_head_matches_replicated_head(W, stage):
    """LM head sharded over the vocabulary (activation all-gather, cross-rank log-sum-exp, reduce-scatter of
    the hidden gradient) must give the single-process parameters; W=3 leaves a ragged last slice."""
    ref_params, ref_losses = _baseline(W, 2, 1)
    full, losses, _ = _run(W, stage, steps=2, accum=1, vocab_parallel=True)
    assert torch.allclose(full[:ref_params.numel()], ref_params, atol=5e-5, rtol=1e-4), \
        (full[:ref_params.numel()] - ref_params).abs().max()
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 1e-5


def test_zero3_world4():
    W = 4
    ref_params, _ = _baseline(W, 1, 1)
    full, _, _ = _run(W, 3, steps=1, accum=1)
    assert torch.allclose(full[:ref_params.numel()], ref_params, atol=1e-5, rtol=1e-4)


def test_single_process_stages_match_plain_model():
    xs, ys = zip(*[_batch(2, 8, seed=i) for i in range(2)])
    base = GPT2(CFG, "fp32", "cpu")
    _train(base, list(xs), list(ys), 2, 1)
    from llm_mojo_b200.parallel.zero import ZeroEngine
    for stage in (1, 2, 3):
        eng = ZeroEngine(stage, 0, 1, torch.device("cpu"))
        m = GPT2(CFG, "fp32", "cpu", zero=eng)
        _train(m, list(xs), list(ys), 2, 1)
        assert torch.allclose(m.full_params()[:base.params.numel()], base.params, atol=1e-6), stage


# ------------------------------------------------------------------------------ liveness
def _abort_worker(rank, W, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    from llm_mojo_b200.parallel.runtime import PeerAborted, init_distributed, shutdown_distributed
    ctx = init_distributed(rank, W, backend="gloo")
    try:
        ctx.barrier(30)
        if rank == 1:
            try:
                raise RuntimeError("injected failure on rank 1")
            except RuntimeError:
                ctx.abort("injected")
                q.put((rank, "raised"))
                return
        try:
            ctx.barrier(30)           # rank 1 never arrives
            q.put((rank, "passed"))
        except PeerAborted:
            q.put((rank, "aborted"))
            try:
                ctx.barrier(30)       # sticky: later waits fail too
                q.put((rank, "not sticky"))
            except PeerAborted:
                q.put((rank, "sticky"))
    finally:
        shutdown_distributed(ctx)


def test_rank_failure_aborts_peers_instead_of_hanging():
    W = 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_abort_worker, args=(r, W, port, q)) for r in range(W)]
    for p in procs:
        p.start()
    seen = [q.get(timeout=60) for _ in range(1 + 2 * (W - 1))]
    for p in procs:
        p.join(timeout=30)
        assert not p.is_alive()
    assert (1, "raised") in seen
    for r in (0, 2):
        assert (r, "aborted") in seen and (r, "sticky") in seen


def test_coordinator_scalar_and_or_and_agreement():
    from torch.distributed import HashStore
    from llm_mojo_b200.parallel.runtime import Coordinator
    import threading
    store = HashStore()
    W = 4
    out = [None] * W

    def run(r):
        c = Coordinator(store, r, W, prefix="t")
        s = c.allreduce_scalar(float(r + 1))
        o = c.allreduce_or([1 << r, 0])
        c.assert_agree([(0, 8), (16, 24)])
        try:
            c.assert_agree([(0, 8)] if r != 2 else [(0, 9)])
            bad = False
        except ValueError:
            bad = True
        except Exception:
            bad = True
        out[r] = (s, o, bad)

    ts = [threading.Thread(target=run, args=(r,)) for r in range(W)]
    [t.start() for t in ts]
    [t.join(30) for t in ts]
    for r in range(W):
        assert out[r][0] == 10.0 and out[r][1] == [15, 0]
    assert out[2][2] or out[0][2]          # divergent ranges are rejected
