"""Process-per-GPU runtime: rendezvous, host-side coordination and failure propagation.

The reference runs its ranks as threads of one process that meet at a generation-counted spin
barrier with a *sticky abort flag* (``llmm/zero.mojo:39-164``): once any rank aborts, every
``wait()`` raises instead of hanging (``tests/test_zero.mojo:254-314``).  Here ranks are
processes (``torchrun``); ``torch.distributed`` provides the rendezvous and the NCCL / Gloo
fallback collectives, and the same abort semantics are rebuilt on the rendezvous key-value
store: ``Coordinator.barrier()`` polls an abort key while it waits, ``abort()`` sets it.
Device-side waits of the peer-memory kernels are bounded separately (they report through a
status word); this module is purely host code and is exercised with Gloo ranks on CPU.
"""
from __future__ import annotations

import datetime
import os
import time
from dataclasses import dataclass, field
from typing import Any, List, Optional

import torch
import torch.distributed as dist


class PeerAborted(RuntimeError):
    """Raised on every rank still waiting once some rank has called ``abort()``."""


class BarrierTimeout(RuntimeError):
    pass


class Coordinator:
    """Store-backed barrier with a sticky abort flag, scalar exchange and OR-reduce.

    Works with any ``torch.distributed`` store (TCPStore / HashStore / FileStore).  ``prefix``
    namespaces the keys so several coordinators can share one store."""

    ABORT_KEY = "abort"

    def __init__(self, store, rank: int, world_size: int, prefix: str = "coord", poll_s: float = 0.002):
        self.store, self.rank, self.world_size = store, rank, world_size
        self.prefix, self.poll_s = prefix, poll_s
        self.generation = 0

    def _k(self, name: str) -> str:
        return f"{self.prefix}/{name}"

    # -- failure propagation -------------------------------------------------------------
    def abort(self, reason: str = "") -> None:
        try:
            self.store.set(self._k(self.ABORT_KEY), f"rank {self.rank}: {reason}")
        except Exception:
            pass

    def aborted(self) -> Optional[str]:
        try:
            if self.store.check([self._k(self.ABORT_KEY)]):
                return self.store.get(self._k(self.ABORT_KEY)).decode()
        except Exception:
            return None
        return None

    def raise_if_aborted(self) -> None:
        why = self.aborted()
        if why is not None:
            raise PeerAborted(f"a peer aborted ({why})")

    # -- barrier ---------------------------------------------------------------------------
    def barrier(self, timeout_s: float = 300.0) -> None:
        """All ranks arrive, or raise ``PeerAborted`` (sticky) / ``BarrierTimeout``."""
        self.raise_if_aborted()
        gen = self.generation
        self.generation += 1
        key = self._k(f"bar/{gen}")
        arrived = self.store.add(key, 1)
        deadline = time.monotonic() + timeout_s
        while arrived < self.world_size:
            self.raise_if_aborted()
            if time.monotonic() > deadline:
                raise BarrierTimeout(f"rank {self.rank}: barrier {gen} timed out with {arrived}/{self.world_size}")
            time.sleep(self.poll_s)
            arrived = self.store.add(key, 0)

    # -- small host-side exchanges (cf. allreduce_scalar / allreduce_or_host, llmm/zero.mojo:417-552)
    def all_gather_object(self, obj: Any, timeout_s: float = 300.0) -> List[Any]:
        import pickle
        gen = self.generation
        self.store.set(self._k(f"obj/{gen}/{self.rank}"), pickle.dumps(obj))
        self.barrier(timeout_s)
        return [pickle.loads(self.store.get(self._k(f"obj/{gen}/{r}"))) for r in range(self.world_size)]

    def allreduce_scalar(self, value: float, timeout_s: float = 300.0) -> float:
        """Sum in rank order (identical result on every rank)."""
        return float(sum(self.all_gather_object(float(value), timeout_s)))

    def allreduce_or(self, words: List[int], timeout_s: float = 300.0) -> List[int]:
        parts = self.all_gather_object(list(words), timeout_s)
        out = [0] * len(words)
        for p in parts:
            if len(p) != len(words):
                raise ValueError("allreduce_or: ranks passed different lengths")
            out = [a | b for a, b in zip(out, p)]
        return out

    def assert_agree(self, payload: Any, what: str = "ranges", timeout_s: float = 300.0) -> None:
        """Every rank must pass an identical payload (``assert_ranges_agree``, llmm/zero.mojo:431-503)."""
        parts = self.all_gather_object(payload, timeout_s)
        for r, p in enumerate(parts):
            if p != parts[0]:
                self.abort(f"{what} disagree between rank 0 and rank {r}")
                raise ValueError(f"{what} disagree between rank 0 and rank {r}")


@dataclass
class DistContext:
    rank: int
    world_size: int
    local_rank: int
    device: torch.device
    backend: str
    coord: Coordinator
    owns_group: bool = True

    def abort(self, reason: str = "exception") -> None:
        self.coord.abort(reason)

    def barrier(self, timeout_s: float = 300.0) -> None:
        self.coord.barrier(timeout_s)


def init_distributed(rank: Optional[int] = None, world_size: Optional[int] = None, backend: Optional[str] = None,
                     timeout_s: float = 600.0) -> DistContext:
    """Join the job.  Reads RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT; NCCL on
    GPUs, Gloo on CPU (``LLMM_USE_CPU``)."""
    rank = int(os.environ.get("RANK", 0)) if rank is None else rank
    world_size = int(os.environ.get("WORLD_SIZE", 1)) if world_size is None else world_size
    local_rank = int(os.environ.get("LOCAL_RANK", rank))
    use_cuda = torch.cuda.is_available() and not os.environ.get("LLMM_USE_CPU")
    backend = backend or ("nccl" if use_cuda else "gloo")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    device = torch.device("cuda", local_rank % torch.cuda.device_count()) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)
    owns = False
    if not dist.is_initialized():
        kw = {"device_id": device} if backend == "nccl" else {}
        dist.init_process_group(backend, rank=rank, world_size=world_size,
                                timeout=datetime.timedelta(seconds=timeout_s), **kw)
        owns = True
    store = dist.distributed_c10d._get_default_store()
    coord = Coordinator(store, rank, world_size, prefix=f"llmb/{os.environ.get('TORCHELASTIC_RUN_ID', 'job')}")
    return DistContext(rank, world_size, local_rank, device, backend, coord, owns)


def shutdown_distributed(ctx: DistContext) -> None:
    if ctx.owns_group and dist.is_initialized():
        try:
            dist.destroy_process_group()
        except Exception:
            pass
