"""DDP and ZeRO stages 1/2/3 over a flat parameter vector.

Parity (what each stage keeps / moves): ``train_gpt2.mojo:1965-2036`` (shard = ceil(P/W) rounded up
to the vector width, rank r owns ``[r·S, (r+1)·S)``), ``:5009-5048`` (stage 0/1: gradients reduced on
the last micro-step), ``:2323-2494``, ``:4921-4929`` (stage 2/3: per-bucket reduce-scatter into a
persistent gradient shard, gradients live in a small recycled pool), ``:1660-1963`` (stage 3:
persistent 1/W parameter shard, per-layer windows gathered just in time in forward and backward,
embedding window), ``:5058-5259`` (sharded AdamW, parameter all-gather after the update for stages
1/2), ``:5261-5383`` (sharded norm + scalar all-reduce).

Two collective backends implement the same five operations on flat ranges:

* ``P2PBackend`` — the product path on GPUs: peer-memory kernels (``csrc/comm.cu``) on a side
  stream, bf16 on the wire, overlapped with backward bucket by bucket; the sharded AdamW kernel
  itself stores the new parameters into every rank's copy.
* ``TorchDistBackend`` — ``torch.distributed`` (Gloo on CPU for the tests, NCCL as a GPU
  fallback / baseline), fp32 on the wire.

Stage 1 is implemented as reduce-scatter → shard update → parameter push (strictly less traffic
than the reference's all-reduce → shard update → all-gather, same result).
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from .. import ops
from ..config import PARAM_NAMES
from ..ops import _lib
from ..utils import checkpointing as ckpt

LAYER_TENSORS = ("ln1w", "ln1b", "qkvw", "qkvb", "attprojw", "attprojb", "ln2w", "ln2b",
                 "fcw", "fcb", "fcprojw", "fcprojb")
Range = Tuple[int, int]
VEC = 8


def shard_size(num_parameters: int, world_size: int) -> int:
    s = (num_parameters + world_size - 1) // world_size
    return (s + VEC - 1) // VEC * VEC


def intersect(a: Range, b: Range) -> Optional[Range]:
    lo, hi = max(a[0], b[0]), min(a[1], b[1])
    return (lo, hi) if lo < hi else None


class _LayerView:
    """``view[l]`` → tensor of layer ``l`` (only the layers currently resident are valid)."""

    def __init__(self):
        self.t: Dict[int, torch.Tensor] = {}

    def __getitem__(self, l: int) -> torch.Tensor:
        return self.t[l]


# ======================================================================================= backends
class TorchDistBackend:
    """Collectives through torch.distributed; synchronous on the current stream."""
    name = "torchdist"
    wire_dtype = torch.float32

    def __init__(self, rank: int, world: int, device: torch.device):
        self.rank, self.world, self.device = rank, world, device

    def reduce_ranges(self, src: torch.Tensor, segs: Sequence[Tuple[int, int, int]], shard: Range,
                      dst: Optional[torch.Tensor], accumulate: bool, allreduce: bool) -> None:
        """``segs``: (flat_begin, length, src_offset).  Mean over ranks.  ``allreduce``: result written
        back into ``src`` in place; else the part of each range inside ``shard`` goes to
        ``dst[flat - shard[0]]`` (+= when ``accumulate``)."""
        for fb, n, so in segs:
            t = src[so:so + n]
            if allreduce:
                if self.world > 1:
                    dist.all_reduce(t)
                    t.div_(self.world)
                continue
            tmp = t.clone()
            if self.world > 1:
                dist.all_reduce(tmp)
                tmp.div_(self.world)
            own = intersect((fb, fb + n), shard)
            if own is not None:
                d = dst[own[0] - shard[0]: own[1] - shard[0]]
                piece = tmp[own[0] - fb: own[1] - fb]
                if accumulate:
                    d += piece
                else:
                    d.copy_(piece)

    def gather_ranges(self, shard_t: torch.Tensor, S: int, segs: Sequence[Tuple[int, int, int]], dst: torch.Tensor) -> None:
        """``segs``: (flat_begin, length, dst_offset); every piece is broadcast by its owner."""
        for fb, n, do in segs:
            for r in range(self.world):
                own = intersect((fb, fb + n), (r * S, (r + 1) * S))
                if own is None:
                    continue
                d = dst[do + own[0] - fb: do + own[1] - fb]
                if r == self.rank:
                    d.copy_(shard_t[own[0] - r * S: own[1] - r * S])
                if self.world > 1:
                    dist.broadcast(d, src=r)

    def push_shard(self, shard_t: torch.Tensor, S: int, full: torch.Tensor) -> None:
        if self.world == 1:
            return
        parts = [torch.empty_like(shard_t) for _ in range(self.world)]
        dist.all_gather(parts, shard_t.contiguous())
        full[:S * self.world].copy_(torch.cat(parts))

    def allreduce_scalar(self, t: torch.Tensor) -> None:
        if self.world > 1:
            dist.all_reduce(t)

    def sync(self) -> None:
        pass

    def rearm_after_timeout(self) -> None:
        pass

    def close(self) -> None:
        pass


class P2PBackend:
    """Peer-memory kernels on a side stream (see csrc/comm.cu)."""
    name = "p2p"
    wire_dtype = torch.bfloat16

    def __init__(self, rank: int, world: int, device: torch.device, send_cap: int, param_elems: int,
                 blocks: int = 296):
        from .symm import SymmetricArena
        self.rank, self.world, self.device = rank, world, device
        self.send_cap = (send_cap + 1023) // 1024 * 1024
        regions = [("send0", self.send_cap * 2), ("send1", self.send_cap * 2),
                   ("recv0", self.send_cap * 2), ("recv1", self.send_cap * 2),
                   ("params", param_elems * 2)]
        self.arena = SymmetricArena(regions, rank, world, device)
        self.stream = torch.cuda.Stream(device=device)
        self.blocks = int(os.environ.get("LLMB_COMM_BLOCKS", blocks))
        self.seq = 0                 # reduce sequence number (same on all ranks)
        self.scalar_seq = 0
        self.param_seq = 0
        self.send_last = [0, 0]      # last seq that used send buffer i
        self.recv_last = [0, 0]
        self.status = _lib.status_word(device)
        self.L = _lib.lib()
        self._declare()
        self.params = self.arena.tensor("params", torch.bfloat16)
        self._pool_events: Dict[int, torch.cuda.Event] = {}

    def _declare(self) -> None:
        L, P, I, LL, F, U = self.L, ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_uint
        LLp = ctypes.POINTER(ctypes.c_longlong)
        Ip = ctypes.POINTER(ctypes.c_int)
        L.llmb_comm_pack.argtypes = [P, P, I, LLp, LLp, LLp, F, P, P, I, I, U, U, P, P, I, P]
        L.llmb_comm_reduce.argtypes = [P, I, LLp, LLp, LLp, I, P, I, P, P, P, P, I, I, U, U, P, P, P, I, P]
        L.llmb_comm_unpack.argtypes = [P, P, I, LLp, LLp, LLp, P, P, I, I, U, P, P, I, P]
        L.llmb_comm_gather.argtypes = [P, P, I, Ip, LLp, LLp, LLp, P, I, U, P, I, P]
        L.llmb_comm_adamw_push.argtypes = [P, LL, P, P, P, P, P, LL, F, F, F, F, F, F, P, I, I, P, I, I, U, P, P]
        L.llmb_comm_wait.argtypes = [P, I, U, I, P, P]
        L.llmb_comm_scalar_allreduce.argtypes = [P, P, P, P, P, P, I, I, U, P, P]

    @staticmethod
    def _arr(vals: Sequence[int], ctype=ctypes.c_longlong):
        return (ctype * max(len(vals), 1))(*vals)

    def reduce_ranges(self, src, segs, shard, dst, accumulate, allreduce, norm_acc=None, scale=None) -> None:
        """Same contract as TorchDistBackend.reduce_ranges; asynchronous on the comm stream.  ``norm_acc``
        (1 fp32) additionally receives the sum of squares of the reduced values this rank owns.  ``scale``
        multiplies every contribution before it goes on the wire (default 1/W: the mean; 1.0: the sum)."""
        A, W, me = self.arena, self.world, self.rank
        total = sum(n for _, n, _ in segs)
        if total > self.send_cap:
            raise ValueError(f"bucket of {total} elements exceeds the send buffer ({self.send_cap})")
        self.seq += 1
        seq, half = self.seq, self.seq & 1
        # k-space: concatenation of the ranges in order
        k_off, src_offs, lens, k = [], [], [], 0
        for fb, n, so in segs:
            k_off.append(k); src_offs.append(so); lens.append(n); k += n
        if allreduce:
            chunk = ((total + W - 1) // W + VEC - 1) // VEC * VEC
            lo, hi = min(me * chunk, total), min((me + 1) * chunk, total)
            owned = [(lo, lo, hi - lo)] if hi > lo else []           # (k, k, len): dst is the recv buffer at k
        else:
            owned = []
            for (fb, n, _), ko in zip(segs, k_off):
                own = intersect((fb, fb + n), shard)
                if own is not None:
                    owned.append((ko + own[0] - fb, own[0] - shard[0], own[1] - own[0]))
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        self.stream.wait_event(ev)
        st = self.stream.cuda_stream
        send_name, recv_name = f"send{half}", f"recv{half}"
        send_ptr = A.base + A.offsets[send_name]
        _lib.check(self.L.llmb_comm_pack(send_ptr, src.data_ptr(), len(segs), self._arr(src_offs), self._arr(k_off),
                                         self._arr(lens), (1.0 / W) if scale is None else float(scale), A.flags_ptr, A.flags_peer_ptrs(), me, W, seq,
                                         self.send_last[half], A.counter_ptr(0), self.status.data_ptr(), self.blocks, st),
                   "comm_pack")
        self.send_last[half] = seq
        packed = torch.cuda.Event()
        packed.record(self.stream)
        self._last_pack_event = packed
        _lib.check(self.L.llmb_comm_reduce(A.peer_ptrs(send_name), len(owned), self._arr([o[0] for o in owned]),
                                           self._arr([o[1] for o in owned]), self._arr([o[2] for o in owned]),
                                           1 if allreduce else 0, dst.data_ptr() if dst is not None else None,
                                           int(accumulate), A.peer_ptrs(recv_name) if allreduce else None, _lib.ptr(norm_acc), A.flags_ptr,
                                           A.flags_peer_ptrs(), me, W, seq, self.recv_last[half] if allreduce else 0,
                                           A.counter_ptr(1), A.counter_ptr(2), self.status.data_ptr(), self.blocks, st),
                   "comm_reduce")
        if allreduce:
            self.recv_last[half] = seq
            _lib.check(self.L.llmb_comm_unpack(src.data_ptr(), A.base + A.offsets[recv_name], len(segs), self._arr(k_off),
                                               self._arr(src_offs), self._arr(lens), A.flags_ptr, A.flags_peer_ptrs(), me, W,
                                               seq, A.counter_ptr(3), self.status.data_ptr(), self.blocks, st), "comm_unpack")
        ops._count(3 if allreduce else 2)

    def pack_done_event(self) -> torch.cuda.Event:
        return self._last_pack_event

    def gather_ranges(self, shard_name_unused, S, segs, dst, stream=None) -> None:
        """Pull ranges from their owners' parameter shards (region 'params' holds each rank's shard)."""
        A, W = self.arena, self.world
        owner, so, do, ln = [], [], [], []
        for fb, n, d0 in segs:
            for r in range(W):
                own = intersect((fb, fb + n), (r * S, (r + 1) * S))
                if own is not None:
                    owner.append(r); so.append(own[0] - r * S); do.append(d0 + own[0] - fb); ln.append(own[1] - own[0])
        st = (stream or torch.cuda.current_stream()).cuda_stream
        _lib.check(self.L.llmb_comm_gather(dst.data_ptr(), A.peer_ptrs("params"), len(owner), self._arr(owner, ctypes.c_int),
                                           self._arr(so), self._arr(do), self._arr(ln), A.flags_ptr, W, self.param_seq,
                                           self.status.data_ptr(), self.blocks, st), "comm_gather")
        ops._count()

    def adamw_push(self, shard_off: int, shard_copy, master, grads, m, v, n, push: bool, **kw) -> None:
        A, W, me = self.arena, self.world, self.rank
        self.param_seq += 1
        _lib.check(self.L.llmb_comm_adamw_push(A.peer_ptrs("params"), shard_off, _lib.ptr(shard_copy), master.data_ptr(),
                                               grads.data_ptr(), m.data_ptr(), v.data_ptr(), n, kw["lr"], kw["beta1"],
                                               kw["beta2"], kw["eps"], kw["weight_decay"], kw["grad_scale"],
                                               _lib.ptr(kw.get("dev_scale")), kw["step"], W if push else 0,
                                               A.flags_peer_ptrs(), me, W, self.param_seq, A.counter_ptr(4),
                                               torch.cuda.current_stream().cuda_stream), "comm_adamw_push")
        ops._count()

    def wait_params(self) -> None:
        """Main stream waits (bounded, on the device) until every rank's parameter push has landed."""
        if self.param_seq:
            _lib.check(self.L.llmb_comm_wait(self.arena.flags_ptr, 3, self.param_seq, self.world, self.status.data_ptr(),
                                             torch.cuda.current_stream().cuda_stream), "comm_wait")
            ops._count()

    def allreduce_scalar(self, t: torch.Tensor) -> None:
        A = self.arena
        self.scalar_seq += 1
        _lib.check(self.L.llmb_comm_scalar_allreduce(t.data_ptr(), t.data_ptr(), A.scalars_ptr, A.scalars_peer_ptrs(),
                                                     A.flags_ptr, A.flags_peer_ptrs(), self.rank, self.world,
                                                     self.scalar_seq, self.status.data_ptr(),
                                                     torch.cuda.current_stream().cuda_stream), "comm_scalar_allreduce")
        ops._count()

    def sync(self) -> None:
        """Main stream waits for everything queued on the comm stream."""
        ev = torch.cuda.Event()
        ev.record(self.stream)
        torch.cuda.current_stream().wait_event(ev)

    def rearm_after_timeout(self) -> None:
        """After a bounded wait expired some blocks of a kernel left early, so the "last block" launch counters
        of this rank's arena can be non-zero; the next launch would then mis-detect its last block.  Zero them."""
        from .symm import _HDR_FLAGS, _HDR_SCALARS, _HDR_COUNTERS
        torch.cuda.synchronize(self.device)
        self.arena._mem[_HDR_FLAGS + _HDR_SCALARS:_HDR_FLAGS + _HDR_SCALARS + _HDR_COUNTERS].zero_()
        torch.cuda.synchronize(self.device)

    def close(self) -> None:
        torch.cuda.synchronize()
        self.arena.close()


# ======================================================================================= fused row gather
class FusedRowGather:
    """All-gather of activation rows fused into the GEMM that consumes them (vocabulary-parallel LM head).

    Every rank owns a [W·n, K] bf16 buffer in a symmetric arena and writes its own n rows in place (chunk ``rank``).
    ``gemm`` launches ONE kernel: two copier warps per CTA pull the other ranks' chunks out of their arenas over
    NVLink into the local buffer while the tensor-core tile loop already works on the local chunk, and a chunk's
    tiles are fetched once it has landed (csrc/gemm.cu, GatherArgs).  Flags: ROWS_READY (6) = "my chunk is written",
    ROWS_DONE (7) = "I have finished reading everybody's chunk"; both are sequence numbers, every wait is bounded."""
    ROWS_READY, ROWS_DONE, STATS_READY, STATS_DONE = 6, 7, 8, 9

    def __init__(self, rank: int, world: int, device: torch.device, rows_per_rank: int, K: int):
        from .symm import SymmetricArena
        if rows_per_rank % 256:
            raise ValueError("fused row gather needs rows per rank to be a multiple of 256")
        self.rank, self.world, self.device, self.n, self.K = rank, world, device, rows_per_rank, K
        self.chunk_bytes = rows_per_rank * K * 2
        self.arena = SymmetricArena([("rows", world * self.chunk_bytes), ("counts", 64),
                                     ("stats", world * rows_per_rank * 16)], rank, world, device)
        # per-row softmax statistics of this rank's vocabulary slice, read by every peer in merge_stats()
        self.stats = self.arena.tensor("stats", torch.float32).view(world * rows_per_rank, 4)
        self.stats_seq = 0
        self.buf = self.arena.tensor("rows", torch.bfloat16).view(world * rows_per_rank, K)
        self.local = self.buf[rank * rows_per_rank:(rank + 1) * rows_per_rank]
        self.counts = self.arena.tensor("counts", torch.int32)
        self.status = ops.status_word(device)
        self.seq = 0
        self.L = _lib.lib()
        P, I, U, LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint, ctypes.c_longlong
        self.L.llmb_comm_signal.argtypes = [P, I, I, I, U, P]
        self.L.llmb_comm_wait.argtypes = [P, I, U, I, P, P]
        self.L.llmb_gemm_set_gather.argtypes = [P, P, P, P, LL, U, I, I, I]
        self.L.llmb_gemm_set_gather.restype = None
        self.L.llmb_comm_ce_stats_merge.argtypes = [P, ctypes.POINTER(P), LL, P, ctypes.POINTER(P), I, I, U, P, P, I, P]
        self._peer_src = (ctypes.c_void_p * 8)()
        off = self.arena.offsets["rows"]
        for r in range(world):                      # chunk r inside rank r's buffer
            self._peer_src[r] = self.arena.peer_bases[r] + off + r * self.chunk_bytes

    def wait_released(self) -> None:
        """Before the local chunk is overwritten: every rank has finished reading the previous contents."""
        if self.seq:
            _lib.check(self.L.llmb_comm_wait(self.arena.flags_ptr, self.ROWS_DONE, self.seq, self.world,
                                             self.status.data_ptr(), _lib.stream()), "rows_wait")

    def stats_writable(self) -> None:
        """Before ``stats`` is rewritten: every rank has read the previous contents."""
        if self.stats_seq:
            _lib.check(self.L.llmb_comm_wait(self.arena.flags_ptr, self.STATS_DONE, self.stats_seq, self.world,
                                             self.status.data_ptr(), _lib.stream()), "stats_wait")

    def merge_stats(self, out: torch.Tensor) -> None:
        """out [W·n, 4] (local) = the ranks' ``stats`` merged into the statistics of the whole vocabulary: one kernel,
        peer loads, no collective library (``csrc/comm.cu``, ce_stats_merge_kernel)."""
        self.stats_seq += 1
        A = self.arena
        _lib.check(self.L.llmb_comm_ce_stats_merge(out.data_ptr(), A.peer_ptrs("stats"), self.stats.shape[0], A.flags_ptr,
                                                   A.flags_peer_ptrs(), self.rank, self.world, self.stats_seq,
                                                   A.counter_ptr(8), self.status.data_ptr(), 148, _lib.stream()), "ce_stats_merge")
        ops._count()

    def gemm(self, D: torch.Tensor, weight: torch.Tensor) -> None:
        """D[W·n, N] = gathered rows · weightᵀ; call after the local chunk has been written on the current stream."""
        self.seq += 1
        st = _lib.stream()
        _lib.check(self.L.llmb_comm_signal(self.arena.flags_peer_ptrs(), self.ROWS_READY, self.rank, self.world, self.seq, st),
                   "rows_signal")
        self.counts.zero_()
        self.L.llmb_gemm_set_gather(self._peer_src, self.buf.data_ptr(), self.arena.flags_ptr, self.counts.data_ptr(),
                                    self.chunk_bytes, self.seq, self.world, self.rank, self.n)
        ops.gemm(D, self.buf, weight)
        _lib.check(self.L.llmb_comm_signal(self.arena.flags_peer_ptrs(), self.ROWS_DONE, self.rank, self.world, self.seq, st),
                   "rows_release")


# ======================================================================================= engine
class ZeroEngine:
    def __init__(self, stage: int, rank: int, world_size: int, device: torch.device, dist_ctx=None,
                 backend: str = "auto"):
        if stage not in (0, 1, 2, 3):
            raise ValueError(f"invalid ZeRO stage {stage}")
        self.stage, self.rank, self.world_size, self.device = stage, rank, world_size, torch.device(device)
        self.dist_ctx = dist_ctx
        if backend == "auto":
            backend = "p2p" if self.device.type == "cuda" and world_size > 1 else "torchdist"
        if backend in ("nccl", "gloo"):
            backend = "torchdist"
        self.backend_name = backend
        self.backend = None
        self.model = None
        self.window_layers: Dict[int, int] = {}       # layer -> window slot (stage 3)
        self.params_dirty = True                       # windows must be re-gathered

    # ------------------------------------------------------------------ setup
    def attach(self, model, flat: torch.Tensor) -> None:
        self.model = model
        W, r, dev = self.world_size, self.rank, self.device
        P = model.num_parameters
        self.P = P
        self.S = S = shard_size(P, W) if W > 1 or self.stage > 0 else P
        self.padded = S * W
        self.shard_range: Range = (r * S, (r + 1) * S)
        dt = model.dtype
        cfg = model.config
        # ---- buckets (ranges in the flat vector)
        self.layer_ranges = [model.layer_ranges(l) for l in range(cfg.num_layer)]
        wte, wpe = model.tensor_range("wte"), model.tensor_range("wpe")
        lnfw, lnfb = model.tensor_range("lnfw"), model.tensor_range("lnfb")
        pooled = self.stage >= 2
        self.buckets: Dict[object, List[Range]] = {"head": ([wte] if pooled else []) + [lnfw, lnfb], "embed": [wte, wpe]}
        for l, rs in enumerate(self.layer_ranges):
            self.buckets[l] = rs
        self.bucket_size = {k: sum(e - b for b, e in v) for k, v in self.buckets.items()}
        max_bucket = max(self.bucket_size.values())

        # ---- backend
        if self.backend_name == "p2p":
            param_elems = 8 if self.stage == 0 else (self.padded if self.stage < 3 else S)
            self.backend = P2PBackend(r, W, dev, max_bucket, param_elems)
        else:
            self.backend = TorchDistBackend(r, W, dev)
        p2p = self.backend_name == "p2p"

        # ---- parameters
        padded_flat = torch.zeros(self.padded, dtype=torch.float32)
        padded_flat[:P] = flat
        my = padded_flat[r * S:(r + 1) * S]
        if self.stage < 3:
            if p2p and self.stage >= 1:
                model.params = self.backend.params          # peers push updated shards into this buffer
                model.params.copy_(padded_flat.to(dt))
            else:
                model.params = padded_flat.to(dev, dt)
            self.param_shard = None
        else:
            model.params = None
            self.param_shard = self.backend.params if p2p else torch.empty(S, dtype=dt, device=dev)
            self.param_shard.copy_(my.to(dt))
            layer_elems = self.bucket_size[0]
            embed_elems = (wte[1] - wte[0]) + (wpe[1] - wpe[0]) + 2 * cfg.channels
            self.windows = [torch.empty(layer_elems, dtype=dt, device=dev) for _ in range(2)]
            self.embed_window = torch.empty(embed_elems, dtype=dt, device=dev)
            self.embed_valid = False
            self.window_layers = {}
            self.window_events = [None, None]
            self._setup_fused_pull(p2p)
        # ---- optimizer state (sharded for stage >= 1)
        n_opt = S if self.stage >= 1 else self.padded if W > 1 else P
        self.n_opt = n_opt
        model.m = torch.zeros(n_opt, dtype=torch.float32, device=dev)
        model.v = torch.zeros(n_opt, dtype=torch.float32, device=dev)
        src = my if self.stage >= 1 else padded_flat[:n_opt]
        if model.precision.use_master or self.stage >= 1:
            model.master = src.to(dev, torch.float32).clone()
        else:
            model.master = None
        # ---- gradients
        if self.stage >= 2:
            self.pools = [torch.zeros(max_bucket, dtype=torch.float32, device=dev) for _ in range(2)]
            self.pool_idx = 0
            self.pool_events: List[Optional[torch.cuda.Event]] = [None, None]
            model.grads = None
            self.grad_shard = torch.zeros(S, dtype=torch.float32, device=dev)
        else:
            model.grads = torch.zeros(self.padded, dtype=torch.float32, device=dev)
            self.grad_shard = torch.zeros(S, dtype=torch.float32, device=dev) if self.stage == 1 else None
        self.norm_sq = torch.zeros(1, dtype=torch.float32, device=dev)
        self.norm_acc = torch.zeros(1, dtype=torch.float32, device=dev)     # fused sum of squares (stage 1, p2p)
        self.norm_fused = False
        self._install_views()
        if dist.is_initialized():
            dist.barrier()

    def _install_views(self) -> None:
        m = self.model
        if self.stage < 3:
            m.p = m._views(m.params)
        else:
            m.p = {n: (_LayerView() if n in LAYER_TENSORS else None) for n in PARAM_NAMES}
        if self.stage < 2:
            m.g = m._views(m.grads)
        else:
            m.g = {n: (_LayerView() if n in LAYER_TENSORS else None) for n in PARAM_NAMES}

    def _segs(self, key, base_offsets: Optional[List[int]] = None) -> List[Tuple[int, int, int]]:
        """(flat_begin, length, local offset) for a bucket: offsets are positions in the pool /
        window (concatenated ranges) or, without pooling, the flat offsets themselves."""
        out, k = [], 0
        for b, e in self.buckets[key]:
            out.append((b, e - b, k))
            k += e - b
        return out

    def _view_bucket(self, key, buf: torch.Tensor, target: Dict[str, object]) -> None:
        """Point the model's parameter / gradient views of bucket ``key`` into ``buf``."""
        m = self.model
        names = {"head": (["wte"] if self.stage >= 2 else []) + ["lnfw", "lnfb"], "embed": ["wte", "wpe"]}
        k = 0
        if isinstance(key, int):
            for n, (b, e) in zip(LAYER_TENSORS, self.buckets[key]):
                shape = m.param_shapes[PARAM_NAMES.index(n)][1:]
                target[n].t[key] = buf[k:k + e - b].view(shape)
                k += e - b
        else:
            for n, (b, e) in zip(names[key], self.buckets[key]):
                target[n] = buf[k:k + e - b].view(m.param_shapes[PARAM_NAMES.index(n)])
                k += e - b

    # ------------------------------------------------------------------ parameter residency (stage 3)
    def _gather_layer(self, l: int, prefetch: bool = False) -> None:
        """Make layer ``l``'s parameters resident in window ``l % 2``.  (Fused mode: its small tensors only.)  With ``prefetch`` (peer-memory
        backend) the pull kernel runs on the comm stream, after everything already queued on the main
        stream (the previous occupant of the window may still be in use there), and the main stream
        only waits for it when the layer is actually needed."""
        if getattr(self, "fused_z3", False):
            return self._gather_layer_small(l, prefetch)
        if l in self.window_layers:
            return
        slot = l % 2
        for victim in [k for k, v in self.window_layers.items() if v == slot]:
            del self.window_layers[victim]
            for n in LAYER_TENSORS:
                self.model.p[n].t.pop(victim, None)
        win = self.windows[slot]
        if prefetch and self.backend_name == "p2p":
            ready = torch.cuda.Event()
            ready.record(torch.cuda.current_stream())
            self.backend.stream.wait_event(ready)
            self.backend.gather_ranges(self.param_shard, self.S, self._segs(l), win, stream=self.backend.stream)
            done = torch.cuda.Event()
            done.record(self.backend.stream)
            self.window_events[slot] = done
        else:
            self.backend.gather_ranges(self.param_shard, self.S, self._segs(l), win)
            self.window_events[slot] = None
        self.window_layers[l] = slot
        self._view_bucket(l, win, self.model.p)


    # ------------------------------------------------------------------ stage 3: weight pulls fused into the layer GEMMs
    WEIGHTS = ("qkvw", "attprojw", "fcw", "fcprojw")
    SITE_WEIGHT = {"qkv": "qkvw", "attproj": "attprojw", "fc": "fcw", "fcproj": "fcprojw"}

    def _setup_fused_pull(self, p2p: bool) -> None:
        """With the peer-memory backend on bf16 tensor-core GEMMs the four weight matrices of a layer are not gathered
        by a collective kernel: the copier warps of the layer's GEMM kernels pull them out of their owners' shards
        while the tile loops run (``csrc/gemm.cu``, PullArgs).  Every GEMM that reads a weight carries the pull of the
        NEXT weight in execution order (forward: qkv, attproj, fc, fcproj, next layer's qkv ...; backward the reverse),
        so a weight has landed when its own GEMM starts; the first GEMM of a pass pulls its own operand as well and
        waits for it.  Only the small tensors of a layer (LayerNorm parameters, biases) still come by the gather kernel.
        ``LLMM_FUSED_Z3=0`` selects the whole-layer gather, prefetched one layer ahead."""
        m = self.model
        self.fused_z3 = bool(p2p and self.world_size > 1 and m.dtype == torch.bfloat16 and m.precision.name == "bf16"
                             and ops.GEMM_IMPL == "tcgen05" and os.environ.get("LLMB_GEMM_PAIR", "1") != "0"
                             and os.environ.get("LLMM_FUSED_Z3", "1") != "0")
        if not self.fused_z3:
            return
        L = m.config.num_layer
        self._pull_counts = torch.zeros(2 * L * 4 + 2, 16, dtype=torch.int32, device=self.device)
        self._pull_order = {False: [(l, w) for l in range(L) for w in self.WEIGHTS],
                            True: [(l, w) for l in reversed(range(L)) for w in reversed(self.WEIGHTS)]}
        self._pull_pos = {ph: {k: i for i, k in enumerate(o)} for ph, o in self._pull_order.items()}
        self._pulled: Dict[Tuple[int, str], Tuple[int, List[Tuple[int, int]]]] = {}    # weight -> (counts row, [(segment, bytes)])
        self._pull_job = 0
        lib = self.backend.L
        P, I, U, LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint, ctypes.c_longlong
        lib.llmb_gemm_set_pull.argtypes = [ctypes.POINTER(P), ctypes.POINTER(P), ctypes.POINTER(LL), ctypes.POINTER(I), I, P, U, P,
                                           ctypes.POINTER(P), ctypes.POINTER(LL), I, I]
        lib.llmb_gemm_set_pull.restype = I
        # window offsets of a layer's tensors (the window holds the bucket's ranges back to back)
        self._win_off, k = {}, 0
        for n, (b, e) in zip(LAYER_TENSORS, self.buckets[0]):
            self._win_off[n] = k
            k += e - b

    def _weight_segments(self, l: int, name: str) -> List[Tuple[int, int, int, int]]:
        """(owner, source address, destination address, bytes) for every piece of weight ``name`` of layer ``l``."""
        A, S = self.backend.arena, self.S
        b, e = self.model.tensor_range(name, l)
        win = self.windows[l % 2]
        out = []
        for r in range(self.world_size):
            own = intersect((b, e), (r * S, (r + 1) * S))
            if own is None:
                continue
            src = A.peer_bases[r] + A.offsets["params"] + (own[0] - r * S) * 2
            dst = win.data_ptr() + (self._win_off[name] + own[0] - b) * 2
            out.append((r, src, dst, (own[1] - own[0]) * 2))
        return out

    def begin_pass(self, backward: bool) -> None:
        """Start of a forward or backward pass: the pull counters are zeroed (stream-ordered behind the previous pass)."""
        if getattr(self, "fused_z3", False):
            self._pull_counts.zero_()
            self._pulled.clear()
            self._pull_job = 0

    def arm_linear(self, site: str, l: int, backward: bool) -> None:
        """Called right before the GEMM that reads the weight of ``site`` in layer ``l`` (forward GEMM, or the input-
        gradient GEMM in backward): arms that GEMM with the pull of the next weight and the wait for its own."""
        if not getattr(self, "fused_z3", False):
            return
        name = self.SITE_WEIGHT[site]
        order, pos = self._pull_order[backward], self._pull_pos[backward][(l, name)]
        todo = []
        if (l, name) not in self._pulled:
            todo.append((l, name))                          # first GEMM of the pass: its own operand
        if pos + 1 < len(order):
            todo.append(order[pos + 1])
        row = self._pull_job
        self._pull_job += 1
        segs = []
        for key in todo:
            mine = []
            for seg in self._weight_segments(*key):
                mine.append((len(segs), seg[3]))
                segs.append(seg)
            self._pulled[key] = (row, mine)
        if len(segs) > 8:
            raise RuntimeError("a weight pull of more than 8 segments does not fit one GEMM launch")
        wrow, wsegs = self._pulled[(l, name)]
        P, LL, I = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int
        n = len(segs)
        src = (P * 8)(*[s_[1] for s_ in segs]); dst = (P * 8)(*[s_[2] for s_ in segs])
        nb = (LL * 8)(*[s_[3] for s_ in segs]); own = (I * 8)(*[s_[0] for s_ in segs])
        base = self._pull_counts.data_ptr()
        wc = (P * 8)(*[base + (wrow * 16 + i) * 4 for i, _ in wsegs]); wb = (LL * 8)(*[nbytes for _, nbytes in wsegs])
        A = self.backend.arena
        _lib.check(self.backend.L.llmb_gemm_set_pull(src, dst, nb, own, n, A.flags_ptr, self.backend.param_seq,
                                                     base + row * 64, wc, wb, len(wsegs), self.world_size), "gemm_set_pull")

    def _gather_layer_small(self, l: int, prefetch: bool = False) -> None:
        """Fused mode: only the LayerNorm parameters and biases of layer ``l`` come by the gather kernel."""
        if l in self.window_layers:
            return
        slot = l % 2
        for victim in [k for k, v in self.window_layers.items() if v == slot]:
            del self.window_layers[victim]
            for n in LAYER_TENSORS:
                self.model.p[n].t.pop(victim, None)
        win = self.windows[slot]
        segs = [sg for n, sg in zip(LAYER_TENSORS, self._segs(l)) if n not in self.WEIGHTS]
        if prefetch:
            ready = torch.cuda.Event()
            ready.record(torch.cuda.current_stream())
            self.backend.stream.wait_event(ready)
            self.backend.gather_ranges(self.param_shard, self.S, segs, win, stream=self.backend.stream)
            done = torch.cuda.Event()
            done.record(self.backend.stream)
            self.window_events[slot] = done
        else:
            self.backend.gather_ranges(self.param_shard, self.S, segs, win)
            self.window_events[slot] = None
        self.window_layers[l] = slot
        self._view_bucket(l, win, self.model.p)

    def _ensure_layer(self, l: int) -> None:
        self._gather_layer(l)
        ev = self.window_events[l % 2]
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
            self.window_events[l % 2] = None

    def _gather_embed(self) -> None:
        if self.embed_valid:
            return
        m = self.model
        wte, wpe = m.tensor_range("wte"), m.tensor_range("wpe")
        lnfw, lnfb = m.tensor_range("lnfw"), m.tensor_range("lnfb")
        segs, k = [], 0
        for b, e in (wte, wpe, lnfw, lnfb):
            segs.append((b, e - b, k)); k += e - b
        self.backend.gather_ranges(self.param_shard, self.S, segs, self.embed_window)
        k = 0
        for n, (b, e) in zip(("wte", "wpe", "lnfw", "lnfb"), (wte, wpe, lnfw, lnfb)):
            m.p[n] = self.embed_window[k:k + e - b].view(m.param_shapes[PARAM_NAMES.index(n)])
            k += e - b
        self.embed_valid = True

    def _params_ready(self) -> None:
        """First parameter use after an optimizer step: wait for the peers' pushes."""
        if self.params_dirty:
            if self.backend_name == "p2p" and self.stage >= 1:
                self.backend.wait_params()
            self.params_dirty = False

    # ------------------------------------------------------------------ hooks called by the model
    def before_embedding(self, backward: bool = False) -> None:
        self._params_ready()
        if not backward:
            self.begin_pass(False)
        if self.stage == 3:
            self._gather_embed()
        if backward and self.stage >= 2:
            self._next_pool("embed")

    def before_head(self, backward: bool) -> None:
        if backward:
            self.begin_pass(True)
        if self.stage == 3:
            self._gather_embed()
        if backward and self.stage >= 2:
            self._next_pool("head")

    def before_layer(self, l: int, backward: bool) -> None:
        if self.stage == 3:
            self._params_ready()
            self._ensure_layer(l)
            nxt = l - 1 if backward else l + 1
            if 0 <= nxt < self.model.config.num_layer:
                self._gather_layer(nxt, prefetch=True)      # overlaps with this layer's compute
        if backward and self.stage >= 2:
            self._next_pool(l)

    def _next_pool(self, key) -> None:
        """Hand the next bucket a zeroed pool; wait until the pack kernel of the pool's previous
        use has finished reading it."""
        self.pool_idx ^= 1
        pool = self.pools[self.pool_idx]
        ev = self.pool_events[self.pool_idx]
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
        pool[:self.bucket_size[key]].zero_()
        self._view_bucket(key, pool, self.model.g)

    def zero_gradients(self) -> None:
        self.norm_acc.zero_()
        self.norm_fused = False
        if self.stage >= 2:
            self.grad_shard.zero_()
        else:
            self.model.grads.zero_()

    def grads_ready(self, key, last_micro_step: bool) -> None:
        """A bucket's gradients are complete for this micro-step."""
        if self.stage >= 2:
            pool = self.pools[self.pool_idx]
            self.backend.reduce_ranges(pool, self._segs(key), self.shard_range, self.grad_shard, True, False)
            if self.backend_name == "p2p":
                self.pool_events[self.pool_idx] = self.backend.pack_done_event()
        elif last_micro_step:
            segs = [(b, e - b, b) for b, e in self.buckets[key]]
            if not segs:
                return
            if self.stage == 0:
                self.backend.reduce_ranges(self.model.grads, segs, self.shard_range, None, False, True)
            elif self.backend_name == "p2p":      # the reduce kernel also emits the norm partial of its ranges
                self.backend.reduce_ranges(self.model.grads, segs, self.shard_range, self.grad_shard, False, False,
                                           norm_acc=self.norm_acc)
                self.norm_fused = True
            else:
                self.backend.reduce_ranges(self.model.grads, segs, self.shard_range, self.grad_shard, False, False)

    def reduce_all(self) -> None:
        """End of the last micro-step's backward: the main stream joins the comm stream."""
        if self.world_size > 1:
            self.backend.sync()

    # ------------------------------------------------------------------ norm / update
    def grad_norm(self) -> torch.Tensor:
        if self.stage == 0:
            ops.global_norm_squared(self.norm_sq, self.model.grads)        # already averaged, identical on all ranks
        else:
            if self.norm_fused:
                self.norm_sq.copy_(self.norm_acc)
            else:
                ops.global_norm_squared(self.norm_sq, self.grad_shard)
            if self.world_size > 1:
                self.backend.allreduce_scalar(self.norm_sq)
        return self.norm_sq.sqrt()

    def optimizer_step(self, **kw) -> None:
        m = self.model
        if self.stage == 0:
            ops.adamw_update(m.params, m.master, m.grads, m.m, m.v, **kw)
            return
        S, r = self.S, self.rank
        if self.backend_name == "p2p":
            kw.pop("seed", None)
            kw.pop("stochastic_rounding", None)
            if self.stage < 3:      # update my shard and store it into every rank's full parameter buffer
                self.backend.adamw_push(r * S, None, m.master, self.grad_shard, m.m, m.v, S, push=True, **kw)
            else:                   # parameters stay sharded: refresh my shard, peers pull what they need
                self.backend.adamw_push(0, self.param_shard, m.master, self.grad_shard, m.m, m.v, S, push=False, **kw)
        else:
            shard_params = m.params[r * S:(r + 1) * S] if self.stage < 3 else self.param_shard
            ops.adamw_update(shard_params, m.master, self.grad_shard, m.m, m.v, **kw)
            if self.stage < 3 and self.world_size > 1:
                self.backend.push_shard(shard_params, S, m.params)
        self.params_dirty = True
        if self.stage == 3:
            self.window_layers = {}
            for n in LAYER_TENSORS:
                m.p[n].t.clear()
            self.embed_valid = False
            self.window_events = [None, None]

    # ------------------------------------------------------------------ misc
    def rearm_after_timeout(self) -> None:
        if self.backend is not None:
            self.backend.rearm_after_timeout()

    def mean_scalar(self, value: float) -> float:
        if self.world_size == 1 or not dist.is_initialized():
            return value
        t = torch.tensor([value], dtype=torch.float64, device=self.device if dist.get_backend() == "nccl" else "cpu")
        dist.all_reduce(t)
        return float(t.item()) / self.world_size

    # ------------------------------------------------------------------ row collectives (vocab-parallel LM head)
    def all_gather_rows(self, t: torch.Tensor) -> torch.Tensor:
        """[n, ...] on every rank → [W·n, ...] in rank order."""
        if self.world_size == 1:
            return t
        out = torch.empty((self.world_size * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, t.contiguous())
        return out

    def reduce_scatter_rows_f32(self, partial: torch.Tensor, out: torch.Tensor) -> None:
        """out [n·C] fp32 = rows [r·n, (r+1)·n) of the SUM over ranks of partial [W·n·C] fp32, through the peer-memory
        reduce kernel (bf16 on the wire), in pieces that fit the send buffers; joins the main stream when done."""
        W, be = self.world_size, self.backend
        total, n = partial.numel(), partial.numel() // W
        lo, hi = self.rank * n, (self.rank + 1) * n
        cap = be.send_cap
        for c0 in range(0, total, cap):
            c1 = min(total, c0 + cap)
            own = intersect((c0, c1), (lo, hi))
            # positions are relative to this piece; ``shard`` is the owned part of it, ``dst`` starts at the first owned element
            shard = (own[0] - c0, own[1] - c0) if own else (0, 0)
            dst = out[own[0] - lo:] if own else out
            be.reduce_ranges(partial[c0:c1], [(0, c1 - c0, 0)], shard, dst, False, False, scale=1.0)
        be.sync()

    def reduce_scatter_rows(self, t: torch.Tensor) -> torch.Tensor:
        """Sum of [W·n, ...] over ranks; rank r keeps rows [r·n, (r+1)·n)."""
        W = self.world_size
        if W == 1:
            return t
        n = t.shape[0] // W
        if dist.get_backend() == "gloo":                 # Gloo has no reduce-scatter
            tmp = t.float().contiguous()
            dist.all_reduce(tmp)
            return tmp[self.rank * n:(self.rank + 1) * n].to(t.dtype)
        out = torch.empty((n,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        dist.reduce_scatter_tensor(out, t.contiguous())
        return out

    def gather_full_params(self) -> torch.Tensor:
        """Full flat parameter vector on this rank (checkpoint write, sampling; ``_z3_gather_full``)."""
        if self.stage < 3:
            return self.model.params[:self.P]
        if self.world_size == 1:
            return self.param_shard[:self.P]
        parts = [torch.empty_like(self.param_shard) for _ in range(self.world_size)]
        dist.all_gather(parts, self.param_shard.contiguous())
        return torch.cat(parts)[:self.P]

    def load_checkpoint(self, model_path: str, state_path: str):
        m, r, S = self.model, self.rank, self.S
        lo, hi = r * S, min((r + 1) * S, self.P)
        if self.stage < 3:
            _, _, flat = ckpt.read_model_checkpoint(model_path, dtype=torch.float32)
            m.params[:self.P].copy_(flat.to(self.device, m.dtype))
            own = m.params[r * S:(r + 1) * S] if self.stage >= 1 else m.params[:self.n_opt]
        else:
            self.param_shard.zero_()
            if hi > lo:
                _, _, part = ckpt.read_model_checkpoint(model_path, dtype=torch.float32, offset=lo, count=hi - lo)
                self.param_shard[:hi - lo].copy_(part.to(self.device, m.dtype))
            own = self.param_shard
            self.window_layers, self.embed_valid = {}, False
        if m.master is not None:
            m.master.copy_(own.float())
        state, mm, vv = ckpt.read_state_checkpoint(state_path, m.m.numel())
        m.m.copy_(mm.to(self.device))
        m.v.copy_(vv.to(self.device))
        # Peers read this rank's parameter memory directly (stage 3 pulls shards, stages 1/2 were pushed into): nobody
        # may start a forward pass before every rank's load has landed in device memory.
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        if self.world_size > 1 and dist.is_initialized():
            dist.barrier()
        return state

    def memory_report(self) -> dict:
        def nb(t):
            return 0 if t is None else t.numel() * t.element_size()
        rep = {"shard_elems": self.S, "grad_shard_bytes": nb(getattr(self, "grad_shard", None))}
        if self.stage >= 2:
            rep["grad_pool_bytes"] = sum(nb(p) for p in self.pools)
        if self.stage == 3:
            rep["param_shard_bytes"] = nb(self.param_shard)
            rep["window_bytes"] = sum(nb(w) for w in self.windows) + nb(self.embed_window)
        if self.backend_name == "p2p" and self.backend is not None:
            rep["comm_arena_bytes"] = self.backend.arena.nbytes
        return rep

    def close(self) -> None:
        if self.backend is not None:
            self.backend.close()
