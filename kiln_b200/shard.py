"""N-sharded column-parallel W4A16 GEMM across the GPUs of one node.

The reference is single-GPU (its wrapper hard-codes device 0,
kiln-marlin-gemm/src/lib.rs:210-215); this module is the multi-GPU extension of the same
call.  Every output column depends on one column of the weight and its scales, and the
Marlin layout is separable along N at 64-column granularity, so a shard is a plain slice
of the packed tensors: b_packed[:, 2*n0:2*n1] and scales[:, n0:n1].  Rank r of g owns
columns [r*N/g, (r+1)*N/g); activations are replicated; the one exchange step is an
all-gather of the bf16 output slices (NCCL over NVLink on GPUs, any backend in tests).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from .marlin_gemm import KilnMarlinError, marlin_w4a16_gemm
from .marlin_proj import MarlinPackedProj


def shard_bounds(n: int, rank: int, world: int) -> tuple:
    """Column range [n0, n1) of `rank`; N/world must keep the kernel's 256-column rule."""
    if world < 1 or not (0 <= rank < world):
        raise KilnMarlinError(f"kiln-marlin-gemm: bad shard rank {rank} of {world}")
    if n % world != 0 or (n // world) % 256 != 0:
        raise KilnMarlinError(
            f"kiln-marlin-gemm: n={n} cannot be split over {world} ranks in multiples of 256 columns")
    per = n // world
    return rank * per, (rank + 1) * per


def shard_packed(b_packed: torch.Tensor, scales: torch.Tensor, rank: int, world: int):
    """Slices of the packed weight [k/16, 2n] and the scales [k/g, n] owned by `rank` (contiguous copies)."""
    n = scales.shape[1]
    if b_packed.shape[1] != 2 * n:
        raise KilnMarlinError(f"kiln-marlin-gemm: b_packed has {b_packed.shape[1]} columns, expected {2 * n}")
    n0, n1 = shard_bounds(n, rank, world)
    return b_packed[:, 2 * n0:2 * n1].contiguous(), scales[:, n0:n1].contiguous()


def shard_proj(proj: MarlinPackedProj, rank: int, world: int) -> MarlinPackedProj:
    b, s = shard_packed(proj.b_packed, proj.scales, rank, world)
    return MarlinPackedProj(b, s, proj.groupsize, proj.k, proj.n // world)


def all_gather_columns(local: torch.Tensor, group=None, out: Optional[torch.Tensor] = None,
                       row_major: bool = False) -> torch.Tensor:
    """All-gather of the [m, n/g] output slices.

    Returns the blocked result [g, m, n/g] (block r = columns of rank r) -- what the collective
    produces without another pass -- or, with row_major=True, the dense [m, n] matrix
    (one extra device copy).  `out` may supply the blocked buffer.
    """
    world = dist.get_world_size(group)
    m, nl = local.shape
    if out is None:
        out = torch.empty((world, m, nl), dtype=local.dtype, device=local.device)
    elif tuple(out.shape) != (world, m, nl) or not out.is_contiguous():
        raise KilnMarlinError("kiln-marlin-gemm: gather buffer must be contiguous [world, m, n/world]")
    dist.all_gather_into_tensor(out.view(world * m, nl), local.contiguous(), group=group)
    if row_major:
        return out.permute(1, 0, 2).reshape(m, world * nl)
    return out


@dataclass
class ColumnParallelLinear:
    """One rank's shard of a W4A16 projection plus the gather of its outputs."""

    shard: MarlinPackedProj
    rank: int
    world: int
    group: object = None

    @classmethod
    def from_full(cls, proj: MarlinPackedProj, group=None) -> "ColumnParallelLinear":
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        return cls(shard_proj(proj, rank, world), rank, world, group)

    def local(self, a: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        return marlin_w4a16_gemm(a, self.shard.b_packed, self.shard.scales, self.shard.groupsize, out=out)

    def forward(self, a: torch.Tensor, gathered: Optional[torch.Tensor] = None, row_major: bool = False,
                m_chunks: int = 1) -> torch.Tensor:
        """GEMM on the local columns, then all-gather.  With m_chunks > 1 the rows are processed in
        chunks and each chunk's gather runs on a side stream while the next chunk's GEMM computes."""
        if m_chunks <= 1 or not a.is_cuda:
            return all_gather_columns(self.local(a), self.group, gathered, row_major)
        m = a.shape[0]
        nl = self.shard.n
        if m % m_chunks != 0:
            raise KilnMarlinError(f"kiln-marlin-gemm: m={m} not divisible by m_chunks={m_chunks}")
        mc = m // m_chunks
        # chunk-major blocked buffer [chunks, world, mc, nl]: each chunk's gather writes one contiguous slab
        buf = torch.empty((m_chunks, self.world, mc, nl), dtype=torch.bfloat16, device=a.device)
        local = torch.empty((m, nl), dtype=torch.bfloat16, device=a.device)
        main = torch.cuda.current_stream(a.device)
        side = _side_stream(a.device)
        for c in range(m_chunks):
            self.local(a[c * mc:(c + 1) * mc], out=local[c * mc:(c + 1) * mc])
            ev = torch.cuda.Event()
            ev.record(main)
            with torch.cuda.stream(side):
                side.wait_event(ev)
                dist.all_gather_into_tensor(buf[c].view(self.world * mc, nl), local[c * mc:(c + 1) * mc],
                                            group=self.group)
        main.wait_stream(side)
        blocked = buf.permute(1, 0, 2, 3)  # [world, chunks, mc, nl] view
        if row_major:
            return blocked.permute(1, 2, 0, 3).reshape(m, self.world * nl)
        out = blocked.reshape(self.world, m, nl)  # copies into the [g, m, n/g] layout
        if gathered is not None:
            gathered.copy_(out)
            return gathered
        return out


class FusedGatherOutput:
    """A row-major [m, n] bf16 result buffer that every GPU of the group can store into: symmetric memory
    (torch.distributed._symmetric_memory), one allocation per rank, peer-mapped after a rendezvous."""

    def __init__(self, m: int, n: int, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        group = group if group is not None else dist.group.WORLD
        self.group = group
        self.tensor = symm_mem.empty((m, n), dtype=torch.bfloat16, device=device)
        self.handle = symm_mem.rendezvous(self.tensor, group)
        world = dist.get_world_size(group)
        ptrs = getattr(self.handle, "buffer_ptrs", None)
        if ptrs is None:
            ptrs = [self.handle.get_buffer(r, (m, n), torch.bfloat16).data_ptr() for r in range(world)]
        self.ptrs = [int(x) for x in ptrs]
        # NVSwitch multicast address of the same buffers (0 when the fabric or the driver offers none)
        self.multicast_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        self._flag = torch.zeros(1, dtype=torch.int32, device=device)
        self._written = False  # a fused launch has stored into the group's buffers since the last reuse barrier

    def barrier(self):
        """Stream-ordered barrier across the group (a one-element NCCL all-reduce): when it completes on a
        rank, every rank's launch before it has finished, so all slices have arrived."""
        dist.all_reduce(self._flag, group=self.group)


def fused_column_parallel_gemm(a: torch.Tensor, lin: "ColumnParallelLinear", out: FusedGatherOutput,
                               barrier: bool = True, multicast: Optional[bool] = None,
                               reuse_barrier: bool = True) -> torch.Tensor:
    """Local columns x all-gather in ONE kernel: the tcgen05 GEMM stores each finished tile into the
    [m, n] buffer of every GPU over NVLink (kiln_w4a16_gemm_bf16_allgather).  Returns this rank's full
    row-major [m, n] result.

    multicast=True writes each piece once to the group's NVSwitch multicast address (multimem.st,
    kiln_w4a16_gemm_bf16_allgather_multicast) instead of once per GPU; None picks it when the buffer has a
    multicast address and the group has more than two GPUs (with two there is nothing to save).

    Buffer reuse: this rank's launch overwrites every OTHER rank's copy of `out`, so the readers of result i on
    every rank must be done before any rank launches call i+1 into the same buffer.  With reuse_barrier=True
    (default) a second stream-ordered barrier is issued before the launch whenever the buffer already holds a
    result: a rank leaves it only after every rank's stream has reached it, i.e. after every rank's kernels that
    read the previous result (enqueued on that stream before this call) have finished.  Pass False only when the
    caller orders readers and writers itself, e.g. by alternating two buffers."""
    import ctypes

    from . import _lib

    m, k = a.shape
    sh = lin.shard
    n_total = sh.n * lin.world
    if tuple(out.tensor.shape) != (m, n_total):
        raise KilnMarlinError(f"kiln-marlin-gemm: fused gather buffer is {tuple(out.tensor.shape)}, expected {(m, n_total)}")
    if k != sh.k or a.dtype != torch.bfloat16 or not a.is_cuda:
        raise KilnMarlinError("kiln-marlin-gemm: a must be a CUDA bf16 [m, k] tensor matching the shard")
    if multicast is None:
        multicast = out.multicast_ptr != 0 and lin.world > 2
    if multicast and out.multicast_ptr == 0:
        raise KilnMarlinError("kiln-marlin-gemm: this buffer has no multicast address")
    arr = (ctypes.c_void_p * lin.world)(*out.ptrs)
    a = a.contiguous()
    if reuse_barrier and out._written:
        out.barrier()
    out._written = True
    with torch.cuda.device(a.device):
        if multicast:
            rc = _lib.lib().kiln_w4a16_gemm_bf16_allgather_multicast(
                a.data_ptr(), sh.b_packed.data_ptr(), sh.scales.data_ptr(), m, sh.n, k, sh.groupsize,
                out.multicast_ptr, n_total, lin.rank * sh.n, torch.cuda.current_stream(a.device).cuda_stream)
        else:
            rc = _lib.lib().kiln_w4a16_gemm_bf16_allgather(
                a.data_ptr(), sh.b_packed.data_ptr(), sh.scales.data_ptr(), m, sh.n, k, sh.groupsize,
                ctypes.cast(arr, ctypes.c_void_p), lin.world, n_total, lin.rank * sh.n,
                torch.cuda.current_stream(a.device).cuda_stream)
    if rc != 0:
        raise KilnMarlinError(f"kiln_w4a16_gemm_bf16_allgather failed: {_lib.STATUS_NAMES.get(rc, rc)}")
    if barrier:
        out.barrier()
    return out.tensor


_side_streams: dict = {}


def _side_stream(device) -> "torch.cuda.Stream":
    s = _side_streams.get(device)
    if s is None:
        s = torch.cuda.Stream(device)
        _side_streams[device] = s
    return s
