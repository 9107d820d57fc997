"""Host logic of the N-sharded column-parallel path on CPU ranks (gloo, world size 2):
shard slicing equals packing the column slice, and the gather reassembles the full output.
Failure cases are made on the host (bad rank, indivisible N, a rank that never joins)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import kiln_b200
import oracle
from oracle import C

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m, k, n = 3, 256, 1024
        a, qn, s = oracle.synth_inputs(m, k, n, seed=4)
        packed, sp = kiln_b200.pack.repack(qn, s, 128)
        b_t, s_t = torch.from_numpy(packed), torch.from_numpy(sp.view(np.int16).copy()).view(torch.float16)
        bs, ss = kiln_b200.shard_packed(b_t, s_t, rank, world)
        n0, n1 = kiln_b200.shard_bounds(n, rank, world)
        # a shard is bit-identical to packing the column slice on its own
        p2, s2 = kiln_b200.pack.repack(qn[:, n0:n1], s[:, n0:n1], 128)
        assert (bs.numpy() == p2).all() and (ss.view(torch.int16).numpy().view(np.uint16) == s2.view(np.uint16)).all()
        # stand-in for the device GEMM on this rank's columns: the CPU oracle on the slice
        local = torch.from_numpy(oracle.f32_to_bf16_bits(C.gemm_fp64(a, qn[:, n0:n1], s[:, n0:n1], 128)).view(np.int16)).view(torch.bfloat16)
        blocked = kiln_b200.all_gather_columns(local)
        assert blocked.shape == (world, m, n // world)
        dense = kiln_b200.all_gather_columns(local, row_major=True)
        full = oracle.f32_to_bf16_bits(C.gemm_fp64(a, qn, s, 128)).view(np.int16)
        assert (dense.contiguous().view(torch.int16).numpy() == full).all()
        assert (blocked[rank].view(torch.int16).numpy() == full[:, n0:n1]).all()
        q.put((rank, "ok"))
    except Exception as e:  # pragma: no cover
        q.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


def test_two_rank_shard_and_gather_on_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(30)
    assert sorted(res) == [(0, "ok"), (1, "ok")], res


def test_shard_rejections_are_host_side():
    b = torch.zeros(8, 2 * 1024, dtype=torch.int32)
    s = torch.zeros(1, 1024, dtype=torch.float16)
    with pytest.raises(kiln_b200.KilnMarlinError, match="bad shard rank"):
        kiln_b200.shard_packed(b, s, 2, 2)
    with pytest.raises(kiln_b200.KilnMarlinError, match="cannot be split"):
        kiln_b200.shard_packed(b, s, 0, 8)  # 1024/8 = 128 columns per rank: below the 256-column rule
    with pytest.raises(kiln_b200.KilnMarlinError, match="cannot be split"):
        kiln_b200.shard_bounds(1024, 0, 3)
    assert kiln_b200.shard_bounds(73728, 7, 8) == (64512, 73728)


def _late_rank(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import datetime

    try:
        # rank 1 never joins: rank 0's rendezvous must end with an error, not hang
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
        q.put("joined")
    except Exception as e:
        q.put("error:" + type(e).__name__)


def test_missing_rank_is_an_error_not_a_hang():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_late_rank, args=(0, 2, _free_port(), q))
    p.start()
    out = q.get(timeout=120)
    p.join(30)
    assert out.startswith("error:"), out
