"""N-sharded column-parallel GEMM on 2 GPUs (NCCL): gathered result equals the single-GPU result
bit for bit and matches the oracle.  Skipped on a box with one GPU.  NVLS is switched off and no rank
leaves mid-step: nothing here faults, traps or hangs a GPU."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    import kiln_b200
    import oracle
    from oracle import C

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    import datetime

    # a short timeout: if one rank fails an assertion and leaves, its peer's next collective ends with an error
    # instead of spinning on the GPU
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=60))
    ok = False
    try:
        for m, k, n, chunks in [(4, 512, 1024, 1), (256, 640, 1024, 1), (256, 640, 1024, 2)]:
            a, qn, s = oracle.synth_inputs(m, k, n, seed=40 + m)
            packed, sp = kiln_b200.pack.repack(qn, s, 128)
            a_t = torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16).to(dev)
            proj = kiln_b200.MarlinPackedProj(torch.from_numpy(packed).to(dev),
                                              torch.from_numpy(sp.view(np.int16).copy()).view(torch.float16).to(dev),
                                              128, k, n)
            full = kiln_b200.matmul_bf16(a_t, proj)
            lin = kiln_b200.ColumnParallelLinear.from_full(proj)
            dense = lin.forward(a_t, row_major=True, m_chunks=chunks)
            blocked = lin.forward(a_t, m_chunks=chunks)
            torch.cuda.synchronize()
            # Bit for bit, the gathered matrix is the column-wise concatenation of the per-shard GEMMs.  Against the single-GPU
            # GEMM over all columns it may differ in the last bit: the K split (cluster size, split-K, stream-K) is chosen per
            # problem shape, and a shard is a narrower problem, so fp32 partial sums can be added in a different order.
            nl = n // world
            mc = m // chunks  # the M-chunked path runs one local GEMM per chunk of rows
            own = torch.cat([kiln_b200.matmul_bf16(a_t[c * mc:(c + 1) * mc], lin.shard) for c in range(chunks)], dim=0)
            torch.cuda.synchronize()
            assert torch.equal(dense[:, rank * nl:(rank + 1) * nl], own), "own columns differ from the local GEMM"
            assert torch.equal(blocked[rank], own)
            assert torch.equal(dense, blocked.permute(1, 0, 2).reshape(m, n)), "row-major and blocked results differ"
            d_full = float((dense.float() - full.float()).abs().max() / full.float().abs().max())
            assert d_full <= 2.0 ** -7, f"gathered result is {d_full} away from the single-GPU result"
            if m >= 64:  # the fused-gather epilogue lives in the tcgen05 kernel
                sym = kiln_b200.FusedGatherOutput(m, n, dev)
                # two calls into the same buffer with different activations: the second may only overwrite a peer's copy
                # after that peer has read the first result (the clone below is enqueued before the second call)
                a_neg = (-a_t).contiguous()
                first = kiln_b200.fused_column_parallel_gemm(a_neg, lin, sym).clone()
                fused = kiln_b200.fused_column_parallel_gemm(a_t, lin, sym)
                torch.cuda.synchronize()
                assert torch.equal(first, -fused), "the first result was overwritten before it was read"
                d = float((fused.float() - full.float()).abs().max() / full.float().abs().max())
                assert d <= 1e-2, f"fused all-gather result differs by {d}"
                # the fused launch never splits K (its epilogue needs whole tiles), the plain one may: same columns to 2^-7
                d_own = float((fused[:, rank * nl:(rank + 1) * nl].float() - own.float()).abs().max() / own.float().abs().max())
                assert d_own <= 2.0 ** -7, f"own slice of the fused result is {d_own} away from the plain local GEMM"
                # the same through the NVSwitch multicast address, where the fabric offers one to every rank
                has_mc = torch.tensor([1 if sym.multicast_ptr else 0], device=dev)
                dist.all_reduce(has_mc, op=dist.ReduceOp.MIN)
                if int(has_mc.item()):
                    keep = fused.clone()
                    sym.tensor.zero_()
                    torch.cuda.synchronize()
                    dist.barrier()
                    mc = kiln_b200.fused_column_parallel_gemm(a_t, lin, sym, multicast=True)
                    torch.cuda.synchronize()
                    assert torch.equal(mc, keep), "multicast stores must give the same matrix as peer stores"
            ref = C.gemm_fp64(a, qn, s, 128)
            got = oracle.bf16_bits_to_f32(dense.cpu().view(torch.int16).numpy().view(np.uint16))
            assert np.abs(got - ref).max() / np.abs(ref).max() <= 1e-2
        ok = True
        q.put((rank, "ok"))
    except Exception as e:  # pragma: no cover
        q.put((rank, repr(e)))
    finally:
        # no collective on the failure path: a rank that failed leaves between steps with nothing of its own in flight
        torch.cuda.synchronize()
        if ok:
            dist.barrier()
            dist.destroy_process_group()


def test_two_gpu_column_parallel():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = []
    try:
        for _ in procs:
            res.append(q.get(timeout=300))
    except Exception as e:  # queue.Empty: a rank never reported
        res.append(("parent", repr(e)))
    for p in procs:
        p.join(90)
    for p in procs:  # a child that outlived both waits is stopped by its exact handle
        if p.is_alive():
            p.terminate()
            p.join(10)
    assert sorted(res, key=str) == [(0, "ok"), (1, "ok")], res
