"""The entry point that allocates nothing: kiln_w4a16_gemm_bf16_noalloc.

Who needs it: a caller that cannot allocate device memory when it calls and has no workspace to lend
either -- for example a server that gave all remaining HBM to its KV-cache pool at start-up, or a
serving loop that cannot take the device-wide synchronisation of cudaMalloc/cudaFree.  The split-K
scratch of the tcgen05 kernel then lives in a 16 MiB array inside the library's device image.

The test calls it through the C ABI twice in a row on shapes where the kernel really splits K (so the
built-in scratch is used, and the second call finds the first call's leftovers in it) and compares with
the regular entry point, which takes the scratch from the caller, within the tolerance all GEMM tests use
(1e-2 of the largest output; the two entry points may pick different tilings, so the fp32 summation order
can differ).  The two calls of the new entry point itself must agree bit for bit, and the oracle is checked too.
This file sorts last so that a run that stops at the first failure has already run everything else."""
import ctypes

import numpy as np
import pytest
import torch

import kiln_b200
from kiln_b200 import _lib
import oracle
from oracle import C
from tests.util import REL_TOL, from_torch_bf16, rel_err, to_torch_bf16

pytestmark = pytest.mark.gpu

SCRATCH_LIMIT = 16 << 20


def _case(m, k, n, seed, device):
    a, q, s = oracle.synth_inputs(m, k, n, seed=seed)
    packed, sp = kiln_b200.pack.repack(q, s, 128)
    return dict(a=a, q=q, s=s, a_t=to_torch_bf16(a, device), b_t=torch.from_numpy(packed).to(device),
                s_t=torch.from_numpy(sp.view(np.int16).copy()).view(torch.float16).to(device))


def _plan(m, k, n):
    out = (ctypes.c_int * 4)()
    _lib.lib().kiln_w4a16_noalloc_plan(m, n, k, out)
    return list(out)


def _noalloc(case, m, k, n, out=None):
    if out is None:
        out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=case["a_t"].device)
    rc = _lib.lib().kiln_w4a16_gemm_bf16_noalloc(case["a_t"].data_ptr(), case["b_t"].data_ptr(), out.data_ptr(),
                                                 case["s_t"].data_ptr(), m, n, k, 128,
                                                 torch.cuda.current_stream().cuda_stream)
    assert rc == 0, _lib.STATUS_NAMES.get(rc, rc)
    return out


def test_noalloc_entry_matches_regular_entry_twice_in_a_row(cuda_device):
    shapes = [(256, 9216, 2560), (384, 9216, 512)]  # both split K: the scratch is really used
    # (with one 128-row M-tile per B stage, which is what this entry point runs, the launch heuristic splits K
    # three ways for both shapes: 7.5 MiB and 6 MiB of partial sums)
    cases = [(_case(m, k, n, 900 + i, cuda_device), m, k, n) for i, (m, k, n) in enumerate(shapes)]
    for _, m, k, n in cases:
        plan = _plan(m, k, n)
        assert plan[1] > 1, f"this test needs a K-splitting tiling, the entry point plans {plan} for {(m, k, n)}"
        assert plan[1] * m * n * 4 <= SCRATCH_LIMIT
    # every tensor the calls touch exists before the free-memory reading: what changes after it would be the library's doing
    bufs = [[torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=cuda_device) for _, m, k, n in cases] for _ in range(2)]
    _noalloc(cases[0][0], *cases[0][1:], out=bufs[0][0])  # first call on this device: symbol look-up, function attributes
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info(cuda_device)[0]
    # two calls in a row, different problems: the second finds the first one's partial sums in the array
    outs = [_noalloc(c, m, k, n, out=o) for (c, m, k, n), o in zip(cases, bufs[0])]
    outs2 = [_noalloc(c, m, k, n, out=o) for (c, m, k, n), o in zip(cases, bufs[1])]
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info(cuda_device)[0] == free_before, "free device memory changed across the calls"
    assert _lib.lib().kiln_w4a16_check_device_status(None, None) == 0
    for (c, m, k, n), o1, o2 in zip(cases, outs, outs2):
        ref_entry = kiln_b200.marlin_w4a16_gemm(c["a_t"], c["b_t"], c["s_t"], 128)  # caller-owned workspace
        torch.cuda.synchronize()
        assert not torch.isnan(o1.float()).any()
        assert torch.equal(o1, o2), "second call (scratch holding the first call's partial sums) changed the result"
        d = float((o1.float() - ref_entry.float()).abs().max() / ref_entry.float().abs().max())
        assert d <= REL_TOL, f"no-alloc entry differs from the regular entry by {d}"
        rows = np.array([0, 1, m // 2, m - 1])
        ref = C.gemm_fp64(c["a"][rows], c["q"], c["s"], 128)
        assert rel_err(from_torch_bf16(o2[torch.from_numpy(rows).to(o2.device)]), ref) <= REL_TOL


def test_noalloc_entry_small_m_and_no_split(cuda_device):
    # any m goes through the tcgen05 kernel here; a shape that does not split K uses no scratch at all
    for m, k, n in [(5, 256, 512), (130, 512, 768)]:
        c = _case(m, k, n, 950 + m, cuda_device)
        out = _noalloc(c, m, k, n)
        torch.cuda.synchronize()
        ref = C.gemm_fp64(c["a"], c["q"], c["s"], 128)
        assert rel_err(from_torch_bf16(out), ref) <= REL_TOL


def test_noalloc_entry_falls_back_to_a_tiling_that_fits(cuda_device):
    """Where the preferred split would need more than the built-in 16 MiB, the entry point takes the best tiling that
    fits instead of refusing (a tiling without a split always fits)."""
    lib = _lib.lib()
    m, k, n = 384, 16384, 4096  # a three-way split would need 18 MiB of partial sums
    plan = _plan(m, k, n)
    assert plan[1] * m * n * 4 <= SCRATCH_LIMIT or plan[1] == 1
    c = _case(m, k, n, 977, cuda_device)
    out = _noalloc(c, m, k, n)
    torch.cuda.synchronize()
    rows = np.array([0, 127, 128, m - 1])
    ref = C.gemm_fp64(c["a"][rows], c["q"], c["s"], 128)
    assert rel_err(from_torch_bf16(out[torch.from_numpy(rows).to(out.device)]), ref) <= REL_TOL
    assert lib.kiln_w4a16_check_device_status(None, None) == 0


def test_noalloc_entry_rejects_what_does_not_fit(cuda_device):
    lib = _lib.lib()
    m, k, n = 1024, 8192, 4096
    # real buffers of the right sizes, so that a regression that launches instead of refusing stays harmless
    a_t = torch.zeros((m, k), dtype=torch.bfloat16, device=cuda_device)
    b_t = torch.zeros((k // 16, 2 * n), dtype=torch.int32, device=cuda_device)
    s_t = torch.ones((k // 128, n), dtype=torch.float16, device=cuda_device)
    out = torch.zeros((m, n), dtype=torch.bfloat16, device=cuda_device)
    args = (a_t.data_ptr(), b_t.data_ptr(), out.data_ptr(), s_t.data_ptr())
    torch.cuda.synchronize()
    before = lib.kiln_w4a16_launch_count()
    try:  # only a tiling forced through the tuning hook can still exceed the array: 8 x 1024 x 4096 x 4 B = 128 MiB
        lib.kiln_w4a16_set_prefill_override(256, 8, 1, 0)
        assert lib.kiln_w4a16_gemm_bf16_noalloc(*args, m, n, k, 128, None) == _lib.ERR_STATIC_SCRATCH
    finally:
        lib.kiln_w4a16_set_prefill_override(0, 0, 0, 0)
    assert lib.kiln_w4a16_launch_count() == before  # refused before anything was launched
    assert lib.kiln_w4a16_gemm_bf16_noalloc(*args, 4, 200, 128, 128, None) == _lib.ERR_PROB_SHAPE
    assert lib.kiln_w4a16_gemm_bf16_noalloc(None, *args[1:], 4, 256, 128, 128, None) == _lib.ERR_ARG
