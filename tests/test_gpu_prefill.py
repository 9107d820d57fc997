"""GPU parity of the tcgen05 prefill kernel (M >= 128), through the C ABI.

The fp64 oracle is evaluated on a sample of rows (every output row depends on one row of A only), and the
whole output is also compared with a float32 torch matmul of the dequantised weight on the GPU.
Tolerance: max|out - ref| / max|ref| <= 1e-2."""
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


@pytest.fixture(autouse=True)
def _force_tcgen05_kernel():
    """This module tests the tcgen05 kernel: route every M to it, whatever the built-in kernel-selection rule says."""
    _lib.lib().kiln_w4a16_set_prefill_min_m(1)
    yield
    _lib.lib().kiln_w4a16_set_prefill_min_m(0)


def _case(m, k, n, seed, groupsize=128, device=None):
    a, q, s = oracle.synth_inputs(m, k, n, seed=seed, groupsize=groupsize)
    packed, sp = kiln_b200.pack.repack(q, s, groupsize)
    return dict(a=a, q=q, s=s, m=m, k=k, n=n, gs=groupsize,
                a_t=to_torch_bf16(a, device), b_t=torch.from_numpy(packed).to(device),
                s_t=torch.from_numpy(sp.view(np.int16).copy()).view(torch.float16).to(device))


def _check(case, out, rows=24):
    torch.cuda.synchronize()
    assert _lib.lib().kiln_w4a16_check_device_status(None, None) == 0, "a bounded device wait gave up"
    m, k, n, gs = case["m"], case["k"], case["n"], case["gs"]
    rng = np.random.default_rng(m + n)
    sel = np.unique(np.concatenate([[0, m - 1, min(m - 1, 127), min(m - 1, 128)], rng.integers(0, m, rows)]))
    ref = C.gemm_fp64(case["a"][sel], case["q"], case["s"], gs)
    got = from_torch_bf16(out[torch.from_numpy(sel).to(out.device)])
    e = rel_err(got, ref)
    assert e <= REL_TOL, f"sampled-row rel err {e}"
    # whole output against float32 torch on the device
    g = k if gs == -1 else gs
    dev = out.device
    w = (torch.from_numpy(case["q"].astype(np.float32)).to(dev) - 8.0) * \
        torch.from_numpy(case["s"].astype(np.float32)).to(dev).repeat_interleave(g, dim=0)
    full = case["a_t"].float() @ w
    e2 = float((out.float() - full).abs().max() / full.abs().max())
    assert e2 <= REL_TOL, f"full-output rel err {e2}"
    return e, e2


@pytest.mark.parametrize("m,k,n", [(128, 128, 256), (128, 256, 512), (256, 2560, 512), (384, 512, 768),
                                   (512, 2560, 4096), (512, 9216, 2560)])
def test_prefill_shapes(cuda_device, m, k, n):
    case = _case(m, k, n, seed=m + k + n, device=cuda_device)
    out = kiln_b200.marlin_w4a16_gemm(case["a_t"], case["b_t"], case["s_t"], 128)
    _check(case, out)


@pytest.mark.parametrize("m", [129, 200, 255, 257, 1000])
def test_prefill_ragged_m(cuda_device, m):
    case = _case(m, 640, 512, seed=m, device=cuda_device)
    buf = torch.full((m + 2, 512), 3.0, dtype=torch.bfloat16, device=cuda_device)
    out = kiln_b200.marlin_w4a16_gemm(case["a_t"], case["b_t"], case["s_t"], 128, out=buf[1:m + 1])
    _check(case, out)
    assert (buf[0] == 3.0).all() and (buf[m + 1] == 3.0).all()  # rows outside [0, m) untouched


def test_prefill_benchmark_shapes(cuda_device):
    """Chunked-prefill configuration: M=2048 on gate+up 2560->18432 and down 9216->2560."""
    for m, k, n in [(2048, 2560, 18432), (2048, 9216, 2560)]:
        case = _case(m, k, n, seed=7, device=cuda_device)
        out = kiln_b200.marlin_w4a16_gemm(case["a_t"], case["b_t"], case["s_t"], 128)
        _check(case, out, rows=8)


@pytest.mark.parametrize("name,k,n", [("gate_up", 2560, 18432), ("down", 9216, 2560)])
def test_prefill_m8192_with_the_rules_own_tiling(cuda_device, name, k, n):
    """Chunked-prefill configuration at its largest M, nothing forced: on the down projection the built-in rule picks
    hybrid stream-K here (320 tiles on 148 SMs), on gate+up pairs of M-tiles."""
    m = 8192
    plan = (ctypes.c_int * 4)()
    _lib.lib().kiln_w4a16_prefill_plan(m, n, k, plan)
    if name == "down":
        assert plan[3] == 1 or plan[1] > 1, f"expected a K-splitting plan for {name}, got {list(plan)}"
    case = _case(m, k, n, seed=8192 + n, device=cuda_device)
    out = kiln_b200.marlin_w4a16_gemm(case["a_t"], case["b_t"], case["s_t"], 128)
    _check(case, out, rows=6)


def test_shard_shape_of_the_column_parallel_configuration(cuda_device):
    """M=16384, K=9216, N=9216: what one of eight GPUs computes in the N-sharded configuration (N=73728)."""
    m, k, n = 16384, 9216, 9216
    case = _case(m, k, n, seed=4, device=cuda_device)
    out = kiln_b200.marlin_w4a16_gemm(case["a_t"], case["b_t"], case["s_t"], 128)
    _check(case, out, rows=4)


def test_prefill_per_column(cuda_device):
    case = _case(256, 512, 512, seed=3, groupsize=-1, device=cuda_device)
    out = kiln_b200.marlin_w4a16_gemm(case["a_t"], case["b_t"], case["s_t"], -1)
    _check(case, out)


def test_prefill_matches_decode_kernel_and_is_reproducible(cuda_device):
    """Both kernels compute the same function; the prefill kernel is bit-reproducible run to run."""
    lib = _lib.lib()
    case = _case(160, 1280, 1024, seed=11, device=cuda_device)
    out1 = kiln_b200.marlin_w4a16_gemm(case["a_t"], case["b_t"], case["s_t"], 128)
    out2 = kiln_b200.marlin_w4a16_gemm(case["a_t"], case["b_t"], case["s_t"], 128)
    torch.cuda.synchronize()
    assert torch.equal(out1, out2)
    try:
        lib.kiln_w4a16_set_prefill_min_m(1 << 30)  # force the decode kernel
        out3 = kiln_b200.marlin_w4a16_gemm(case["a_t"], case["b_t"], case["s_t"], 128)
        torch.cuda.synchronize()
    finally:
        lib.kiln_w4a16_set_prefill_min_m(0)
    d = float((out1.float() - out3.float()).abs().max() / out3.float().abs().max())
    assert d < 1e-2
    _check(case, out1)
