"""GPU parity of the small-batch tcgen05 kernel (at most 128 rows; the dequantised weights live in tensor memory),
through the C ABI.

Each case is checked against the fp64 oracle (every row), against a float32 torch matmul of the dequantised weight,
and bit for bit against the general tcgen05 kernel on the same inputs: both dequantise with the same two bf16 roundings
and accumulate the same products in fp32 tensor-core accumulators, K split the same way.
Tolerance against the oracle: max|out - ref| / max|ref| <= 1e-2."""
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
def _restore_hooks():
    yield
    _lib.lib().kiln_w4a16_set_prefill_min_m(0)
    _lib.lib().kiln_w4a16_set_small_batch_kernel(1)


def _case(m, k, n, seed, device, groupsize=128):
    a, q, s = oracle.synth_inputs(m, k, n, seed=seed, groupsize=groupsize)
    packed, sp = kiln_b200.pack.repack(q, s, groupsize)
    return dict(a=a, q=q, s=s, a_t=to_torch_bf16(a, device), b_t=torch.from_numpy(packed).to(device),
                s_t=torch.from_numpy(sp.view(np.int16).copy()).view(torch.float16).to(device))


def _run(case, small_batch, m, n, device, groupsize=128):
    lib = _lib.lib()
    lib.kiln_w4a16_set_prefill_min_m(1)  # a tcgen05 kernel whatever the built-in rule says
    lib.kiln_w4a16_set_small_batch_kernel(1 if small_batch else 0)
    buf = torch.full((m + 2, n), 3.0, dtype=torch.bfloat16, device=device)
    out = kiln_b200.marlin_w4a16_gemm(case["a_t"], case["b_t"], case["s_t"], groupsize, out=buf[1:m + 1])
    torch.cuda.synchronize()
    assert lib.kiln_w4a16_check_device_status(None, None) == 0, "a bounded device wait gave up"
    assert (buf[0] == 3.0).all() and (buf[m + 1] == 3.0).all()  # rows outside [0, m) untouched
    return out


# one K stage, one tile; ragged row counts around the MMA's N steps of 16; K splits (q: 4, down: 6); many tiles per CTA;
# the 128-row variant (65..128 rows: one accumulator buffer), also with several tiles per CTA
@pytest.mark.parametrize("m,k,n", [(1, 128, 256), (16, 256, 256), (17, 640, 512), (31, 2560, 4096), (33, 4096, 2560),
                                   (47, 9216, 2560), (48, 2560, 8192), (64, 2560, 18432), (64, 128, 256),
                                   (63, 1152, 38400), (65, 2560, 4096), (100, 9216, 2560),
                                   (128, 2560, 18432), (127, 640, 512), (100, 640, 38400)])
def test_small_batch_kernel_matches_the_oracle_and_the_general_kernel(cuda_device, m, k, n):
    case = _case(m, k, n, seed=3 * m + k + n, device=cuda_device)
    out = _run(case, True, m, n, cuda_device)
    ref = C.gemm_fp64(case["a"], case["q"], case["s"], 128)
    e = rel_err(from_torch_bf16(out), ref)
    assert e <= REL_TOL, f"oracle rel err {e}"
    w = (torch.from_numpy(case["q"].astype(np.float32)).to(cuda_device) - 8.0) * \
        torch.from_numpy(case["s"].astype(np.float32)).to(cuda_device).repeat_interleave(128, dim=0)
    full = case["a_t"].float() @ w
    assert float((out.float() - full).abs().max() / full.abs().max()) <= REL_TOL
    general = _run(case, False, m, n, cuda_device)
    assert torch.equal(out.view(torch.int16), general.view(torch.int16)), "differs from the general tcgen05 kernel"


# per-column scales (group size -1): dequantised unscaled, the scale applied by the epilogue or by the split-K reduction
@pytest.mark.parametrize("m,k,n", [(24, 640, 512), (100, 2560, 4096), (64, 9216, 2560)])
def test_small_batch_kernel_with_per_column_scales(cuda_device, m, k, n):
    case = _case(m, k, n, seed=m + k + n, device=cuda_device, groupsize=-1)
    out = _run(case, True, m, n, cuda_device, groupsize=-1)
    assert rel_err(from_torch_bf16(out), C.gemm_fp64(case["a"], case["q"], case["s"], -1)) <= REL_TOL
    general = _run(case, False, m, n, cuda_device, groupsize=-1)
    assert torch.equal(out.view(torch.int16), general.view(torch.int16)), "differs from the general tcgen05 kernel"


def test_built_in_rule_routes_17_to_64_rows_of_wide_projections_here(cuda_device):
    """Without any hook the dispatcher takes the tcgen05 path from 17 rows for projections of more than 1024 columns (the
    workspace query says so: q splits K four ways) and keeps narrow projections and up to 16 rows on the decode kernel."""
    lib = _lib.lib()
    assert lib.kiln_w4a16_workspace_bytes(17, 4096, 2560) == 4 * 17 * 4096 * 4
    assert lib.kiln_w4a16_workspace_bytes(64, 4096, 2560) == 4 * 64 * 4096 * 4
    assert lib.kiln_w4a16_workspace_bytes(16, 4096, 2560) == 0
    assert lib.kiln_w4a16_workspace_bytes(64, 512, 2560) == 0
    m, k, n = 24, 2560, 4096
    case = _case(m, k, n, seed=5, device=cuda_device)
    out = kiln_b200.marlin_w4a16_gemm(case["a_t"], case["b_t"], case["s_t"], 128)
    torch.cuda.synchronize()
    assert lib.kiln_w4a16_check_device_status(None, None) == 0
    assert rel_err(from_torch_bf16(out), C.gemm_fp64(case["a"], case["q"], case["s"], 128)) <= REL_TOL


def test_small_batch_kernel_with_extreme_nibbles_and_scales(cuda_device):
    """All-0 and all-15 nibbles (weights -8 and +7) with the largest and smallest scales of the synthetic distribution."""
    m, k, n = 40, 512, 512
    a, q, s = oracle.synth_inputs(m, k, n, seed=11, groupsize=128)
    q[:, ::2] = 0
    q[:, 1::2] = 15
    s[0, :] = s.max()
    s[1, :] = s.min()
    packed, sp = kiln_b200.pack.repack(q, s, 128)
    case = dict(a=a, q=q, s=s, a_t=to_torch_bf16(a, cuda_device), b_t=torch.from_numpy(packed).to(cuda_device),
                s_t=torch.from_numpy(sp.view(np.int16).copy()).view(torch.float16).to(cuda_device))
    out = _run(case, True, m, n, cuda_device)
    assert rel_err(from_torch_bf16(out), C.gemm_fp64(a, q, s, 128)) <= REL_TOL


def test_swiglu_is_fused_from_17_rows_under_the_built_in_rule(cuda_device):
    """gate+up with SwiGLU at 24 rows: no hook, no workspace, one launch of the small-batch kernel (the decode kernel below
    17 rows, which fuses it too)."""
    import ctypes

    from tests.test_gpu_epilogue import _gate_up_case, _silu

    lib = _lib.lib()
    ep = _lib.Epilogue()
    ep.swiglu = 1
    for m in (16, 24):
        assert int(lib.kiln_w4a16_workspace_bytes_ex(m, 18432, 2560, ctypes.byref(ep))) == 0
        a, fused, g, u = _gate_up_case(m, 2560, 9216, seed=40 + m, dev=cuda_device)
        before = lib.kiln_w4a16_launch_count()
        out = kiln_b200.swiglu_gate_up(to_torch_bf16(a, cuda_device), fused)
        torch.cuda.synchronize()
        assert lib.kiln_w4a16_check_device_status(None, None) == 0
        assert lib.kiln_w4a16_launch_count() - before == 1
        assert rel_err(from_torch_bf16(out), (_silu(g) * u).astype(np.float32)) <= REL_TOL
