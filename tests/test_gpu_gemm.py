"""GPU parity of the W4A16 GEMM, called through the C ABI, against the CPU oracle.
Tolerance: max|out - oracle| / max|oracle| <= 1e-2 against the fp64-accumulated oracle."""
import ctypes

import numpy as np
import pytest
import torch

import kiln_b200
import oracle
from kiln_b200 import _lib
from oracle import C
from tests.util import QWEN_SHAPES, REL_TOL, from_torch_bf16, make_case, rel_err, to_torch_bf16

pytestmark = pytest.mark.gpu


def run(case, **kw):
    return kiln_b200.marlin_w4a16_gemm(case["a_t"], case["b_t"], case["s_t"], case["groupsize"], **kw)


def check(case, out, tol=REL_TOL):
    torch.cuda.synchronize()
    e = rel_err(from_torch_bf16(out), case["ref"])
    assert e <= tol, f"rel err {e} > {tol} for m={case['m']} k={case['k']} n={case['n']}"
    return e


@pytest.mark.parametrize("name", list(QWEN_SHAPES))
@pytest.mark.parametrize("m", [1, 4, 8, 16])
def test_decode_sweep_shapes(cuda_device, name, m):
    k, n = QWEN_SHAPES[name]
    case = make_case(m, k, n, seed=100 + m, device=cuda_device)
    e = check(case, run(case))
    assert e < 5e-3  # bf16 output rounding alone is 2^-9; anything near 1e-2 would be a real defect


@pytest.mark.parametrize("m,k,n", [(1, 128, 256), (16, 128, 256), (1, 2560, 8192), (16, 2560, 1024), (1, 2560, 9216)])
def test_reference_parity_shapes(cuda_device, m, k, n):
    """Shapes of kiln-marlin-gemm/tests/parity.rs:172-198 and marlin_qproj_parity.rs, with the
    reference's own LCG inputs; weights go through quantize_and_pack like there."""
    import oracle
    from oracle import C

    w = oracle.kiln_lcg_fill(k * n, 0xC0FFEE_5EED ^ k ^ (n << 16), 0.5).reshape(k, n) if k * n <= 1 << 20 else (
        np.random.default_rng(k ^ n).uniform(-0.25, 0.25, (k, n)).astype(np.float32))
    acts = oracle.kiln_lcg_fill(m * k, 0xDEAD_BEEF ^ m ^ (k << 24), 0.25).reshape(m, k)
    packed, scales, dequant = kiln_b200.pack.quantize_and_pack(w, k, n, 128)
    a_bits = oracle.f32_to_bf16_bits(acts)
    ref = (oracle.bf16_bits_to_f32(a_bits).astype(np.float64) @ dequant.astype(np.float64)).astype(np.float32)
    out = kiln_b200.marlin_w4a16_gemm(
        to_torch_bf16(a_bits, cuda_device), torch.from_numpy(packed).to(cuda_device),
        torch.from_numpy(scales.view(np.int16).copy()).view(torch.float16).to(cuda_device), 128)
    torch.cuda.synchronize()
    assert out.shape == (m, n) and out.dtype == torch.bfloat16
    assert rel_err(from_torch_bf16(out), ref) <= REL_TOL


@pytest.mark.parametrize("name", ["q", "k", "o", "gate_up", "down", "gdn_in"])
def test_stack_shapes_at_m64(cuda_device, name):
    """Continuous-batch M=64 on the six distinct projection shapes of the 32-layer stack configuration, with whatever
    kernel the built-in rule picks.  fp64 oracle on sampled rows, float32 torch matmul on the whole output."""
    k, n = QWEN_SHAPES[name]
    m = 64
    a, q, s = oracle.synth_inputs(m, k, n, seed=640 + len(name))
    packed, sp = kiln_b200.pack.repack(q, s, 128)
    a_t = to_torch_bf16(a, cuda_device)
    out = kiln_b200.marlin_w4a16_gemm(a_t, torch.from_numpy(packed).to(cuda_device),
                                      torch.from_numpy(sp.view(np.int16).copy()).view(torch.float16).to(cuda_device), 128)
    torch.cuda.synchronize()
    sel = np.array([0, 7, 8, 15, 16, 31, 47, 63])
    ref = C.gemm_fp64(a[sel], q, s, 128)
    assert rel_err(from_torch_bf16(out[torch.from_numpy(sel).to(cuda_device)]), ref) <= REL_TOL
    w = (torch.from_numpy(q.astype(np.float32)).to(cuda_device) - 8.0) * \
        torch.from_numpy(s.astype(np.float32)).to(cuda_device).repeat_interleave(128, dim=0)
    full = a_t.float() @ w
    assert float((out.float() - full).abs().max() / full.abs().max()) <= REL_TOL


@pytest.mark.parametrize("m", [2, 3, 5, 7, 9, 15, 17, 31, 32, 33, 63, 64, 65, 100])
def test_ragged_m(cuda_device, m):
    case = make_case(m, 384, 512, seed=m, device=cuda_device)
    check(case, run(case))


@pytest.mark.parametrize("k", [128, 256, 1152, 1408])
@pytest.mark.parametrize("n", [256, 768])
def test_small_shape_grid(cuda_device, k, n):
    for m in (1, 6, 16, 24):
        case = make_case(m, k, n, seed=k + n + m, device=cuda_device)
        check(case, run(case))


@pytest.mark.parametrize("m,k,n", [(1, 256, 256), (16, 256, 256), (5, 2560, 512)])
def test_per_column_scales(cuda_device, m, k, n):
    """groupsize = -1 (kiln-marlin-gemm/tests/parity.rs:202-215)."""
    case = make_case(m, k, n, seed=77, groupsize=-1, device=cuda_device)
    check(case, run(case))


@pytest.mark.parametrize("cfg", [(1, 1, 1), (1, 4, 1), (2, 3, 2), (4, 2, 4), (8, 1, 1), (8, 2, 2), (4, 5, 1), (2, 1, 4)])
def test_every_decomposition_gives_the_same_answer(cuda_device, cfg):
    """Forces (cluster_k, warps_k, warps_n) through the tuning hook: split-K over warps and over the
    cluster must not change the result beyond fp32 summation order."""
    lib = _lib.lib()
    try:
        for m, k, n in [(1, 1408, 512), (16, 2560, 256), (13, 640, 768)]:
            case = make_case(m, k, n, seed=sum(cfg) + m, device=cuda_device)
            lib.kiln_w4a16_set_decode_override(*cfg)
            check(case, run(case))
    finally:
        lib.kiln_w4a16_set_decode_override(0, 0, 0)


@pytest.mark.parametrize("m,k,n,cfg", [(16, 5120, 256, (1, 2, 1)), (8, 49152 + 128, 256, None), (16, 9216, 512, (1, 1, 2))])
def test_long_k_is_staged_in_passes(cuda_device, m, k, n, cfg):
    """A K range whose activations do not fit the shared-memory stage at once is staged in several passes
    (the reference walks K in tiles of 64 or 128 whatever its length, marlin_kernel.cu:207-279)."""
    lib = _lib.lib()
    plan = (ctypes.c_int * 4)()
    try:
        if cfg:
            lib.kiln_w4a16_set_decode_override(*cfg)
        lib.kiln_w4a16_decode_plan(m, n, k, plan)
        assert plan[3] * plan[0] < k // 128, "this case is meant to need more than one pass"
        case = make_case(m, k, n, seed=k % 1000 + m, device=cuda_device)
        check(case, run(case))
    finally:
        lib.kiln_w4a16_set_decode_override(0, 0, 0)


def test_bit_reproducible_and_in_bounds(cuda_device):
    """Fixed reduction order: two runs agree bit for bit; canaries around the output survive."""
    case = make_case(7, 2560, 4096, seed=5, device=cuda_device)
    m, n = 7, 4096
    buf = torch.full((m + 2, n), 7.0, dtype=torch.bfloat16, device=cuda_device)
    out = buf[1:m + 1]
    run(case, out=out)
    first = out.clone()
    run(case, out=out)
    torch.cuda.synchronize()
    assert torch.equal(first, out)
    assert (buf[0] == 7.0).all() and (buf[m + 1] == 7.0).all()
    check(case, out)


def test_legacy_symbol_and_stream(cuda_device):
    """kiln_marlin_w4a16_gemm with the reference's argument order, on a non-default stream."""
    lib = _lib.lib()
    case = make_case(4, 2560, 512, seed=9, device=cuda_device)
    out = torch.empty((4, 512), dtype=torch.bfloat16, device=cuda_device)
    st = torch.cuda.Stream()
    st.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(st):
        rc = lib.kiln_marlin_w4a16_gemm(case["a_t"].data_ptr(), case["b_t"].data_ptr(), out.data_ptr(),
                                        case["s_t"].data_ptr(), 4, 512, 2560, None, 128, 0, st.cuda_stream,
                                        -1, -1, -1, 16)
    assert rc == 0
    st.synchronize()
    check(case, out)
    assert lib.kiln_w4a16_launch_count() > 0
    assert lib.kiln_w4a16_check_device_status(None, None) == 0


def test_legacy_symbol_never_touches_the_references_small_workspace(cuda_device):
    """An unmodified reference wrapper passes its (n / 128) * 16 int32 lock array (kiln-marlin-gemm/src/lib.rs:174-178).
    At a batch size where the regular entry point would split K into a caller-sized workspace, the legacy symbol must
    leave that small buffer, and what surrounds it, alone."""
    lib = _lib.lib()
    m, k, n = 256, 9216, 2560
    assert lib.kiln_w4a16_workspace_bytes(m, n, k) > (n // 128) * 16 * 4, "the regular entry point would use scratch here"
    case = make_case(8, k, n, seed=77, device=cuda_device)
    a = torch.cat([case["a_t"]] * (m // 8), dim=0).contiguous()
    words = (n // 128) * 16
    buf = torch.full((words + 2048,), 0x5A5A5A5A, dtype=torch.int32, device=cuda_device)
    ws = buf[1024:1024 + words]
    out = torch.empty((m, n), dtype=torch.bfloat16, device=cuda_device)
    rc = lib.kiln_marlin_w4a16_gemm(a.data_ptr(), case["b_t"].data_ptr(), out.data_ptr(), case["s_t"].data_ptr(), m, n, k,
                                    ws.data_ptr(), 128, 0, torch.cuda.current_stream().cuda_stream, -1, -1, -1, 16)
    assert rc == 0
    torch.cuda.synchronize()
    assert (buf == 0x5A5A5A5A).all(), "the legacy entry point wrote into or around the reference-sized workspace"
    assert rel_err(from_torch_bf16(out[:8]), case["ref"]) <= REL_TOL
    assert torch.equal(out[:8], out[m - 8:])


def test_gemm_right_after_a_device_pack_on_the_same_stream(cuda_device):
    """The GEMM kernels read weights before their grid-dependency wait; the device pack entry points end with an
    ordinary launch so that a GEMM enqueued right behind a pack still sees the packed weights."""
    k, n, m = 2560, 4096, 4
    g = torch.Generator(device=cuda_device)
    g.manual_seed(3)
    a_t = torch.randn((m, k), device=cuda_device, generator=g).to(torch.bfloat16)
    for i in range(4):  # a fresh weight each time: the packed tensors of the previous round must not be what is read
        w = (torch.randn((k, n), device=cuda_device, generator=g) * 0.02).to(torch.bfloat16)
        proj = kiln_b200.pack_from_bf16(w)
        out = kiln_b200.matmul_bf16(a_t, proj)  # no synchronisation between the pack and the GEMM
        ref = a_t.float() @ w.float()
        torch.cuda.synchronize()
        assert float((out.float() - ref).abs().max() / ref.abs().max()) < 0.2  # int4 quantisation error, not garbage
        again = kiln_b200.matmul_bf16(a_t, proj)
        torch.cuda.synchronize()
        assert torch.equal(out, again), "the GEMM right behind the pack read something else than the packed weights"


def test_rank3_activation_through_marlin_proj(cuda_device):
    """matmul_bf16 flattens [b, s, k] like kiln-model/src/marlin_proj.rs:285-319."""
    case = make_case(6, 256, 512, seed=21, device=cuda_device)
    proj = kiln_b200.MarlinPackedProj(case["b_t"], case["s_t"], 128, 256, 512)
    y = kiln_b200.matmul_bf16(case["a_t"].reshape(2, 3, 256), proj)
    assert y.shape == (2, 3, 512)
    check(case, y.reshape(6, 512))
    with pytest.raises(kiln_b200.KilnMarlinError):
        kiln_b200.matmul_bf16(case["a_t"].reshape(6, 2, 128), proj)


def test_wrapper_rejections_on_device(cuda_device):
    case = make_case(1, 256, 256, seed=1, device=cuda_device)
    with pytest.raises(kiln_b200.KilnMarlinError, match="groupsize must be -1 or 128"):
        kiln_b200.marlin_w4a16_gemm(case["a_t"], case["b_t"], case["s_t"], 64)
    with pytest.raises(kiln_b200.KilnMarlinError, match="a must be bf16"):
        kiln_b200.marlin_w4a16_gemm(case["a_t"].float(), case["b_t"], case["s_t"], 128)
    with pytest.raises(kiln_b200.KilnMarlinError, match="does not match expected"):
        kiln_b200.marlin_w4a16_gemm(case["a_t"], case["b_t"][:, :256], case["s_t"], 128)
    with pytest.raises(kiln_b200.KilnMarlinError, match="scales rows"):
        kiln_b200.marlin_w4a16_gemm(case["a_t"], case["b_t"], torch.cat([case["s_t"], case["s_t"]]), 128)


def test_cuda_graph_replay(cuda_device):
    """The call is stream-ordered and capturable (kiln-model/src/cuda_graph.rs:10-17 replays decode as a graph)."""
    case = make_case(1, 2560, 4096, seed=31, device=cuda_device)
    out = torch.zeros((1, 4096), dtype=torch.bfloat16, device=cuda_device)
    run(case, out=out)  # warm-up: attributes set outside capture
    torch.cuda.synchronize()
    out.zero_()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(3):
            run(case, out=out)
    out.zero_()
    g.replay()
    check(case, out)
