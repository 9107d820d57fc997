"""GPU parity of the fused epilogue options and the grouped launch, through the C ABI, against the fp64 oracle.

SwiGLU: silu(gate) * up of the gate+up projection (kiln-model/src/forward.rs:2769-2839); LoRA: base + x @ A^T @ B^T * scale
(kiln-model/src/lora_loader.rs:213-233); grouped: sibling projections in one launch.  Tolerance: max|out - ref| / max|ref|
<= 1e-2, as for the plain GEMM."""
import numpy as np
import pytest
import torch

import kiln_b200
import oracle
from kiln_b200 import _lib
from oracle import C
from tests.util import REL_TOL, from_torch_bf16, rel_err, to_torch_bf16

pytestmark = pytest.mark.gpu


def _proj(q, s, gs, dev):
    packed, sp = kiln_b200.pack.repack(q, s, gs)
    k, n = q.shape
    return kiln_b200.MarlinPackedProj(torch.from_numpy(packed).to(dev),
                                      torch.from_numpy(sp.view(np.int16).copy()).view(torch.float16).to(dev), gs, k, n)


def _gate_up_case(m, k, n_half, seed, dev):
    """Separate gate and up projections, fused by the product's own interleave, and the fp64 reference."""
    a, qg, sg = oracle.synth_inputs(m, k, n_half, seed=seed)
    _, qu, su = oracle.synth_inputs(1, k, n_half, seed=seed + 1)
    fused = kiln_b200.interleave_gate_up(_proj(qg, sg, 128, dev), _proj(qu, su, 128, dev))
    g = C.gemm_fp64(a, qg, sg, 128).astype(np.float64)
    u = C.gemm_fp64(a, qu, su, 128).astype(np.float64)
    return a, fused, g, u


def _silu(x):
    return x / (1.0 + np.exp(-x))


@pytest.mark.parametrize("m,k,n_half", [(1, 2560, 9216), (16, 2560, 9216), (4, 512, 256), (8, 1152, 640), (40, 640, 512)])
def test_swiglu_fused_into_the_gate_up_gemm(cuda_device, m, k, n_half):
    a, fused, g, u = _gate_up_case(m, k, n_half, seed=m + k, dev=cuda_device)
    out = kiln_b200.swiglu_gate_up(to_torch_bf16(a, cuda_device), fused)
    torch.cuda.synchronize()
    assert out.shape == (m, n_half)
    assert rel_err(from_torch_bf16(out), (_silu(g) * u).astype(np.float32)) <= REL_TOL


@pytest.mark.parametrize("m,k,n_half,fused_expected", [(64, 2560, 9216, True), (24, 2560, 9216, True), (128, 2560, 9216, True),
                                                        (48, 2560, 2048, False), (384, 512, 2048, False), (300, 2560, 9216, True),
                                                        (600, 1152, 4096, True), (2048, 640, 1024, True)])
def test_swiglu_at_the_batch_sizes_of_the_tcgen05_kernel(cuda_device, m, k, n_half, fused_expected):
    """Batch sizes of the tcgen05 kernels: the small-batch kernel without a K split (its gate and up warps meet through
    shared memory) and the general kernel's tilings that write whole tiles from one accumulator per M-tile compute
    silu(gate) * up in the epilogue (no workspace needed); the others compose the GEMM with a second pass.  Rows outside
    [0, m) stay untouched."""
    import ctypes

    lib = _lib.lib()
    lib.kiln_w4a16_set_prefill_min_m(1)
    try:
        ep = _lib.Epilogue()
        ep.swiglu = 1
        need = int(lib.kiln_w4a16_workspace_bytes_ex(m, 2 * n_half, k, ctypes.byref(ep)))
        assert (need == 0) == fused_expected, f"workspace {need} bytes"
        a, fused, g, u = _gate_up_case(m, k, n_half, seed=m + k, dev=cuda_device)
        buf = torch.full((m + 2, n_half), 3.0, dtype=torch.bfloat16, device=cuda_device)
        out = kiln_b200.swiglu_gate_up(to_torch_bf16(a, cuda_device), fused, out=buf[1:m + 1])
        torch.cuda.synchronize()
        assert lib.kiln_w4a16_check_device_status(None, None) == 0
        assert rel_err(from_torch_bf16(out), (_silu(g) * u).astype(np.float32)) <= REL_TOL
        assert (buf[0] == 3.0).all() and (buf[m + 1] == 3.0).all()
    finally:
        lib.kiln_w4a16_set_prefill_min_m(0)


@pytest.mark.parametrize("cfg", [(1, 2, 1), (2, 3, 2), (3, 2, 1), (4, 2, 4), (5, 1, 2), (8, 1, 1), (8, 2, 2)])
def test_swiglu_with_every_cluster_split(cuda_device, cfg):
    """The gate pair and its up pair must meet in one cluster rank whatever the decomposition."""
    lib = _lib.lib()
    try:
        for m in (1, 7, 16):
            a, fused, g, u = _gate_up_case(m, 1408, 512, seed=sum(cfg) + m, dev=cuda_device)
            lib.kiln_w4a16_set_decode_override(*cfg)
            out = kiln_b200.swiglu_gate_up(to_torch_bf16(a, cuda_device), fused)
            torch.cuda.synchronize()
            assert rel_err(from_torch_bf16(out), (_silu(g) * u).astype(np.float32)) <= REL_TOL
    finally:
        lib.kiln_w4a16_set_decode_override(0, 0, 0)


def _lora(rng, r, k, n):
    la = oracle.f32_to_bf16_bits((rng.standard_normal((r, k)) * 0.05).astype(np.float32))
    lb = oracle.f32_to_bf16_bits((rng.standard_normal((n, r)) * 0.05).astype(np.float32))
    return la, lb


@pytest.mark.parametrize("r", [8, 20, 64, 128])
@pytest.mark.parametrize("m,k,n", [(1, 2560, 4096), (16, 2560, 4096), (5, 640, 768), (512, 640, 1024),
                                   (40, 2560, 4096), (100, 640, 2560), (128, 4096, 2560)])  # (the last three: small-batch kernel)
def test_lora_delta_in_the_epilogue(cuda_device, m, k, n, r):
    a, q, s = oracle.synth_inputs(m, k, n, seed=r + m)
    rng = np.random.default_rng(r * 7 + m)
    la, lb = _lora(rng, r, k, n)
    scale = 2.0
    x = oracle.bf16_bits_to_f32(a).astype(np.float64)
    delta = (x @ oracle.bf16_bits_to_f32(la).astype(np.float64).T) @ oracle.bf16_bits_to_f32(lb).astype(np.float64).T * scale
    base = C.gemm_fp64(a, q, s, 128).astype(np.float64)
    assert np.abs(delta).max() > 0.05 * np.abs(base).max(), "the delta must matter for this test to mean anything"
    out = kiln_b200.matmul_bf16_lora(to_torch_bf16(a, cuda_device), _proj(q, s, 128, cuda_device),
                                     to_torch_bf16(la, cuda_device), to_torch_bf16(lb, cuda_device), scale)
    torch.cuda.synchronize()
    assert rel_err(from_torch_bf16(out), (base + delta).astype(np.float32)) <= REL_TOL


@pytest.mark.parametrize("m,k,nh", [(3, 640, 512), (300, 640, 512), (300, 1152, 4096), (64, 2560, 9216), (48, 640, 2048)])
def test_lora_and_swiglu_together(cuda_device, m, k, nh):
    """Separate LoRA adapters on gate and up are one adapter of twice the rank on the fused matrix: A = [A_g; A_u],
    B = [[B_g, 0]; [0, B_u]] with its rows in the fused column order.  m = 3: decode kernel; m = 300: tcgen05 kernel with
    the delta as extra K-steps, SwiGLU composed (narrow tiles) or in the epilogue (pairs of 256-column tiles); m = 64 and
    48: small-batch kernel, the delta as an extra stage and SwiGLU in its epilogue (or composed when K is split)."""
    r = 8
    a, fused, g, u = _gate_up_case(m, k, nh, seed=99, dev=cuda_device)
    rng = np.random.default_rng(5)
    ag, bg = _lora(rng, r, k, nh)
    au, bu = _lora(rng, r, k, nh)
    f = lambda bits: oracle.bf16_bits_to_f32(bits).astype(np.float64)
    x = f(a)
    g2 = g + (x @ f(ag).T) @ f(bg).T * 1.5
    u2 = u + (x @ f(au).T) @ f(bu).T * 1.5
    t = lambda bits: to_torch_bf16(bits, cuda_device)
    la = torch.cat([t(ag), t(au)], dim=0)
    zero = torch.zeros((nh, r), dtype=torch.bfloat16, device=cuda_device)
    lb = kiln_b200.interleave_columns_32(torch.cat([t(bg), zero], dim=1), torch.cat([zero, t(bu)], dim=1))
    out = kiln_b200.swiglu_gate_up(t(a), fused, la, lb, 1.5)
    torch.cuda.synchronize()
    assert rel_err(from_torch_bf16(out), (_silu(g2) * u2).astype(np.float32)) <= REL_TOL


@pytest.mark.parametrize("m", [1, 8, 16])
def test_grouped_qkv_in_one_launch(cuda_device, m):
    """q, k, v of an attention layer (2560 -> 4096, 512, 512) on the same activations, one launch."""
    lib = _lib.lib()
    k = 2560
    a, qq, sq = oracle.synth_inputs(m, k, 4096, seed=300 + m)
    _, qk, sk = oracle.synth_inputs(1, k, 512, seed=301 + m)
    _, qv, sv = oracle.synth_inputs(1, k, 512, seed=302 + m)
    projs = [_proj(qq, sq, 128, cuda_device), _proj(qk, sk, 128, cuda_device), _proj(qv, sv, 128, cuda_device)]
    a_t = to_torch_bf16(a, cuda_device)
    c0 = lib.kiln_w4a16_launch_count()
    outs = kiln_b200.grouped_matmul_bf16([a_t, a_t, a_t], projs)
    torch.cuda.synchronize()
    assert lib.kiln_w4a16_launch_count() - c0 == 1, "three sibling projections must be one launch at a decode batch size"
    for o, (q_, s_) in zip(outs, [(qq, sq), (qk, sk), (qv, sv)]):
        assert rel_err(from_torch_bf16(o), C.gemm_fp64(a, q_, s_, 128)) <= REL_TOL


def test_grouped_problems_may_differ_in_everything(cuda_device):
    """Different activations, K, N and row counts within one batch class; and a mixed list falls back to one launch each."""
    shapes = [(3, 640, 256), (8, 1152, 768), (1, 2560, 512), (5, 128, 1024)]
    xs, projs, refs = [], [], []
    for i, (m, k, n) in enumerate(shapes):
        a, q, s = oracle.synth_inputs(m, k, n, seed=500 + i)
        xs.append(to_torch_bf16(a, cuda_device))
        projs.append(_proj(q, s, 128, cuda_device))
        refs.append(C.gemm_fp64(a, q, s, 128))
    lib = _lib.lib()
    c0 = lib.kiln_w4a16_launch_count()
    outs = kiln_b200.grouped_matmul_bf16(xs, projs)
    torch.cuda.synchronize()
    assert lib.kiln_w4a16_launch_count() - c0 == 1
    for o, r in zip(outs, refs):
        assert rel_err(from_torch_bf16(o), r) <= REL_TOL
    # one problem with more than eight rows: two batch classes, so one launch per problem, same results
    a, q, s = oracle.synth_inputs(12, 640, 256, seed=600)
    outs = kiln_b200.grouped_matmul_bf16(xs[:2] + [to_torch_bf16(a, cuda_device)], projs[:2] + [_proj(q, s, 128, cuda_device)])
    torch.cuda.synchronize()
    assert rel_err(from_torch_bf16(outs[2]), C.gemm_fp64(a, q, s, 128)) <= REL_TOL
    assert rel_err(from_torch_bf16(outs[0]), refs[0]) <= REL_TOL
