"""Device packer against the oracle (bit-exact) and round trips at full size."""
import numpy as np
import pytest
import torch

import kiln_b200
from kiln_b200 import _lib
from oracle import C
import oracle

pytestmark = pytest.mark.gpu


def _dev_pack(w_t, gs, want_dequant=True):
    k, n = w_t.shape
    g = k if gs == -1 else gs
    dev = w_t.device
    p = torch.empty((k // 16, 2 * n), dtype=torch.int32, device=dev)
    s = torch.empty((k // g, n), dtype=torch.float16, device=dev)
    d = torch.empty((k, n), dtype=torch.float32, device=dev) if want_dequant else None
    rc = _lib.lib().kiln_w4a16_quantize_and_pack_device(
        w_t.data_ptr(), 1 if w_t.dtype == torch.bfloat16 else 0, k, n, gs, p.data_ptr(), s.data_ptr(),
        d.data_ptr() if d is not None else None, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    return p.cpu().numpy(), s.cpu().view(torch.int16).numpy().view(np.uint16), None if d is None else d.cpu().numpy()


@pytest.mark.parametrize("k,n,gs", [(128, 256, 128), (256, 512, -1), (2560, 512, 128), (2560, 4096, 128), (4096, 2560, -1)])
def test_device_pack_f32_bit_exact(cuda_device, k, n, gs):
    rng = np.random.default_rng(k + n)
    w = (rng.standard_normal((k, n)) * 0.05).astype(np.float32)
    w[:, 2] = 0
    w[1, :] *= 64
    p, s, d = _dev_pack(torch.from_numpy(w).to(cuda_device), gs)
    p2, s2, d2 = kiln_b200.pack.quantize_and_pack(w, k, n, gs)  # native host packer == oracle (CPU suite)
    assert (p == p2).all() and (s == s2.view(np.uint16)).all() and (d == d2).all()
    if k * n <= 2560 * 512:
        po, so, do, _ = C.quantize_and_pack(w, gs)
        assert (p == po).all() and (s == so.view(np.uint16)).all() and (d == do).all()


def test_device_pack_unaligned_weight_takes_the_two_kernel_path(cuda_device):
    """A weight that does not start on a 16-byte boundary cannot use the one-pass kernel's vector loads."""
    k, n = 256, 256
    rng = np.random.default_rng(5)
    w = (rng.standard_normal((k, n)) * 0.05).astype(np.float32)
    flat = torch.zeros(k * n + 1, dtype=torch.float32, device=cuda_device)
    flat[1:] = torch.from_numpy(w).to(cuda_device).reshape(-1)
    p, s, d = _dev_pack(flat[1:].view(k, n), 128)
    p2, s2, d2 = kiln_b200.pack.quantize_and_pack(w, k, n, 128)
    assert (p == p2).all() and (s == s2.view(np.uint16)).all() and (d == d2).all()


def test_device_pack_bf16_full_size(cuda_device):
    """One gate projection (2560 x 9216, bf16, grouped) through the one-pass kernel against the host packer."""
    k, n = 2560, 9216
    w = (torch.randn(k, n, generator=torch.Generator().manual_seed(11)) * 0.02).to(torch.bfloat16)
    w[5, :] *= 40
    w[:, 7] = 0
    proj = kiln_b200.pack_from_bf16(w.to(cuda_device), 128)
    torch.cuda.synchronize()
    p2, s2, _ = kiln_b200.pack.quantize_and_pack(w.float().numpy(), k, n, 128)
    assert (proj.b_packed.cpu().numpy() == p2).all()
    assert (proj.scales.cpu().view(torch.int16).numpy().view(np.uint16) == s2.view(np.uint16)).all()


def test_device_pack_bf16_and_proj_helper(cuda_device):
    k, n = 2560, 1024
    w = (torch.randn(k, n, generator=torch.Generator().manual_seed(3)) * 0.05).to(torch.bfloat16)
    proj = kiln_b200.pack_from_bf16(w.to(cuda_device), 128)
    torch.cuda.synchronize()
    assert proj is not None and (proj.k, proj.n, proj.groupsize) == (k, n, 128)
    p2, s2, _ = kiln_b200.pack.quantize_and_pack(w.float().numpy(), k, n, 128)
    assert (proj.b_packed.cpu().numpy() == p2).all()
    assert (proj.scales.cpu().view(torch.int16).numpy().view(np.uint16) == s2.view(np.uint16)).all()
    assert kiln_b200.pack_from_bf16(w[:, :100].contiguous().to(cuda_device)) is None  # unsupported shape
    assert kiln_b200.pack_from_bf16(w) is None  # not on CUDA


def test_device_repack_prequantised_full_size_roundtrip(cuda_device):
    """Full benchmark size (gate+up 2560x18432): pack on device, unpack with the consumer-side formula."""
    k, n = 2560, 18432
    a, q, s = oracle.synth_inputs(1, k, n, seed=8)
    qd = torch.from_numpy(q).to(cuda_device)
    sd = torch.from_numpy(s.view(np.int16).copy()).to(cuda_device)
    p = torch.empty((k // 16, 2 * n), dtype=torch.int32, device=cuda_device)
    sp = torch.empty((k // 128, n), dtype=torch.int16, device=cuda_device)
    rc = _lib.lib().kiln_w4a16_repack_device(qd.data_ptr(), sd.data_ptr(), k, n, 128, p.data_ptr(), sp.data_ptr(),
                                             torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    pn = p.cpu().numpy()
    assert (C.unpack_fragment(pn, k, n) == q).all()
    ph, sph = kiln_b200.pack.repack(q, s, 128)
    assert (pn == ph).all() and (sp.cpu().numpy().view(np.uint16) == sph.view(np.uint16)).all()


def test_gptq_repack_on_device(cuda_device):
    import oracle

    rng = np.random.default_rng(11)
    k, n, g = 2560, 1024, 128
    q = rng.integers(0, 16, (k, n), dtype=np.uint8)
    s = (0.01 * np.abs(rng.standard_normal((k // g, n))) + 1e-3).astype(np.float16)
    zeros = np.full((k // g, n), 8, np.uint8)
    qw, qz = oracle.np_gptq_pack(q, zeros)
    proj = kiln_b200.pack_from_gptq(torch.from_numpy(qw).to(cuda_device), torch.from_numpy(qz).to(cuda_device),
                                    torch.from_numpy(s.view(np.int16).copy()).view(torch.float16).to(cuda_device), g)
    assert proj is not None
    assert (proj.b_packed.cpu().numpy() == oracle.C.pack_nibbles(q)).all()
    assert (proj.scales.cpu().view(torch.int16).numpy().view(np.uint16) == oracle.C.permute_scales(s, g).view(np.uint16)).all()
    # the packed projection multiplies like kiln's dequantised GPTQ weight
    a = rng.standard_normal((4, k)).astype(np.float32)
    a_t = torch.from_numpy(a).to(cuda_device).to(torch.bfloat16)
    out = kiln_b200.matmul_bf16(a_t, proj).float().cpu().numpy()
    w = oracle.np_gptq_dequant(qw, qz, s, g).astype(np.float64)
    ref = a_t.float().cpu().numpy().astype(np.float64) @ w
    assert np.abs(out - ref).max() / np.abs(ref).max() <= 1e-2
    # asymmetric: refused (None), nothing raised
    zeros[3, 5] = 0
    qw2, qz2 = oracle.np_gptq_pack(q, zeros)
    assert kiln_b200.pack_from_gptq(torch.from_numpy(qw2).to(cuda_device), torch.from_numpy(qz2).to(cuda_device),
                                    torch.from_numpy(s.view(np.int16).copy()).view(torch.float16).to(cuda_device), g) is None


def test_packed_cache_round_trip(cuda_device, tmp_path):
    cache = kiln_b200.PackedCache(str(tmp_path))
    w = (torch.randn((512, 768), device=cuda_device) * 0.02).to(torch.bfloat16)
    first = cache.get_or_pack("layers.0.mlp.gate", w)
    files = list(tmp_path.iterdir())
    assert len(files) == 1
    second = cache.get_or_pack("layers.0.mlp.gate", w)  # from disk
    assert torch.equal(first.b_packed, second.b_packed) and torch.equal(first.scales, second.scales)
    direct = kiln_b200.pack_from_bf16(w)
    assert torch.equal(direct.b_packed, second.b_packed)
    # a different weight under the same name is repacked, not served from the stale entry
    w2 = w.clone()
    w2[3, 5] += 0.5
    third = cache.get_or_pack("layers.0.mlp.gate", w2)
    assert torch.equal(third.b_packed, kiln_b200.pack_from_bf16(w2).b_packed)
    assert len(list(tmp_path.iterdir())) == 1
    # two rows swapped: same multiset of words, different weight -> repacked as well
    w3 = w2.clone()
    w3[[1, 2]] = w3[[2, 1]]
    fourth = cache.get_or_pack("layers.0.mlp.gate", w3)
    assert torch.equal(fourth.b_packed, kiln_b200.pack_from_bf16(w3).b_packed)
    assert not torch.equal(fourth.b_packed, third.b_packed)
    assert cache.get_or_pack("odd", torch.zeros((100, 256), device=cuda_device, dtype=torch.bfloat16)) is None
