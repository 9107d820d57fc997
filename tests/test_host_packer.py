"""Native host packer (C ABI) against the oracle: bit-exact, including digests of full-size matrices."""
import hashlib
import json
import os

import numpy as np
import pytest

import oracle
from oracle import C
from kiln_b200 import _lib, pack

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _digest(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def test_perm_tables_match_oracle():
    assert pack.build_weight_perm() == C.weight_perm().tolist()
    assert pack.build_scale_perm() == C.scale_perm().tolist()
    assert pack.build_scale_perm_single() == C.scale_perm_single().tolist()
    assert pack.MAX_Q == 15 and pack.Q_OFFSET == 8


@pytest.mark.parametrize("k,n,gs", [(128, 256, 128), (128, 256, -1), (256, 512, 128), (640, 768, 128), (512, 256, -1)])
@pytest.mark.parametrize("threads", [1, 0])
def test_quantize_and_pack_bit_exact(k, n, gs, threads):
    rng = np.random.default_rng(k + n)
    w = (rng.standard_normal((k, n)) * 0.2).astype(np.float32)
    w[:, 1] = 0
    w[3, :] *= 50
    p, s, d = pack.quantize_and_pack(w, k, n, gs, num_threads=threads)
    p2, s2, d2, _ = C.quantize_and_pack(w, gs)
    assert (p == p2).all() and (s.view(np.uint16) == s2.view(np.uint16)).all() and (d == d2).all()


def test_full_size_digests():
    from tests.golden.make_pack_hashes import CASES, synth_weight

    with open(os.path.join(GOLD, "pack_hashes.json")) as f:
        gold = json.load(f)
    for k, n, gs, seed in CASES:
        p, s, d = pack.quantize_and_pack(synth_weight(k, n, seed), k, n, gs)
        g = gold[f"{k}x{n}_g{gs}_s{seed}"]
        assert _digest(p) == g["packed"], (k, n, gs)
        assert _digest(s.view(np.uint16)) == g["scales"] and _digest(d) == g["dequant"]


def test_reference_lcg_inputs():
    # the reference parity test's own weight generator and seeds (parity.rs:33-43, 55)
    k, n = 128, 256
    w = oracle.kiln_lcg_fill(k * n, 0xC0FFEE_5EED ^ k ^ (n << 16), 0.5).reshape(k, n)
    p, s, d = pack.quantize_and_pack(w, k, n, 128)
    p2, s2, d2, _ = C.quantize_and_pack(w, 128)
    assert (p == p2).all() and (s.view(np.uint16) == s2.view(np.uint16)).all() and (d == d2).all()


def test_repack_prequantised():
    a, q, s = oracle.synth_inputs(1, 2560, 512, seed=3)
    p, sp = pack.repack(q, s, 128)
    assert (p == C.pack_nibbles(q)).all()
    assert (sp.view(np.uint16) == C.permute_scales(s, 128).view(np.uint16)).all()
    assert (C.unpack_fragment(p, 2560, 512) == q).all()


def test_rejects_what_the_reference_asserts():
    w = np.zeros((100, 256), np.float32)
    with pytest.raises(AssertionError):
        pack.quantize_and_pack(w, 100, 256, 128)  # k % 128
    with pytest.raises(AssertionError):
        pack.quantize_and_pack(np.zeros((128, 200), np.float32), 128, 200, 128)  # n % 256
    with pytest.raises(AssertionError):
        pack.quantize_and_pack(np.zeros((256, 256), np.float32), 256, 256, 96)  # k % g
    lib = _lib.lib()
    out = np.zeros(16, np.int32)
    assert lib.kiln_w4a16_quantize_and_pack_host(None, 128, 256, 128, out.ctypes.data, out.ctypes.data, None, 1) == _lib.ERR_ARG
    assert lib.kiln_w4a16_quantize_and_pack_host(out.ctypes.data, 120, 256, 128, out.ctypes.data, out.ctypes.data, None, 1) == _lib.ERR_PROB_SHAPE


def test_concat_projections_equals_packing_the_concatenated_weight():
    import torch

    import kiln_b200

    k = 256
    ws = [np.random.default_rng(i).standard_normal((k, n)).astype(np.float32) * 0.05 for i, n in enumerate((512, 128, 128))]
    parts = []
    for w in ws:
        n = w.shape[1]
        # pack each projection on its own (n % 64 == 0 suffices for the format; pad the call to the 256 rule)
        pad = (-n) % 256
        wp = np.concatenate([w, np.zeros((k, pad), np.float32)], 1) if pad else w
        p, s, _ = pack.quantize_and_pack(wp, k, n + pad, 128)
        parts.append(kiln_b200.MarlinPackedProj(torch.from_numpy(p[:, :2 * n].copy()),
                                                torch.from_numpy(s[:, :n].copy().view(np.int16)).view(torch.float16), 128, k, n))
    fused = kiln_b200.concat_projections(parts)
    pf, sf, _ = pack.quantize_and_pack(np.concatenate(ws, 1), k, 768, 128)
    assert fused.n == 768 and (fused.b_packed.numpy() == pf).all()
    assert (fused.scales.view(torch.int16).numpy().view(np.uint16) == sf.view(np.uint16)).all()
    with pytest.raises(kiln_b200.KilnMarlinError):
        kiln_b200.concat_projections(parts[:2])  # 640 columns: not a multiple of 256


def test_gptq_repack_is_exact_for_symmetric_checkpoints_and_refused_otherwise():
    """GPTQ tensors in kiln's layout (quantized.rs:6-14) -> the packed format: same words as packing the nibbles directly,
    and the packed weight dequantises to exactly kiln's GPTQ dequantisation (quantized.rs:118-145)."""
    rng = np.random.default_rng(7)
    k, n, g = 256, 512, 128
    q = rng.integers(0, 16, (k, n), dtype=np.uint8)
    s = (0.01 * np.abs(rng.standard_normal((k // g, n))) + 1e-3).astype(np.float16)
    zeros = np.full((k // g, n), 8, np.uint8)
    qw, qz = oracle.np_gptq_pack(q, zeros)
    packed, sp = pack.repack_gptq(qw, qz, s, g)
    ref_p, ref_s = pack.repack(q, s, g)
    assert (packed == ref_p).all() and (sp.view(np.uint16) == ref_s.view(np.uint16)).all()
    assert (packed == oracle.C.pack_nibbles(q)).all()
    # the format's value (nibble - 8) * scale against kiln's GPTQ formula (nibble - zero) * scale
    want = oracle.np_gptq_dequant(qw, qz, s, g)
    got = (q.astype(np.int32) - 8).astype(np.float32) * s.astype(np.float32)[np.arange(k) // g]
    assert (want == got).all()
    # per-column mode: one scale row, one zero row
    s1 = s[:1]
    qw1, qz1 = oracle.np_gptq_pack(q, zeros[:1])
    p1, sp1 = pack.repack_gptq(qw1, qz1, s1, -1)
    r1, rs1 = pack.repack(q, s1, -1)
    assert (p1 == r1).all() and (sp1.view(np.uint16) == rs1.view(np.uint16)).all()
    # an asymmetric checkpoint is refused, with the count
    zeros[1, 37] = 7
    zeros[0, 500] = 9
    qw, qz = oracle.np_gptq_pack(q, zeros)
    with pytest.raises(ValueError, match="2 zero-points"):
        pack.repack_gptq(qw, qz, s, g)


@pytest.mark.parametrize("gs", [128, -1])
def test_interleave_gate_up_is_the_packed_interleaved_matrix(gs):
    """Fusing packed gate and up projections by shuffling words gives bit for bit what packing the matrix with its
    columns interleaved in runs of 32 gives."""
    import torch

    import kiln_b200

    k, n = 256, 256
    rng = np.random.default_rng(1)
    qg, qu = rng.integers(0, 16, (k, n), dtype=np.uint8), rng.integers(0, 16, (k, n), dtype=np.uint8)
    ng = k // 128 if gs == 128 else 1
    sg, su = rng.random((ng, n)).astype(np.float16), rng.random((ng, n)).astype(np.float16)

    def proj(q, s):
        return kiln_b200.MarlinPackedProj(torch.from_numpy(C.pack_nibbles(q)),
                                          torch.from_numpy(C.permute_scales(s, gs).view(np.int16).copy()).view(torch.float16), gs, k, n)

    f = kiln_b200.interleave_gate_up(proj(qg, sg), proj(qu, su))
    qi = np.stack([qg.reshape(k, n // 32, 32), qu.reshape(k, n // 32, 32)], axis=2).reshape(k, 2 * n)
    si = np.stack([sg.reshape(ng, n // 32, 32), su.reshape(ng, n // 32, 32)], axis=2).reshape(ng, 2 * n)
    assert (f.b_packed.numpy() == C.pack_nibbles(qi)).all()
    assert (f.scales.view(torch.int16).numpy().view(np.uint16) == C.permute_scales(si, gs).view(np.uint16)).all()
    assert f.n == 2 * n and f.k == k
