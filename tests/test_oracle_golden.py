"""Pins the CPU oracle: against the reference's own numpy quantiser fixture, against an
independent numpy restatement, against the fragment-formula unpacker, and against frozen digests."""
import hashlib
import json
import os

import numpy as np
import pytest

import oracle
from oracle import C

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _digest(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def test_quantiser_matches_reference_numpy_fixture():
    """Fixture made by kiln's scripts/c11_marlin_audit.py:208-241 (see golden/make_quantiser_golden.py).
    That script rounds ties to even, the Rust packer away from zero: exact ties are excluded."""
    z = np.load(os.path.join(GOLD, "quantiser_c11.npz"))
    w, w_dq, scales = z["w"], z["w_dq"], z["scales"]
    _, s_perm, deq, q = C.quantize_and_pack(w, 128)
    s_nat = oracle.np_quantize(w, 128)[1].astype(np.float32)
    assert (s_nat == scales).all()
    ratio = np.abs(w.reshape(-1, 128, w.shape[1]) / scales[:, None, :]).reshape(w.shape)
    ties = np.abs(ratio - np.floor(ratio) - 0.5) == 0
    assert ties.mean() < 1e-3
    assert (deq[~ties] == w_dq[~ties]).all()
    assert q[:, 7].tolist() == [8] * w.shape[0]  # all-zero column -> scale from max_abs = 1
    assert q.min() == 0 and q.max() == 15  # outlier row reaches both clamps


@pytest.mark.parametrize("k,n,gs", [(128, 256, 128), (128, 256, -1), (384, 512, 128), (256, 768, -1)])
def test_c_oracle_equals_numpy_restatement(k, n, gs):
    rng = np.random.default_rng(k * 7 + n)
    w = (rng.standard_normal((k, n)) * 0.1).astype(np.float32)
    p, s, d, q = C.quantize_and_pack(w, gs)
    p2, s2, d2, q2 = oracle.np_quantize_and_pack(w, gs)
    assert (p == p2).all()
    assert (s.view(np.uint16) == s2.view(np.uint16)).all()
    assert (d == d2).all() and (q == q2).all()
    assert (C.unpack_fragment(p, k, n) == q).all()  # consumer-side formula inverts the packer


def test_round_half_away_from_zero_on_exact_ties():
    # scale = 2*max/15 with max = 7.5 -> s = 1.0 exactly; w = +-0.5, +-1.5, 2.5 are exact ties
    k, n = 128, 256
    w = np.zeros((k, n), np.float32)
    w[0, :] = 7.5
    w[1, 0], w[2, 0], w[3, 0], w[4, 0], w[5, 0] = 0.5, -0.5, 1.5, -1.5, 2.5
    _, _, d, q = C.quantize_and_pack(w, 128)
    assert q[1:6, 0].tolist() == [9, 7, 10, 6, 11]
    assert (oracle.np_quantize(w, 128)[0] == q).all()
    assert q[0, 0] == 15 and d[0, 0] == 7.0  # round(7.5)=8 -> 16 clamps to 15


def test_permutation_tables():
    assert (C.weight_perm() == oracle.np_weight_perm()).all()
    assert sorted(C.weight_perm().tolist()) == list(range(1024))
    assert C.scale_perm().tolist() == [i + 8 * j for i in range(8) for j in range(8)]
    assert C.scale_perm_single().tolist() == [2 * i + j for i in range(4) for j in [0, 1, 8, 9, 16, 17, 24, 25]]


def test_packed_format_is_separable_along_n():
    a, q, s = oracle.synth_inputs(1, 256, 512, seed=9)
    full, sfull = C.pack_nibbles(q), C.permute_scales(s, 128)
    for n0, n1 in [(0, 64), (64, 320), (256, 512)]:
        assert (C.pack_nibbles(q[:, n0:n1]) == full[:, 2 * n0:2 * n1]).all()
        assert (C.permute_scales(s[:, n0:n1].copy(), 128).view(np.uint16) == sfull[:, n0:n1].view(np.uint16)).all()


def test_frozen_digests():
    from tests.golden.make_pack_hashes import CASES, synth_weight

    with open(os.path.join(GOLD, "pack_hashes.json")) as f:
        gold = json.load(f)
    for k, n, gs, seed in CASES:
        if k * n > 2560 * 4096:
            continue  # the scalar oracle needs seconds per large matrix; digests of those are checked via the native packer
        p, s, d, q = C.quantize_and_pack(synth_weight(k, n, seed), gs)
        g = gold[f"{k}x{n}_g{gs}_s{seed}"]
        assert _digest(p) == g["packed"] and _digest(s.view(np.uint16)) == g["scales"]
        assert _digest(d) == g["dequant"] and _digest(q) == g["q"]


def test_gemm_oracles_agree():
    a, q, s = oracle.synth_inputs(5, 384, 256, seed=11)
    o = C.gemm_fp64(a, q, s, 128)
    assert np.abs(o - oracle.np_gemm_fp64(a, q, s, 128)).max() <= 1e-6 * np.abs(o).max()
    ob = oracle.bf16_bits_to_f32(C.gemm_cpu_reference(a, q, s, 128))
    assert np.abs(ob - o).max() / np.abs(o).max() < 1e-2
    # per-column mode
    a, q, s = oracle.synth_inputs(3, 256, 256, seed=12, groupsize=-1)
    o = C.gemm_fp64(a, q, s, -1)
    assert np.abs(o - oracle.np_gemm_fp64(a, q, s, -1)).max() <= 1e-6 * np.abs(o).max()


def test_kiln_lcg_restated():
    # first outputs of the reference test's LCG (parity.rs:22-31) computed by hand from its recurrence
    v = oracle.kiln_lcg_fill(3, 1, 1.0)
    state = 1
    exp = []
    for _ in range(3):
        state = (state * 6364136223846793005 + 1442695040888963407) & (2**64 - 1)
        exp.append(np.float32(np.float32((state >> 33) & 0x7FFFFFFF) / np.float32(2147483647)) - np.float32(0.5))
    assert v.tolist() == [float(e) for e in exp]
    assert np.abs(v).max() <= 0.5


def test_gptq_layout_matches_the_references_known_answers():
    """The oracle's restatement of kiln's GPTQ layout (quantized.rs:118-145) reproduces the two known-answer tests
    the reference holds for it (quantized.rs:311-372: all nibbles 5, zero-point 8, scale 0.5 -> -1.5 everywhere;
    :374-415: nibbles 0..7 in one word, zero-point 0, scale 1 -> 0..7 by input row, which fixes the nibble order),
    and `np_gptq_pack` is its inverse on both."""
    import json
    import os

    with open(os.path.join(os.path.dirname(__file__), "golden", "gptq_known_answers.json")) as f:
        cases = json.load(f)["cases"]
    for c in cases:
        k, n, g = c["in_features"], c["out_features"], c["group_size"]
        qw = np.array(c["qweight_words_u32"], np.uint32).reshape(c["qweight_shape"]).view(np.int32)
        qz = np.array(c["qzeros_words_u32"], np.uint32).reshape(c["qzeros_shape"]).view(np.int32)
        sc = np.array(c["scales"], np.float16).reshape(c["scales_shape"])
        npad = qz.shape[1] * 8  # the zero-point words cover eight output columns each
        qw_p = np.zeros((k // 8, npad), np.int32)
        qw_p[:, :n] = qw
        sc_p = np.zeros((k // g, npad), np.float16)
        sc_p[:, :n] = sc
        w = oracle.np_gptq_dequant(qw_p, qz, sc_p, g)[:, :n]
        assert w.shape == (k, n)
        if "expected_every_element" in c:
            assert (w == c["expected_every_element"]).all()
        else:
            assert (w[:, 0] == np.array(c["expected_by_input_row"], np.float32)).all()
        # the packer of the same layout is the inverse: nibbles and zero-points in, the same words out
        rows = np.arange(k)
        nib = ((qw_p.view(np.uint32)[rows // 8] >> (4 * (rows % 8)).astype(np.uint32)[:, None]) & 0xF).astype(np.uint8)
        cols = np.arange(npad)
        zer = ((qz.view(np.uint32)[:, cols // 8] >> (4 * (cols % 8)).astype(np.uint32)[None, :]) & 0xF).astype(np.uint8)
        qw2, qz2 = oracle.np_gptq_pack(nib, zer)
        assert (qw2 == qw_p).all() and (qz2 == qz).all()
