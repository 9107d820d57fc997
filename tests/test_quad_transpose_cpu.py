"""The quad exchange of the small-batch tcgen05 kernel (kiln_b200/csrc/smallm_w4a16_tmem.cu), restated with numpy and checked
against the oracle's packer on the CPU.

The kernel needs every K of ONE weight column in a lane (a tensor-memory lane is a row of the MMA's weight operand), while a
lane of the packed layout holds two K pairs of eight columns.  Per 16-row K tile each lane reads the 8-byte half of its 16-byte
piece that holds its warp's 32 columns, the four lanes of a quad transpose their 16-bit items (even-K byte, odd-K byte of a
column) with two `shfl.xor` and six `prmt`, and four shifts + eight `lop3` then yield the eight K pairs of the lane's column.
This test runs exactly that sequence (same selectors, same shifts) on a block packed by the oracle and compares every lane's
result with the nibbles it must hold: column 16 * (2 * hf + qd / 2) + 8 * (qd % 2) + c of the chunk, K pairs 0..7 in order."""
import numpy as np
import pytest

from oracle import C


def _prmt(a, b, sel):
    """PTX prmt.b32 in its default mode: result byte i = byte (sel >> 4i) & 7 of the 64-bit value {b, a}."""
    v = (np.asarray(b, dtype=np.uint64) << np.uint64(32)) | np.asarray(a, dtype=np.uint64)
    out = np.zeros_like(v)
    sel = np.asarray(sel, dtype=np.uint64) + np.zeros_like(v)
    for i in range(4):
        idx = (sel >> np.uint64(4 * i)) & np.uint64(7)
        out |= ((v >> (idx * np.uint64(8))) & np.uint64(0xFF)) << np.uint64(8 * i)
    return out.astype(np.uint32)


def _shfl_xor(v, mask):
    return v[np.arange(32) ^ mask]


@pytest.mark.parametrize("hf", [0, 1])
def test_quad_exchange_gives_each_lane_one_column(hf):
    rng = np.random.default_rng(7 + hf)
    q = rng.integers(0, 16, size=(16, 64), dtype=np.uint8)          # one K tile x one 64-column chunk of nibbles
    block = np.asarray(C.pack_nibbles(q)).view(np.uint32).reshape(32, 4)  # 512 bytes: lane L holds words 4L .. 4L+3
    lane = np.arange(32)
    c, qd = lane >> 2, lane & 3
    x, y = block[:, 2 * hf], block[:, 2 * hf + 1]                  # the warp's half of every 16-byte piece

    # the selectors of the kernel
    b0, b1 = (qd & 1) != 0, (qd & 2) != 0
    sel_k = np.where(b0, 0x7531, 0x6420)
    sel_s = np.where(b0, 0x6420, 0x7531)
    sel_u = np.where(b0, 0x1054, 0x5410)
    sel_v = np.where(b0, 0x3276, 0x7632)
    sel_k2 = np.where(b1, sel_v, sel_u)
    sel_s2 = np.where(b1, sel_u, sel_v)
    sel_ra = np.where(b1, 0x7564, 0x3120)
    sel_rb = np.where(b1, 0x3120, 0x7564)

    keep1 = _prmt(x, y, sel_k)
    recv1 = _shfl_xor(_prmt(x, y, sel_s), 1)
    keep2 = _prmt(keep1, recv1, sel_k2)
    recv2 = _shfl_xor(_prmt(keep1, recv1, sel_s2), 2)
    ra, rb = _prmt(keep2, recv2, sel_ra), _prmt(keep2, recv2, sel_rb)

    # (word >> shift) & 0x000F000F: even-K nibble in bits 0..3, odd-K nibble in bits 16..19 of K pair `kp`
    order = [(ra, 0, 0), (ra, 4, 4), (ra, 8, 1), (ra, 12, 5), (rb, 0, 2), (rb, 4, 6), (rb, 8, 3), (rb, 12, 7)]
    got = np.zeros((32, 16), dtype=np.uint8)                        # [lane][k]
    for word, shift, kp in order:
        v = (word >> np.uint32(shift)) & np.uint32(0x000F000F)
        got[:, 2 * kp] = v & 0xF
        got[:, 2 * kp + 1] = (v >> 16) & 0xF

    col = 16 * (2 * hf + (qd >> 1)) + 8 * (qd & 1) + c
    assert sorted(col.tolist()) == list(range(32 * hf, 32 * hf + 32))  # the warp's lanes cover its 32 columns once each
    want = q[:, col].T                                              # [lane][k]
    assert np.array_equal(got, want)


def test_scale_position_of_a_lane():
    """The scale of natural column `col` of a chunk sits at position 8 * (col % 8) + col / 8 of the chunk's scale order
    (kiln-marlin-gemm/src/lib.rs:333-341); for the lane's column above that is 8c + 4hf + qd."""
    s = np.arange(64, dtype=np.float32).reshape(1, 64) + 1.0       # scale value = natural column + 1
    perm = np.asarray(C.permute_scales(s.astype(np.float16), 128)).astype(np.float32).reshape(64)
    for hf in (0, 1):
        for lane in range(32):
            c, qd = lane >> 2, lane & 3
            col = 16 * (2 * hf + (qd >> 1)) + 8 * (qd & 1) + c
            assert perm[8 * c + 4 * hf + qd] == col + 1.0
