"""The bit tricks that turn packed nibbles into floating-point numbers, restated with numpy (no GPU).

Decode kernel (fp16, kiln_b200/csrc/decode_w4a16.cu): `(x & 0x000F000F) | 0x64006400` is the fp16 pair {1024 + nib}, whose unit in
the last place is 1; `(x & 0x00F000F0) | 0x54005400` is {64 + nib} for the nibbles that sit at bits 4..7, because the unit in the
last place of 64.0 is 1/16.  The constants -1032 and -72 of the offset MMA remove 1024 + 8 and 64 + 8.
tcgen05 kernels (bf16, prefill_w4a16_umma.cu and smallm_w4a16_tmem.cu): `(x & 0x000F000F) | 0x43004300` is the bf16 pair {128 + nib};
subtracting 136 gives nib - 8 exactly, and one multiplication by the bf16 group scale rounds once."""
import numpy as np


def _f16(bits):
    return np.array(bits, dtype=np.uint16).view(np.float16).astype(np.float64)


def _bf16(bits):
    return (np.array(bits, dtype=np.uint32) << 16).view(np.float32).astype(np.float64)


def test_fp16_magic_numbers_of_the_decode_kernel():
    nib = np.arange(16, dtype=np.uint32)
    lo = (nib & 0x000F) | 0x6400                  # a nibble at bits 0..3 of a 16-bit half
    hi = ((nib << 4) & 0x00F0) | 0x5400           # a nibble at bits 4..7
    assert np.array_equal(_f16(lo), 1024.0 + nib)
    assert np.array_equal(_f16(hi), 64.0 + nib)
    assert _f16([0xE408])[0] == -1032.0 and _f16([0xD480])[0] == -72.0
    # (1024 + nib) - 1032 and (64 + nib) - 72 are the signed weights -8..7
    assert np.array_equal(_f16(lo) + _f16([0xE408])[0], nib.astype(np.float64) - 8.0)
    assert np.array_equal(_f16(hi) + _f16([0xD480])[0], nib.astype(np.float64) - 8.0)


def test_bf16_magic_numbers_of_the_tcgen05_kernels():
    nib = np.arange(16, dtype=np.uint32)
    v = (nib & 0x000F) | 0x4300
    assert np.array_equal(_bf16(v), 128.0 + nib)
    assert _bf16([0x4308])[0] == 136.0
    assert np.array_equal(_bf16(v) - 136.0, nib.astype(np.float64) - 8.0)
    # bf16 has 7 mantissa bits: a nibble at bits 4..7 would reach the exponent, which is why these kernels shift
    assert not np.array_equal(_bf16(((nib << 4) & 0x00F0) | 0x4300), 128.0 + 16.0 * nib)
    # -136 * scale is not a bf16 number in general, so subtract and multiply cannot be one fused multiply-add
    s = _bf16([0x3C23])[0]                        # some scale with a full mantissa
    prod = np.float32(-136.0 * s)
    assert (prod.view(np.uint32) & 0xFFFF) != 0
