"""Invariants of the decode kernel's decomposition rule (`choose_config` in kiln_b200/csrc/decode_w4a16.cu), read through
`kiln_w4a16_decode_plan` without a GPU (148 SMs assumed): whatever the rule or its table of measured configurations says
must be launchable - a power-of-two number of 64-column chunks per CTA that divides the matrix, no more warps than the
kernel's launch bounds, a portable cluster that does not exceed the K groups, and the whole grid resident in one wave
(CTAs of a cluster wait for each other, and the next kernel's CTAs move in as this one's drain)."""
import ctypes

import pytest

from kiln_b200 import _lib

SHAPES = [(2560, 4096), (2560, 512), (4096, 2560), (2560, 18432), (9216, 2560), (2560, 8192),  # the benchmark's projections
          (128, 256), (640, 768), (1152, 38400), (49152, 256), (256, 1024)]


@pytest.mark.parametrize("k,n", SHAPES)
def test_every_plan_is_launchable(k, n):
    lib = _lib.lib()
    out = (ctypes.c_int * 4)()
    groups, chunks = k // 128, n // 64
    for m in list(range(1, 17)) + [24, 32]:
        lib.kiln_w4a16_decode_plan(m, n, k, out)
        ck, wk, wn, pass_groups = list(out)
        rows = 8 if (m <= 8 or (n <= 1024 and m <= 32)) else 16      # rows per block of CTAs
        max_warps = 20 if rows == 8 else 16
        assert wn in (1, 2, 4, 8) and chunks % wn == 0, (m, list(out))
        assert 1 <= wk and wk * wn <= max_warps, (m, list(out))
        assert 1 <= ck <= 8 and ck <= groups, (m, list(out))
        per_cta = -(-groups // ck)
        assert 1 <= pass_groups <= per_cta, (m, list(out))
        ctas = (chunks // wn) * -(-m // rows) * ck
        resident = 148 * max(1, max_warps // (wk * wn))
        assert ctas <= resident, (m, list(out), ctas, resident)


def test_override_is_reported_and_restored():
    lib = _lib.lib()
    out = (ctypes.c_int * 4)()
    lib.kiln_w4a16_decode_plan(1, 4096, 2560, out)
    rule = list(out)
    try:
        lib.kiln_w4a16_set_decode_override(2, 3, 2)
        lib.kiln_w4a16_decode_plan(1, 4096, 2560, out)
        assert list(out)[:3] == [2, 3, 2]
    finally:
        lib.kiln_w4a16_set_decode_override(0, 0, 0)
    lib.kiln_w4a16_decode_plan(1, 4096, 2560, out)
    assert list(out) == rule
