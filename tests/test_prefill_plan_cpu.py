"""Invariants of the tcgen05 kernels' tiling rule (`choose_prefill` in kiln_b200/csrc/prefill_w4a16_umma.cu), read through
`kiln_w4a16_prefill_plan` without a GPU (148 SMs assumed): the tile width divides the matrix, a K split leaves every split
at least one 64-deep step, and `kiln_w4a16_workspace_bytes` is exactly what the chosen tiling writes (fp32 slabs of the
whole output per split, or two tile-shaped slabs per CTA for hybrid stream-K)."""
import ctypes

import pytest

from kiln_b200 import _lib

SHAPES = [(2560, 4096), (4096, 2560), (2560, 18432), (9216, 2560), (2560, 8192), (128, 256), (640, 768), (1152, 38400),
          (9216, 9216), (9216, 73728)]


@pytest.mark.parametrize("k,n", SHAPES)
def test_plans_and_workspace_agree(k, n):
    lib = _lib.lib()
    out = (ctypes.c_int * 4)()
    try:
        lib.kiln_w4a16_set_prefill_min_m(1)  # ask the tcgen05 rule at every row count
        for m in (1, 17, 33, 64, 100, 128, 129, 256, 300, 512, 1000, 2048, 8192, 16384):
            lib.kiln_w4a16_prefill_plan(m, n, k, out)
            bn, splits, mt, stream_k = list(out)
            assert bn in (128, 256) and n % bn == 0, (m, list(out))
            assert mt in (1, 2) and stream_k in (0, 1), (m, list(out))
            assert 1 <= splits <= 8 and splits <= k // 64, (m, list(out))
            assert not (stream_k and splits > 1), (m, list(out))
            need = lib.kiln_w4a16_workspace_bytes(m, n, k)
            if stream_k:
                assert need == 2 * 148 * (128 * mt) * bn * 4, (m, list(out), need)
            else:
                assert need == (splits * m * n * 4 if splits > 1 else 0), (m, list(out), need)
    finally:
        lib.kiln_w4a16_set_prefill_min_m(0)
