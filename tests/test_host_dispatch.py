"""Host-side kernel selection and workspace rules, through the C ABI, without a GPU (148 SMs are assumed when no device is
present).  The workspace a caller must lend follows from which kernel a problem goes to and how that kernel splits K:
  * up to 16 rows, and projections of at most 1024 columns up to 256 rows: decode kernel, no workspace;
  * from 17 rows on wider projections: a tcgen05 kernel, `splits * m * n * 4` bytes when the planner splits K;
  * epilogue options add the fp32 [m, rank] projection of a LoRA delta and, when an option is not fused, a bf16 copy of
    the GEMM result for the second pass."""
import ctypes

from kiln_b200 import _lib


def _align256(x):
    return (x + 255) // 256 * 256


def _plan(lib, m, n, k):
    out = (ctypes.c_int * 4)()
    lib.kiln_w4a16_prefill_plan(m, n, k, out)
    return list(out)  # columns per tile, K splits, M-tiles per CTA, stream-K


def test_plain_gemm_workspace_follows_the_kernel_choice():
    lib = _lib.lib()
    assert lib.kiln_w4a16_workspace_bytes(16, 4096, 2560) == 0          # decode kernel
    assert lib.kiln_w4a16_workspace_bytes(256, 512, 2560) == 0          # narrow projection: decode kernel up to 256 rows
    for m in (17, 64, 128):                                             # small-batch tcgen05 kernel, the planner's K splits
        bn, splits, mt, sk = _plan(lib, m, 4096, 2560)
        assert (bn, mt, sk) == (128, 1, 0) and splits > 1
        assert lib.kiln_w4a16_workspace_bytes(m, 4096, 2560) == splits * m * 4096 * 4
    assert _plan(lib, 64, 18432, 2560)[:2] == [128, 1]
    assert lib.kiln_w4a16_workspace_bytes(64, 18432, 2560) == 0         # one tile per SM already: K is not split
    assert lib.kiln_w4a16_workspace_bytes(0, 4096, 2560) == 0


def test_epilogue_options_workspace():
    lib = _lib.lib()
    ep = _lib.Epilogue()
    ep.swiglu = 1
    # gate+up: K not split, SwiGLU fused in the epilogue from 17 rows (small-batch kernel) and below (decode kernel)
    for m in (1, 16, 24, 128, 2048):
        assert lib.kiln_w4a16_workspace_bytes_ex(m, 18432, 2560, ctypes.byref(ep)) == 0
    # a split tiling cannot fuse it: bf16 copy of the GEMM result + the split's fp32 slabs
    m, n, k = 48, 4096, 2560
    splits = _plan(lib, m, n, k)[1]
    assert splits > 1
    assert lib.kiln_w4a16_workspace_bytes_ex(m, n, k, ctypes.byref(ep)) == _align256(m * n * 2) + _align256(splits * m * n * 4)
    # LoRA: the projection t = scale * x * A^T always; on the tcgen05 kernels also the buffer of the composed pass (the
    # query does not know the group size) and the split's slabs
    ep.swiglu, ep.lora_rank = 0, 64
    assert lib.kiln_w4a16_workspace_bytes_ex(8, n, k, ctypes.byref(ep)) == _align256(8 * 64 * 4)
    m = 64
    splits = _plan(lib, m, n, k)[1]
    assert lib.kiln_w4a16_workspace_bytes_ex(m, n, k, ctypes.byref(ep)) == \
        _align256(m * 64 * 4) + _align256(m * n * 2) + _align256(splits * m * n * 4)


def test_tuning_hooks_change_the_rule_and_restore_it():
    lib = _lib.lib()
    try:
        lib.kiln_w4a16_set_prefill_min_m(1 << 30)                       # decode kernel only
        assert lib.kiln_w4a16_workspace_bytes(64, 4096, 2560) == 0
        lib.kiln_w4a16_set_prefill_min_m(1)                             # tcgen05 kernels from one row
        assert lib.kiln_w4a16_workspace_bytes(4, 4096, 2560) == _plan(lib, 4, 4096, 2560)[1] * 4 * 4096 * 4
    finally:
        lib.kiln_w4a16_set_prefill_min_m(0)
    assert lib.kiln_w4a16_workspace_bytes(4, 4096, 2560) == 0
