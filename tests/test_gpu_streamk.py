"""Hybrid stream-K tiling of the tcgen05 kernel, forced through the tuning hook: same answer as the built-in rule
(<= 1e-2 against the fp64 oracle), for tile counts below, at and above the number of SMs and for ragged M."""
import numpy as np
import pytest
import torch

import kiln_b200
from kiln_b200 import _lib
from tests.util import REL_TOL, from_torch_bf16, make_case, rel_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,k,n,cfg", [
    (64, 2560, 4096, (128, 1, 1, 1)),      # 32 tiles: every tile shared by several CTAs
    (300, 1024, 2560, (256, 1, 2, 1)),     # ragged M, pairs of M-tiles, 20 tiles
    (1024, 640, 9728, (256, 1, 2, 1)),     # 152 tiles on 148 SMs: one whole wave + 4 tiles in shares
    (1024, 9216, 2560, (256, 1, 2, 1)),    # the down projection: 40 tiles of 144 K-steps
    (128, 36864, 256, (256, 1, 1, 1)),     # one tile, 576 K-steps: the share floor keeps the slab count in bounds
])
def test_forced_stream_k_matches_oracle(cuda_device, m, k, n, cfg):
    lib = _lib.lib()
    case = make_case(m, k, n, seed=700 + m, device=cuda_device)
    lib.kiln_w4a16_set_prefill_min_m(1)
    try:
        ref = kiln_b200.marlin_w4a16_gemm(case["a_t"], case["b_t"], case["s_t"], 128).clone()
        lib.kiln_w4a16_set_prefill_override(*cfg)
        for _ in range(2):
            out = kiln_b200.marlin_w4a16_gemm(case["a_t"], case["b_t"], case["s_t"], 128)
        torch.cuda.synchronize()
    finally:
        lib.kiln_w4a16_set_prefill_override(0, 0, 0, 0)
        lib.kiln_w4a16_set_prefill_min_m(0)
    assert lib.kiln_w4a16_check_device_status(None, None) == _lib.OK
    assert rel_err(from_torch_bf16(out), case["ref"]) <= REL_TOL
    # against the rule's tiling: same math, different fp32 summation order
    d = float((out.float() - ref.float()).abs().max() / ref.float().abs().max())
    assert d <= 1e-2
