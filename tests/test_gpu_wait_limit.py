"""The give-up path of the bounded device-side waits, exercised without faulting, trapping or hanging anything.

The reference's inter-CTA barrier spins without a limit (kiln-marlin-gemm/csrc/marlin_kernel.cu:162-171).  Here every
wait of the tcgen05 kernel polls against a time limit; when it runs out the kernel records a code, stops its other waits,
drains its copies, frees its tensor memory and returns.  The test shortens the limit to 2 ms and uses the test hook that
announces one activation tile to its barrier without ever copying it, so that exactly one wait (the MMA issuer's wait for
that stage, and with it the waits that depend on it) runs out: the status call must report the timeout, and the next launch on the same
stream must be clean and correct."""
import ctypes

import numpy as np
import pytest
import torch

import kiln_b200
import oracle
from kiln_b200 import _lib
from oracle import C
from tests.util import REL_TOL, from_torch_bf16, rel_err, to_torch_bf16

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_is_reported_and_the_next_launch_is_clean(cuda_device):
    lib = _lib.lib()
    m, k, n = 256, 512, 512  # eight K-steps, too short for split-K: one kernel per call
    a, q, s = oracle.synth_inputs(m, k, n, seed=4242)
    packed, sp = kiln_b200.pack.repack(q, s, 128)
    a_t = to_torch_bf16(a, cuda_device)
    b_t = torch.from_numpy(packed).to(cuda_device)
    s_t = torch.from_numpy(sp.view(np.int16).copy()).view(torch.float16).to(cuda_device)
    out = torch.zeros((m, n), dtype=torch.bfloat16, device=cuda_device)
    assert lib.kiln_w4a16_check_device_status(None, None) == 0
    lib.kiln_w4a16_set_prefill_min_m(1)
    try:
        lib.kiln_w4a16_set_wait_limit_ns(2_000_000)
        lib.kiln_w4a16_test_drop_activation_load(1)
        kiln_b200.marlin_w4a16_gemm(a_t, b_t, s_t, 128, out=out)
        torch.cuda.synchronize()  # the launch returns by itself: no wait outlasts its limit
    finally:
        lib.kiln_w4a16_test_drop_activation_load(-1)
        lib.kiln_w4a16_set_wait_limit_ns(0)
    detail = ctypes.c_uint32(0)
    assert lib.kiln_w4a16_check_device_status(None, ctypes.byref(detail)) == _lib.ERR_TIMEOUT
    # the first wait to run out records its code: the MMA issuer's wait for the stage to fill (0x3..) or a wait that
    # started earlier and depends on it, the epilogue's wait for the accumulator (0x5..)
    assert detail.value & 0xF00 in (0x300, 0x500), hex(detail.value)
    assert lib.kiln_w4a16_check_device_status(None, None) == 0  # read and cleared
    try:
        kiln_b200.marlin_w4a16_gemm(a_t, b_t, s_t, 128, out=out)
        torch.cuda.synchronize()
    finally:
        lib.kiln_w4a16_set_prefill_min_m(0)
    assert lib.kiln_w4a16_check_device_status(None, None) == 0
    assert rel_err(from_torch_bf16(out), C.gemm_fp64(a, q, s, 128)) <= REL_TOL
