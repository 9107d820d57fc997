"""Pins the packed format against the reference's OWN CUDA kernel (compiled unmodified into
oracle/_ref): weights packed here, multiplied by that kernel, must reproduce the oracle GEMM.
The reference kernel is fp16-in/fp16-out with a zeroed int32 lock workspace
(kiln-marlin-gemm/src/lib.rs:169-178)."""
import ctypes
import os

import numpy as np
import pytest
import torch

import kiln_b200
import oracle
from tests.util import make_case, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref_lib():
    if not os.path.exists(oracle.REF_KERNEL_PATH):
        pytest.skip("oracle/_ref/libkiln_marlin_ref.so not built (kiln sources absent at build time)")
    lib = ctypes.CDLL(oracle.REF_KERNEL_PATH)
    vp, i = ctypes.c_void_p, ctypes.c_int
    lib.kiln_marlin_w4a16_gemm.restype = i
    lib.kiln_marlin_w4a16_gemm.argtypes = [vp, vp, vp, vp, i, i, i, vp, i, i, vp, i, i, i, i]
    return lib


def ref_gemm(lib, a_bf16, b, s, groupsize):
    m, k = a_bf16.shape
    n = s.shape[1]
    a16 = a_bf16.to(torch.float16).contiguous()
    c16 = torch.zeros((m, n), dtype=torch.float16, device=a16.device)
    ws = torch.zeros((n // 128) * 16, dtype=torch.int32, device=a16.device)
    rc = lib.kiln_marlin_w4a16_gemm(a16.data_ptr(), b.data_ptr(), c16.data_ptr(), s.data_ptr(), m, n, k,
                                    ws.data_ptr(), groupsize, 0, torch.cuda.current_stream().cuda_stream,
                                    -1, -1, -1, 16)
    assert rc == 0
    torch.cuda.synchronize()
    return c16


@pytest.mark.parametrize("m,k,n,gs", [(1, 128, 256, 128), (16, 2560, 4096, 128), (1, 9216, 2560, 128),
                                      (4, 2560, 9216, 128), (16, 256, 256, -1), (64, 2560, 1024, 128)])
def test_reference_kernel_reads_our_packed_format(cuda_device, ref_lib, m, k, n, gs):
    case = make_case(m, k, n, seed=m + k, groupsize=gs, device=cuda_device)
    # (1) the oracle's packing and (2) the native packer's packing are the same bytes (CPU suite);
    # here the reference kernel consumes them
    out = ref_gemm(ref_lib, case["a_t"], case["b_t"], case["s_t"], gs)
    e = rel_err(out.float().cpu().numpy(), case["ref"])
    assert e < 2e-2, e  # the reference's own bar (tests/parity.rs:150-157); fp16 partial sums
    # and our kernel agrees with the reference kernel on the same bytes
    ours = kiln_b200.marlin_w4a16_gemm(case["a_t"], case["b_t"], case["s_t"], gs)
    torch.cuda.synchronize()
    assert rel_err(ours.float().cpu().numpy(), out.float().cpu().numpy()) < 2e-2
