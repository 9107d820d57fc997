"""The C-ABI library loads and exports every symbol include/kiln_w4a16.h declares; argument
validation that needs no GPU behaves like the reference's (no compute is launched here)."""
import ctypes
import os
import re

import pytest
import torch

import kiln_b200
from kiln_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "kiln_w4a16.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(kiln_(?:marlin_)?w4a16_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    names = _declared()
    assert len(names) >= 15
    cdll = ctypes.CDLL(_lib.LIB_PATH)
    for name in names:
        assert hasattr(cdll, name), f"{name} declared in the header but not exported"
    assert sorted(_lib.SIGNATURES) == names


def test_version_and_shape_rule():
    lib = _lib.lib()
    assert lib.kiln_w4a16_version() >= 100
    assert lib.kiln_w4a16_shape_is_supported(2560, 9216) == 1
    assert lib.kiln_w4a16_shape_is_supported(2560, 9216 + 64) == 0
    assert lib.kiln_w4a16_shape_is_supported(2500, 256) == 0
    assert kiln_b200.shape_is_supported(4096, 2560) and not kiln_b200.shape_is_supported(4096, 100)


def test_status_codes_before_any_launch():
    lib = _lib.lib()
    p = ctypes.c_void_p(0x1000)
    # reference: k % 128, n % 256, groupsize -> ERR_PROB_SHAPE (marlin_kernel.cu:770-771, lib.rs:112-130)
    assert lib.kiln_w4a16_gemm_bf16(p, p, p, p, 1, 256, 100, 128, None, 0, None) == _lib.ERR_PROB_SHAPE
    assert lib.kiln_w4a16_gemm_bf16(p, p, p, p, 1, 200, 128, 128, None, 0, None) == _lib.ERR_PROB_SHAPE
    assert lib.kiln_w4a16_gemm_bf16(p, p, p, p, 1, 256, 128, 64, None, 0, None) == _lib.ERR_PROB_SHAPE
    # zero-size problem is a no-op success (marlin_kernel.cu:772-773)
    assert lib.kiln_w4a16_gemm_bf16(p, p, p, p, 0, 256, 128, 128, None, 0, None) == _lib.OK
    assert lib.kiln_w4a16_gemm_bf16(None, p, p, p, 1, 256, 128, 128, None, 0, None) == _lib.ERR_ARG
    assert lib.kiln_w4a16_gemm_bf16(ctypes.c_void_p(0x1004), p, p, p, 1, 256, 128, 128, None, 0, None) == _lib.ERR_ALIGNMENT
    # legacy symbol: tile overrides follow the reference's rejections
    assert lib.kiln_marlin_w4a16_gemm(p, p, p, p, 1, 256, 192, None, 128, 0, None, 64, 256, -1, 16) == _lib.ERR_PROB_SHAPE
    assert lib.kiln_marlin_w4a16_gemm(p, p, p, p, 1, 256, 192, None, 128, 0, None, 128, 128, -1, 16) == _lib.ERR_PROB_SHAPE
    assert lib.kiln_marlin_w4a16_gemm(p, p, p, p, 1, 256, 128, None, 128, 0, None, 32, 32, -1, 16) == _lib.ERR_KERN_SHAPE
    assert lib.kiln_marlin_w4a16_gemm(p, p, p, p, 0, 256, 128, None, 128, 0, None, -1, -1, -1, 16) == _lib.OK
    # fused all-gather entry: argument checks happen before any launch
    peers = (ctypes.c_void_p * 2)(0x1000, 0x2000)
    pp = ctypes.cast(peers, ctypes.c_void_p)
    assert lib.kiln_w4a16_gemm_bf16_allgather(p, p, p, 128, 256, 128, 128, pp, 9, 512, 0, None) == _lib.ERR_ARG
    assert lib.kiln_w4a16_gemm_bf16_allgather(p, p, p, 128, 256, 128, 128, pp, 2, 256, 256, None) == _lib.ERR_ARG
    assert lib.kiln_w4a16_gemm_bf16_allgather(p, p, p, 128, 200, 128, 128, pp, 2, 512, 0, None) == _lib.ERR_PROB_SHAPE
    assert lib.kiln_w4a16_gemm_bf16_allgather(p, p, p, 0, 256, 128, 128, pp, 2, 512, 0, None) == _lib.OK


def test_wrapper_messages_match_reference():
    a = torch.zeros(1, 128, dtype=torch.bfloat16)
    b = torch.zeros(8, 512, dtype=torch.int32)
    s = torch.zeros(1, 256, dtype=torch.float16)
    with pytest.raises(kiln_b200.KilnMarlinError, match="kiln-marlin-gemm: a must be on CUDA"):
        kiln_b200.marlin_w4a16_gemm(a, b, s, 128)


def test_product_does_not_import_the_oracle():
    for dirpath, _, files in os.walk(os.path.join(ROOT, "kiln_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.replace("fp32 oracle", ""), f"{f} mentions the oracle"
