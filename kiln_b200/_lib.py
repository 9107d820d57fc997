"""ctypes loader for libkiln_w4a16.so (the C ABI declared in include/kiln_w4a16.h).

There is no fallback: if the shared library is missing or does not load, importing
the product raises.  Build it with `python -m kiln_b200.build`.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# KILN_W4A16_LIB may point at another build of the same library (same C ABI)
LIB_PATH = os.environ.get("KILN_W4A16_LIB") or os.path.join(_HERE, "libkiln_w4a16.so")

OK = 0
ERR_PROB_SHAPE = 1
ERR_KERN_SHAPE = 2
ERR_ALIGNMENT = 3
ERR_WORKSPACE = 4
ERR_CUDA = 5
ERR_TIMEOUT = 6
ERR_ARG = 7
ERR_STATIC_SCRATCH = 8

STATUS_NAMES = {
    0: "OK", 1: "ERR_PROB_SHAPE", 2: "ERR_KERN_SHAPE", 3: "ERR_ALIGNMENT", 4: "ERR_WORKSPACE",
    5: "ERR_CUDA", 6: "ERR_TIMEOUT", 7: "ERR_ARG", 8: "ERR_STATIC_SCRATCH",
}

_vp, _i, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t


class Epilogue(ctypes.Structure):
    """kiln_w4a16_epilogue_t."""

    _fields_ = [("swiglu", _i), ("lora_a", _vp), ("lora_b", _vp), ("lora_rank", _i), ("lora_scale", ctypes.c_float)]


class Problem(ctypes.Structure):
    """kiln_w4a16_problem_t."""

    _fields_ = [("A", _vp), ("B", _vp), ("C", _vp), ("s", _vp), ("m", _i), ("n", _i), ("k", _i), ("groupsize", _i)]


# name -> (restype, argtypes); must list every symbol include/kiln_w4a16.h declares
SIGNATURES = {
    "kiln_marlin_w4a16_gemm": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp, _i, _i, _vp, _i, _i, _i, _i]),
    "kiln_w4a16_gemm_bf16": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _sz, _vp]),
    "kiln_w4a16_workspace_bytes_ex": (_sz, [_i, _i, _i, ctypes.POINTER(Epilogue)]),
    "kiln_w4a16_gemm_bf16_ex": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, ctypes.POINTER(Epilogue), _vp, _sz, _vp]),
    "kiln_w4a16_gemm_bf16_grouped": (_i, [ctypes.POINTER(Problem), _i, _vp, _sz, _vp]),
    "kiln_w4a16_gemm_bf16_noalloc": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "kiln_w4a16_noalloc_plan": (None, [_i, _i, _i, ctypes.POINTER(ctypes.c_int)]),
    "kiln_w4a16_gemm_bf16_allgather": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _vp, _i, _i, _i, _vp]),
    "kiln_w4a16_gemm_bf16_allgather_multicast": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _vp, _i, _i, _vp]),
    "kiln_w4a16_workspace_bytes": (_sz, [_i, _i, _i]),
    "kiln_w4a16_shape_is_supported": (_i, [_i, _i]),
    "kiln_w4a16_build_weight_perm": (None, [_vp]),
    "kiln_w4a16_build_scale_perm": (None, [_vp]),
    "kiln_w4a16_build_scale_perm_single": (None, [_vp]),
    "kiln_w4a16_quantize_and_pack_host": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp, _i]),
    "kiln_w4a16_quantize_and_pack_device": (_i, [_vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "kiln_w4a16_repack_host": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, _i]),
    "kiln_w4a16_repack_device": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, _vp]),
    "kiln_w4a16_repack_gptq_host": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _i]),
    "kiln_w4a16_repack_gptq_device": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "kiln_w4a16_last_cuda_error": (_i, []),
    "kiln_w4a16_check_device_status": (_i, [_vp, _vp]),
    "kiln_w4a16_set_decode_override": (None, [_i, _i, _i]),
    "kiln_w4a16_decode_plan": (None, [_i, _i, _i, ctypes.POINTER(ctypes.c_int)]),
    "kiln_w4a16_set_prefill_override": (None, [_i, _i, _i, _i]),
    "kiln_w4a16_set_small_batch_kernel": (None, [_i]),
    "kiln_w4a16_set_wait_limit_ns": (None, [ctypes.c_ulonglong]),
    "kiln_w4a16_test_drop_activation_load": (None, [_i]),
    "kiln_w4a16_prefill_plan": (None, [_i, _i, _i, ctypes.POINTER(ctypes.c_int)]),
    "kiln_w4a16_set_prefill_min_m": (None, [_i]),
    "kiln_w4a16_version": (_i, []),
    "kiln_w4a16_launch_count": (ctypes.c_ulonglong, []),
}

_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: the CUDA library has not been built "
                "(run `python -m kiln_b200.build`). There is no CPU or PyTorch fallback."
            )
        cdll = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(cdll, name)  # AttributeError if the .so lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = cdll
    return _lib
