"""Mirror of `kiln_marlin_gemm::pack` (kiln-marlin-gemm/src/lib.rs:284-529) over the native packer."""
from __future__ import annotations

import numpy as np

from . import _lib

MAX_Q = 15  # lib.rs:288
Q_OFFSET = 8  # lib.rs:289


def _ptr(a: np.ndarray):
    return a.ctypes.data


def build_weight_perm() -> list:
    """lib.rs:296-327 -> 1024 indices."""
    out = np.zeros(1024, np.int32)
    _lib.lib().kiln_w4a16_build_weight_perm(_ptr(out))
    return out.tolist()


def build_scale_perm() -> list:
    """lib.rs:333-341 -> 64 indices."""
    out = np.zeros(64, np.int32)
    _lib.lib().kiln_w4a16_build_scale_perm(_ptr(out))
    return out.tolist()


def build_scale_perm_single() -> list:
    """lib.rs:348-357 -> 32 indices."""
    out = np.zeros(32, np.int32)
    _lib.lib().kiln_w4a16_build_scale_perm_single(_ptr(out))
    return out.tolist()


def quantize_and_pack(weight, k: int, n: int, groupsize: int, num_threads: int = 0):
    """lib.rs:370-491.  weight: f32 row-major [k, n] (flat or 2-D, numpy).

    Returns (b_packed int32 [k/16, 2n], scales float16 [k/g, n], dequant float32 [k, n]).
    Like the reference it asserts on shapes it does not support.
    """
    w = np.ascontiguousarray(weight, dtype=np.float32).reshape(-1)
    assert w.size == k * n, "weight.len() must equal k * n"
    assert k % 128 == 0, "k must be %128 == 0"
    assert n % 256 == 0, "n must be %256 == 0"
    g = k if groupsize == -1 else int(groupsize)
    assert g > 0 and k % g == 0, f"k={k} must be divisible by groupsize={g}"
    packed = np.empty((k // 16, 2 * n), np.int32)
    scales = np.empty((k // g, n), np.uint16)
    dequant = np.empty((k, n), np.float32)
    rc = _lib.lib().kiln_w4a16_quantize_and_pack_host(
        _ptr(w), k, n, int(groupsize), _ptr(packed), _ptr(scales), _ptr(dequant), int(num_threads)
    )
    if rc != 0:
        raise AssertionError(f"kiln_w4a16_quantize_and_pack_host failed: {_lib.STATUS_NAMES.get(rc, rc)}")
    return packed, scales.view(np.float16), dequant


def repack(q, scales_f16, groupsize: int, num_threads: int = 0):
    """Steps 3-5 of lib.rs:429-488 for already-quantised weights.

    q: uint8 [k, n] with values 0..15; scales_f16: float16 [k/g, n] in natural column order.
    Returns (b_packed int32 [k/16, 2n], scales float16 [k/g, n] in Marlin order).
    """
    q = np.ascontiguousarray(q, np.uint8)
    k, n = q.shape
    s = np.ascontiguousarray(scales_f16).view(np.uint16)
    g = k if groupsize == -1 else int(groupsize)
    if s.shape != (k // g, n):
        raise ValueError(f"scales shape {s.shape} != {(k // g, n)}")
    packed = np.empty((k // 16, 2 * n), np.int32)
    sp = np.empty_like(s)
    rc = _lib.lib().kiln_w4a16_repack_host(_ptr(q), _ptr(s), k, n, int(groupsize), _ptr(packed), _ptr(sp), int(num_threads))
    if rc != 0:
        raise ValueError(f"kiln_w4a16_repack_host failed: {_lib.STATUS_NAMES.get(rc, rc)}")
    return packed, sp.view(np.float16)


def repack_gptq(qweight, qzeros, scales_f16, groupsize: int, num_threads: int = 0):
    """GPTQ checkpoint tensors (kiln-model/src/quantized.rs:6-14) -> (b_packed, scales) without dequantising.

    qweight int32 [k/8, n], qzeros int32 [k/g, n/8], scales float16 [k/g, n].  Exact for symmetric checkpoints
    (every zero-point 8); raises ValueError for any other (the caller then takes kiln's dequantise-and-requantise route).
    """
    qw = np.ascontiguousarray(qweight, np.int32)
    qz = np.ascontiguousarray(qzeros, np.int32)
    k, n = qw.shape[0] * 8, qw.shape[1]
    s = np.ascontiguousarray(scales_f16).view(np.uint16)
    g = k if groupsize == -1 else int(groupsize)
    if s.shape != (k // g, n) or qz.shape != (k // g, n // 8):
        raise ValueError(f"scales {s.shape} / qzeros {qz.shape} do not match k={k}, n={n}, groupsize={groupsize}")
    packed = np.empty((k // 16, 2 * n), np.int32)
    sp = np.empty_like(s)
    bad = np.zeros(1, np.uint32)
    rc = _lib.lib().kiln_w4a16_repack_gptq_host(_ptr(qw), _ptr(qz), _ptr(s), k, n, int(groupsize), _ptr(packed), _ptr(sp),
                                                _ptr(bad), int(num_threads))
    if rc != 0:
        why = f": {int(bad[0])} zero-points are not 8 (asymmetric checkpoint)" if bad[0] else ""
        raise ValueError(f"kiln_w4a16_repack_gptq_host failed: {_lib.STATUS_NAMES.get(rc, rc)}{why}")
    return packed, sp.view(np.float16)
