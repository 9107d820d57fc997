"""TEST INFRASTRUCTURE ONLY -- Python face of the CPU oracle.

Two things live here, both restating kiln's `kiln-marlin-gemm` packer and its
dequantise-then-matmul semantics on the CPU (paths relative to the kiln tree):

* `C` -- ctypes bindings to `oracle/w4a16_oracle.c` (a scalar restatement that
  keeps the loop order of crates/kiln-marlin-gemm/src/lib.rs:370-491);
* `np_*` -- an independent, vectorised numpy restatement of the same steps, used
  to cross-check the C file bit for bit.

Nothing under `kiln_b200/` may import this package.  Only `tests/`, the smoke
check and the benchmark's CPU-baseline leg use it, as the checker or as the timed
CPU baseline.  See the header of `w4a16_oracle.c` for what pins it.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

MAX_Q = 15
Q_OFFSET = 8


def build(force: bool = False) -> None:
    """Compile the C oracle."""
    src = os.path.join(_HERE, "w4a16_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "liboracle.so"], stdout=subprocess.DEVNULL)


_lib = None


def _load():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.oracle_f16_bits_to_f32.restype = ctypes.c_float
        _lib.oracle_f16_bits_to_f32.argtypes = [ctypes.c_uint16]
        _lib.oracle_f32_to_f16_bits.restype = ctypes.c_uint16
        _lib.oracle_f32_to_f16_bits.argtypes = [ctypes.c_float]
        _lib.oracle_f32_to_bf16_bits.restype = ctypes.c_uint16
        _lib.oracle_f32_to_bf16_bits.argtypes = [ctypes.c_float]
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dtype):
    a = np.ascontiguousarray(a, dtype=dtype)
    return a


# ----------------------------------------------------------------------------
# ctypes face of w4a16_oracle.c
# ----------------------------------------------------------------------------
class C:
    @staticmethod
    def set_num_threads(n: int) -> None:
        """Threads the OpenMP loops of the C oracle use from now on (a launcher may have exported OMP_NUM_THREADS=1)."""
        _load().oracle_set_num_threads(int(n))

    @staticmethod
    def num_threads() -> int:
        return int(_load().oracle_num_threads())

    @staticmethod
    def weight_perm() -> np.ndarray:
        out = np.zeros(1024, np.int32)
        _load().oracle_build_weight_perm(_p(out))
        return out

    @staticmethod
    def scale_perm() -> np.ndarray:
        out = np.zeros(64, np.int32)
        _load().oracle_build_scale_perm(_p(out))
        return out

    @staticmethod
    def scale_perm_single() -> np.ndarray:
        out = np.zeros(32, np.int32)
        _load().oracle_build_scale_perm_single(_p(out))
        return out

    @staticmethod
    def pack_nibbles(q: np.ndarray) -> np.ndarray:
        q = _c(q, np.uint8)
        k, n = q.shape
        out = np.zeros((k // 16, 2 * n), np.int32)
        rc = _load().oracle_pack_nibbles(_p(q), k, n, _p(out))
        if rc:
            raise ValueError(f"oracle_pack_nibbles rc={rc}")
        return out

    @staticmethod
    def unpack_fragment(packed: np.ndarray, k: int, n: int) -> np.ndarray:
        packed = _c(packed, np.int32)
        q = np.zeros((k, n), np.uint8)
        rc = _load().oracle_unpack_fragment(_p(packed), k, n, _p(q))
        if rc:
            raise ValueError(f"oracle_unpack_fragment rc={rc}")
        return q

    @staticmethod
    def permute_scales(scales_f16: np.ndarray, groupsize: int) -> np.ndarray:
        s = _c(scales_f16.view(np.uint16), np.uint16)
        g, n = s.shape
        out = np.zeros_like(s)
        rc = _load().oracle_permute_scales(_p(s), g, n, groupsize, _p(out))
        if rc:
            raise ValueError(f"oracle_permute_scales rc={rc}")
        return out.view(np.float16)

    @staticmethod
    def quantize_and_pack(weight: np.ndarray, groupsize: int):
        """-> (packed i32 [k/16,2n], scales f16 [k/g,n] permuted, dequant f32 [k,n], q u8 [k,n])"""
        w = _c(weight, np.float32)
        k, n = w.shape
        g = k if groupsize == -1 else groupsize
        if k % 128 or n % 256 or g <= 0 or k % g:
            raise ValueError("shape rejected (k%128, n%256, k%g)")
        packed = np.zeros((k // 16, 2 * n), np.int32)
        scales = np.zeros((k // g, n), np.uint16)
        dequant = np.zeros((k, n), np.float32)
        q = np.zeros((k, n), np.uint8)
        rc = _load().oracle_quantize_and_pack(_p(w), k, n, groupsize, _p(packed), _p(scales), _p(dequant), _p(q))
        if rc:
            raise ValueError(f"oracle_quantize_and_pack rc={rc}")
        return packed, scales.view(np.float16), dequant, q

    @staticmethod
    def gemm_fp64(a_bf16_bits: np.ndarray, q: np.ndarray, scales_f16: np.ndarray, groupsize: int) -> np.ndarray:
        """fp32-semantics oracle (exact operands, f64 accumulation).  scales UNPERMUTED."""
        a = _c(a_bf16_bits, np.uint16)
        q = _c(q, np.uint8)
        s = _c(scales_f16.view(np.uint16), np.uint16)
        m, k = a.shape
        n = q.shape[1]
        out = np.zeros((m, n), np.float32)
        rc = _load().oracle_gemm_fp64(_p(a), _p(q), _p(s), m, n, k, groupsize, _p(out))
        if rc:
            raise ValueError(f"oracle_gemm_fp64 rc={rc}")
        return out

    @staticmethod
    def gemm_cpu_reference(a_bf16_bits, q, scales_f16, groupsize, scratch=None) -> np.ndarray:
        """The reference's CPU dequantise(bf16)-then-matmul path; returns bf16 bits [m,n]."""
        a = _c(a_bf16_bits, np.uint16)
        q = _c(q, np.uint8)
        s = _c(scales_f16.view(np.uint16), np.uint16)
        m, k = a.shape
        n = q.shape[1]
        if scratch is None:
            scratch = np.empty((k, n), np.uint16)
        out = np.zeros((m, n), np.uint16)
        rc = _load().oracle_w4a16_gemm_cpu(_p(a), _p(q), _p(s), m, n, k, groupsize, _p(scratch), _p(out))
        if rc:
            raise ValueError(f"oracle_w4a16_gemm_cpu rc={rc}")
        return out


# ----------------------------------------------------------------------------
# independent numpy restatement
# ----------------------------------------------------------------------------
def np_weight_perm() -> np.ndarray:
    """crates/kiln-marlin-gemm/src/lib.rs:296-327, stated with array ops."""
    i = np.arange(32)
    col = i // 4
    rows = np.stack([2 * (i % 4), 2 * (i % 4) + 1, 2 * (i % 4 + 4), 2 * (i % 4 + 4) + 1], 1)  # [32,4]
    perm1 = np.concatenate([16 * rows + col[:, None] + 8 * b for b in (0, 1)], 1)  # [32,8]
    perm = (perm1[:, None, :] + 256 * np.arange(4)[None, :, None]).reshape(-1)  # [1024]
    inter = np.array([0, 2, 4, 6, 1, 3, 5, 7])
    return perm.reshape(-1, 8)[:, inter].reshape(-1).astype(np.int32)


def np_pack_nibbles(q: np.ndarray) -> np.ndarray:
    """crates/kiln-marlin-gemm/src/lib.rs:429-479 as reshape/transpose/gather."""
    k, n = q.shape
    t = q.astype(np.uint32).reshape(k // 16, 16, n // 16, 16).transpose(0, 2, 1, 3).reshape(k // 16, n * 16)
    r = t.reshape(-1, 1024)[:, np_weight_perm()].reshape(t.shape)
    out = np.zeros((k // 16, n * 2), np.uint32)
    for i in range(8):
        out |= (r[:, i::8] & 0xF) << np.uint32(4 * i)
    return out.view(np.int32)


def np_permute_scales(scales_f16: np.ndarray, groupsize: int) -> np.ndarray:
    """crates/kiln-marlin-gemm/src/lib.rs:496-528."""
    s = np.ascontiguousarray(scales_f16)
    g, n = s.shape
    if groupsize == -1:
        inner = np.array([0, 1, 8, 9, 16, 17, 24, 25])
        sp = (2 * np.arange(4)[:, None] + inner[None, :]).reshape(-1)
        return s.reshape(-1, 32)[:, sp].reshape(g, n)
    sp = (np.arange(8)[:, None] + 8 * np.arange(8)[None, :]).reshape(-1)
    return s.reshape(-1, 64)[:, sp].reshape(g, n)


def np_round_half_away(x: np.ndarray) -> np.ndarray:
    """Rust `f32::round` (crates/kiln-marlin-gemm/src/lib.rs:422): ties away from zero."""
    x = x.astype(np.float32)
    return (np.sign(x) * np.floor(np.abs(x).astype(np.float64) + 0.5)).astype(np.float32)


def np_quantize(weight: np.ndarray, groupsize: int):
    """Steps 1-2 of crates/kiln-marlin-gemm/src/lib.rs:393-427 -> (q u8 [k,n], scales f16 [k/g,n], dequant f32)."""
    w = np.ascontiguousarray(weight, np.float32)
    k, n = w.shape
    g = k if groupsize == -1 else groupsize
    wg = w.reshape(k // g, g, n)
    max_abs = np.abs(wg).max(1)
    max_abs = np.where(max_abs == 0, np.float32(1.0), max_abs).astype(np.float32)
    s32 = (np.float32(2.0) * max_abs) / np.float32(MAX_Q)
    s16 = s32.astype(np.float16)
    s = s16.astype(np.float32)
    raw = np_round_half_away(wg / s[:, None, :]).astype(np.int64)
    qq = np.clip(raw + Q_OFFSET, 0, MAX_Q)
    deq = ((qq - Q_OFFSET).astype(np.float32) * s[:, None, :]).reshape(k, n)
    return qq.reshape(k, n).astype(np.uint8), s16, deq


def np_quantize_and_pack(weight: np.ndarray, groupsize: int):
    q, s16, deq = np_quantize(weight, groupsize)
    return np_pack_nibbles(q), np_permute_scales(s16, groupsize), deq, q


def np_gemm_fp64(a_bf16_bits: np.ndarray, q: np.ndarray, scales_f16: np.ndarray, groupsize: int) -> np.ndarray:
    a = bf16_bits_to_f32(a_bf16_bits).astype(np.float64)
    k, n = q.shape
    g = k if groupsize == -1 else groupsize
    w = (q.astype(np.float64) - Q_OFFSET) * np.repeat(scales_f16.astype(np.float64), g, axis=0)
    return (a @ w).astype(np.float32)


# ----------------------------------------------------------------------------
# bf16 helpers and the seeded synthetic inputs the benchmark configurations use
# ----------------------------------------------------------------------------
def np_gptq_pack(q: np.ndarray, zeros: np.ndarray):
    """Builds GPTQ checkpoint tensors from nibbles q uint8 [k, n] and zero-points uint8 [k/g, n], in the layout kiln reads
    (kiln-model/src/quantized.rs:6-14, 125-135): qweight int32 [k/8, n], nibble i of a word = input row 8*row + i;
    qzeros int32 [k/g, n/8], nibble j of a word = output column 8*col + j."""
    k, n = q.shape
    qw = np.zeros((k // 8, n), np.uint32)
    for i in range(8):
        qw |= q[i::8].astype(np.uint32) << np.uint32(4 * i)
    qz = np.zeros((zeros.shape[0], n // 8), np.uint32)
    for j in range(8):
        qz |= zeros[:, j::8].astype(np.uint32) << np.uint32(4 * j)
    return qw.view(np.int32), qz.view(np.int32)


def np_gptq_dequant(qweight: np.ndarray, qzeros: np.ndarray, scales_f16: np.ndarray, group_size: int) -> np.ndarray:
    """kiln's GPTQ dequantisation (kiln-model/src/quantized.rs:118-145) as float32 [k, n] (the reference stores the
    transpose, rounded to bf16): (nibble - zero) * scale."""
    qw, qz = qweight.view(np.uint32), qzeros.view(np.uint32)
    k, n = qw.shape[0] * 8, qw.shape[1]
    rows = np.arange(k)
    w = (qw[rows // 8] >> (4 * (rows % 8)).astype(np.uint32)[:, None]) & np.uint32(0xF)
    cols = np.arange(n)
    z = (qz[:, cols // 8] >> (4 * (cols % 8)).astype(np.uint32)[None, :]) & np.uint32(0xF)
    grp = rows // group_size
    return (w.astype(np.int32) - z[grp].astype(np.int32)).astype(np.float32) * scales_f16.astype(np.float32)[grp]


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    return ((u + 0x7FFF + lsb) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def synth_inputs(m: int, k: int, n: int, seed: int = 1234, groupsize: int = 128):
    """Seeded synthetic tensors with the benchmark's distributions: activations
    bf16(N(0,1)) [m,k]; nibbles uniform in [0,15] [k,n]; scales
    f16(0.01*|N(0,1)|+1e-3) [k/g,n] (unpermuted)."""
    rng = np.random.default_rng(seed)
    g = k if groupsize == -1 else groupsize
    a = f32_to_bf16_bits(rng.standard_normal((m, k), dtype=np.float32))
    q = rng.integers(0, 16, size=(k, n), dtype=np.uint8)
    s = (0.01 * np.abs(rng.standard_normal((k // g, n), dtype=np.float32)) + 1e-3).astype(np.float16)
    return a, q, s


def kiln_lcg_fill(count: int, seed: int, scale: float) -> np.ndarray:
    """The reference parity test's own 64-bit LCG
    (crates/kiln-marlin-gemm/tests/parity.rs:22-52): value = (bits31 / i32::MAX - 0.5) * scale."""
    out = np.empty(count, np.float32)
    state = seed & 0xFFFFFFFFFFFFFFFF
    mul, inc, mask = 6364136223846793005, 1442695040888963407, 0xFFFFFFFFFFFFFFFF
    i32max = np.float32(2147483647)
    for i in range(count):
        state = (state * mul + inc) & mask
        bits = (state >> 33) & 0x7FFFFFFF
        out[i] = (np.float32(bits) / i32max - np.float32(0.5)) * np.float32(scale)
    return out
