"""Mirror of `kiln_marlin_gemm::marlin_w4a16_gemm` (kiln-marlin-gemm/src/lib.rs:97-275)."""
from __future__ import annotations

import torch

from . import _lib, nvtx


class KilnMarlinError(RuntimeError):
    """Stands in for `candle_core::Error` raised by the reference's `bail!` sites."""


_workspaces: dict = {}
_retired: list = []


def workspace_bytes(m: int, n: int, k: int) -> int:
    return int(_lib.lib().kiln_w4a16_workspace_bytes(m, n, k))


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Scratch that only grows, one buffer per (device, stream): GEMMs on different streams may overlap on the GPU and
    must not share split-K partial sums.  Replaces the reference's per-call `Tensor::zeros` workspace (lib.rs:176-178).
    A buffer that is outgrown is kept alive until the process ends (a kernel of an earlier call may still use it)."""
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        if ws is not None:
            _retired.append(ws)
        ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def marlin_w4a16_gemm(a: torch.Tensor, b_packed: torch.Tensor, scales: torch.Tensor, groupsize: int,
                      out: torch.Tensor | None = None) -> torch.Tensor:
    """a [m,k] bf16 x b_packed [k/16, 2n] i32 (Marlin layout) x scales [k/g, n] f16 -> [m,n] bf16.

    Same checks, in the same order and with the same messages, as lib.rs:103-166.
    `out` (optional, beyond the reference) receives the result in place.
    """
    if not a.is_cuda:
        raise KilnMarlinError("kiln-marlin-gemm: a must be on CUDA")
    if a.dim() != 2 or b_packed.dim() != 2 or scales.dim() != 2:
        raise KilnMarlinError("kiln-marlin-gemm: a, b_packed and scales must be rank-2")
    m, k = a.shape
    b_rows, b_cols = b_packed.shape
    s_rows, n = scales.shape
    if k % 128 != 0:
        raise KilnMarlinError(f"kiln-marlin-gemm: k must be a multiple of 128 (got {k})")
    if n % 256 != 0:
        raise KilnMarlinError(f"kiln-marlin-gemm: n must be a multiple of 256 (got {n})")
    if b_rows != k // 16 or b_cols != n * 16 // 8:
        raise KilnMarlinError(
            f"kiln-marlin-gemm: b_packed shape [{b_rows}, {b_cols}] does not match expected "
            f"[k/16={k // 16}, n*16/8={n * 16 // 8}] for k={k}, n={n}"
        )
    if not (groupsize == -1 or groupsize == 128):
        raise KilnMarlinError(f"kiln-marlin-gemm: groupsize must be -1 or 128 (got {groupsize})")
    g = k if groupsize == -1 else groupsize
    if g > k or k % g != 0:
        raise KilnMarlinError(f"kiln-marlin-gemm: k={k} must be divisible by groupsize={groupsize}")
    if s_rows != k // g:
        raise KilnMarlinError(
            f"kiln-marlin-gemm: scales rows {s_rows} != expected {k // g} (k={k}, groupsize={groupsize})"
        )
    if a.dtype != torch.bfloat16:
        raise KilnMarlinError(f"kiln-marlin-gemm: a must be bf16 (got {a.dtype})")
    if b_packed.dtype != torch.int32:
        raise KilnMarlinError(f"kiln-marlin-gemm: b_packed must be i32 (got {b_packed.dtype})")
    if scales.dtype != torch.float16:
        raise KilnMarlinError(f"kiln-marlin-gemm: scales must be f16 (got {scales.dtype})")
    if not (b_packed.is_cuda and scales.is_cuda):
        raise KilnMarlinError("kiln-marlin-gemm: b_packed must be on CUDA")

    a = a.contiguous()
    b_packed = b_packed.contiguous()
    scales = scales.contiguous()
    if out is None:
        out = torch.empty((m, n), dtype=torch.bfloat16, device=a.device)
    elif out.shape != (m, n) or out.dtype != torch.bfloat16 or not out.is_contiguous() or out.device != a.device:
        raise KilnMarlinError("kiln-marlin-gemm: out must be a contiguous bf16 [m, n] tensor on a's device")
    if m == 0:
        return out
    with torch.cuda.device(a.device), nvtx.range("kiln/marlin/gemm"):
        nbytes = workspace_bytes(m, n, k)
        ws = _workspace(a.device, nbytes) if nbytes else None
        stream = torch.cuda.current_stream(a.device).cuda_stream
        status = _lib.lib().kiln_w4a16_gemm_bf16(
            a.data_ptr(), b_packed.data_ptr(), out.data_ptr(), scales.data_ptr(), m, n, k, groupsize,
            ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0, stream,
        )
    if status != 0:
        raise KilnMarlinError(
            f"kiln_marlin_w4a16_gemm failed with status {status} "
            f"(1=ERR_PROB_SHAPE, 2=ERR_KERN_SHAPE) for m={m}, n={n}, k={k}, groupsize={groupsize}"
            f" [{_lib.STATUS_NAMES.get(status, '?')}, cuda={_lib.lib().kiln_w4a16_last_cuda_error()}]"
        )
    return out
