"""Mirror of kiln's caller-side helpers (kiln-model/src/marlin_proj.rs)."""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from . import _lib
from .marlin_gemm import KilnMarlinError, marlin_w4a16_gemm


@dataclass
class MarlinPackedProj:
    """marlin_proj.rs:38-50."""

    b_packed: torch.Tensor  # [k/16, 2n] int32, Marlin layout
    scales: torch.Tensor  # [k/g, n] float16, Marlin order
    groupsize: int  # -1 or 128
    k: int
    n: int


def shape_is_supported(k: int, n: int) -> bool:
    """marlin_proj.rs:53-55."""
    return k % 128 == 0 and n % 256 == 0


def w4a16_enabled() -> bool:
    """marlin_proj.rs:330-338: KILN_W4A16 in {1, true, yes} (case-insensitive)."""
    return os.environ.get("KILN_W4A16", "").strip().lower() in ("1", "true", "yes")


def pack_from_bf16(weight_t: torch.Tensor, groupsize: int = 128) -> Optional[MarlinPackedProj]:
    """marlin_proj.rs:198-227: pack a pre-transposed [k, n] weight living on the GPU.

    Returns None for an unsupported shape or a non-CUDA tensor (caller keeps its bf16 path).
    Unlike the reference's download -> CPU pack -> upload (marlin_proj.rs:87-182) the
    quantise+pack runs on the device, straight from the tensor.
    """
    if not weight_t.is_cuda:
        return None
    if weight_t.dim() != 2:
        raise KilnMarlinError("marlin_proj: weight_t must be a 2D [k, n] tensor")
    k, n = weight_t.shape
    if not shape_is_supported(k, n):
        return None
    if not (groupsize == -1 or groupsize == 128):
        raise KilnMarlinError(f"marlin_proj: groupsize must be -1 or 128 (got {groupsize})")
    if weight_t.dtype not in (torch.bfloat16, torch.float32):
        weight_t = weight_t.to(torch.float32)
    w = weight_t.contiguous()
    g = k if groupsize == -1 else groupsize
    dev = w.device
    b_packed = torch.empty((k // 16, 2 * n), dtype=torch.int32, device=dev)
    scales = torch.empty((k // g, n), dtype=torch.float16, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().kiln_w4a16_quantize_and_pack_device(
            w.data_ptr(), 1 if w.dtype == torch.bfloat16 else 0, k, n, groupsize,
            b_packed.data_ptr(), scales.data_ptr(), None, torch.cuda.current_stream(dev).cuda_stream,
        )
    if rc != 0:
        raise KilnMarlinError(f"marlin_proj: device pack failed: {_lib.STATUS_NAMES.get(rc, rc)}")
    return MarlinPackedProj(b_packed, scales, groupsize, k, n)


def pack_from_gptq(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor,
                   groupsize: int = 128) -> Optional[MarlinPackedProj]:
    """GPTQ tensors already on the GPU (qweight i32 [k/8, n], qzeros i32 [k/g, n/8], scales f16 [k/g, n]) -> packed
    projection, on the device and without dequantising (kiln: CPU dequantise to bf16, kiln-model/src/quantized.rs:70-163,
    then re-quantise).  Returns None when the shape is unsupported or the checkpoint is not symmetric (a zero-point other
    than 8): the caller then keeps kiln's route.  Reads one counter back from the device."""
    if not (qweight.is_cuda and qzeros.is_cuda and scales.is_cuda):
        return None
    k, n = qweight.shape[0] * 8, qweight.shape[1]
    if not shape_is_supported(k, n) or not (groupsize == -1 or groupsize == 128):
        return None
    g = k if groupsize == -1 else groupsize
    if tuple(scales.shape) != (k // g, n) or tuple(qzeros.shape) != (k // g, n // 8):
        raise KilnMarlinError("marlin_proj: GPTQ scales / qzeros shapes do not match qweight")
    if qweight.dtype != torch.int32 or qzeros.dtype != torch.int32:
        raise KilnMarlinError("marlin_proj: GPTQ qweight and qzeros must be i32")
    dev = qweight.device
    sc = scales.to(torch.float16).contiguous()
    b_packed = torch.empty((k // 16, 2 * n), dtype=torch.int32, device=dev)
    s_perm = torch.empty((k // g, n), dtype=torch.float16, device=dev)
    bad = torch.zeros(1, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().kiln_w4a16_repack_gptq_device(
            qweight.contiguous().data_ptr(), qzeros.contiguous().data_ptr(), sc.data_ptr(), k, n, groupsize,
            b_packed.data_ptr(), s_perm.data_ptr(), bad.data_ptr(), torch.cuda.current_stream(dev).cuda_stream)
    if rc != 0:
        raise KilnMarlinError(f"marlin_proj: GPTQ repack failed: {_lib.STATUS_NAMES.get(rc, rc)}")
    if int(bad.item()) != 0:
        return None
    return MarlinPackedProj(b_packed, s_perm, groupsize, k, n)


def pack_from_bf16_batch(weights: Sequence[torch.Tensor], groupsize: int = 128):
    """marlin_proj.rs:229-262: pack many projections; order preserved, None where unsupported."""
    return [pack_from_bf16(w, groupsize) for w in weights]


def concat_projections(projs: Sequence[MarlinPackedProj]) -> MarlinPackedProj:
    """Fuses sibling projections that read the same activations (q+k+v, gate+up) into one packed weight.

    The Marlin layout is separable along N at 64-column granularity, so the fused tensors are plain
    concatenations: one GEMM launch then replaces several (kiln issues one Marlin call per projection,
    kiln-model/src/forward.rs:2771-2839; its profiling notes list the gate/up merge as the next lever).
    The caller splits the [.., sum(n)] output by columns.
    """
    if not projs:
        raise KilnMarlinError("marlin_proj: nothing to concatenate")
    k, g = projs[0].k, projs[0].groupsize
    for pr in projs:
        if pr.k != k or pr.groupsize != g:
            raise KilnMarlinError("marlin_proj: projections must share k and groupsize to be fused")
        if pr.n % 64 != 0:
            raise KilnMarlinError("marlin_proj: every fused projection needs n % 64 == 0")
    n = sum(pr.n for pr in projs)
    if n % 256 != 0:
        raise KilnMarlinError(f"marlin_proj: fused n={n} must be a multiple of 256")
    b = torch.cat([pr.b_packed for pr in projs], dim=1).contiguous()
    s = torch.cat([pr.scales for pr in projs], dim=1).contiguous()
    return MarlinPackedProj(b, s, g, k, n)


def matmul_bf16(x: torch.Tensor, proj: MarlinPackedProj) -> torch.Tensor:
    """marlin_proj.rs:285-319: x [.., k] bf16 -> [.., n] bf16 (rank 2 or 3)."""
    if x.dim() == 2:
        lead = None
        if x.shape[1] != proj.k:
            raise KilnMarlinError(f"marlin_proj: x last dim {x.shape[1]} != k={proj.k}")
        x2 = x
    elif x.dim() == 3:
        b, s, kk = x.shape
        if kk != proj.k:
            raise KilnMarlinError(f"marlin_proj: x last dim {kk} != k={proj.k}")
        lead = (b, s)
        x2 = x.reshape(b * s, kk)
    else:
        raise KilnMarlinError(f"marlin_proj: matmul_bf16 expects rank-2 or rank-3 input, got rank {x.dim()}")
    out = marlin_w4a16_gemm(x2.contiguous(), proj.b_packed, proj.scales, proj.groupsize)
    return out if lead is None else out.reshape(lead[0], lead[1], proj.n)


class PackedCache:
    """On-disk cache of packed projections, so that a model is quantised and packed once, not at every load
    (kiln packs at every load: kiln-model/src/marlin_proj.rs:87-182, 16.9 s for its 96 MLP projections).

    An entry is keyed by a caller-chosen name plus the shape, dtype and groupsize, and carries a checksum of the
    source weight (the wrapping int64 sum of its 32-bit words, computed where the tensor lives), so a changed
    checkpoint under the same name is repacked, not trusted.  Files are numpy .npz archives.
    """

    def __init__(self, directory: str):
        import os

        self.dir = directory
        os.makedirs(directory, exist_ok=True)

    @staticmethod
    def _checksum(w: torch.Tensor) -> int:
        flat = w.contiguous().view(torch.uint8).flatten()
        pad = (-flat.numel()) % 4
        if pad:
            flat = torch.cat([flat, flat.new_zeros(pad)])
        return int(flat.view(torch.int32).to(torch.int64).sum().item())

    def _path(self, name: str, w: torch.Tensor, groupsize: int) -> str:
        import hashlib
        import os

        tag = f"{name}|{tuple(w.shape)}|{w.dtype}|{groupsize}"
        return os.path.join(self.dir, hashlib.sha256(tag.encode()).hexdigest()[:24] + ".npz")

    def get_or_pack(self, name: str, weight_t: torch.Tensor, groupsize: int = 128) -> Optional[MarlinPackedProj]:
        """pack_from_bf16 with the cache in front of it; the result lives on weight_t's device."""
        import os

        import numpy as np

        k, n = weight_t.shape
        if not weight_t.is_cuda or not shape_is_supported(k, n):
            return None
        path, chk = self._path(name, weight_t, groupsize), self._checksum(weight_t)
        if os.path.exists(path):
            with np.load(path) as z:
                if int(z["checksum"]) == chk and z["b_packed"].shape == (k // 16, 2 * n):
                    dev = weight_t.device
                    return MarlinPackedProj(torch.from_numpy(z["b_packed"]).to(dev),
                                            torch.from_numpy(z["scales_bits"].view(np.int16).copy()).view(torch.float16).to(dev),
                                            groupsize, k, n)
        proj = pack_from_bf16(weight_t, groupsize)
        if proj is not None:
            tmp = path + f".tmp{os.getpid()}.npz"
            np.savez(tmp, b_packed=proj.b_packed.cpu().numpy(),
                     scales_bits=proj.scales.cpu().view(torch.int16).numpy().view(np.uint16), checksum=np.int64(chk))
            os.replace(tmp, path)
        return proj
