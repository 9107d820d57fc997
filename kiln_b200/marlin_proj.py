"""Mirror of kiln's caller-side helpers (kiln-model/src/marlin_proj.rs)."""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from . import _lib, nvtx
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
    with torch.cuda.device(dev), nvtx.range("kiln/marlin/pack"):
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


def interleave_gate_up(gate: MarlinPackedProj, up: MarlinPackedProj) -> MarlinPackedProj:
    """Fuses the gate and up projections of an MLP into ONE packed weight whose columns alternate in runs of 32 (fused
    columns 64c .. 64c+31 = gate columns 32c .. 32c+31, 64c+32 .. 64c+63 = the up columns of the same indices): the
    layout `swiglu_gate_up` needs, so that a gate column and its up column are finished by the same threads.

    No weight is touched: in the Marlin layout a 16-column tile of a 64-column chunk is one 32-bit word per lane, so the
    fused matrix is a shuffle of whole words, and the scale order (position 8i + j of a chunk holds column i + 8j) is
    undone, interleaved and redone.  kiln keeps gate and up as two Marlin calls (kiln-model/src/forward.rs:2769-2839)."""
    if gate.k != up.k or gate.n != up.n or gate.groupsize != up.groupsize:
        raise KilnMarlinError("marlin_proj: gate and up must have the same shape and groupsize")
    k, n, g = gate.k, gate.n, gate.groupsize
    if n % 128 != 0 or (2 * n) % 256 != 0:
        raise KilnMarlinError(f"marlin_proj: n={n} must be a multiple of 128 to interleave gate and up")
    ch = n // 64
    # words: [k/16, chunk, lane, tile]; fused chunk 2c takes tiles 0,1 of gate chunk c then tiles 0,1 of up chunk c,
    # fused chunk 2c+1 takes tiles 2,3 of both
    gw = gate.b_packed.view(k // 16, ch, 32, 2, 2)  # [.., lane, half, tile in half]
    uw = up.b_packed.view(k // 16, ch, 32, 2, 2)
    fused = torch.stack([gw, uw], dim=4)  # [k/16, ch, lane, half, (gate|up), tile]
    fused = fused.permute(0, 1, 3, 2, 4, 5).reshape(k // 16, 2 * ch * 32 * 4).contiguous()  # chunk 2c+half
    if g == -1:
        nat = _scales_single_to_natural
        perm = _scales_natural_to_single
    else:
        nat = _scales_grouped_to_natural
        perm = _scales_natural_to_grouped
    gs, us = nat(gate.scales), nat(up.scales)  # natural column order
    rows = gs.shape[0]
    fs = torch.stack([gs.view(rows, n // 32, 32), us.view(rows, n // 32, 32)], dim=2).reshape(rows, 2 * n)
    return MarlinPackedProj(fused, perm(fs).contiguous(), g, k, 2 * n)


def _grouped_perm(device):
    t = torch.arange(64, device=device)
    return (t // 8) + 8 * (t % 8)  # position t of a 64-column run holds column perm[t] (kiln-marlin-gemm/src/lib.rs:333-341)


def _single_perm(device):
    t = torch.arange(32, device=device)
    off = torch.tensor([0, 1, 8, 9, 16, 17, 24, 25], device=device)
    return 2 * (t // 8) + off[t % 8]  # kiln-marlin-gemm/src/lib.rs:348-357


def _scales_grouped_to_natural(s: torch.Tensor) -> torch.Tensor:
    r, n = s.shape
    out = torch.empty_like(s)
    out.view(r, n // 64, 64)[:, :, _grouped_perm(s.device)] = s.view(r, n // 64, 64)
    return out


def _scales_natural_to_grouped(s: torch.Tensor) -> torch.Tensor:
    r, n = s.shape
    return s.view(r, n // 64, 64)[:, :, _grouped_perm(s.device)].reshape(r, n)


def _scales_single_to_natural(s: torch.Tensor) -> torch.Tensor:
    r, n = s.shape
    out = torch.empty_like(s)
    out.view(r, n // 32, 32)[:, :, _single_perm(s.device)] = s.view(r, n // 32, 32)
    return out


def _scales_natural_to_single(s: torch.Tensor) -> torch.Tensor:
    r, n = s.shape
    return s.view(r, n // 32, 32)[:, :, _single_perm(s.device)].reshape(r, n)


def interleave_columns_32(gate_cols: torch.Tensor, up_cols: torch.Tensor) -> torch.Tensor:
    """Row-wise companion of `interleave_gate_up` for anything indexed by output column (LoRA B matrices [n, r], biases):
    rows 64c .. 64c+31 of the result are rows 32c .. 32c+31 of the first argument, the next 32 those of the second."""
    n = gate_cols.shape[0]
    rest = gate_cols.shape[1:]
    return torch.stack([gate_cols.reshape(n // 32, 32, *rest), up_cols.reshape(n // 32, 32, *rest)], dim=1).reshape(2 * n, *rest)


_ex_workspaces: dict = {}


def _gemm_ex(x2: torch.Tensor, proj: MarlinPackedProj, swiglu: bool, lora_a, lora_b, lora_scale: float,
             out: Optional[torch.Tensor] = None) -> torch.Tensor:
    import ctypes

    m, k = x2.shape
    if k != proj.k:
        raise KilnMarlinError(f"marlin_proj: x last dim {k} != k={proj.k}")
    if x2.dtype != torch.bfloat16 or not x2.is_cuda:
        raise KilnMarlinError("marlin_proj: x must be a CUDA bf16 tensor")
    ep = _lib.Epilogue()
    ep.swiglu = 1 if swiglu else 0
    keep = []
    if lora_a is not None:
        r = lora_a.shape[0]
        if tuple(lora_a.shape) != (r, k) or tuple(lora_b.shape) != (proj.n, r):
            raise KilnMarlinError(f"marlin_proj: LoRA A must be [r, {k}] and B [{proj.n}, r]")
        a_ = lora_a.to(device=x2.device, dtype=torch.bfloat16).contiguous()
        b_ = lora_b.to(device=x2.device, dtype=torch.bfloat16).contiguous()
        if r % 8:  # pad the rank to a multiple of 8 with zeros
            pad = 8 - r % 8
            a_ = torch.cat([a_, a_.new_zeros((pad, k))], dim=0).contiguous()
            b_ = torch.cat([b_, b_.new_zeros((proj.n, pad))], dim=1).contiguous()
            r += pad
        keep += [a_, b_]
        ep.lora_a, ep.lora_b, ep.lora_rank, ep.lora_scale = a_.data_ptr(), b_.data_ptr(), r, float(lora_scale)
    n_out = proj.n // 2 if swiglu else proj.n
    if out is None:
        out = torch.empty((m, n_out), dtype=torch.bfloat16, device=x2.device)
    elif tuple(out.shape) != (m, n_out) or out.dtype != torch.bfloat16 or not out.is_contiguous() or out.device != x2.device:
        raise KilnMarlinError("marlin_proj: out must be a contiguous bf16 [m, n_out] tensor on x's device")
    if m == 0:
        return out
    lib = _lib.lib()
    name = "kiln/mlp/gate_up_swiglu" if swiglu else ("kiln/marlin/gemm_lora" if lora_a is not None else "kiln/marlin/gemm")
    with torch.cuda.device(x2.device), nvtx.range(name):
        need = int(lib.kiln_w4a16_workspace_bytes_ex(m, proj.n, k, ctypes.byref(ep)))
        ws = _ex_workspaces.get(x2.device)
        if need and (ws is None or ws.numel() < need):
            ws = torch.empty(max(need, 1 << 20), dtype=torch.uint8, device=x2.device)
            _ex_workspaces[x2.device] = ws
        rc = lib.kiln_w4a16_gemm_bf16_ex(
            x2.contiguous().data_ptr(), proj.b_packed.data_ptr(), out.data_ptr(), proj.scales.data_ptr(), m, proj.n, k,
            proj.groupsize, ctypes.byref(ep), ws.data_ptr() if need else None, ws.numel() if need else 0,
            torch.cuda.current_stream(x2.device).cuda_stream)
    if rc != 0:
        raise KilnMarlinError(f"kiln_w4a16_gemm_bf16_ex failed: {_lib.STATUS_NAMES.get(rc, rc)}")
    return out


def _flatten(x: torch.Tensor, k: int):
    if x.dim() == 2:
        return x, None
    if x.dim() == 3:
        b, s_, kk = x.shape
        return x.reshape(b * s_, kk), (b, s_)
    raise KilnMarlinError(f"marlin_proj: expects rank-2 or rank-3 input, got rank {x.dim()}")


def matmul_bf16_lora(x: torch.Tensor, proj: MarlinPackedProj, lora_a: torch.Tensor, lora_b: torch.Tensor,
                     lora_scale: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """`mlp_proj_forward` / `linear_with_lora` on the Marlin path (kiln-model/src/forward.rs:2925-2945): base GEMM plus
    the LoRA delta x @ A^T @ B^T * scale (lora_loader.rs:213-233), the delta added inside the GEMM's epilogue.
    lora_a [r, k], lora_b [n, r]."""
    x2, lead = _flatten(x, proj.k)
    out = _gemm_ex(x2, proj, False, lora_a, lora_b, lora_scale, out)
    return out if lead is None else out.reshape(lead[0], lead[1], -1)


def swiglu_gate_up(x: torch.Tensor, fused: MarlinPackedProj, lora_a: Optional[torch.Tensor] = None,
                   lora_b: Optional[torch.Tensor] = None, lora_scale: float = 1.0,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """silu(x @ gate) * (x @ up) in one GEMM launch (kiln: two Marlin calls, a SiLU kernel and a multiply,
    kiln-model/src/forward.rs:2769-2839).  `fused` comes from `interleave_gate_up`; the result is [.., n/2] and feeds
    the down projection directly.  An optional LoRA pair applies to the fused matrix (lora_b rows in the same
    interleaved column order, see `interleave_columns_32`)."""
    x2, lead = _flatten(x, fused.k)
    out = _gemm_ex(x2, fused, True, lora_a, lora_b, lora_scale, out)
    return out if lead is None else out.reshape(lead[0], lead[1], -1)


def grouped_matmul_bf16(xs: Sequence[torch.Tensor], projs: Sequence[MarlinPackedProj],
                        outs: Optional[Sequence[torch.Tensor]] = None) -> list:
    """Several independent projections (the q, k, v of an attention layer, say) in ONE launch when the batch is at a
    decode size; xs[i] [m_i, k_i] bf16 (rank 2) goes with projs[i].  Returns the list of outputs."""
    import ctypes

    if len(xs) != len(projs) or not 1 <= len(xs) <= 8:
        raise KilnMarlinError("marlin_proj: grouped_matmul_bf16 takes 1..8 (x, projection) pairs")
    dev = xs[0].device
    given = outs
    outs, arr, keep = [], (_lib.Problem * len(xs))(), []
    need = 0
    lib = _lib.lib()
    for i, (x, pr) in enumerate(zip(xs, projs)):
        if x.dim() != 2 or x.shape[1] != pr.k or x.dtype != torch.bfloat16 or x.device != dev:
            raise KilnMarlinError("marlin_proj: every x must be a rank-2 bf16 tensor [m, k] on one device")
        xc = x.contiguous()
        keep.append(xc)
        o = given[i] if given is not None else torch.empty((x.shape[0], pr.n), dtype=torch.bfloat16, device=dev)
        if tuple(o.shape) != (x.shape[0], pr.n) or o.dtype != torch.bfloat16 or not o.is_contiguous():
            raise KilnMarlinError("marlin_proj: every out must be a contiguous bf16 [m, n] tensor")
        outs.append(o)
        arr[i] = _lib.Problem(xc.data_ptr(), pr.b_packed.data_ptr(), o.data_ptr(), pr.scales.data_ptr(), x.shape[0], pr.n, pr.k,
                              pr.groupsize)
        need = max(need, int(lib.kiln_w4a16_workspace_bytes(x.shape[0], pr.n, pr.k)))
    with torch.cuda.device(dev), nvtx.range("kiln/proj/grouped"):
        ws = _ex_workspaces.get(dev)
        if need and (ws is None or ws.numel() < need):
            ws = torch.empty(max(need, 1 << 20), dtype=torch.uint8, device=dev)
            _ex_workspaces[dev] = ws
        rc = lib.kiln_w4a16_gemm_bf16_grouped(arr, len(xs), ws.data_ptr() if need else None, ws.numel() if need else 0,
                                              torch.cuda.current_stream(dev).cuda_stream)
    if rc != 0:
        raise KilnMarlinError(f"kiln_w4a16_gemm_bf16_grouped failed: {_lib.STATUS_NAMES.get(rc, rc)}")
    return outs


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

    An entry is keyed by a caller-chosen name plus the shape, dtype and groupsize, and carries a digest of the
    source weight computed where the tensor lives: the wrapping int64 sum of word[i] * (2 * (i mod 2^20) + 1) over its
    32-bit words plus their plain sum, i.e. position-dependent, so that rows swapped or words re-ordered under the
    same name are repacked, not trusted.  Files are numpy .npz archives.
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
        words = flat.view(torch.int32).to(torch.int64)
        mult = 2 * (torch.arange(words.numel(), device=words.device, dtype=torch.int64) & ((1 << 20) - 1)) + 1
        return int(((words * mult).sum() + words.sum() * 0x9E3779B1).item())

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
