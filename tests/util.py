"""Shared helpers for the parity tests (oracle side lives in `oracle/`)."""
import numpy as np
import torch

import oracle
from oracle import C

# max |diff| / max |oracle| bound stated by the path's accuracy contract
REL_TOL = 1e-2

QWEN_SHAPES = {  # name: (k, n) of the benchmark's projection sweep
    "q": (2560, 4096), "k": (2560, 512), "v": (2560, 512), "o": (4096, 2560),
    "gate_up": (2560, 18432), "down": (9216, 2560), "gdn_in": (2560, 8192), "gdn_out": (4096, 2560),
}


def to_torch_bf16(bits: np.ndarray, device) -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16).to(device)


def from_torch_bf16(t: torch.Tensor) -> np.ndarray:
    return oracle.bf16_bits_to_f32(t.detach().cpu().view(torch.int16).numpy().view(np.uint16))


def make_case(m, k, n, seed=1234, groupsize=128, device=None):
    """Synthetic benchmark-distribution inputs, packed by the ORACLE packer, plus the fp64 oracle output."""
    a, q, s = oracle.synth_inputs(m, k, n, seed=seed, groupsize=groupsize)
    packed = C.pack_nibbles(q)
    sp = C.permute_scales(s, groupsize)
    ref = C.gemm_fp64(a, q, s, groupsize)
    case = dict(a=a, q=q, s=s, packed=packed, sp=sp, ref=ref, m=m, k=k, n=n, groupsize=groupsize)
    if device is not None:
        case["a_t"] = to_torch_bf16(a, device)
        case["b_t"] = torch.from_numpy(packed).to(device)
        case["s_t"] = torch.from_numpy(sp.view(np.int16).copy()).view(torch.float16).to(device)
    return case


def rel_err(out_f32: np.ndarray, ref: np.ndarray) -> float:
    return float(np.abs(out_f32.astype(np.float64) - ref.astype(np.float64)).max() / max(np.abs(ref).max(), 1e-30))
