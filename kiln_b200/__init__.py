"""kiln_b200: B200 (sm_100a) W4A16 quantised-linear path behind kiln's `kiln-marlin-gemm` API.

Host-side mirror of the reference crate's public surface
(kiln-marlin-gemm/src/lib.rs: `marlin_w4a16_gemm`, `mod pack`) and of its caller-side
helpers (kiln-model/src/marlin_proj.rs), on top of the C ABI in include/kiln_w4a16.h.
"""
from . import nvtx, pack  # noqa: F401
from .marlin_gemm import KilnMarlinError, marlin_w4a16_gemm, workspace_bytes  # noqa: F401
from .shard import (  # noqa: F401
    ColumnParallelLinear,
    FusedGatherOutput,
    fused_column_parallel_gemm,
    all_gather_columns,
    shard_bounds,
    shard_packed,
    shard_proj,
)
from .marlin_proj import (  # noqa: F401
    MarlinPackedProj,
    concat_projections,
    interleave_gate_up,
    interleave_columns_32,
    swiglu_gate_up,
    matmul_bf16_lora,
    grouped_matmul_bf16,
    pack_from_gptq,
    PackedCache,
    matmul_bf16,
    pack_from_bf16,
    pack_from_bf16_batch,
    shape_is_supported,
)

__all__ = [
    "pack", "marlin_w4a16_gemm", "workspace_bytes", "KilnMarlinError", "MarlinPackedProj",
    "matmul_bf16", "concat_projections", "interleave_gate_up", "interleave_columns_32", "swiglu_gate_up", "matmul_bf16_lora", "grouped_matmul_bf16", "pack_from_gptq", "PackedCache", "pack_from_bf16", "pack_from_bf16_batch", "shape_is_supported",
    "ColumnParallelLinear", "FusedGatherOutput", "fused_column_parallel_gemm", "all_gather_columns", "shard_bounds", "shard_packed", "shard_proj",
]
