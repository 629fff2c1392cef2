"""Megakernel host runtime: op protocol, scheduler, launch.

Usage, as with the reference (src/machete/megakernel/__init__.py:9-16)::

    from machete_b200.megakernel import Megakernel
    from machete_b200.kernels.rms_norm import RMSNormOp

    ops = RMSNormOp.schedule(x=x, weight=w, y=y)
    Megakernel(ops).run()
"""

from .lowering import LowerCtx, NativeOp, Region
from .megakernel import Megakernel, MegakernelConfig, create_megakernel
from .ops import (DEFAULT_PAGE_SIZE, BFloat16, Float16, Float32, Int32, Int64, Op, PipelineSpec, ScheduledOp,
                  TensorMeta, Uint8, build_op_config, is_compile_static_dim, last_dim_slice_region,
                  tensor_meta_overlaps)
from .scheduling import (INSTRUCTION_WORDS, BackwardScheduler, BuiltProgram, InstructionStreamBuilder,
                         OverlapTileScheduler, TileScheduler, infer_dependencies, simulate)

__all__ = [
    "DEFAULT_PAGE_SIZE", "Op", "ScheduledOp", "TensorMeta", "PipelineSpec", "build_op_config",
    "is_compile_static_dim", "last_dim_slice_region", "tensor_meta_overlaps",
    "Float16", "BFloat16", "Float32", "Int32", "Int64", "Uint8",
    "INSTRUCTION_WORDS", "TileScheduler", "BackwardScheduler", "OverlapTileScheduler",
    "InstructionStreamBuilder", "BuiltProgram", "infer_dependencies", "simulate",
    "Megakernel", "MegakernelConfig", "create_megakernel", "NativeOp", "Region", "LowerCtx",
]
