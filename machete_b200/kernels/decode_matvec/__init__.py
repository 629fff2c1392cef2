"""Decode matvec ops (bf16 and NVFP4 weights) and layer schedules."""

from .nvfp4 import (FinalRmsLmHeadNvfp4Sm120Op, MatvecNvfp4Sm120Op, MatvecResidualNvfp4Sm120Op,
                    RmsGateUpSiluNvfp4Sm120Op, RmsKMatvecRopeCacheNvfp4Sm120Op, RmsMatvecNvfp4Sm120Op,
                    RmsQMatvecRopeNvfp4Sm120Op, RmsVMatvecCacheNvfp4Sm120Op)
from .norm import RmsAddNormSm100Op, RmsAddNormSm120Op
from .sm100 import DecodeLayerSchedule as DecodeLayerScheduleSm100
from .sm100 import (FinalRmsLmHeadSm100Op, MatvecResidualSm100Op, MatvecSm100Op, ResidualAddSm100Op,
                    RmsGateUpSiluSm100Op, RmsKMatvecRopeCacheSm100Op, RmsQMatvecRopeSm100Op,
                    RmsVMatvecCacheSm100Op, schedule_decode_layer_sm100, schedule_final_sm100)
from .top1 import (FinalAddRmsTop1LmHeadNvfp4Sm100Op, FinalAddRmsTop1LmHeadSm100Op, ReduceTop1Sm100Op,
                   schedule_final_top1_sm100)

# The NVFP4 ops run on sm_100a here; both suffixes name the same classes.
RmsQMatvecRopeNvfp4Sm100Op = RmsQMatvecRopeNvfp4Sm120Op
RmsKMatvecRopeCacheNvfp4Sm100Op = RmsKMatvecRopeCacheNvfp4Sm120Op
RmsVMatvecCacheNvfp4Sm100Op = RmsVMatvecCacheNvfp4Sm120Op
RmsMatvecNvfp4Sm100Op = RmsMatvecNvfp4Sm120Op
MatvecNvfp4Sm100Op = MatvecNvfp4Sm120Op
MatvecResidualNvfp4Sm100Op = MatvecResidualNvfp4Sm120Op
RmsGateUpSiluNvfp4Sm100Op = RmsGateUpSiluNvfp4Sm120Op
FinalRmsLmHeadNvfp4Sm100Op = FinalRmsLmHeadNvfp4Sm120Op

__all__ = [n for n in dir() if n.endswith("Op") or n.startswith("schedule_") or n.startswith("DecodeLayer")]
