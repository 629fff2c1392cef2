"""Op protocol: declarations, schedule-time validation, tile counts, config packing, aliasing.

Known answers re-derived from the behaviours the reference's host tests pin
(tests/megakernel/test_ops.py: declaration processing, tile counts = ceil(dim / tile),
dim conflicts, rank checks, config tensor layout).
"""

import struct

import pytest
import torch

from machete_b200.megakernel import (BFloat16, Float32, Op, ScheduledOp, TensorMeta, last_dim_slice_region,
                                     tensor_meta_overlaps)
from machete_b200.megakernel.lowering import meta_of


class ToyOp(Op):
    reads = {"x": (None, ("M", "D")), "w": (Float32, ("D",))}
    writes = {"y": (None, ("M", "D"))}
    tile = ("M",)


def test_declaration_metadata():
    assert ToyOp.INPUTS == ["x", "w"] and ToyOp.OUTPUTS == ["y"]
    assert ToyOp.DIM_NAMES == {"M": 0}
    assert ToyOp.gen_tensor_param_names() == ["x", "w", "y"]
    assert ToyOp._CONFIG_PTR_I32_OFFSET == {"x": 0, "w": 2, "y": 4}
    assert ToyOp._CONFIG_DYNAMIC_I32_OFFSET == {"D": 6}     # non-tile dims are dynamic


def test_tile_dim_must_exist():
    with pytest.raises(ValueError, match="not found"):
        class Bad(Op):
            reads = {"x": (None, ("M",))}
            writes = {"y": (None, ("M",))}
            tile = ("Q",)


def test_too_many_tile_dims():
    with pytest.raises(ValueError, match="max is 4"):
        class Bad(Op):
            reads = {"x": (None, ("A", "B", "C", "D", "E"))}
            writes = {"y": (None, ("A", "B", "C", "D", "E"))}
            tile = ("A", "B", "C", "D", "E")


def test_schedule_counts_and_config():
    x = torch.zeros(10, 8, dtype=torch.bfloat16)
    w = torch.zeros(8)
    y = torch.zeros(10, 8, dtype=torch.bfloat16)
    (op,) = ToyOp.schedule(x=x, w=w, y=y, tile_sizes={"M": 4})
    assert isinstance(op, ScheduledOp)
    assert op.tile_counts == (3,) and op.tile_sizes == {"M": 4} and op.total_tiles == 3
    assert op.static_dims == {"M": 10, "D": 8}
    assert op.tensor_dtypes == {"x": BFloat16, "y": BFloat16}
    cfg = op.config_data
    assert cfg.dtype == torch.int32 and cfg.numel() == 7
    lo, hi = struct.unpack("<2i", struct.pack("<Q", x.data_ptr()))
    assert cfg[0].item() == lo and cfg[1].item() == hi and cfg[6].item() == 8
    # unspecified tile size = whole extent, one tile
    (op2,) = ToyOp.schedule(x=x, w=w, y=y)
    assert op2.tile_counts == (1,) and op2.tile_sizes == {"M": 10}
    # a tile larger than the extent is clamped
    (op3,) = ToyOp.schedule(x=x, w=w, y=y, tile_sizes={"M": 64})
    assert op3.tile_counts == (1,) and op3.tile_sizes == {"M": 10}


def test_schedule_rejects_rank_and_dim_conflicts():
    x = torch.zeros(10, 8)
    with pytest.raises(ValueError, match="declared as 2D"):
        ToyOp.schedule(x=x[0], w=torch.zeros(8), y=x)
    with pytest.raises(ValueError, match="conflict"):
        ToyOp.schedule(x=x, w=torch.zeros(9), y=x)


def test_tile_count_limit():
    with pytest.raises(ValueError, match="65535"):
        ScheduledOp(op_cls=ToyOp, tile_counts=(70000,))


def test_overlap_rules():
    buf = torch.zeros(4, 2, 96, dtype=torch.bfloat16)          # packed q|k|v on the last dim
    q, k, v = buf[..., :32], buf[..., 32:64], buf[..., 64:]
    mq, mk, mv, mb = (meta_of(t) for t in (q, k, v, buf))
    assert not tensor_meta_overlaps(mq, mk) and not tensor_meta_overlaps(mk, mv)
    assert tensor_meta_overlaps(mb, mk) and tensor_meta_overlaps(mq, mq)
    assert last_dim_slice_region(mb, mk) == (32, 32, 96)
    other = torch.zeros(4, 2, 96, dtype=torch.bfloat16)
    assert not tensor_meta_overlaps(mb, meta_of(other))
    # row ranges of one cache
    cache = torch.zeros(2, 16, 4, 8)
    assert not tensor_meta_overlaps(meta_of(cache[:, :8]), meta_of(cache[:, 8:]))
    assert tensor_meta_overlaps(meta_of(cache[:, :9]), meta_of(cache[:, 8:]))
    # different ranks over the same bytes fall back to address spans
    assert tensor_meta_overlaps(meta_of(buf.view(8, 96)), mb)


def test_op_without_native_handler_is_rejected():
    from machete_b200.megakernel import Megakernel, MegakernelConfig

    x = torch.zeros(4, 8)
    ops = ToyOp.schedule(x=x, w=torch.zeros(8), y=x.clone())
    with pytest.raises(NotImplementedError, match="no native"):
        Megakernel(ops, config=MegakernelConfig(num_sms=4))
