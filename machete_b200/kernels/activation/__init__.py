from .add import AddOp

ACT_MAP = {"relu": 1, "silu": 2, "identity": 0, None: 0}

__all__ = ["AddOp", "ACT_MAP"]
