"""machete_b200: the decode-step megakernel of b-albar/machete, rebuilt for B200 (sm_100a).

Package layout mirrors the reference's ``machete`` package for the decode path
(``megakernel``, ``kernels.*``, ``quantization``); ``install_as_machete()``
registers the same modules under the ``machete`` name so that code written
against the reference imports unchanged.
"""

from __future__ import annotations

import importlib
import sys

__version__ = "0.1.0"

_ALIASED = [
    "megakernel", "megakernel.ops", "megakernel.scheduling", "megakernel.megakernel",
    "kernels", "kernels.gemm", "kernels.rms_norm", "kernels.rope", "kernels.qknorm_rope", "kernels.glu",
    "kernels.activation", "kernels.activation.add", "kernels.attention", "kernels.attention.flash_decoding",
    "kernels.decode_matvec", "kernels.decode_matvec.sm100", "kernels.llama1b", "quantization",
    "quantization.nvfp4",
]


def install_as_machete() -> None:
    """Make ``import machete...`` resolve to this package (refuses to shadow a real ``machete``)."""
    existing = sys.modules.get("machete")
    if existing is not None and not getattr(existing, "__machete_b200_alias__", False):
        raise RuntimeError("a different 'machete' package is already imported")
    root = sys.modules[__name__]
    root.__machete_b200_alias__ = True
    sys.modules["machete"] = root
    for name in _ALIASED:
        sys.modules[f"machete.{name}"] = importlib.import_module(f"{__name__}.{name}")
