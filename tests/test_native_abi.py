"""The C-ABI library: it loads, exports every declared symbol, and the struct layouts agree."""

import ctypes
import re
from pathlib import Path

import numpy as np
import pytest

from machete_b200 import _native as N

HEADER = Path(__file__).resolve().parents[1] / "include" / "machete_b200.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(mk_[a-z0-9_]+)\s*\(", text)))


def test_header_functions_are_exported():
    lib = N.lib()
    names = declared_functions()
    assert set(N.EXPORTS) == set(names)
    for name in names:
        assert hasattr(lib, name), name
    assert lib.mk_abi_version() == N.ABI_VERSION


def test_struct_layouts_match_header():
    assert N.OP_DTYPE.itemsize == 384
    assert N.OP_DTYPE.fields["i"][1] == 16 and N.OP_DTYPE.fields["f"][1] == 112
    assert N.OP_DTYPE.fields["p"][1] == 128 and N.OP_DTYPE.fields["s"][1] == 256
    assert N.INSTR_DTYPE.itemsize == 64 and N.EVENT_DTYPE.itemsize == 64 and N.WAIT_DTYPE.itemsize == 8
    assert ctypes.sizeof(N.Program) == 12 * 4 + 9 * 8 + 2 * 4


def test_enum_values_match_header():
    text = HEADER.read_text()
    for name, value in (("MK_OP_MATVEC", N.OP_MATVEC), ("MK_OP_ATTN_SPLIT", N.OP_ATTN_SPLIT),
                        ("MK_OP_TOP1_FINAL", N.OP_TOP1_FINAL)):
        assert re.search(rf"{name} = {value}\b", text), name
    assert f"#define MK_ABI_VERSION {N.ABI_VERSION}" in text
    # the attention op's integer slots, in header order (the last one is filled in by the library)
    slots = re.search(r"MK_AT_B = 0,(.*?)\};", text, re.S).group(1)
    names = ["MK_AT_B"] + re.findall(r"\b(MK_AT_[A-Z0-9_]+)\b(?=\s*[,/\n}])", re.sub(r"/\*.*?\*/", "", slots, flags=re.S))
    assert names[-2:] == ["MK_AT_DYNPOS", "MK_AT_GROUP"] and len(names) == N.AT_GROUP + 1 <= 24


def test_host_errors_without_a_gpu():
    lib = N.lib()
    assert lib.mk_workspace_bytes(None) == 0
    assert lib.mk_standalone_workspace_bytes() >= 1 << 20
    handle = ctypes.c_void_p()
    rc = lib.mk_create(None, ctypes.byref(handle))
    assert rc != 0 and b"null program" in lib.mk_last_error()
    assert lib.mk_run(None, None) != 0


def test_public_calls_refuse_cpu_tensors():
    """There is no CPU path behind the operator API: CPU tensors are refused with a message, and the
    C entry points of the tensor-core kernels refuse bad arguments before touching a device."""
    import pytest
    import torch

    from machete_b200.kernels.attention import flash_prefill
    from machete_b200.kernels.gemm.gemm_sm100 import gemm_sm100

    bf = torch.bfloat16
    q = torch.zeros(1, 2, 128, 64, dtype=bf)
    with pytest.raises(RuntimeError, match="no CPU path"):
        flash_prefill(q, q, q, torch.zeros_like(q))
    with pytest.raises(ValueError, match="layout"):
        flash_prefill(q, q, q, torch.zeros_like(q), layout="hbmd")
    a, w, c = torch.zeros(1, 64, 256, dtype=bf), torch.zeros(128, 256, dtype=bf), torch.zeros(1, 64, 128, dtype=bf)
    with pytest.raises(RuntimeError, match="no CPU path"):
        gemm_sm100(a, w, c)
    lib = N.lib()
    strides = (ctypes.c_int64 * 3)(1, 1, 1)
    rc = lib.mk_flash_prefill_bf16(None, None, None, None, None, 1, 1, 1, 1, 1, 64, strides, strides, strides, strides,
                                   ctypes.c_float(1.0), 0, None, 0, 0, None)
    assert rc != 0 and b"null pointer" in lib.mk_flash_prefill_last_error()
    assert lib.mk_gemm_bf16_workspace_bytes(64, 4096, 4096, 4) > 0


def test_a_missing_library_is_an_error_not_a_fallback(tmp_path):
    """With no loadable native library the package refuses to work: there is no CPU path to fall back to."""
    import os
    import subprocess
    import sys

    code = ("import machete_b200._native as N\n"
            "try:\n    N.lib()\nexcept RuntimeError as e:\n    print('refused:', str(e)[:60])\nelse:\n    print('loaded')\n")
    env = dict(os.environ, MACHETE_B200_LIB=str(tmp_path / "no_such_library.so"))
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True,
                         cwd=str(HEADER.parent.parent), timeout=300)
    assert "refused: machete_b200: cannot load" in out.stdout, out.stdout + out.stderr
