"""Ahead-of-time build of the native library (``libmachete_b200.so``).

The reference JIT-compiles its device code through CuTe DSL on every new op
configuration (``Megakernel.compile``, src/machete/megakernel/megakernel.py:1594).
This build compiles one fixed persistent kernel for sm_100a with ``nvcc`` and
nothing else; the output lands next to this file so that it travels with the
source tree.

Run ``python -m machete_b200.build`` or call :func:`build`.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libmachete_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--use_fast_math",
    "-Xcompiler", "-fPIC",
]


def _sources() -> list[Path]:
    """The host side plus one translation unit per group of kernel variants."""
    return [CSRC / "megakernel.cu", CSRC / "gemm_sm100.cu", CSRC / "attn_prefill_sm100.cu"] + sorted(CSRC.glob("variants_*.cu"))


def _deps() -> list[Path]:
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.inc"))
    deps.append(PKG_DIR.parent / "include" / "machete_b200.h")
    return deps


def is_stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    return any(p.stat().st_mtime > built for p in _deps() if p.exists())


def build(force: bool = False, verbose: bool = False, defines: tuple = (), out: Path | None = None) -> Path:
    """Compile the library if it is missing or older than its sources.

    The translation units are compiled side by side (one ``nvcc -c`` each) and
    linked into one shared object; objects go to a scratch directory.
    """
    target = Path(out) if out else LIB_PATH
    if not force and out is None and not is_stale():
        return LIB_PATH
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: cannot build libmachete_b200.so")
    import tempfile
    from concurrent.futures import ThreadPoolExecutor

    flags = [*NVCC_FLAGS, *[f"-D{d}" for d in defines]]
    if verbose:
        flags += ["-Xptxas", "-v"]
    with tempfile.TemporaryDirectory(prefix="machete_b200_build_") as tmp:
        def compile_one(src: Path):
            obj = Path(tmp) / (src.stem + ".o")
            cmd = [nvcc, *flags, "-c", str(src), "-o", str(obj)]
            proc = subprocess.run(cmd, capture_output=True, text=True)
            if proc.returncode != 0:
                raise RuntimeError(f"nvcc failed:\n{' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
            return obj, proc.stderr

        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
            results = list(pool.map(compile_one, _sources()))
        if verbose:
            for _, err in results:
                sys.stderr.write(err)
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a",
               *[str(o) for o, _ in results], "-o", str(target)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    return target


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
