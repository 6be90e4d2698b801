"""In-tree build of libb200_bridge.so (nvcc, sm_100a only).

``python m4-prefill-engine_b200/build.py`` or ``build()`` from Python.  Objects go to
``csrc/_obj`` and the shared library next to this file, so it travels with a source snapshot.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = CSRC / "_obj"
LIB = HERE / "libb200_bridge.so"
SOURCES = ["qgemm.cu", "qgemm_small.cu", "qgemv.cu", "bridge.cu", "attention.cu", "layer_ops.cu", "transformer_layer.cu", "transformer_model.cu", "peer_reduce.cu", "no_alloc.cu", "quant_registry.cpp", "gguf_loader.cpp"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v", "-I", str(HERE.parent / "include")]
# development builds only: extra nvcc flags (e.g. -DATTN_TRACE, -DQG_TRACE=1) from the environment
NVCC_FLAGS += os.environ.get("B200_EXTRA_NVCC_FLAGS", "").split()


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found: the CUDA extension cannot be built")
    return exe


def _deps(src: Path) -> list[Path]:
    return [src, *CSRC.glob("*.cuh"), *CSRC.glob("*.h"), *(HERE.parent / "include").glob("*.h")]


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps if d.exists())


def _compile(src: Path, verbose: bool) -> Path:
    obj = OBJ / (src.stem + ".o")
    if _stale(obj, _deps(src)):
        cmd = [nvcc(), *NVCC_FLAGS, "-x", "cu", "-c", str(src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        (OBJ / (src.stem + ".log")).write_text(res.stdout + res.stderr)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError(f"nvcc failed on {src.name}")
        if verbose:
            sys.stderr.write(res.stderr)
    return obj


def build(verbose: bool = False, force: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    srcs = [CSRC / s for s in SOURCES if (CSRC / s).exists()]
    if force:
        for o in OBJ.glob("*.o"):
            o.unlink()
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose), srcs))
    if force or _stale(LIB, objs):
        cmd = [nvcc(), "-shared", "-o", str(LIB), *map(str, objs), "-lcudart", "-Xlinker", "-z,noexecstack"]
        subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
