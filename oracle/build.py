"""Build recipe for the CPU checkers (test infrastructure, never the product path).

  liboracle.so  <- oracle/oracle.cpp              (our restatement; always built)
  _ref/libm4ref.so <- the reference's own CPU verifier sources, compiled where they lie in
                   the reference checkout (only when that checkout is present; on machines
                   without it the previously built file is used as is).

The reference sources use two things g++ lacks: the `__fp16` type name and Apple's
`dispatch_apply(n, queue, ^(size_t i){...});` blocks.  They are rewritten on the fly by sed
into a temporary directory (`__fp16` -> `_Float16` by a -D define; each dispatch_apply block
-> an OpenMP for loop with the same body) and only the shared object is kept.
"""
from __future__ import annotations

import os
import re
import subprocess
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
BUILD = HERE / "_build"
REF_OUT = HERE / "_ref"
CXXFLAGS = ["-O2", "-std=c++17", "-fopenmp", "-fPIC", "-shared", "-fno-fast-math", "-ffp-contract=off"]

_DISPATCH = re.compile(
    r"dispatch_apply\((\w+),\s*dispatch_get_global_queue\([^)]*\),\s*\^\(size_t (\w+)\)\s*\{")


def _newer(target: Path, *sources: Path) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(s.exists() and s.stat().st_mtime <= t for s in sources)


def build_oracle(force: bool = False) -> Path:
    BUILD.mkdir(exist_ok=True)
    out = BUILD / "liboracle.so"
    src = HERE / "oracle.cpp"
    hdr = HERE.parent / "include" / "quant_router.h"
    if force or not _newer(out, src, hdr):
        subprocess.check_call(["g++", *CXXFLAGS, str(src), "-o", str(out)])
    return out


def _rewrite(text: str) -> str:
    """dispatch_apply blocks -> OpenMP loops; drop the libdispatch include."""
    text = text.replace("#include <dispatch/dispatch.h>", "")
    text = _DISPATCH.sub(
        r'_Pragma("omp parallel for schedule(dynamic)") for (size_t \2 = 0; \2 < (size_t)(\1); ++\2) {', text)
    return re.sub(r"^(\s*)\}\);\s*$", r"\1}", text, flags=re.M)


def _section(text: str, start: str, stop: str) -> str:
    """Lines from the first one that starts with `start` up to (not including) the first later
    line that starts with `stop`."""
    lines = text.splitlines()
    i0 = next(i for i, l in enumerate(lines) if l.startswith(start))
    i1 = next(i for i in range(i0 + 1, len(lines)) if lines[i].startswith(stop))
    return "\n".join(lines[i0:i1]) + "\n"


def reference_root() -> Path:
    """Where the reference checkout lies: $M4_PREFILL_REFERENCE_ROOT, else a directory named `reference` beside this
    repository.  It does not have to exist (then the previously built verifier, if any, is used as is)."""
    env = os.environ.get("M4_PREFILL_REFERENCE_ROOT")
    return Path(env) if env else HERE.parent.parent / "reference"


def build_ref(ref_root: str | os.PathLike | None = None, force: bool = False) -> Path | None:
    ref = Path(ref_root) if ref_root is not None else reference_root()
    out = REF_OUT / "libm4ref.so"
    gold = ref / "tests" / "e2e" / "cpu_gold_reference.h"
    if not gold.exists():
        return out if out.exists() else None
    shim = HERE / "ref_shim.cpp"
    if not force and _newer(out, shim, gold):
        return out
    REF_OUT.mkdir(exist_ok=True)
    with tempfile.TemporaryDirectory(prefix="m4ref_") as tmp:
        t = Path(tmp)
        g = _rewrite(gold.read_text()).replace('"../../quant_router.h"', f'"{ref / "quant_router.h"}"')
        (t / "gold.h").write_text(g)
        common = (ref / "tests" / "e2e" / "test_common.h").read_text()
        (t / "gen.inc").write_text(_section(common, "static uint32_t g_prng_state", "// Shader Path Resolver"))
        b3 = (ref / "brick3_swiglu_bench.mm").read_text()
        (t / "brick3.inc").write_text(_section(b3, "static uint32_t prng_state", "struct VariantConfig"))
        b4 = (ref / "brick4_attn_bench.mm").read_text()
        (t / "brick4.inc").write_text(_section(b4, "static uint32_t prng_state", "// BENCHMARK CONFIGURATION"))
        l8 = (ref / "bench_8b_engine.mm").read_text()
        (t / "layer.inc").write_text(_rewrite(_section(l8, "static uint32_t prng_state", "// TIMING & PROFILING")))
        defs = ["-D__fp16=_Float16",
                f'-DREF_GOLD_H="{t / "gold.h"}"', f'-DREF_GEN_INC="{t / "gen.inc"}"',
                f'-DREF_BRICK3="{t / "brick3.inc"}"', f'-DREF_BRICK4="{t / "brick4.inc"}"',
                f'-DREF_LAYER="{t / "layer.inc"}"']
        subprocess.check_call(["g++", *CXXFLAGS, "-w", *defs, str(shim), "-o", str(out)])
    return out


if __name__ == "__main__":
    print(build_oracle(force=True))
    print(build_ref(force=True))
