import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with -m gpu)")


def _has_gpu() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_terminal_summary(terminalreporter, exitstatus, config):
    """Parity table of the GPU tests: per checked configuration the largest difference from the oracle's gold, the
    number of outputs over the strict criterion max(1/128, one fp16 ulp) and by what factor, and (where the test
    computed it) the same against the gold built from the exact fp16 weights the kernel uses."""
    try:
        import gpu_util
    except Exception:
        return
    rows = gpu_util.PARITY_REPORT
    if not rows:
        return
    gpu_util.write_report()
    tr = terminalreporter
    tr.section("parity against the CPU oracle (strict criterion: max(1/128, 1 fp16 ulp))")
    for r in rows:
        ob = r["over_by"]
        line = (f"{r['what'][:44]:44s} n={r['outputs']:>9d} max|d|={r['max_abs']:.5f} rms={r['rms_gold']:.2f} "
                f"over={r['over_strict']} [(1,2]x {ob['(1,2]x']}, (2,3]x {ob['(2,3]x']}, >3x {ob['>3x']}]")
        if "vs_device_weights" in r:
            d = r["vs_device_weights"]
            line += f" | fp16-weight gold: max|d|={d['max_abs']:.5f} over={d['over_strict']}"
        tr.write_line(line)


@pytest.fixture(scope="session")
def pkg():
    from __graft_entry__ import load_package
    return load_package()


@pytest.fixture(scope="session")
def lib_path():
    p = ROOT / "m4-prefill-engine_b200" / "libb200_bridge.so"
    if not p.exists():
        from __graft_entry__ import _load_build_module
        _load_build_module().build()
    return p


@pytest.fixture(scope="session")
def bridge(pkg, lib_path):
    """Initialised bridge on cuda:0.  Fails loudly if the CUDA library cannot come up: there is no
    CPU path to fall back to."""
    import torch
    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    br = pkg.B200Bridge.get_instance()
    assert br.init(), br.lib.b200_bridge_last_error_string()
    yield br
    br.synchronize()
    assert br.device_error() == 0
