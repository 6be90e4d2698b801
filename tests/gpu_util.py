"""Helpers shared by the GPU parity tests (all calls go through the C ABI via the ctypes bridge)."""
import ctypes
import json
import os
import subprocess
import tempfile
from pathlib import Path

import numpy as np
import torch

import oracle as o

TOL = 0.0078125      # 1/128: the reference's tier-1 tolerance (tests/e2e/test_tier1_feature_coverage.mm:149,213,222)
ROOT = Path(__file__).resolve().parent.parent

# One row per checked configuration: what was compared, the largest difference, how many outputs are over the
# strict criterion max(1/128, one fp16 ulp of the gold), and how far over they are.  conftest.py prints the table
# at the end of the run and writes it to the file named by B200_PARITY_REPORT (if set).
PARITY_REPORT: list = []


def dev(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def run_gemm(br, fmt, X, W, N, layout=0, H=0, D=0, residual=None, host=False, ex=False):
    M, K = X.shape
    to = (lambda a: torch.from_numpy(np.ascontiguousarray(a))) if host else dev
    Xd, Wd = to(X), to(W)
    shape = (H, M, D) if layout == 1 else (M, N)
    Yd = torch.full(shape, float("nan"), dtype=torch.float16, device="cpu" if host else "cuda")
    if ex or layout or residual is not None or fmt > 5:
        Rd = to(residual) if residual is not None else None
        br.dispatch_gemm_ex(Xd, Wd, Yd, fmt, M, K, N, layout, H, D, Rd)
    else:
        br.dispatch_gemm(Xd, Wd, Yd, fmt, M, K, N)
    br.synchronize()
    assert br.device_error() == 0
    return Yd.cpu().numpy()


def strict_bound(gold64: np.ndarray) -> np.ndarray:
    """max(1/128, one fp16 ulp of the gold): the reference's tier-1 tolerance, widened only where the fp16 output
    grid itself is coarser than 1/128 (|y| >= 8)."""
    ulp = np.spacing(np.abs(gold64).astype(np.float16)).astype(np.float64)
    return np.maximum(TOL, ulp)


def tolerance(gold64: np.ndarray, rms_factor: float = 1.0) -> np.ndarray:
    """Pass line for fp16 outputs against the double-precision gold:
        |diff| <= max(1/128, ulp_fp16(gold), 2^-9 * rms(gold)).
    1/128 is the reference's tolerance on its own test distribution (output rms about 1); one fp16 ulp
    covers outputs above 8 where the fp16 grid itself is coarser than 1/128; the rms term scales the
    bound with the output magnitude for the heavier benchmark distributions (fp16 weights carry a relative
    rounding error of 2^-11 each, which a K = 4096 contraction turns into about 2^-11 * rms(y) of noise).  rms_factor
    widens that term for codecs whose fp16 weight is built from several rounded terms (the variable-rate affine codec
    rounds its sub-scale, its sub-bias and their multiply-add: three roundings per weight instead of one)."""
    rms = float(np.sqrt(np.mean(gold64 ** 2)))
    return np.maximum(strict_bound(gold64), rms_factor * 2.0 ** -9 * rms)


def parity_stats(Y, gold64, what="") -> dict:
    """Difference statistics against the strict criterion: how many outputs exceed it and by what factor."""
    diff = np.abs(Y.astype(np.float64) - gold64)
    ratio = diff / strict_bound(gold64)
    over = ratio > 1.0
    return {"what": what, "outputs": int(diff.size), "max_abs": float(diff.max()) if diff.size else 0.0,
            "rms_gold": float(np.sqrt(np.mean(gold64 ** 2))) if diff.size else 0.0,
            "over_strict": int(over.sum()),
            "over_by": {"(1,2]x": int(((ratio > 1.0) & (ratio <= 2.0)).sum()), "(2,3]x": int(((ratio > 2.0) & (ratio <= 3.0)).sum()),
                        ">3x": int((ratio > 3.0).sum())},
            "max_over_factor": float(ratio.max()) if diff.size else 0.0}


_codec_lib = None


def codec_lib():
    """The device unpackers of csrc/codecs.cuh compiled for the host (tests/codec_host_shim.cpp)."""
    global _codec_lib
    if _codec_lib is None:
        out = Path(tempfile.mkdtemp(prefix="codec_host_")) / "codec_host.so"
        subprocess.check_call(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", str(ROOT / "tests" / "codec_host_shim.cpp"), "-o", str(out)])
        _codec_lib = ctypes.CDLL(str(out))
    return _codec_lib


def device_weight_gold(fmt, X, W, N):
    """Double-precision contraction of X with the exact fp16 weights the kernel feeds to the tensor core (the
    device unpackers run on the host, bit for bit).  What separates the kernel's output from this gold is the fp32
    accumulation and the final fp16 rounding only, so the strict criterion must hold against it outright; what
    separates this gold from the oracle's is the one fp16 rounding per weight that the reference's device
    unpackers (half arithmetic, quant_router_kernels.metal:111-436) perform as well."""
    M, K = X.shape
    out = np.empty((N, K), np.uint16)
    assert codec_lib().codec_host_dequant(int(fmt), o._ptr(W), o._ptr(out), N, K) == 0
    Wd = out.view(np.float16).astype(np.float64)
    Y = X.astype(np.float64) @ Wd.T
    if fmt == o.TERNARY_ROW:            # integers code-1 in the tensor core; the row's scale multiplies the accumulator
        Y = Y * W[N * K // 4:N * K // 4 + 2 * N].view(np.float16).astype(np.float64)[None, :]
    return Y


def check(Y, gold64, what="", dev_gold=None, rms_factor=1.0):
    """Pass line: every output within tolerance() of the oracle's double-precision gold.  With `dev_gold` (see
    device_weight_gold) the strict criterion max(1/128, 1 ulp) must hold against it with no exception, which shows
    that anything the rms term of the pass line covers is fp16 weight rounding, not a defect of the kernel.  The
    statistics against the strict criterion go to the parity report either way."""
    diff = np.abs(Y.astype(np.float64) - gold64)
    assert np.all(np.isfinite(Y.astype(np.float32))), f"{what}: non-finite output"
    st = parity_stats(Y, gold64, what)
    if dev_gold is not None:
        sd = parity_stats(Y, dev_gold, what)
        st["vs_device_weights"] = {"max_abs": sd["max_abs"], "over_strict": sd["over_strict"], "max_over_factor": sd["max_over_factor"]}
    PARITY_REPORT.append(st)
    tol = tolerance(gold64, rms_factor)
    bad = diff > tol
    assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} outputs over tolerance, max-abs {diff.max():.5f}"
    if dev_gold is not None:
        assert st["vs_device_weights"]["over_strict"] == 0, \
            f"{what}: {st['vs_device_weights']['over_strict']} outputs over max(1/128, ulp) against the fp16-weight gold"
    return float(diff.max())


def write_report(path=None):
    path = path or os.environ.get("B200_PARITY_REPORT")
    if path and PARITY_REPORT:
        Path(path).parent.mkdir(parents=True, exist_ok=True)
        Path(path).write_text(json.dumps(PARITY_REPORT, indent=1))


def cfloat(x):
    return ctypes.c_float(float(x))


def check_swiglu(Y, g64, u64, what=""):
    """SwiGLU outputs multiply two contractions, so the GEMM criterion is propagated through the product:
        tol = 1.1*|u|*tol(g) + |silu(g)|*tol(u) + max(1/128, ulp_fp16(out))
    (|silu'| <= 1.1), with tol() the per-GEMM criterion above on the gate and up golds."""
    sig = 1.0 / (1.0 + np.exp(-g64))
    out = g64 * sig * u64
    tol = 1.1 * np.abs(u64) * tolerance(g64) + np.abs(g64 * sig) * tolerance(u64) + \
        np.maximum(TOL, np.spacing(np.abs(out).astype(np.float16)).astype(np.float64))
    diff = np.abs(Y.astype(np.float64) - out)
    assert np.all(np.isfinite(Y.astype(np.float32))), f"{what}: non-finite output"
    PARITY_REPORT.append(parity_stats(Y, out, what))
    bad = diff > tol
    assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} outputs over tolerance, max-abs {diff.max():.5f}"
    return float(diff.max())
