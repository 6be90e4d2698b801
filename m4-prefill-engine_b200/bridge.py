"""ctypes wrapper over libb200_bridge.so.

Mirrors ``core/bridge/m4_bridge.py:18-281`` of the reference: the ``QuantFormat`` enum, a singleton
bridge class with ``init / dispatch_gemm / dispatch_gemv / synchronize / get_uma_footprint_mb /
shutdown`` and module-level ``m4_bridge_*`` functions.  Arrays are ``torch`` tensors: CUDA tensors
are used in place, CPU tensors are staged by the library (host pointer in, host pointer out).
As in the reference, tensors are kept alive until ``synchronize()`` and a non-zero status raises
``RuntimeError`` carrying the code.
"""
from __future__ import annotations

import ctypes
import os
from enum import IntEnum
from pathlib import Path
from typing import Optional, Union

import torch


class QuantFormat(IntEnum):
    QUANT_Q4_0 = 0
    QUANT_MLX_4BIT = 1
    QUANT_Q4_K = 2
    QUANT_TERNARY_1_58 = 3
    QUANT_VAR_RATE_AFFINE = 4
    QUANT_EXL3 = 5
    # registry-only in the reference (quant_router.h:21-22); accepted by the *_ex entry points
    QUANT_PRISM_Q2_0 = 7
    # extension layouts of this library
    QUANT_MLX_4BIT_G64 = 100
    QUANT_TERNARY_ROW = 101
    QUANT_MLX_4BIT_PLANAR = 102


def library_path() -> Path:
    """Location of the shared library: $B200_BRIDGE_SO_PATH, else next to this file
    (the reference's M4_BRIDGE_DYLIB_PATH rule, core/bridge/m4_bridge.py:27-44)."""
    env = os.environ.get("B200_BRIDGE_SO_PATH")
    if env and Path(env).is_file():
        return Path(env)
    cand = Path(__file__).resolve().parent / "libb200_bridge.so"
    if cand.is_file():
        return cand
    raise FileNotFoundError(
        f"libb200_bridge.so not found at {cand}; build it with `python m4-prefill-engine_b200/build.py` "
        "or set B200_BRIDGE_SO_PATH (there is no CPU fallback)")


_vp, _sz, _u32, _i = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_uint32, ctypes.c_int


def bind(lib: ctypes.CDLL) -> ctypes.CDLL:
    """Declare argument and result types of every exported entry point (include/b200_bridge.h)."""
    lib.m4_bridge_init.argtypes = [ctypes.c_char_p]
    lib.m4_bridge_init.restype = ctypes.c_bool
    lib.m4_bridge_get_expected_weight_bytes.argtypes = [_i, _u32, _u32]
    lib.m4_bridge_get_expected_weight_bytes.restype = _sz
    lib.m4_bridge_dispatch_gemm.argtypes = [_vp, _sz, _vp, _sz, _vp, _sz, _i, _u32, _u32, _u32]
    lib.m4_bridge_dispatch_gemm.restype = _i
    lib.m4_bridge_dispatch_gemv.argtypes = [_vp, _sz, _vp, _sz, _vp, _sz, _i, _u32, _u32]
    lib.m4_bridge_dispatch_gemv.restype = _i
    lib.m4_bridge_synchronize.argtypes = []
    lib.m4_bridge_synchronize.restype = None
    lib.m4_bridge_get_uma_footprint_mb.argtypes = []
    lib.m4_bridge_get_uma_footprint_mb.restype = ctypes.c_double
    lib.m4_bridge_is_initialized.argtypes = []
    lib.m4_bridge_is_initialized.restype = ctypes.c_bool
    lib.m4_bridge_shutdown.argtypes = []
    lib.m4_bridge_shutdown.restype = None
    lib.b200_bridge_weight_bytes.argtypes = [_i, _u32, _u32]
    lib.b200_bridge_weight_bytes.restype = _sz
    lib.b200_bridge_dispatch_gemm_ex.argtypes = [_vp, _sz, _vp, _sz, _vp, _sz, _i, _u32, _u32, _u32, _i, _u32, _u32, _vp, _sz]
    lib.b200_bridge_dispatch_gemm_ex.restype = _i
    lib.b200_bridge_dispatch_swiglu.argtypes = [_vp, _sz, _vp, _vp, _sz, _vp, _sz, _i, _u32, _u32, _u32]
    lib.b200_bridge_dispatch_swiglu.restype = _i
    lib.b200_bridge_register_weights.argtypes = [_vp, _sz]
    lib.b200_bridge_register_weights.restype = _i
    lib.b200_bridge_unregister_weights.argtypes = [_vp]
    lib.b200_bridge_unregister_weights.restype = _i
    lib.b200_bridge_device_error.argtypes = []
    lib.b200_bridge_device_error.restype = _i
    lib.b200_bridge_last_error_string.argtypes = []
    lib.b200_bridge_last_error_string.restype = ctypes.c_char_p
    lib.b200_bridge_kernel_launches.argtypes = []
    lib.b200_bridge_kernel_launches.restype = ctypes.c_uint64
    lib.b200_bridge_stream.argtypes = []
    lib.b200_bridge_stream.restype = _vp
    lib.b200_bridge_force_generic.argtypes = [_i]
    lib.b200_bridge_force_generic.restype = None
    lib.b200_bridge_force_legacy_attention.argtypes = [_i]
    lib.b200_bridge_dispatch_gemm_grouped.argtypes = [_vp, ctypes.POINTER(_vp), ctypes.POINTER(_vp), ctypes.POINTER(ctypes.c_uint32),
                                                      ctypes.c_uint32, _i, ctypes.c_uint32, ctypes.c_uint32, _i, ctypes.c_uint32]
    lib.b200_bridge_dispatch_gemm_grouped.restype = _i
    lib.b200_bridge_force_legacy_attention.restype = None
    for name, args in _OPTIONAL.items():
        if hasattr(lib, name):
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = args
    return lib


_f = ctypes.c_float
# entry points of later translation units (attention, layer); bound when present
_OPTIONAL = {
    "b200_bridge_quantize_kv_q8_0": ([_vp, _sz, _vp, _sz, _sz], _i),
    "b200_bridge_dequantize_q8_0": ([_vp, _sz, _vp, _sz, _sz], _i),
    "b200_bridge_dispatch_attention_q8kv": ([_vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _f, _u32, _i, _i], _i),
    "b200_bridge_rmsnorm": ([_vp, _vp, _vp, _u32, _u32, _f], _i),
    "b200_bridge_rope": ([_vp, _u32, _u32, _u32, _f, _u32], _i),
    "b200_bridge_gemm_scratch_static": ([_vp, _sz, _vp, _sz, _vp, _sz, _i, _u32, _u32, _u32], _i),
    "b200_bridge_dispatch_qkv_fused": ([_vp] * 7 + [_i] + [_u32] * 5 + [_f, _u32, _i, _u32], _i),
}


def _addr(t: torch.Tensor) -> tuple[int, int]:
    return t.data_ptr(), t.numel() * t.element_size()


class B200Bridge:
    """Singleton over the shared library (shape of the reference's MetalUMABridge)."""

    _instance: Optional["B200Bridge"] = None

    def __init__(self, so_path: Optional[Union[str, Path]] = None) -> None:
        path = Path(so_path) if so_path else library_path()
        self._lib = bind(ctypes.CDLL(str(path)))
        self._in_flight: list[tuple[torch.Tensor, ...]] = []
        self._pending_finite: list[torch.Tensor] = []

    @property
    def lib(self) -> ctypes.CDLL:
        return self._lib

    @classmethod
    def get_instance(cls, so_path: Optional[Union[str, Path]] = None) -> "B200Bridge":
        if cls._instance is None:
            cls._instance = cls(so_path)
        return cls._instance

    @staticmethod
    def extract_buffer_address_and_size(t: torch.Tensor) -> tuple[torch.Tensor, int, int]:
        """Pointer and byte size of a tensor; non-contiguous views are made contiguous first
        (core/bridge/m4_bridge.py:112-134)."""
        if not t.is_contiguous():
            t = t.contiguous()
        p, n = _addr(t)
        return t, p, n

    def init(self, ignored: Optional[str] = None) -> bool:
        if torch.cuda.is_available():
            torch.cuda.current_device()   # make torch's context the current one before the library asks for it
        return bool(self._lib.m4_bridge_init(ignored.encode() if ignored else None))

    def is_initialized(self) -> bool:
        return bool(self._lib.m4_bridge_is_initialized())

    def _wait_torch(self, *tensors: torch.Tensor) -> None:
        # inputs produced on torch's stream must be complete before the bridge stream reads them
        if any(t.is_cuda for t in tensors):
            torch.cuda.current_stream().synchronize()

    def dispatch_gemm(self, X, W, Y, format, M=None, K=None, N=None, check_finite: bool = False) -> int:
        Xc, xp, xb = self.extract_buffer_address_and_size(X)
        Wc, wp, wb = self.extract_buffer_address_and_size(W)
        if not Y.is_contiguous():
            raise ValueError("output tensor must be contiguous")
        yp, yb = _addr(Y)
        if M is None:
            M = X.shape[0] if X.dim() >= 2 else 1
        if K is None:
            K = X.shape[1] if X.dim() >= 2 else X.shape[0]
        if N is None:
            N = Y.shape[1] if Y.dim() >= 2 else Y.shape[0]
        self._wait_torch(Xc, Wc, Y)
        ret = self._lib.m4_bridge_dispatch_gemm(xp, xb, wp, wb, yp, yb, int(format), int(M), int(K), int(N))
        if ret != 0:
            raise RuntimeError(f"m4_bridge_dispatch_gemm failed with status code {ret}")
        self._in_flight.append((Xc, Wc, Y))
        if check_finite:
            self._pending_finite.append(Y)
        return ret

    def dispatch_gemv(self, x, W, y, format, K=None, N=None, check_finite: bool = False) -> int:
        xc, xp, xb = self.extract_buffer_address_and_size(x)
        Wc, wp, wb = self.extract_buffer_address_and_size(W)
        yp, yb = _addr(y)
        if K is None:
            K = x.shape[-1]
        if N is None:
            N = y.shape[-1]
        self._wait_torch(xc, Wc, y)
        ret = self._lib.m4_bridge_dispatch_gemv(xp, xb, wp, wb, yp, yb, int(format), int(K), int(N))
        if ret != 0:
            raise RuntimeError(f"m4_bridge_dispatch_gemv failed with status code {ret}")
        self._in_flight.append((xc, Wc, y))
        if check_finite:
            self._pending_finite.append(y)
        return ret

    def dispatch_gemm_ex(self, X, W, Y, format, M, K, N, layout=0, H=0, D=0, residual=None) -> int:
        Xc, xp, xb = self.extract_buffer_address_and_size(X)
        Wc, wp, wb = self.extract_buffer_address_and_size(W)
        yp, yb = _addr(Y)
        rp, rb, Rc = None, 0, None
        if residual is not None:
            Rc, rp, rb = self.extract_buffer_address_and_size(residual)
        self._wait_torch(Xc, Wc, Y)
        ret = self._lib.b200_bridge_dispatch_gemm_ex(xp, xb, wp, wb, yp, yb, int(format), M, K, N, layout, H, D, rp, rb)
        if ret != 0:
            raise RuntimeError(f"b200_bridge_dispatch_gemm_ex failed with status code {ret}")
        self._in_flight.append((Xc, Wc, Y, Rc))
        return ret

    def dispatch_swiglu(self, X, Wg, Wu, Out, format, M, K, F) -> int:
        Xc, xp, xb = self.extract_buffer_address_and_size(X)
        Gc, gp, gb = self.extract_buffer_address_and_size(Wg)
        Uc, up, ub = self.extract_buffer_address_and_size(Wu)
        op, ob = _addr(Out)
        self._wait_torch(Xc, Gc, Uc, Out)
        ret = self._lib.b200_bridge_dispatch_swiglu(xp, xb, gp, up, min(gb, ub), op, ob, int(format), M, K, F)
        if ret != 0:
            raise RuntimeError(f"b200_bridge_dispatch_swiglu failed with status code {ret}")
        self._in_flight.append((Xc, Gc, Uc, Out))
        return ret

    def register_weights(self, W: torch.Tensor) -> int:
        p, n = _addr(W)
        return int(self._lib.b200_bridge_register_weights(p, n))

    def synchronize(self) -> None:
        self._lib.m4_bridge_synchronize()
        self._in_flight.clear()
        if self._pending_finite:
            checks, self._pending_finite = self._pending_finite, []
            for t in checks:
                if not bool(torch.isfinite(t).all().item()):
                    raise FloatingPointError("Tripwire assertion failed: Non-finite values (NaN/Inf) detected in output tensor.")

    def device_error(self) -> int:
        return int(self._lib.b200_bridge_device_error())

    def kernel_launches(self) -> int:
        return int(self._lib.b200_bridge_kernel_launches())

    def get_uma_footprint_mb(self) -> float:
        return float(self._lib.m4_bridge_get_uma_footprint_mb())

    def shutdown(self) -> None:
        self._in_flight.clear()
        self._pending_finite.clear()
        self._lib.m4_bridge_shutdown()


MetalUMABridge = B200Bridge   # the reference's class name, for callers written against it


def m4_bridge_init(ignored: Optional[str] = None) -> bool:
    return B200Bridge.get_instance().init(ignored)


def m4_bridge_dispatch_gemm(X, W, Y, format, M=None, K=None, N=None, check_finite: bool = False) -> int:
    return B200Bridge.get_instance().dispatch_gemm(X, W, Y, format, M, K, N, check_finite=check_finite)


def m4_bridge_dispatch_gemv(x, W, y, format, K=None, N=None, check_finite: bool = False) -> int:
    return B200Bridge.get_instance().dispatch_gemv(x, W, y, format, K, N, check_finite=check_finite)


def m4_bridge_synchronize() -> None:
    B200Bridge.get_instance().synchronize()


def m4_bridge_get_uma_footprint_mb() -> float:
    return B200Bridge.get_instance().get_uma_footprint_mb()
