"""Decoder layer over the C ABI, single GPU or tensor parallel.

``TransformerLayerConfig`` / ``TransformerLayerCoordinator`` mirror ``models/transformer_layer.h``
(:12-47) of the reference; the coordinator here is a thin handle on the C++ class of the same name
in the shared library.  ``shard_layer_weights`` cuts whole-model weights into the column / row
shards of one tensor-parallel rank, and ``torch_allreduce_hook`` provides the sum-reduction the
row-split projections need through ``torch.distributed`` (NCCL on GPUs).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Callable, Optional

import numpy as np
import torch

from .bridge import B200Bridge, QuantFormat
from .modules import FORMAT_SPECS, normalize_format


@dataclass
class TransformerLayerConfig:
    M: int = 128
    K: int = 2048
    H: int = 32
    D: int = 64
    N_mlp: int = 8192
    attn_scale: float = 0.125
    weight_format: int = int(QuantFormat.QUANT_Q4_0)
    num_kv_heads: int = 0
    rms_eps: float = 0.0
    rope_theta: float = 0.0
    kv_q8_0: bool = False
    tp_size: int = 1


class _CConfig(ctypes.Structure):
    _fields_ = [("M", ctypes.c_uint32), ("K", ctypes.c_uint32), ("H", ctypes.c_uint32), ("D", ctypes.c_uint32),
                ("N_mlp", ctypes.c_uint32), ("attn_scale", ctypes.c_float), ("weight_format", ctypes.c_int),
                ("num_kv_heads", ctypes.c_uint32), ("rms_eps", ctypes.c_float), ("rope_theta", ctypes.c_float),
                ("kv_q8_0", ctypes.c_int), ("tp_size", ctypes.c_uint32)]


_ALLREDUCE_CB = ctypes.CFUNCTYPE(None, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t)


def _bind_layer(lib) -> None:
    if getattr(lib, "_layer_bound", False):
        return
    vp = ctypes.c_void_p
    lib.b200_layer_create.argtypes = [ctypes.POINTER(_CConfig)]
    lib.b200_layer_create.restype = vp
    lib.b200_layer_destroy.argtypes = [vp]
    lib.b200_layer_destroy.restype = None
    lib.b200_layer_set_norm_weights.argtypes = [vp, vp, vp]
    lib.b200_layer_set_norm_weights.restype = ctypes.c_int
    lib.b200_layer_set_allreduce.argtypes = [vp, _ALLREDUCE_CB, vp]
    lib.b200_layer_set_allreduce.restype = ctypes.c_int
    lib.b200_layer_forward.argtypes = [vp] * 10
    lib.b200_layer_forward.restype = ctypes.c_int
    lib.b200_layer_kernels_per_forward.argtypes = [vp]
    lib.b200_layer_kernels_per_forward.restype = ctypes.c_uint32
    lib._layer_bound = True


class TransformerLayerCoordinator:
    """Handle on the C++ coordinator.  ``forward`` only enqueues on the bridge stream; call
    ``bridge.synchronize()`` (or order your own stream after it) before reading the output."""

    def __init__(self, config: TransformerLayerConfig, bridge: Optional[B200Bridge] = None) -> None:
        self.bridge = bridge or B200Bridge.get_instance()
        if not self.bridge.is_initialized() and not self.bridge.init():
            raise RuntimeError("bridge initialisation failed")
        self.lib = self.bridge.lib
        _bind_layer(self.lib)
        self.config = config
        c = _CConfig(config.M, config.K, config.H, config.D, config.N_mlp, config.attn_scale, int(config.weight_format),
                     config.num_kv_heads, config.rms_eps, config.rope_theta, int(config.kv_q8_0), config.tp_size)
        self._h = self.lib.b200_layer_create(ctypes.byref(c))
        if not self._h:
            raise RuntimeError("b200_layer_create failed: " + (self.lib.b200_bridge_last_error_string() or b"").decode())
        self._keep: list = []
        self._cb = None

    def initialize_pipelines(self, library=None) -> bool:
        return bool(self._h)     # binding happens at creation; kept for the reference's call sequence

    def set_norm_weights(self, attn_norm: torch.Tensor, mlp_norm: torch.Tensor) -> None:
        self._keep = [attn_norm, mlp_norm]
        rc = self.lib.b200_layer_set_norm_weights(self._h, attn_norm.data_ptr(), mlp_norm.data_ptr())
        if rc:
            raise RuntimeError(f"b200_layer_set_norm_weights failed with status code {rc}")

    def set_allreduce(self, fn: Callable[[int, int], None]) -> None:
        """fn(device_pointer, count) must sum-reduce `count` fp32 values in place across ranks, ordered on
        the bridge stream."""
        def _cb(_ctx, buf, count):
            fn(int(buf), int(count))
        self._cb = _ALLREDUCE_CB(_cb)
        rc = self.lib.b200_layer_set_allreduce(self._h, self._cb, None)
        if rc:
            raise RuntimeError(f"b200_layer_set_allreduce failed with status code {rc}")

    def forward(self, X_in, W_q, W_k, W_v, W_o, W_gate, W_up, W_down, X_out) -> None:
        ts = (X_in, W_q, W_k, W_v, W_o, W_gate, W_up, W_down, X_out)
        if any(t.is_cuda for t in ts):
            torch.cuda.current_stream().synchronize()
        rc = self.lib.b200_layer_forward(self._h, *[t.data_ptr() for t in ts])
        if rc:
            raise RuntimeError(f"b200_layer_forward failed with status code {rc}")

    def kernels_per_forward(self) -> int:
        return int(self.lib.b200_layer_kernels_per_forward(self._h))

    def close(self) -> None:
        if self._h:
            self.lib.b200_layer_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def torch_allreduce_hook(bridge: B200Bridge, group=None) -> Callable[[int, int], None]:
    """All-reduce for ``set_allreduce`` built on torch.distributed: wraps the device buffer as a tensor
    without copying and reduces it on the bridge stream, so it is ordered between the layer's kernels."""
    import torch.distributed as dist

    stream = torch.cuda.ExternalStream(bridge.lib.b200_bridge_stream()) if torch.cuda.is_available() else None

    class _Raw:                       # __cuda_array_interface__ view of a raw device pointer
        def __init__(self, ptr, n):
            self.__cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (ptr, False), "version": 3}

    def hook(ptr: int, count: int) -> None:
        t = torch.as_tensor(_Raw(ptr, count), device="cuda")
        with torch.cuda.stream(stream):
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)

    return hook


# ---------------------------------------------------------------------------------------------
# tensor-parallel sharding of packed weights (host side, numpy; pure byte slicing)
# ---------------------------------------------------------------------------------------------
def shard_rows(W: np.ndarray, fmt, K: int, N: int, rank: int, tp: int) -> np.ndarray:
    """Column split of Y = X.W^T: rows [rank*N/tp, (rank+1)*N/tp) of the packed [N][K/blk] matrix."""
    spec = FORMAT_SPECS[normalize_format(fmt)]
    row_bytes = (K // spec["block_size"]) * spec["struct_size"]
    n_loc = N // tp
    return np.ascontiguousarray(W.reshape(N, row_bytes)[rank * n_loc:(rank + 1) * n_loc]).reshape(-1)


def shard_cols(W: np.ndarray, fmt, K: int, N: int, rank: int, tp: int) -> np.ndarray:
    """Row split of Y = X.W^T: input columns [rank*K/tp, (rank+1)*K/tp) of every row, i.e. a strided gather
    of whole blocks; K/tp must be a multiple of the block size."""
    spec = FORMAT_SPECS[normalize_format(fmt)]
    bs, ss = spec["block_size"], spec["struct_size"]
    k_loc = K // tp
    if k_loc % bs:
        raise ValueError(f"K/tp = {k_loc} is not a multiple of the block size {bs}")
    blocks = W.reshape(N, K // bs, ss)
    b_loc = k_loc // bs
    return np.ascontiguousarray(blocks[:, rank * b_loc:(rank + 1) * b_loc]).reshape(-1)


def shard_layer_weights(fmt, weights: dict, cfg: TransformerLayerConfig, rank: int, tp: int) -> dict:
    """weights: {'q','k','v','o','gate','up','down'} whole-model packed arrays -> this rank's shards."""
    hkv = cfg.num_kv_heads or cfg.H
    QD, KD = cfg.H * cfg.D, hkv * cfg.D
    return {
        "q": shard_rows(weights["q"], fmt, cfg.K, QD, rank, tp),
        "k": shard_rows(weights["k"], fmt, cfg.K, KD, rank, tp),
        "v": shard_rows(weights["v"], fmt, cfg.K, KD, rank, tp),
        "o": shard_cols(weights["o"], fmt, QD, cfg.K, rank, tp),
        "gate": shard_rows(weights["gate"], fmt, cfg.K, cfg.N_mlp, rank, tp),
        "up": shard_rows(weights["up"], fmt, cfg.K, cfg.N_mlp, rank, tp),
        "down": shard_cols(weights["down"], fmt, cfg.N_mlp, cfg.K, rank, tp),
    }
