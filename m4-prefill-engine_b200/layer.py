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
    u32, pp = ctypes.c_uint32, ctypes.POINTER(ctypes.c_void_p)
    lib.b200_peer_alloc.argtypes = [ctypes.c_size_t, pp, ctypes.c_char_p]
    lib.b200_peer_open.argtypes = [ctypes.c_char_p, pp]
    lib.b200_peer_close.argtypes = [vp]
    lib.b200_peer_free.argtypes = [vp]
    lib.b200_layer_set_peer_exchange.argtypes = [vp, u32, u32, pp, pp, pp, pp]
    lib.b200_peer_gemm_scatter.argtypes = [vp, vp, ctypes.c_int, u32, u32, u32, u32, u32, pp, pp, u32]
    lib.b200_peer_reduce_broadcast.argtypes = [u32, u32, pp, pp, pp, u32, vp, u32, u32]
    lib.b200_peer_wait_rows.argtypes = [u32, u32, pp, u32]
    lib.b200_peer_reduce_norm_broadcast.argtypes = [u32, u32, pp, pp, pp, u32, vp, u32, u32, vp, ctypes.c_float, vp]
    lib.b200_peer_reduce_norm_broadcast.restype = ctypes.c_int
    lib.b200_peer_exchange_create.argtypes = [u32, u32, pp, pp, pp, pp, ctypes.c_int]
    lib.b200_peer_exchange_create.restype = vp
    lib.b200_peer_exchange_destroy.argtypes = [vp]
    lib.b200_peer_exchange_destroy.restype = None
    lib.b200_layer_attach_peer_exchange.argtypes = [vp, vp]
    lib.b200_layer_set_profiling.argtypes = [vp, ctypes.c_int]
    lib.b200_layer_set_fused_kv_epilogue.argtypes = [vp, ctypes.c_int]
    lib.b200_layer_set_fused_kv_epilogue.restype = ctypes.c_int
    lib.b200_layer_profile.argtypes = [vp, ctypes.c_char_p, ctypes.c_size_t, ctypes.POINTER(ctypes.c_float), ctypes.c_size_t]
    for f in ("b200_peer_alloc", "b200_peer_open", "b200_peer_close", "b200_peer_free", "b200_layer_set_peer_exchange",
              "b200_peer_gemm_scatter", "b200_peer_reduce_broadcast", "b200_peer_wait_rows", "b200_layer_attach_peer_exchange",
              "b200_layer_set_profiling", "b200_layer_profile"):
        getattr(lib, f).restype = ctypes.c_int
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

    def set_peer_exchange(self, rank: int, world: int, recv: list, out0: list, out1: list, flags: list) -> None:
        """Lists of `world` device addresses indexed by rank (this rank's own buffers and the mapped buffers of the
        others); see ``PeerExchange.setup`` for the usual way to get them."""
        arr = lambda xs: (ctypes.c_void_p * world)(*xs)
        rc = self.lib.b200_layer_set_peer_exchange(self._h, rank, world, arr(recv), arr(out0), arr(out1), arr(flags))
        if rc:
            raise RuntimeError(f"b200_layer_set_peer_exchange failed with status code {rc} "
                               "(needs tp_size == world and M / world a multiple of 256)")

    def attach_peer_exchange(self, px: "PeerExchange") -> None:
        """Use an exchange that other layers use as well (the layers of a model take turns on one set of buffers)."""
        rc = self.lib.b200_layer_attach_peer_exchange(self._h, px.handle)
        if rc:
            raise RuntimeError(f"b200_layer_attach_peer_exchange failed with status code {rc} "
                               "(needs tp_size == world and M / world a multiple of 256)")

    def set_fused_kv_epilogue(self, on: bool) -> None:
        """Rotary embedding and Q8_0 K/V compression inside the Q/K/V projection's epilogue (default) or as separate
        kernels behind it; the layer's output is the same bit for bit."""
        self.lib.b200_layer_set_fused_kv_epilogue(self._h, int(on))

    def profile_forward(self, *tensors) -> list:
        """A forward with a CUDA event after every launch: [(what ran, microseconds), ...] in launch order.  Two forwards
        run back to back and the second one is reported: in a tensor-parallel group the first one's exchanges bring the
        ranks into step, so the second one's waits show the exchange itself rather than the ranks' start-up skew."""
        self.lib.b200_layer_set_profiling(self._h, 1)
        try:
            self.forward(*tensors)
            self.forward(*tensors)
            cap, lb = 64, 96
            labels = ctypes.create_string_buffer(cap * lb)
            us = (ctypes.c_float * cap)()
            n = self.lib.b200_layer_profile(self._h, labels, lb, us, cap)
        finally:
            self.lib.b200_layer_set_profiling(self._h, 0)
        if n < 0:
            raise RuntimeError(f"b200_layer_profile failed with status code {n}")
        raw = labels.raw
        return [(raw[i * lb:(i + 1) * lb].split(b"\0", 1)[0].decode(), round(float(us[i]), 2)) for i in range(n)]

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


class PeerExchange:
    """Buffers of the tensor-parallel reduction over peer memory (one instance per rank and layer shape, shared by
    every layer of that shape: the epoch counter lives with the buffers): this rank's receive buffer, two result
    buffers and flag words, allocated so that the other processes of the node can map them, plus the mappings of every
    other rank's buffers.  Handles travel through torch.distributed (any backend)."""

    KINDS = ("recv", "out0", "out1", "flags")

    def __init__(self, bridge: B200Bridge, M: int, K: int, rank: int, world: int, partial_fp16: Optional[bool] = None) -> None:
        self.bridge, self.rank, self.world = bridge, rank, world
        # Partial sums cross NVLink as fp16 by default (the exchange is bound by NVLink bytes at 4 and 8 ranks); fp32
        # with B200_EXCHANGE_FP32=1 or partial_fp16=False.  Every rank of a group must choose the same.
        if partial_fp16 is None:
            import os
            partial_fp16 = os.environ.get("B200_EXCHANGE_FP32", "0") != "1"
        self.partial_fp16 = bool(partial_fp16)
        _bind_layer(bridge.lib)
        self.sizes = {"recv": M * K * 4, "out0": M * K * 2, "out1": M * K * 2, "flags": 64}
        self.own: dict = {}
        self.handles: dict = {}
        self.ptrs: dict = {k: [0] * world for k in self.KINDS}
        self._opened: list = []
        self.handle = None
        for kind in self.KINDS:
            p = ctypes.c_void_p()
            h = ctypes.create_string_buffer(64)
            rc = bridge.lib.b200_peer_alloc(self.sizes[kind], ctypes.byref(p), h)
            if rc:
                raise RuntimeError(f"b200_peer_alloc failed with status code {rc}")
            self.own[kind] = p.value
            self.handles[kind] = h.raw
            self.ptrs[kind][rank] = p.value

    def connect(self, all_handles: list) -> None:
        """all_handles[r] = the ``handles`` dict of rank r (e.g. from dist.all_gather_object)."""
        for r, hs in enumerate(all_handles):
            if r == self.rank:
                continue
            for kind in self.KINDS:
                p = ctypes.c_void_p()
                rc = self.bridge.lib.b200_peer_open(hs[kind], ctypes.byref(p))
                if rc:
                    raise RuntimeError(f"b200_peer_open failed with status code {rc}: " +
                                       (self.bridge.lib.b200_bridge_last_error_string() or b"").decode())
                self.ptrs[kind][r] = p.value
                self._opened.append(p.value)
        arr = lambda xs: (ctypes.c_void_p * self.world)(*xs)
        self.handle = self.bridge.lib.b200_peer_exchange_create(self.rank, self.world, arr(self.ptrs["recv"]), arr(self.ptrs["out0"]),
                                                                arr(self.ptrs["out1"]), arr(self.ptrs["flags"]), int(self.partial_fp16))
        if not self.handle:
            raise RuntimeError("b200_peer_exchange_create failed")

    @classmethod
    def setup(cls, layer: "TransformerLayerCoordinator", group=None) -> Optional["PeerExchange"]:
        """Allocate, exchange handles over `group` and attach to `layer` (collective: every rank calls it).  Returns
        None on every rank when any rank could not allocate, map a peer's buffers or attach them (the ranks agree
        through one all-gather), so that the group can fall back to ``set_allreduce`` together."""
        import torch.distributed as dist
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        px, err = None, None
        try:
            px = cls(layer.bridge, layer.config.M, layer.config.K, rank, world)
        except Exception as e:                      # noqa: BLE001 - reported to the group below
            err = repr(e)
        gathered: list = [None] * world
        dist.all_gather_object(gathered, None if err else px.handles, group=group)
        if err is None and all(h is not None for h in gathered):
            try:
                px.connect(gathered)
                layer.attach_peer_exchange(px)
            except Exception as e:                  # noqa: BLE001
                err = repr(e)
        else:
            err = err or "another rank failed to allocate"
        status: list = [None] * world
        dist.all_gather_object(status, err, group=group)
        if any(s is not None for s in status):
            if px is not None:
                px.close()
            return None
        return px

    def result_tensor(self, M: int, K: int) -> torch.Tensor:
        """This rank's copy of the exchange's second result buffer as an fp16 [M, K] tensor (no copy).  Passed to
        ``forward`` as X_out it receives the layer's output directly from the owners' reductions; any other X_out costs
        one device-to-device copy at the end of the layer.  Valid until ``close``."""
        class _Raw:
            __cuda_array_interface__ = {"shape": (M, K), "typestr": "<f2", "data": (self.own["out1"], False), "version": 3}
        return torch.as_tensor(_Raw(), device="cuda")

    def close(self) -> None:
        if self.handle:
            self.bridge.lib.b200_peer_exchange_destroy(self.handle)
            self.handle = None
        for p in self._opened:
            self.bridge.lib.b200_peer_close(p)
        self._opened = []
        for p in self.own.values():
            self.bridge.lib.b200_peer_free(p)
        self.own = {}


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


def shard_rows_any(W: np.ndarray, fmt, K: int, N: int, rank: int, tp: int) -> np.ndarray:
    """Column split of Y = X.W^T for every layout the projection accepts, the planar extension layouts included
    (formats 100 and 102: nibble plane, scale plane, bias plane; format 101: 2-bit plane, one scale per row): each plane
    is an [N][x] matrix and keeps rows [rank*N/tp, (rank+1)*N/tp); the planes of format 102 start on 16-byte boundaries.  This is how the N-sharded ternary projection of the
    benchmark (K=4096, N=14336 over 1/2/4/8 GPUs) is cut; no collective follows it."""
    fmt = int(fmt)
    n_loc = N // tp
    if fmt == 100:
        planes = [N * K // 2, N * (K // 64) * 2, N * (K // 64) * 2]
    elif fmt == 101:
        planes = [N * K // 4, N * 2]
    elif fmt == 102:
        planes = [N * K // 2, N * (K // 32) * 2, N * (K // 32) * 2]
    elif fmt == 7:
        planes = [N * (K // 128) * 34]
    else:
        return shard_rows(W, fmt, K, N, rank, tp)
    pad = 16 if fmt == 102 else 1
    out, at = [], 0
    for nbytes in planes:
        at = (at + pad - 1) // pad * pad
        part = np.ascontiguousarray(W[at:at + nbytes].reshape(N, -1)[rank * n_loc:(rank + 1) * n_loc]).reshape(-1)
        have = sum(len(x) for x in out)
        out.append(np.zeros((have + pad - 1) // pad * pad - have, np.uint8))
        out.append(part)
        at += nbytes
    return np.concatenate(out)


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
