"""GGUF ingest over the C surface of the shared library (``b200_gguf_*``).

``GGUFLoader`` and ``GGUFLayerStreamer`` follow the reference's classes of the same names
(``core/weights/gguf_loader.h:46-127``, ``core/weights/gguf_layer_streamer.h:36-95``): parse a GGUF v2/v3 file (memory
mapped) or an in-memory buffer, query metadata and the tensor directory, get tensor payloads without copying, extract
PrismML Q2_0 blocks, and serve a model layer by layer with a bounded number of layers resident -- resident in device
memory here.  ``write_gguf`` builds a container from numpy arrays (test fixtures, conversion scripts).
"""
from __future__ import annotations

import ctypes
import struct
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from .bridge import library_path

GGML_F32, GGML_F16, GGML_Q4_0, GGML_Q8_0, GGML_PRISM_Q2_0 = 0, 1, 2, 8, 100
_T_U32, _T_F32, _T_STRING, _T_U64 = 4, 6, 8, 10

_lib = None


def _load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    L = ctypes.CDLL(str(library_path()))
    vp, cp, u64, u32, i = ctypes.c_void_p, ctypes.c_char_p, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_int
    sig = {
        "b200_gguf_open": ([cp], vp), "b200_gguf_parse": ([vp, ctypes.c_size_t], vp), "b200_gguf_close": ([vp], None),
        "b200_gguf_error": ([], cp), "b200_gguf_version": ([vp], u32), "b200_gguf_alignment": ([vp], u32),
        "b200_gguf_data_offset": ([vp], u64), "b200_gguf_tensor_count": ([vp], u64), "b200_gguf_metadata_count": ([vp], u64),
        "b200_gguf_get_uint": ([vp, cp, ctypes.POINTER(u64)], i), "b200_gguf_get_string": ([vp, cp, cp, ctypes.c_size_t], i),
        "b200_gguf_tensor_name": ([vp, u64, cp, ctypes.c_size_t], i),
        "b200_gguf_tensor_info": ([vp, cp, ctypes.POINTER(u32), ctypes.POINTER(u64), ctypes.POINTER(u32), ctypes.POINTER(u64),
                                   ctypes.POINTER(u64)], i),
        "b200_gguf_tensor_data": ([vp, cp], vp), "b200_gguf_tensor_format": ([vp, cp], i),
        "b200_gguf_extract_prism_q2_0": ([vp, cp, vp, u64, ctypes.POINTER(u64), ctypes.POINTER(u64)], ctypes.c_int64),
        "b200_gguf_streamer_open": ([cp, u64, i], vp), "b200_gguf_streamer_close": ([vp], None),
        "b200_gguf_streamer_acquire": ([vp, i], i), "b200_gguf_streamer_is_resident": ([vp, i], i),
        "b200_gguf_streamer_tensor": ([vp, cp], vp), "b200_gguf_streamer_stat": ([vp, i], u64),
        "b200_gguf_parse_layer_index": ([cp], i),
    }
    for name, (args, res) in sig.items():
        fn = getattr(L, name)
        fn.argtypes, fn.restype = args, res
    _lib = L
    return L


class GGUFLoader:
    def __init__(self) -> None:
        self._h = None
        self._buf = None           # keeps an in-memory buffer alive while it is parsed in place

    def open(self, path: str) -> bool:
        self.close()
        self._h = _load().b200_gguf_open(str(path).encode())
        return bool(self._h)

    def parse_from_buffer(self, data: bytes) -> bool:
        self.close()
        self._buf = ctypes.create_string_buffer(bytes(data), len(data))
        self._h = _load().b200_gguf_parse(ctypes.addressof(self._buf), len(data))
        if not self._h:
            self._buf = None
        return bool(self._h)

    def close(self) -> None:
        if self._h:
            _load().b200_gguf_close(self._h)
        self._h, self._buf = None, None

    @staticmethod
    def last_error() -> str:
        return (_load().b200_gguf_error() or b"").decode()

    def is_open(self) -> bool:
        return bool(self._h)

    def version(self) -> int:
        return int(_load().b200_gguf_version(self._h))

    def alignment(self) -> int:
        return int(_load().b200_gguf_alignment(self._h))

    def tensor_data_offset(self) -> int:
        return int(_load().b200_gguf_data_offset(self._h))

    def tensor_count(self) -> int:
        return int(_load().b200_gguf_tensor_count(self._h))

    def metadata_count(self) -> int:
        return int(_load().b200_gguf_metadata_count(self._h))

    def get_uint_metadata(self, key: str, default: int = 0) -> int:
        v = ctypes.c_uint64()
        return int(v.value) if _load().b200_gguf_get_uint(self._h, key.encode(), ctypes.byref(v)) else default

    def has_metadata(self, key: str) -> bool:
        v = ctypes.c_uint64()
        buf = ctypes.create_string_buffer(8)
        return bool(_load().b200_gguf_get_uint(self._h, key.encode(), ctypes.byref(v)) or
                    _load().b200_gguf_get_string(self._h, key.encode(), buf, 8))

    def get_string_metadata(self, key: str, default: str = "") -> str:
        buf = ctypes.create_string_buffer(4096)
        return buf.value.decode() if _load().b200_gguf_get_string(self._h, key.encode(), buf, 4096) else default

    def tensor_names(self) -> List[str]:
        out, buf = [], ctypes.create_string_buffer(1024)
        for i in range(self.tensor_count()):
            if _load().b200_gguf_tensor_name(self._h, i, buf, 1024):
                out.append(buf.value.decode())
        return out

    def has_tensor(self, name: str) -> bool:
        return self.get_tensor_info(name) is not None

    def get_tensor_info(self, name: str) -> Optional[dict]:
        nd, ty, off, nb = ctypes.c_uint32(), ctypes.c_uint32(), ctypes.c_uint64(), ctypes.c_uint64()
        dims = (ctypes.c_uint64 * 4)()
        if not _load().b200_gguf_tensor_info(self._h, name.encode(), ctypes.byref(nd), dims, ctypes.byref(ty), ctypes.byref(off), ctypes.byref(nb)):
            return None
        return {"name": name, "n_dims": nd.value, "dims": [int(d) for d in dims][:nd.value], "type": ty.value,
                "file_offset": int(off.value), "size_bytes": int(nb.value), "format": int(_load().b200_gguf_tensor_format(self._h, name.encode()))}

    def get_tensor_raw_data(self, name: str) -> Optional[np.ndarray]:
        """Zero-copy uint8 view of the tensor's payload inside the mapping (valid while the loader is open)."""
        info = self.get_tensor_info(name)
        p = _load().b200_gguf_tensor_data(self._h, name.encode()) if info else None
        if not p:
            return None
        return np.ctypeslib.as_array((ctypes.c_uint8 * info["size_bytes"]).from_address(p))

    def extract_q2_0_tensor(self, name: str) -> Optional[Tuple[np.ndarray, int, int]]:
        """(blocks [n, 34] uint8, K, N) of a PrismML Q2_0 tensor, or None where the reference's extractor refuses."""
        info = self.get_tensor_info(name)
        if info is None or not info["dims"]:
            return None
        n_el = int(np.prod([int(d) for d in info["dims"]], dtype=np.uint64))
        cap = max(1, n_el // 128)
        out = np.empty((cap, 34), np.uint8)
        K, N = ctypes.c_uint64(), ctypes.c_uint64()
        n = _load().b200_gguf_extract_prism_q2_0(self._h, name.encode(), out.ctypes.data, cap, ctypes.byref(K), ctypes.byref(N))
        return None if n < 0 else (out[:n], int(K.value), int(N.value))

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class GGUFLayerStreamer:
    """Layer-by-layer weight serving with at most `resident_layer_count` layers in device memory (upload=False keeps the
    bytes on the host: directory and accounting only)."""

    def __init__(self) -> None:
        self._h = None

    def open(self, path: str, resident_layer_count: int = 2, upload: bool = True) -> bool:
        self.close()
        self._h = _load().b200_gguf_streamer_open(str(path).encode(), int(resident_layer_count), int(upload))
        return bool(self._h)

    def close(self) -> None:
        if self._h:
            _load().b200_gguf_streamer_close(self._h)
        self._h = None

    def acquire_layer(self, layer: int) -> bool:
        return bool(_load().b200_gguf_streamer_acquire(self._h, int(layer)))

    def is_resident(self, layer: int) -> bool:
        return bool(_load().b200_gguf_streamer_is_resident(self._h, int(layer)))

    def tensor_data(self, name: str) -> Optional[int]:
        """Device address (host address with upload=False) of a tensor of a resident layer, else None."""
        p = _load().b200_gguf_streamer_tensor(self._h, name.encode())
        return int(p) if p else None

    def _stat(self, what: int) -> int:
        return int(_load().b200_gguf_streamer_stat(self._h, what))

    def current_resident_bytes(self) -> int:
        return self._stat(0)

    def peak_resident_bytes(self) -> int:
        return self._stat(1)

    def total_model_bytes(self) -> int:
        return self._stat(2)

    def shared_bytes(self) -> int:
        return self._stat(3)

    def num_layers(self) -> int:
        return self._stat(4)

    @staticmethod
    def parse_layer_index(name: str) -> int:
        return int(_load().b200_gguf_parse_layer_index(name.encode()))

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def write_gguf(tensors: Sequence[Tuple[str, Sequence[int], int, np.ndarray]], metadata: Optional[Dict[str, object]] = None,
               alignment: int = 32, version: int = 3) -> bytes:
    """Serialise a GGUF container.  tensors: (name, dims with dims[0] the contiguous dimension, ggml type id, payload as a
    uint8 array); metadata values: int (UINT32, or UINT64 above 2**32), float (FLOAT32) or str."""
    def s(x: str) -> bytes:
        b = x.encode()
        return struct.pack("<Q", len(b)) + b
    meta = dict(metadata or {})
    meta.setdefault("general.alignment", int(alignment))
    out = bytearray(b"GGUF" + struct.pack("<IQQ", version, len(tensors), len(meta)))
    for k, v in meta.items():
        out += s(k)
        if isinstance(v, str):
            out += struct.pack("<I", _T_STRING) + s(v)
        elif isinstance(v, float):
            out += struct.pack("<If", _T_F32, v)
        elif int(v) >= 2 ** 32:
            out += struct.pack("<IQ", _T_U64, int(v))
        else:
            out += struct.pack("<II", _T_U32, int(v))
    offsets, at = [], 0
    for _, _, _, payload in tensors:
        offsets.append(at)
        at = (at + int(payload.size) + alignment - 1) // alignment * alignment
    for (name, dims, ty, _), off in zip(tensors, offsets):
        out += s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", int(d)) for d in dims) + struct.pack("<IQ", ty, off)
    out += b"\0" * ((len(out) + alignment - 1) // alignment * alignment - len(out))
    base = len(out)
    for (_, _, _, payload), off in zip(tensors, offsets):
        out += b"\0" * (base + off - len(out))
        out += np.ascontiguousarray(payload, dtype=np.uint8).tobytes()
    return bytes(out)
