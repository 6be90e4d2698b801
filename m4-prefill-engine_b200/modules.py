"""Linear-layer wrapper and format tables above the bridge.

Mirrors the parts of the reference's ``src/engine/modules.py`` that call the bridge:
``FORMAT_SPECS`` (:38-81), ``normalize_format`` (:84-99), ``compute_quantized_weight_bytes``
(:102-113), the unit-pattern branch of ``generate_synthetic_quantized_weights`` (:115-199, used by
the reference's known-answer tests) and ``M4QuantizedLinear`` (:290-429) with the same argument
checks and error types.  Tensors are ``torch`` tensors; outputs are allocated on the input's device.
"""
from __future__ import annotations

from typing import Optional, Union

import numpy as np
import torch

from .bridge import B200Bridge, QuantFormat, m4_bridge_dispatch_gemm, m4_bridge_dispatch_gemv, m4_bridge_init, m4_bridge_synchronize


def _spec(name, block, size, bpw, sup):
    return {"name": name, "block_size": block, "struct_size": size, "bits_per_weight": bpw, "is_super_block": sup}


FORMAT_SPECS = {
    QuantFormat.QUANT_Q4_0: _spec("QUANT_Q4_0", 32, 18, 4.5, False),
    QuantFormat.QUANT_MLX_4BIT: _spec("QUANT_MLX_4BIT", 32, 20, 5.0, False),
    QuantFormat.QUANT_Q4_K: _spec("QUANT_Q4_K", 256, 144, 4.5, True),
    QuantFormat.QUANT_TERNARY_1_58: _spec("QUANT_TERNARY_1_58", 32, 12, 3.0, False),
    QuantFormat.QUANT_VAR_RATE_AFFINE: _spec("QUANT_VAR_RATE_AFFINE", 256, 160, 5.0, True),
    QuantFormat.QUANT_EXL3: _spec("QUANT_EXL3", 256, 144, 4.5, True),
}


def normalize_format(format_val: Union[int, QuantFormat, str]) -> QuantFormat:
    if isinstance(format_val, QuantFormat):
        return format_val
    if isinstance(format_val, (int, np.integer)):
        return QuantFormat(int(format_val))
    if isinstance(format_val, str):
        key = format_val.upper().strip()
        if not key.startswith("QUANT_"):
            key = "QUANT_" + key
        for qf in QuantFormat:
            if qf.name == key:
                return qf
        raise ValueError(f"Unknown quantization format string: '{format_val}'")
    raise TypeError(f"Invalid format type: {type(format_val)}")


def compute_quantized_weight_bytes(format_val, in_features: int, out_features: int) -> int:
    if in_features <= 0 or out_features <= 0:
        raise ValueError(f"in_features ({in_features}) and out_features ({out_features}) must be positive integers > 0")
    fmt = normalize_format(format_val)
    spec = FORMAT_SPECS[fmt]
    if in_features % spec["block_size"] != 0:
        raise ValueError(f"in_features ({in_features}) must be divisible by {spec['block_size']} for {fmt.name}")
    return (in_features // spec["block_size"]) * out_features * spec["struct_size"]


def unit_weights(format_val, in_features: int, out_features: int, scale: float = 1.0) -> torch.Tensor:
    """The reference's unit pattern: every weight dequantises to `scale` (Q4_0 nibble 9, MLX nibble 1
    with zero bias, ternary code 2, Q4_K with d = scale, sub-scale 1, minimum 0 and nibble 1), so an
    all-ones input gives Y == K * scale.  The two codebook super-block formats only get a header scale."""
    fmt = normalize_format(format_val)
    spec = FORMAT_SPECS[fmt]
    nb = (in_features // spec["block_size"]) * out_features
    raw = np.zeros((nb, spec["struct_size"]), dtype=np.uint8)
    s = np.frombuffer(np.float16(scale).tobytes(), dtype=np.uint8)
    if fmt == QuantFormat.QUANT_Q4_0:
        raw[:, 0:2] = s
        raw[:, 2:18] = 0x99
    elif fmt == QuantFormat.QUANT_MLX_4BIT:
        raw[:, 0:2] = s
        raw[:, 4:20] = 0x11
    elif fmt == QuantFormat.QUANT_TERNARY_1_58:
        raw[:, 0:2] = s
        raw[:, 4:12] = 0xAA
    elif fmt == QuantFormat.QUANT_Q4_K:
        raw[:, 0:2] = s                 # d = scale, sub-scale 1, minimum 0, nibble 1
        raw[:, 4:12] = 1
        raw[:, 16:144] = 0x11
    else:
        raw[:, 0:2] = s
    return torch.from_numpy(raw.reshape(-1))


class M4QuantizedLinear(torch.nn.Module):
    """Quantised linear layer over the bridge (reference: src/engine/modules.py:290-429).

    ``forward`` accepts any number of leading dimensions, casts to fp16, returns zeros-shaped
    empties for zero-length inputs without touching the bridge, sends a single row through the
    GEMV entry point and everything else through the GEMM entry point.
    """

    def __init__(self, in_features: int, out_features: int, format=QuantFormat.QUANT_Q4_0,
                 weight: Optional[torch.Tensor] = None, device: Optional[Union[str, torch.device]] = None) -> None:
        super().__init__()
        self.in_features = int(in_features)
        self.out_features = int(out_features)
        self.format = normalize_format(format)
        if self.format not in FORMAT_SPECS:
            raise ValueError(f"format {self.format.name} is not served by the bridge's GEMM entry points")
        self.spec = FORMAT_SPECS[self.format]
        if self.in_features <= 0 or self.out_features <= 0:
            raise ValueError(
                f"in_features ({self.in_features}) and out_features ({self.out_features}) must be positive integers > 0")
        if self.in_features % self.spec["block_size"] != 0:
            raise ValueError(
                f"in_features={self.in_features} must be divisible by {self.spec['block_size']} for format {self.format.name}")
        if self.spec["is_super_block"] and self.in_features % 256 != 0:
            raise ValueError(f"Super-block format {self.format.name} requires in_features ({self.in_features}) % 256 == 0")
        expected = compute_quantized_weight_bytes(self.format, self.in_features, self.out_features)
        dev = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        if weight is None:
            weight = torch.zeros(expected, dtype=torch.uint8, device=dev)
        else:
            if not isinstance(weight, torch.Tensor):
                weight = torch.as_tensor(np.frombuffer(bytes(weight), dtype=np.uint8).copy()
                                         if isinstance(weight, (bytes, bytearray)) else np.asarray(weight))
            nbytes = weight.numel() * weight.element_size()
            if nbytes != expected:
                raise ValueError(
                    f"Weight buffer size mismatch for {self.format.name}: expected {expected} bytes, got {nbytes} bytes")
            weight = weight.contiguous().view(torch.uint8).reshape(-1).to(dev)
        self.register_buffer("weight", weight, persistent=True)
        if not B200Bridge.get_instance().is_initialized():
            if not m4_bridge_init():
                raise RuntimeError("bridge initialisation failed: " +
                                   (B200Bridge.get_instance().lib.b200_bridge_last_error_string() or b"").decode())

    @classmethod
    def from_quantized(cls, weights, format, in_features: int, out_features: int, device=None) -> "M4QuantizedLinear":
        return cls(in_features, out_features, format=format, weight=weights, device=device)

    def init_synthetic_weights(self, scale: float = 1.0) -> None:
        self.weight = unit_weights(self.format, self.in_features, self.out_features, scale).to(self.weight.device)

    def forward(self, x: torch.Tensor, check_finite: bool = False) -> torch.Tensor:
        if x.dim() < 1:
            raise ValueError(f"Input tensor must have at least 1 dimension, got ndim={x.dim()} with shape {tuple(x.shape)}")
        K, N = self.in_features, self.out_features
        if x.shape[-1] != K:
            raise ValueError(f"Input feature dimension {x.shape[-1]} does not match layer in_features {K}")
        dev = self.weight.device
        if x.numel() == 0:
            return torch.zeros((*x.shape[:-1], N), dtype=torch.float16, device=dev)
        if x.dtype != torch.float16:
            x = x.to(torch.float16)
        x = x.to(dev)
        if x.dim() == 1:
            y = torch.zeros((N,), dtype=torch.float16, device=dev)
            m4_bridge_dispatch_gemv(x, self.weight, y, self.format, K, N, check_finite=check_finite)
            m4_bridge_synchronize()
            return y
        x2 = x.reshape(-1, K)
        m = x2.shape[0]
        y2 = torch.zeros((m, N), dtype=torch.float16, device=dev)
        if m == 1:
            m4_bridge_dispatch_gemv(x2, self.weight, y2, self.format, K, N, check_finite=check_finite)
        else:
            m4_bridge_dispatch_gemm(x2, self.weight, y2, self.format, m, K, N, check_finite=check_finite)
        # the result is handed back to torch code that runs on another stream: wait here
        m4_bridge_synchronize()
        return y2.reshape(*x.shape[:-1], N)
