"""B200-native prefill hot path behind the reference's bridge / registry / layer surfaces.

The directory name is not a Python identifier; load it with
``__graft_entry__.load_package()`` (registers it as ``m4_prefill_engine_b200``).

* ``bridge``   -- ctypes wrapper over ``libb200_bridge.so`` mirroring the reference's
  ``core/bridge/m4_bridge.py`` (class ``MetalUMABridge`` and the ``m4_bridge_*`` functions),
  taking ``torch`` tensors (device or host) in place of ``mlx`` arrays.
* ``modules``  -- ``FORMAT_SPECS``, ``M4QuantizedLinear`` and helpers mirroring
  ``src/engine/modules.py``.
* ``layer``    -- the decoder layer (``TransformerLayerConfig`` / ``TransformerLayerCoordinator``
  of ``models/transformer_layer.h``) including its tensor-parallel form.

There is no CPU fallback: importing works anywhere, but every compute call raises unless the
CUDA library is built and a B200 is present.
"""
from .bridge import (  # noqa: F401
    B200Bridge,
    MetalUMABridge,
    QuantFormat,
    library_path,
    m4_bridge_dispatch_gemm,
    m4_bridge_dispatch_gemv,
    m4_bridge_get_uma_footprint_mb,
    m4_bridge_init,
    m4_bridge_synchronize,
)

__all__ = [
    "B200Bridge", "MetalUMABridge", "QuantFormat", "library_path", "m4_bridge_init", "m4_bridge_dispatch_gemm",
    "m4_bridge_dispatch_gemv", "m4_bridge_synchronize", "m4_bridge_get_uma_footprint_mb",
]
