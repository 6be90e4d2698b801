"""Multi-layer model over the C ABI: token embedding, L decoder layers, final RMSNorm, lm_head.

``EngineConfig`` and ``TransformerModel`` mirror ``src/engine/config.py:13-95`` and
``src/engine/model.py:273-368`` of the reference (same field names, same checks and error types, an
``IndexError`` for token ids outside the vocabulary, ``init_synthetic_weights`` for runs without weight
files); the loop itself runs inside the shared library (``b200_model_*``), one stream, no host
synchronisation between layers.  ``forward`` is the stateless prefill (the reference's
``use_cache=False`` path: rotary positions from 0, keys and values of this call only).
"""
from __future__ import annotations

import ctypes
import math
import statistics
from dataclasses import dataclass
from typing import List, Optional, Union

import numpy as np
import torch

from .bridge import B200Bridge, QuantFormat
from .layer import PeerExchange, _CConfig, _bind_layer, torch_allreduce_hook, _ALLREDUCE_CB
from .modules import FORMAT_SPECS, compute_quantized_weight_bytes, normalize_format


@dataclass
class EngineConfig:
    num_layers: int = 4
    hidden_dim: int = 512
    num_q_heads: int = 8
    num_kv_heads: int = 2
    head_dim: int = 64
    intermediate_dim: int = 1024
    vocab_size: int = 1024
    rope_theta: float = 10000.0
    activation: str = "swiglu"
    norm_type: str = "rmsnorm"
    weight_format: Union[int, QuantFormat, str] = 0
    max_context_length: int = 2048
    norm_eps: float = 1e-5
    kv_q8_0: bool = True          # keys and values compressed to Q8_0 before attention (the engine's KV cache format)
    tp_size: int = 1

    def __post_init__(self) -> None:
        for name in ("num_layers", "hidden_dim", "num_q_heads", "num_kv_heads", "head_dim", "intermediate_dim", "vocab_size",
                     "max_context_length"):
            if getattr(self, name) <= 0:
                raise ValueError(f"{name} must be > 0, got {getattr(self, name)}")
        if self.num_q_heads % self.num_kv_heads != 0:
            raise ValueError(f"num_q_heads ({self.num_q_heads}) must be divisible by num_kv_heads ({self.num_kv_heads}) for GQA/MHA")
        if self.norm_eps <= 0:
            raise ValueError(f"norm_eps must be positive, got {self.norm_eps}")
        if self.rope_theta <= 0:
            raise ValueError(f"rope_theta must be positive, got {self.rope_theta}")
        self.activation = self.activation.lower().strip()
        if self.activation != "swiglu":
            raise ValueError(f"Unsupported activation '{self.activation}': the fused gate/up kernel computes SwiGLU")
        self.norm_type = self.norm_type.lower().strip()
        if self.norm_type != "rmsnorm":
            raise ValueError(f"Unsupported norm_type '{self.norm_type}'. Must be 'rmsnorm'.")
        if self.head_dim not in (64, 128):
            raise ValueError(f"head_dim must be 64 or 128, got {self.head_dim}")
        self.weight_format = normalize_format(self.weight_format)

    @property
    def scale(self) -> float:
        return 1.0 / math.sqrt(self.head_dim)

    @property
    def q_dim(self) -> int:
        return self.num_q_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_kv_heads * self.head_dim


class _CModelConfig(ctypes.Structure):
    _fields_ = [("layer", _CConfig), ("num_layers", ctypes.c_uint32), ("vocab_size", ctypes.c_uint32)]


def _bind_model(lib) -> None:
    if getattr(lib, "_model_bound", False):
        return
    _bind_layer(lib)
    vp, u32, i = ctypes.c_void_p, ctypes.c_uint32, ctypes.c_int
    lib.b200_model_create.argtypes = [ctypes.POINTER(_CModelConfig)]
    lib.b200_model_create.restype = vp
    lib.b200_model_destroy.argtypes = [vp]
    lib.b200_model_destroy.restype = None
    lib.b200_model_set_embedding.argtypes = [vp, vp]
    lib.b200_model_set_layer.argtypes = [vp, u32] + [vp] * 9
    lib.b200_model_set_head.argtypes = [vp, vp, vp, u32]
    lib.b200_model_attach_peer_exchange.argtypes = [vp, vp]
    lib.b200_model_set_allreduce.argtypes = [vp, _ALLREDUCE_CB, vp]
    lib.b200_model_forward.argtypes = [vp, vp, u32, vp, vp]
    for f in ("b200_model_set_embedding", "b200_model_set_layer", "b200_model_set_head", "b200_model_attach_peer_exchange",
              "b200_model_set_allreduce", "b200_model_forward"):
        getattr(lib, f).restype = i
    lib.b200_model_kernels_per_forward.argtypes = [vp]
    lib.b200_model_kernels_per_forward.restype = u32
    lib._model_bound = True


LAYER_KEYS = ("q", "k", "v", "o", "gate", "up", "down")


class TransformerModel:
    """Prefill of a fixed number of tokens per call (``tokens_per_call``) through L decoder layers.

    Weights are ``torch.uint8`` tensors of packed blocks in ``config.weight_format`` (device tensors; for tensor
    parallelism this rank's shards, see ``layer.shard_layer_weights``), norms and the embedding table fp16."""

    def __init__(self, config: EngineConfig, tokens_per_call: int, bridge: Optional[B200Bridge] = None) -> None:
        self.config = config
        self.M = int(tokens_per_call)
        if self.M <= 0 or self.M > config.max_context_length:
            raise ValueError(f"tokens_per_call must be in (0, max_context_length], got {tokens_per_call}")
        self.bridge = bridge or B200Bridge.get_instance()
        if not self.bridge.is_initialized() and not self.bridge.init():
            raise RuntimeError("bridge initialisation failed")
        self.lib = self.bridge.lib
        _bind_model(self.lib)
        c = config
        lc = _CConfig(self.M, c.hidden_dim, c.num_q_heads, c.head_dim, c.intermediate_dim, c.scale, int(c.weight_format), c.num_kv_heads,
                      c.norm_eps, c.rope_theta, int(c.kv_q8_0), c.tp_size)
        mc = _CModelConfig(lc, c.num_layers, c.vocab_size)
        self._h = self.lib.b200_model_create(ctypes.byref(mc))
        if not self._h:
            raise RuntimeError("b200_model_create failed: " + (self.lib.b200_bridge_last_error_string() or b"").decode())
        self._keep: dict = {}
        self._cb = None
        self.vocab_rows = c.vocab_size // c.tp_size
        self.px: Optional[PeerExchange] = None

    # ---- weights ----
    def _rc(self, rc: int, what: str) -> None:
        if rc:
            raise RuntimeError(f"{what} failed with status code {rc}")

    def set_embedding(self, table: torch.Tensor) -> None:
        if table.dtype != torch.float16 or tuple(table.shape) != (self.config.vocab_size, self.config.hidden_dim):
            raise ValueError("embedding table must be fp16 [vocab_size, hidden_dim]")
        self._keep["emb"] = table
        self._rc(self.lib.b200_model_set_embedding(self._h, table.data_ptr()), "b200_model_set_embedding")

    def set_layer(self, index: int, weights: dict, attn_norm: torch.Tensor, mlp_norm: torch.Tensor) -> None:
        ts = [weights[k] for k in LAYER_KEYS] + [attn_norm, mlp_norm]
        self._keep[("layer", index)] = ts
        self._rc(self.lib.b200_model_set_layer(self._h, index, *[t.data_ptr() for t in ts]), "b200_model_set_layer")

    def set_head(self, final_norm: torch.Tensor, lm_head: torch.Tensor, vocab_rows: Optional[int] = None) -> None:
        rows = int(vocab_rows if vocab_rows is not None else self.vocab_rows)
        need = compute_quantized_weight_bytes(self.config.weight_format, self.config.hidden_dim, rows)
        if lm_head.numel() < need:
            raise ValueError(f"lm_head holds {lm_head.numel()} bytes, {need} needed for {rows} rows")
        self._keep["head"] = (final_norm, lm_head)
        self.vocab_rows = rows
        self._rc(self.lib.b200_model_set_head(self._h, final_norm.data_ptr(), lm_head.data_ptr(), rows), "b200_model_set_head")

    def init_synthetic_weights(self, seed: int = 42, scale_lo: float = 0.0003, scale_hi: float = 0.0033, rank: int = 0) -> None:
        """Random-init weights generated on the device (no weight files): Q4_0 blocks with uniform nibbles and fp16
        scales ~ U(scale_lo, scale_hi) (the range of the reference's layer bench, bench_8b_engine.mm:44-53), unit norm
        weights, embedding ~ N(0, 0.02) as in the reference's init_synthetic_weights (src/engine/model.py:330-333).
        Tensor-parallel ranks generate their own shards (seeded by rank)."""
        c = self.config
        if c.weight_format != QuantFormat.QUANT_Q4_0:
            raise ValueError("init_synthetic_weights generates Q4_0 blocks; pass packed weights for other formats")
        dev = torch.device("cuda")
        tp = c.tp_size
        gen = torch.Generator(device=dev); gen.manual_seed(seed)
        self.set_embedding((torch.randn(c.vocab_size, c.hidden_dim, device=dev, generator=gen) * 0.02).to(torch.float16))
        gw = torch.Generator(device=dev); gw.manual_seed(seed * 1000 + rank)

        def q4_0(rows: int, k: int) -> torch.Tensor:
            nb = rows * (k // 32)
            blocks = torch.randint(0, 256, (nb, 18), dtype=torch.uint8, device=dev, generator=gw)
            d = (torch.rand(nb, device=dev, generator=gw) * (scale_hi - scale_lo) + scale_lo).to(torch.float16)
            blocks[:, 0:2] = d.view(torch.uint8).reshape(nb, 2)
            return blocks.reshape(-1)
        ones = torch.ones(c.hidden_dim, dtype=torch.float16, device=dev)
        for l in range(c.num_layers):
            w = {"q": q4_0(c.q_dim // tp, c.hidden_dim), "k": q4_0(c.kv_dim // tp, c.hidden_dim), "v": q4_0(c.kv_dim // tp, c.hidden_dim),
                 "o": q4_0(c.hidden_dim, c.q_dim // tp), "gate": q4_0(c.intermediate_dim // tp, c.hidden_dim),
                 "up": q4_0(c.intermediate_dim // tp, c.hidden_dim), "down": q4_0(c.hidden_dim, c.intermediate_dim // tp)}
            self.set_layer(l, w, ones, ones)
        self.set_head(ones, q4_0(c.vocab_size // tp, c.hidden_dim), c.vocab_size // tp)

    # ---- tensor parallel ----
    def setup_tensor_parallel(self, group=None, prefer_peer: bool = True) -> str:
        """Collective over `group`: the fused exchange over peer memory where it is available (M / world a multiple of
        256 and peer mappings on every rank), else an NCCL all-reduce hook.  Returns "peer" or "nccl"."""
        import torch.distributed as dist
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        if prefer_peer and (self.M // world) % 256 == 0 and self.M % world == 0:
            px, err = None, None
            try:
                px = PeerExchange(self.bridge, self.M, self.config.hidden_dim, rank, world)
            except Exception as e:                      # noqa: BLE001 - agreed on with the group below
                err = repr(e)
            gathered: list = [None] * world
            dist.all_gather_object(gathered, None if err else px.handles, group=group)
            if err is None and all(h is not None for h in gathered):
                try:
                    px.connect(gathered)
                    if self.lib.b200_model_attach_peer_exchange(self._h, px.handle):
                        err = "attach failed"
                except Exception as e:                  # noqa: BLE001
                    err = repr(e)
            else:
                err = err or "another rank failed"
            status: list = [None] * world
            dist.all_gather_object(status, err, group=group)
            if not any(s is not None for s in status):
                self.px = px
                return "peer"
            if px is not None:
                px.close()
        hook = torch_allreduce_hook(self.bridge, group)
        self._cb = _ALLREDUCE_CB(lambda _ctx, buf, count: hook(int(buf), int(count)))
        self._rc(self.lib.b200_model_set_allreduce(self._h, self._cb, None), "b200_model_set_allreduce")
        return "nccl"

    # ---- forward ----
    def forward(self, tokens, logits: Optional[torch.Tensor] = None, hidden: Optional[torch.Tensor] = None, want_logits: bool = True):
        """tokens: list of ints or an int32 tensor of tokens_per_call ids (host ids are checked: IndexError outside the
        vocabulary, as the reference's Embedding).  Enqueues the prefill on the bridge's stream and returns the logits
        tensor [M, vocab_rows] (fp16, on the device unless one was passed); call bridge.synchronize() before reading."""
        if isinstance(tokens, (list, tuple)):
            tokens = torch.tensor(tokens, dtype=torch.int32)
        tokens = tokens.to(torch.int32).contiguous()
        if tokens.numel() != self.M:
            raise ValueError(f"expected {self.M} token ids, got {tokens.numel()}")
        if not tokens.is_cuda and tokens.numel() and (int(tokens.min()) < 0 or int(tokens.max()) >= self.config.vocab_size):
            raise IndexError(f"Token ID out of vocabulary bounds [0, {self.config.vocab_size})")
        if want_logits and logits is None:
            logits = torch.empty(self.M, self.vocab_rows, dtype=torch.float16, device="cuda")
        if any(t is not None and t.is_cuda for t in (tokens, logits, hidden)):
            torch.cuda.current_stream().synchronize()
        rc = self.lib.b200_model_forward(self._h, tokens.data_ptr(), self.M, logits.data_ptr() if logits is not None else None,
                                         hidden.data_ptr() if hidden is not None else None)
        if rc == -8:
            raise IndexError(f"Token ID out of vocabulary bounds [0, {self.config.vocab_size})")
        self._rc(rc, "b200_model_forward")
        self._keep["io"] = (tokens, logits, hidden)
        return logits

    __call__ = forward

    def kernels_per_forward(self) -> int:
        return int(self.lib.b200_model_kernels_per_forward(self._h))

    def close(self) -> None:
        if self._h:
            self.lib.b200_model_destroy(self._h)
            self._h = None
        if self.px is not None:
            self.px.close()
            self.px = None
        self._keep.clear()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def bench_prefill(bridge: B200Bridge, world: int, rank: int, layers: int = 32, steps: int = 5) -> dict:
    """End-to-end prefill of the 8B-shape model (32 layers, hidden 4096, 32/8 heads of 128, MLP 14336, vocabulary
    128256, Q4_0, 2048 tokens per call) with random-init weights: embedding gather, every layer, final norm and the
    lm_head inside the timed region, CUDA events on the library's stream, maximum over ranks."""
    import torch.distributed as dist
    cfg = EngineConfig(num_layers=layers, hidden_dim=4096, num_q_heads=32, num_kv_heads=8, head_dim=128, intermediate_dim=14336,
                       vocab_size=128256, rope_theta=500000.0, weight_format=0, max_context_length=2048, tp_size=world)
    M = 2048
    if cfg.num_kv_heads % world or cfg.intermediate_dim % world or cfg.vocab_size % world:
        return {"skipped": f"shape does not shard over {world} ranks"}
    model = TransformerModel(cfg, M, bridge)
    model.init_synthetic_weights(seed=11, rank=rank)
    mode = model.setup_tensor_parallel() if world > 1 else "single"
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev); gen.manual_seed(5)
    tokens = torch.randint(0, cfg.vocab_size, (M,), dtype=torch.int32, device=dev, generator=gen)
    logits = torch.empty(M, model.vocab_rows, dtype=torch.float16, device=dev)
    stream = torch.cuda.ExternalStream(bridge.lib.b200_bridge_stream())
    for _ in range(2):
        model.forward(tokens, logits)
    bridge.synchronize()
    err0 = bridge.device_error()
    times = []
    for _ in range(steps):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        model.forward(tokens, logits)
        e1.record(stream)
        bridge.synchronize(); e1.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        times.append(float(t.item()))
    ms = statistics.median(times)
    finite = bool(torch.isfinite(logits.float()).all().item())
    kernels = model.kernels_per_forward()
    if world > 1:
        dist.barrier()
    model.close()
    torch.cuda.empty_cache()
    c = cfg
    per_layer = 2.0 * M * c.hidden_dim * (c.q_dim + 2 * c.kv_dim) + 2.0 * c.num_q_heads * M * (M + 1) * c.head_dim + \
        2.0 * M * c.q_dim * c.hidden_dim + 4.0 * M * c.hidden_dim * c.intermediate_dim + 2.0 * M * c.intermediate_dim * c.hidden_dim
    flops = layers * per_layer + 2.0 * M * c.hidden_dim * c.vocab_size
    return {"workload": f"{layers}-layer 8B-shape model prefill, {M} tokens, Q4_0 weights (random init), vocabulary {c.vocab_size}: "
                        "embedding, layers, final norm, lm_head", "parallelism": f"tp{world} ({mode})", "scaling": "strong",
            "ms": ms, "ms_all": times, "prefill_tokens_per_s": M / ms * 1e3, "tflops": flops / ms / 1e9, "kernels_per_forward": kernels,
            "finite": finite, "device_error": err0}
