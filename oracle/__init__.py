"""CPU oracle for the prefill hot path -- TEST INFRASTRUCTURE ONLY.

numpy front end over ``oracle/_build/liboracle.so`` (our restatement of the reference's
double-precision CPU verifier, ``oracle/oracle.cpp``) and, when it has been built,
``oracle/_ref/libm4ref.so`` (the reference's own verifier sources compiled as they are).

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may
import this package.  The product package never does.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import numpy as np

from . import build as _build

HERE = Path(__file__).resolve().parent

# format ids (include/quant_router.h)
Q4_0, MLX_4BIT, Q4_K, TERNARY_1_58, VAR_RATE_AFFINE, EXL3, Q8_0, PRISM_Q2_0 = range(8)
MLX_4BIT_G64, TERNARY_ROW, MLX_4BIT_PLANAR = 100, 101, 102
BLOCK = {Q4_0: (32, 18), MLX_4BIT: (32, 20), Q4_K: (256, 144), TERNARY_1_58: (32, 12),
         VAR_RATE_AFFINE: (256, 160), EXL3: (256, 144), Q8_0: (32, 34), PRISM_Q2_0: (128, 34)}
FORMAT_NAMES = {Q4_0: "q4_0", MLX_4BIT: "mlx_4bit", Q4_K: "q4_k", TERNARY_1_58: "ternary_1_58",
                VAR_RATE_AFFINE: "var_rate_affine", EXL3: "exl3", PRISM_Q2_0: "prism_q2_0",
                MLX_4BIT_G64: "mlx_4bit_g64", TERNARY_ROW: "ternary_row", MLX_4BIT_PLANAR: "mlx_4bit_planar"}


def weight_bytes(fmt: int, K: int, N: int) -> int:
    if fmt == MLX_4BIT_G64:
        return N * (K // 8) * 4 + 2 * N * (K // 64) * 2
    if fmt == TERNARY_ROW:
        return N * (K // 16) * 4 + N * 2
    if fmt == MLX_4BIT_PLANAR:
        blocks = N * (K // 32)
        scales_off = (blocks * 16 + 15) & ~15
        return ((scales_off + blocks * 2 + 15) & ~15) + blocks * 2
    be, bb = BLOCK[fmt]
    return N * (K // be) * bb


_vp, _u32, _sz, _i, _f = C.c_void_p, C.c_uint32, C.c_size_t, C.c_int, C.c_float


def _ptr(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.c_void_p)


def _load_oracle() -> C.CDLL:
    lib = C.CDLL(str(_build.build_oracle()))
    lib.orc_gemm.argtypes = [_i, _vp, _vp, _vp, _u32, _u32, _u32, _i, _u32, _u32]
    lib.orc_gemm.restype = _i
    lib.orc_gemm_f64.argtypes = [_i, _vp, _vp, _vp, _u32, _u32, _u32]
    lib.orc_gemm_f64.restype = _i
    lib.orc_dequant_matrix.argtypes = [_i, _vp, _vp, _u32, _u32]
    lib.orc_dequant_matrix.restype = _i
    lib.orc_swiglu_fused.argtypes = [_i, _vp, _vp, _vp, _vp, _u32, _u32, _u32]
    lib.orc_swiglu_fused.restype = _i
    lib.orc_swiglu_elementwise.argtypes = [_vp, _vp, _vp, _u32]
    lib.orc_quantize_q8_0.argtypes = [_vp, _vp, _sz]
    lib.orc_dequantize_q8_0.argtypes = [_vp, _vp, _sz]
    lib.orc_attention.argtypes = [_vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _f, _u32, _i]
    lib.orc_rmsnorm.argtypes = [_vp, _vp, _vp, _u32, _u32, _f]
    lib.orc_rope.argtypes = [_vp, _u32, _u32, _u32, _f, _u32]
    lib.orc_layer.argtypes = [_i] + [_vp] * 9 + [_u32] * 6 + [_f, _f, _vp, _vp, _f, _i]
    lib.orc_layer.restype = _i
    lib.orc_gen_activations.argtypes = [_u32, _vp, _sz]
    lib.orc_gen_activations.restype = _u32
    lib.orc_gen_weights.argtypes = [_u32, _i, _vp, _sz]
    lib.orc_gen_weights.restype = _u32
    lib.orc_gen_brick3_activations.argtypes = [_u32, _vp, _sz]
    lib.orc_gen_brick3_activations.restype = _u32
    lib.orc_gen_q4_0_affine_scale.argtypes = [_u32, _vp, _sz, _f, _f]
    lib.orc_gen_q4_0_affine_scale.restype = _u32
    lib.orc_num_threads.restype = _i
    return lib


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = _load_oracle()
    return _lib


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int = 0) -> int:
    """Make the CPU checkers (restatement and, where built, the reference's own verifier) use n OpenMP threads
    (0: every core this process may run on) and return the team size a parallel region really gets.  Needed under
    launchers that export OMP_NUM_THREADS=1 to their children."""
    if n <= 0:
        n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    got = int(lib().orc_set_num_threads(int(n)))
    r = ref_lib()
    if r is not None and hasattr(r, "ref_set_threads"):
        got = min(got, int(r.ref_set_threads(int(n))))
    return got


# ---------------------------------------------------------------------------------------
# golds
# ---------------------------------------------------------------------------------------
def gemm(fmt: int, A: np.ndarray, W: np.ndarray, N: int, direct_head: bool = False, H: int = 0, D: int = 0) -> np.ndarray:
    """fp16 GEMM gold.  A [M,K] float16, W raw uint8 weight bytes.  Returns [M,N] (or [H,M,D])."""
    A = np.ascontiguousarray(A, dtype=np.float16)
    M, K = A.shape
    assert W.dtype == np.uint8 and W.size >= weight_bytes(fmt, K, N)
    out = np.empty((H, M, D) if direct_head else (M, N), dtype=np.float16)
    rc = lib().orc_gemm(fmt, _ptr(A), _ptr(W), _ptr(out), M, N, K, int(direct_head), H, D)
    if rc:
        raise ValueError(f"orc_gemm rc={rc}")
    return out


def gemm_f64(fmt: int, A: np.ndarray, W: np.ndarray, N: int) -> np.ndarray:
    A = np.ascontiguousarray(A, dtype=np.float16)
    M, K = A.shape
    out = np.empty((M, N), dtype=np.float64)
    rc = lib().orc_gemm_f64(fmt, _ptr(A), _ptr(W), _ptr(out), M, N, K)
    if rc:
        raise ValueError(f"orc_gemm_f64 rc={rc}")
    return out


def dequant_matrix(fmt: int, W: np.ndarray, N: int, K: int) -> np.ndarray:
    out = np.empty((N, K), dtype=np.float64)
    rc = lib().orc_dequant_matrix(fmt, _ptr(W), _ptr(out), N, K)
    if rc:
        raise ValueError(f"orc_dequant_matrix rc={rc}")
    return out


def swiglu_fused(fmt: int, A: np.ndarray, Wg: np.ndarray, Wu: np.ndarray, F: int) -> np.ndarray:
    A = np.ascontiguousarray(A, dtype=np.float16)
    M, K = A.shape
    out = np.empty((M, F), dtype=np.float16)
    rc = lib().orc_swiglu_fused(fmt, _ptr(A), _ptr(Wg), _ptr(Wu), _ptr(out), M, F, K)
    if rc:
        raise ValueError(f"orc_swiglu_fused rc={rc}")
    return out


def swiglu_elementwise(g: np.ndarray, u: np.ndarray) -> np.ndarray:
    g = np.ascontiguousarray(g, dtype=np.float16)
    u = np.ascontiguousarray(u, dtype=np.float16)
    out = np.empty_like(g)
    lib().orc_swiglu_elementwise(_ptr(g), _ptr(u), _ptr(out), g.size)
    return out


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    """fp16 array (size % 32 == 0) -> raw block_q8_0 bytes (34 per 32 values)."""
    x = np.ascontiguousarray(x, dtype=np.float16)
    out = np.empty(x.size // 32 * 34, dtype=np.uint8)
    lib().orc_quantize_q8_0(_ptr(x), _ptr(out), x.size)
    return out


def dequantize_q8_0(blocks: np.ndarray, shape) -> np.ndarray:
    out = np.empty(shape, dtype=np.float16)
    lib().orc_dequantize_q8_0(_ptr(blocks), _ptr(out), out.size)
    return out


def attention(Q, K, V, scale: float, pos0: int = 0, tokens_major: bool = False) -> np.ndarray:
    """Q [Hq,M,D], K/V [Hkv,Mkv,D] fp16 -> O [Hq,M,D] (or [M,Hq*D])."""
    Q = np.ascontiguousarray(Q, dtype=np.float16)
    K = np.ascontiguousarray(K, dtype=np.float16)
    V = np.ascontiguousarray(V, dtype=np.float16)
    Hq, M, D = Q.shape
    Hkv, Mkv, _ = K.shape
    out = np.empty((M, Hq * D) if tokens_major else (Hq, M, D), dtype=np.float16)
    lib().orc_attention(_ptr(Q), _ptr(K), _ptr(V), _ptr(out), Hq, Hkv, M, Mkv, D, scale, pos0, int(tokens_major))
    return out


def rmsnorm(X, weight, eps: float) -> np.ndarray:
    X = np.ascontiguousarray(X, dtype=np.float16)
    weight = np.ascontiguousarray(weight, dtype=np.float16)
    out = np.empty_like(X)
    lib().orc_rmsnorm(_ptr(X), _ptr(weight), _ptr(out), X.shape[0], X.shape[1], eps)
    return out


def rope(X, theta: float, pos0: int = 0) -> np.ndarray:
    """X [H,M,D] fp16 -> rotated copy."""
    X = np.array(X, dtype=np.float16, order="C", copy=True)
    H, M, D = X.shape
    lib().orc_rope(_ptr(X), H, M, D, theta, pos0)
    return X


def layer(fmt, X, Wq, Wk, Wv, Wo, Wg, Wu, Wd, H, Hkv, D, F, attn_scale, rms_eps=0.0, norm1=None, norm2=None,
          rope_theta=0.0, kv_q8=False) -> np.ndarray:
    X = np.ascontiguousarray(X, dtype=np.float16)
    M, K = X.shape
    out = np.empty_like(X)
    n1 = _ptr(np.ascontiguousarray(norm1, dtype=np.float16)) if norm1 is not None else None
    n2 = _ptr(np.ascontiguousarray(norm2, dtype=np.float16)) if norm2 is not None else None
    rc = lib().orc_layer(fmt, _ptr(X), _ptr(Wq), _ptr(Wk), _ptr(Wv), _ptr(Wo), _ptr(Wg), _ptr(Wu), _ptr(Wd),
                         _ptr(out), M, K, H, Hkv, D, F, attn_scale, rms_eps, n1, n2, rope_theta, int(kv_q8))
    if rc:
        raise ValueError(f"orc_layer rc={rc}")
    return out


# ---------------------------------------------------------------------------------------
# seeded generators
# ---------------------------------------------------------------------------------------
class RefLcg:
    """The reference's test generators (tests/e2e/test_common.h:253-427): one LCG state threaded
    through weights then activations."""

    def __init__(self, seed: int = 1337):
        self.state = seed & 0xFFFFFFFF

    def activations(self, *shape) -> np.ndarray:
        out = np.empty(shape, dtype=np.float16)
        self.state = lib().orc_gen_activations(self.state, _ptr(out), out.size)
        return out

    def weights(self, fmt: int, K: int, N: int) -> np.ndarray:
        be, bb = BLOCK[fmt]
        nblk = N * (K // be)
        out = np.empty(nblk * bb, dtype=np.uint8)
        self.state = lib().orc_gen_weights(self.state, fmt, _ptr(out), nblk)
        return out

    def brick3_activations(self, *shape) -> np.ndarray:
        out = np.empty(shape, dtype=np.float16)
        self.state = lib().orc_gen_brick3_activations(self.state, _ptr(out), out.size)
        return out

    def q4_0_bench(self, K: int, N: int, rng: float = 0.04, offset: float = 0.002) -> np.ndarray:
        nblk = N * (K // 32)
        out = np.empty(nblk * 18, dtype=np.uint8)
        self.state = lib().orc_gen_q4_0_affine_scale(self.state, _ptr(out), nblk, rng, offset)
        return out


def baseline_inputs(fmt: int, M: int, K: int, N: int, seed: int = 0):
    """Seeded inputs with the value distributions the benchmark contract names: X ~ N(0,1) fp16;
    Q4_0 d~U(0.005,0.02), q~U{0..15}; MLX s~U(0.005,0.02), b=-8s+U(-0.01,0.01); Q4_K, var-rate, EXL3
    with the reference generator's ranges; ternary codes with p=(0.25,0.5,0.25), scale U(0.01,0.05)
    per block (per row for TERNARY_ROW).  Returns (X [M,K] float16, W uint8)."""
    rng = np.random.default_rng(seed)
    X = rng.standard_normal((M, K), dtype=np.float32).astype(np.float16)
    return X, baseline_weights(fmt, K, N, rng)


def mlx_aos_to_planar(W: np.ndarray, K: int, N: int) -> np.ndarray:
    """20-byte MLX blocks {d, bias, qs[16]} -> the three planes of the reference's layer benchmarks
    (bench_all_scales.mm:62-95): qs | scales | biases, each plane starting on a 16-byte boundary."""
    nb = N * (K // 32)
    blk = np.ascontiguousarray(W).reshape(nb, 20)
    out = np.zeros(weight_bytes(MLX_4BIT_PLANAR, K, N), np.uint8)
    scales_off = (nb * 16 + 15) & ~15
    biases_off = (scales_off + nb * 2 + 15) & ~15
    out[:nb * 16] = blk[:, 4:].reshape(-1)
    out[scales_off:scales_off + nb * 2] = blk[:, 0:2].reshape(-1)
    out[biases_off:biases_off + nb * 2] = blk[:, 2:4].reshape(-1)
    return out


def baseline_weights(fmt: int, K: int, N: int, rng) -> np.ndarray:
    if isinstance(rng, (int, np.integer)):
        rng = np.random.default_rng(int(rng))
    if fmt == Q4_0:
        nb = N * (K // 32)
        W = np.empty((nb, 18), dtype=np.uint8)
        W[:, 0:2] = rng.uniform(0.005, 0.02, nb).astype(np.float16).view(np.uint8).reshape(nb, 2)
        W[:, 2:] = rng.integers(0, 256, (nb, 16), dtype=np.uint8)
        return W.reshape(-1)
    if fmt == MLX_4BIT:
        nb = N * (K // 32)
        s = rng.uniform(0.005, 0.02, nb)
        b = -8.0 * s + rng.uniform(-0.01, 0.01, nb)
        W = np.empty((nb, 20), dtype=np.uint8)
        W[:, 0:2] = s.astype(np.float16).view(np.uint8).reshape(nb, 2)
        W[:, 2:4] = b.astype(np.float16).view(np.uint8).reshape(nb, 2)
        W[:, 4:] = rng.integers(0, 256, (nb, 16), dtype=np.uint8)
        return W.reshape(-1)
    if fmt == MLX_4BIT_PLANAR:
        return mlx_aos_to_planar(baseline_weights(MLX_4BIT, K, N, rng), K, N)
    if fmt == MLX_4BIT_G64:
        qs = rng.integers(0, 2**32, (N, K // 8), dtype=np.uint32)
        s = rng.uniform(0.005, 0.02, (N, K // 64))
        b = -8.0 * s + rng.uniform(-0.01, 0.01, (N, K // 64))
        return np.concatenate([qs.view(np.uint8).reshape(-1), s.astype(np.float16).view(np.uint8).reshape(-1),
                               b.astype(np.float16).view(np.uint8).reshape(-1)])
    if fmt == TERNARY_1_58:
        nb = N * (K // 32)
        codes = rng.choice(np.array([0, 1, 2], dtype=np.uint32), size=(nb, 2, 16), p=[0.25, 0.5, 0.25])
        words = (codes << (2 * np.arange(16, dtype=np.uint32))).sum(axis=2, dtype=np.uint32)
        W = np.zeros((nb, 12), dtype=np.uint8)
        W[:, 0:2] = rng.uniform(0.01, 0.05, nb).astype(np.float16).view(np.uint8).reshape(nb, 2)
        W[:, 4:] = words.view(np.uint8).reshape(nb, 8)
        return W.reshape(-1)
    if fmt == TERNARY_ROW:
        codes = rng.choice(np.array([0, 1, 2], dtype=np.uint32), size=(N, K // 16, 16), p=[0.25, 0.5, 0.25])
        words = (codes << (2 * np.arange(16, dtype=np.uint32))).sum(axis=2, dtype=np.uint32)
        rs = rng.uniform(0.01, 0.05, N).astype(np.float16)
        return np.concatenate([words.view(np.uint8).reshape(-1), rs.view(np.uint8).reshape(-1)])
    # Q4_K / var-rate / EXL3 / Prism: the reference generator's own ranges, seeded from rng
    g = RefLcg(int(rng.integers(1, 2**31)))
    return g.weights(fmt, K, N)


# ---------------------------------------------------------------------------------------
# the reference's own verifier (present only where oracle/_ref was built)
# ---------------------------------------------------------------------------------------
_ref = None


def ref_lib():
    """ctypes handle on oracle/_ref/libm4ref.so, or None when it has not been built."""
    global _ref
    if _ref is None:
        p = _build.build_ref()
        if p is None or not Path(p).exists():
            return None
        r = C.CDLL(str(p))
        r.ref_gemm.argtypes = [_i, _vp, _vp, _vp, _u32, _u32, _u32, _i, _u32, _u32]
        r.ref_gemm.restype = _i
        r.ref_attention.argtypes = [_vp, _vp, _vp, _vp, _u32, _u32, _u32, _f]
        r.ref_swiglu_elementwise.argtypes = [_vp, _vp, _vp, _u32]
        r.ref_gen_activations.argtypes = [_u32, _vp, _sz]
        r.ref_gen_activations.restype = _u32
        r.ref_gen_weights.argtypes = [_u32, _i, _vp, _sz]
        r.ref_gen_weights.restype = _u32
        r.ref_brick3_swiglu.argtypes = [_u32, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _i]
        r.ref_quantize_q8_0.argtypes = [_vp, _vp, _sz]
        r.ref_dequantize_q8_0.argtypes = [_vp, _vp, _sz]
        r.ref_brick4_attention.argtypes = [_vp, _vp, _vp, _vp, _u32, _u32, _u32, _f]
        r.ref_layer_gen_q4_0.argtypes = [_u32, _vp, _sz, _f]
        r.ref_layer_gen_q4_0.restype = _u32
        r.ref_layer.argtypes = [_vp] * 9 + [_u32] * 5 + [_f]
        _ref = r
    return _ref


def ref_gemm(fmt: int, A: np.ndarray, W: np.ndarray, N: int, direct_head=False, H=0, D=0) -> np.ndarray:
    A = np.ascontiguousarray(A, dtype=np.float16)
    M, K = A.shape
    out = np.empty((H, M, D) if direct_head else (M, N), dtype=np.float16)
    rc = ref_lib().ref_gemm(fmt, _ptr(A), _ptr(W), _ptr(out), M, N, K, int(direct_head), H, D)
    if rc:
        raise ValueError(f"ref_gemm rc={rc}")
    return out
