"""CPU-only checks of the host side: the shared library loads and exports every declared symbol,
the registry answers like the reference's, the device unpackers (built for the host) agree with
the oracle, the Linear wrapper validates like the reference's, and tensor-parallel sharding of
packed weights is exact (including a 2-rank gloo run)."""
import ctypes
import os
import re
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import oracle as o

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    names = set()
    for hdr in (ROOT / "include").glob("*.h"):
        text = hdr.read_text()
        for block in re.findall(r'extern "C" \{(.*?)\n\}', text, flags=re.S):
            names.update(re.findall(r"\b((?:m4_bridge|b200_bridge|b200_layer|b200_registry|b200_model|b200_peer|b200_gguf)_\w+)\s*\(", block))
    return names


def test_library_exports_every_declared_symbol(lib_path):
    lib = ctypes.CDLL(str(lib_path))
    names = declared_symbols()
    assert len(names) >= 30
    missing = [n for n in sorted(names) if not hasattr(lib, n)]
    assert not missing, f"declared in include/*.h but not exported: {missing}"


def test_public_headers_compile_as_c(tmp_path):
    """The C entry points are declared for C callers too: every header under include/ that declares one compiles as C11
    (the C++ classes that mirror the reference's own headers are hidden from a C compiler)."""
    inc = Path(__file__).resolve().parent.parent / "include"
    for h in ("b200_bridge.h", "transformer_layer.h", "transformer_model.h", "gguf_loader.h", "quant_registry.h"):
        src = tmp_path / (h + ".c")
        src.write_text(f'#include "{h}"\nint main(void) {{ return 0; }}\n')
        r = subprocess.run(["gcc", "-std=c11", "-Wall", "-Werror", "-I", str(inc), "-fsyntax-only", str(src)], capture_output=True, text=True)
        assert r.returncode == 0, f"{h}: {r.stderr[:400]}"


def test_no_compute_without_init(lib_path, pkg):
    lib = pkg.bridge.bind(ctypes.CDLL(str(lib_path)))
    if lib.m4_bridge_is_initialized():
        pytest.skip("bridge already initialised in this process")
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.addressof(buf)
    # -1 comes first, as in the reference (core/bridge/m4_mlx_bridge.mm:201-203)
    assert lib.m4_bridge_dispatch_gemm(p, 4096, p, 4096, p, 4096, 0, 1, 32, 1) == -1
    assert lib.m4_bridge_get_expected_weight_bytes(0, 4096, 4096) == 4096 * 4096 // 32 * 18
    assert lib.m4_bridge_get_expected_weight_bytes(6, 4096, 4096) == 0
    assert lib.m4_bridge_get_expected_weight_bytes(-1, 4096, 4096) == 0


def test_init_fails_loudly_without_gpu(lib_path, pkg):
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    lib = pkg.bridge.bind(ctypes.CDLL(str(lib_path)))
    assert lib.m4_bridge_init(None) is False
    assert b"no CPU path" in lib.b200_bridge_last_error_string()


# ---- registry (tests/test_quant_registry.mm:10-123) ----
REG = {0: ("Q4_0", 32, 18, 4.5, "q4_0"), 1: ("MLX_4BIT", 32, 20, 5.0, "mlx_4bit"), 2: ("Q4_K", 256, 144, 4.5, "q4_k"),
       3: ("TERNARY_1_58", 32, 12, 3.0, "ternary_1_58"), 4: ("VAR_RATE_AFFINE", 256, 160, 5.0, "var_rate_affine"),
       5: ("EXL3", 256, 144, 4.5, "exl3"), 6: ("Q8_0", 32, 34, 8.5, "q8_0"), 7: ("PRISM_Q2_0", 128, 34, 2.125, "prism_q2_0")}


def _describe(lib, fmt):
    name = ctypes.create_string_buffer(64); gk = ctypes.create_string_buffer(96); hk = ctypes.create_string_buffer(96)
    bs = ctypes.c_uint32(); ss = ctypes.c_size_t(); bpw = ctypes.c_double()
    lib.b200_registry_describe.argtypes = [ctypes.c_int, ctypes.c_char_p, ctypes.c_size_t, ctypes.POINTER(ctypes.c_uint32),
                                           ctypes.POINTER(ctypes.c_size_t), ctypes.POINTER(ctypes.c_double), ctypes.c_char_p,
                                           ctypes.c_size_t, ctypes.c_char_p, ctypes.c_size_t]
    ok = lib.b200_registry_describe(fmt, name, 64, ctypes.byref(bs), ctypes.byref(ss), ctypes.byref(bpw), gk, 96, hk, 96)
    return ok, name.value.decode(), bs.value, ss.value, bpw.value, gk.value.decode(), hk.value.decode()


def test_registry_builtin_descriptors(lib_path):
    lib = ctypes.CDLL(str(lib_path))
    lib.b200_registry_weight_bytes.restype = ctypes.c_size_t
    lib.b200_registry_weight_bytes.argtypes = [ctypes.c_int, ctypes.c_size_t]
    assert lib.b200_registry_count() >= 8
    for fmt, (name, bs, ss, bpw, stem) in REG.items():
        ok, n, b, s, w, gk, hk = _describe(lib, fmt)
        assert ok == 1 and (n, b, s, w) == (name, bs, ss, bpw)
        assert gk == f"quant_router_gemm_{stem}_64x64" and hk == f"quant_router_head_gemm_{stem}_64x64"
        assert lib.b200_registry_weight_bytes(fmt, 4096 * 4096) == 4096 * 4096 // bs * ss
        assert lib.b200_registry_format_by_name(name.encode()) == fmt
    assert _describe(lib, 42)[0] == 0
    assert lib.b200_registry_weight_bytes(42, 1024) == 0           # unknown format sizes to 0
    f, l, i = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    assert lib.b200_registry_resolve_kernel(b"quant_router_head_gemm_q4_k_64x64", ctypes.byref(f), ctypes.byref(l), ctypes.byref(i)) == 1
    assert (f.value, l.value, i.value) == (2, 1, 1)
    assert lib.b200_registry_resolve_kernel(b"quant_router_gemm_q8_0_64x64", ctypes.byref(f), ctypes.byref(l), ctypes.byref(i)) == 1
    assert (f.value, i.value) == (6, 0)                              # name registered, no such kernel
    assert lib.b200_registry_resolve_kernel(b"nope", ctypes.byref(f), ctypes.byref(l), ctypes.byref(i)) == 0


def test_registry_dynamic_registration(lib_path):
    lib = ctypes.CDLL(str(lib_path))
    lib.b200_registry_register.argtypes = [ctypes.c_int, ctypes.c_char_p, ctypes.c_uint32, ctypes.c_size_t, ctypes.c_double,
                                           ctypes.c_char_p, ctypes.c_char_p]
    n0 = lib.b200_registry_count()
    assert lib.b200_registry_register(99, b"CUSTOM_3BIT", 64, 26, 3.25, b"custom_gemm", b"custom_head_gemm") == 0
    assert lib.b200_registry_count() == n0 + 1
    ok, n, b, s, w, gk, hk = _describe(lib, 99)
    assert (ok, n, b, s, w, gk) == (1, "CUSTOM_3BIT", 64, 26, 3.25, "custom_gemm")
    assert lib.b200_registry_format_by_name(b"CUSTOM_3BIT") == 99


# ---- device unpackers compiled for the host ----
@pytest.fixture(scope="module")
def codec_lib(tmp_path_factory):
    out = tmp_path_factory.mktemp("codec") / "codec_host.so"
    subprocess.check_call(["g++", "-O1", "-std=c++17", "-fPIC", "-shared", str(ROOT / "tests" / "codec_host_shim.cpp"), "-o", str(out)])
    return ctypes.CDLL(str(out))


@pytest.mark.parametrize("fmt,exact", [(o.Q4_0, True), (o.MLX_4BIT, True), (o.Q4_K, False), (o.TERNARY_1_58, True),
                                       (o.VAR_RATE_AFFINE, False), (o.EXL3, True), (o.PRISM_Q2_0, True)])
def test_unpackers_match_oracle(codec_lib, fmt, exact):
    K, N = 1024, 48
    for seed in (1337, 7):
        W = o.RefLcg(seed).weights(fmt, K, N)
        if fmt == o.VAR_RATE_AFFINE and seed == 7:      # every bit depth and permutation at every position
            Wb = W.reshape(-1, 160)
            rng = np.random.default_rng(0)
            Wb[:, 20:28] = ((rng.integers(0, 4, (Wb.shape[0], 8)) << 3) | rng.choice([3, 4, 5], (Wb.shape[0], 8))).astype(np.uint8)
        out = np.empty((N, K), np.uint16)
        assert codec_lib.codec_host_dequant(fmt, o._ptr(W), o._ptr(out), N, K) == 0
        got = out.view(np.float16).astype(np.float64)
        ref = o.dequant_matrix(fmt, W, N, K)
        if exact:   # one rounding of the exact value: bit-identical to fp16(gold)
            assert np.array_equal(got, ref.astype(np.float16).astype(np.float64))
        else:       # a sub-block term (minimum / bias / scale) is itself rounded to fp16 first: allow 2 ulps of
                    # the result plus one rounding of a term of the size these generators produce (< 0.13)
            ulp = np.spacing(np.abs(ref).astype(np.float16)).astype(np.float64)
            assert np.all(np.abs(got - ref) <= 2 * ulp + 0.13 * 2.0 ** -11)


def test_unpackers_baseline_distribution(codec_lib):
    K, N = 512, 32
    for fmt in (o.Q4_0, o.MLX_4BIT, o.TERNARY_1_58):
        _, W = o.baseline_inputs(fmt, 1, K, N, 11)
        out = np.empty((N, K), np.uint16)
        codec_lib.codec_host_dequant(fmt, o._ptr(W), o._ptr(out), N, K)
        ref = o.dequant_matrix(fmt, W, N, K)
        assert np.array_equal(out.view(np.float16).astype(np.float64), ref.astype(np.float16).astype(np.float64))


def test_planar_unpackers_match_oracle(codec_lib):
    """The planar layouts (the reference's group-32 MLX planes and the two extension layouts): nibble / 2-bit plane through the tensor-core codec, metadata planes beside it."""
    K, N = 1024, 40
    for fmt in (o.MLX_4BIT_G64, o.TERNARY_ROW, o.MLX_4BIT_PLANAR):
        _, W = o.baseline_inputs(fmt, 1, K, N, 5)
        out = np.empty((N, K), np.uint16)
        assert codec_lib.codec_host_dequant(fmt, o._ptr(W), o._ptr(out), N, K) == 0
        got = out.view(np.float16).astype(np.float64)
        ref = o.dequant_matrix(fmt, W, N, K)
        if fmt == o.TERNARY_ROW:            # the codec yields the integers code-1; the row scale is applied to the accumulator
            assert set(np.unique(got)) <= {-1.0, 0.0, 1.0}
            got = got * W[N * K // 4:].view(np.float16).astype(np.float64)[:, None]
            assert np.array_equal(got, ref)
        else:
            assert np.array_equal(got, ref.astype(np.float16).astype(np.float64))


# ---- Linear wrapper argument contract (tests/redteam_modules.py:122-176) ----
def test_linear_wrapper_rejects_bad_shapes(pkg):
    from m4_prefill_engine_b200.modules import M4QuantizedLinear, compute_quantized_weight_bytes, normalize_format
    for bad in [(0, 64), (64, 0), (-32, 64), (48, 64)]:
        with pytest.raises(ValueError):
            M4QuantizedLinear(bad[0], bad[1], format="q4_0")
    for fmt in ("q4_k", "var_rate_affine", "exl3"):
        with pytest.raises(ValueError):
            M4QuantizedLinear(128, 64, format=fmt)
    with pytest.raises(ValueError):
        M4QuantizedLinear(64, 64, format="q4_0", weight=np.zeros(10, np.uint8))
    with pytest.raises(ValueError):
        normalize_format("no_such_format")
    assert compute_quantized_weight_bytes("Q4_K", 4096, 4096) == 4096 * 4096 // 256 * 144
    assert normalize_format(3).name == "QUANT_TERNARY_1_58"


# ---- tensor-parallel sharding ----
def test_shards_reassemble_exactly(pkg):
    from m4_prefill_engine_b200.layer import shard_cols, shard_rows
    K, N, M, tp = 1024, 96, 7, 4
    for fmt in (o.Q4_0, o.Q4_K, o.TERNARY_1_58):
        g = o.RefLcg(21)
        W = g.weights(fmt, K, N)
        X = g.activations(M, K)
        full = o.gemm_f64(fmt, X, W, N)
        cols = np.concatenate([o.gemm_f64(fmt, X, shard_rows(W, fmt, K, N, r, tp), N // tp) for r in range(tp)], axis=1)
        assert np.array_equal(cols, full)
        part = sum(o.gemm_f64(fmt, X[:, r * K // tp:(r + 1) * K // tp], shard_cols(W, fmt, K, N, r, tp), N) for r in range(tp))
        assert np.abs(part - full).max() < 1e-9


def test_planar_shards_reassemble_exactly(pkg):
    """Column split of the planar layouts (every plane keeps the rank's rows; the group-32 MLX layout pads its planes to
    16 bytes, also where a shard's plane sizes are not multiples of 16)."""
    from m4_prefill_engine_b200.layer import shard_rows_any
    M = 5
    for fmt, K, N, tp in ((o.MLX_4BIT_G64, 512, 96, 4), (o.TERNARY_ROW, 512, 96, 4), (o.MLX_4BIT_PLANAR, 512, 96, 4),
                          (o.MLX_4BIT_PLANAR, 96, 6, 2), (o.PRISM_Q2_0, 512, 96, 4)):
        X, W = o.baseline_inputs(fmt, M, K, N, 31) if fmt != o.PRISM_Q2_0 else (o.RefLcg(3).activations(M, K), o.RefLcg(3).weights(fmt, K, N))
        full = o.gemm_f64(fmt, X, W, N)
        shards = [shard_rows_any(W, fmt, K, N, r, tp) for r in range(tp)]
        for sh in shards:
            assert sh.size == o.weight_bytes(fmt, K, N // tp)
        cols = np.concatenate([o.gemm_f64(fmt, X, sh, N // tp) for sh in shards], axis=1)
        assert np.array_equal(cols, full)


GLOO_WORKER = r'''
import os, sys, numpy as np, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
import oracle as o
from __graft_entry__ import load_package
load_package()
from m4_prefill_engine_b200.layer import shard_cols
dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{sys.argv[2]}", rank=int(sys.argv[3]), world_size=2)
r = dist.get_rank()
K, N, M = 512, 64, 9
g = o.RefLcg(77); W = g.weights(o.Q4_0, K, N); X = g.activations(M, K)
part = o.gemm_f64(o.Q4_0, X[:, r * K // 2:(r + 1) * K // 2], shard_cols(W, o.Q4_0, K, N, r, 2), N)
t = torch.from_numpy(part.astype(np.float32)); dist.all_reduce(t)
full = o.gemm_f64(o.Q4_0, X, W, N)
assert np.abs(t.numpy() - full).max() < 1e-4, np.abs(t.numpy() - full).max()
dist.barrier(); dist.destroy_process_group()
print("rank", r, "ok")
'''


def test_row_split_all_reduce_two_gloo_ranks(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(GLOO_WORKER)
    port = 29500 + (os.getpid() % 500)
    procs = [subprocess.Popen([sys.executable, str(script), str(ROOT), str(port), str(r)], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=180)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
