"""CPU oracle pinned three ways: the reference's known-answer tests, the committed fixtures that
the reference's own verifier produced, and (where it has been built) that verifier itself."""
import numpy as np
import pytest

import oracle as o

GOLD = __import__("pathlib").Path(__file__).resolve().parent / "golden"
FORMATS = (o.Q4_0, o.MLX_4BIT, o.Q4_K, o.TERNARY_1_58, o.VAR_RATE_AFFINE, o.EXL3, o.PRISM_Q2_0)


def h(a):
    return np.ascontiguousarray(a).view(np.float16)


# ---- known-answer tests (tests/e2e/test_tier1_feature_coverage.mm:248-257,287-297,363-376) ----
def test_kat_q4_0_zero_offset():
    blk = np.zeros(18, np.uint8)
    blk[0:2] = np.frombuffer(np.float16(1.0).tobytes(), np.uint8)
    blk[2:] = 0x88
    out = o.gemm(o.Q4_0, np.ones((1, 32), np.float16), blk, 1)
    assert abs(float(out[0, 0])) <= 1e-4


def test_kat_mlx_bias_application():
    blk = np.zeros(20, np.uint8)
    blk[2:4] = np.frombuffer(np.float16(0.5).tobytes(), np.uint8)
    out = o.gemm(o.MLX_4BIT, np.ones((1, 32), np.float16), blk, 1)
    assert abs(float(out[0, 0]) - 16.0) <= 1e-2


def test_kat_ternary_zero_trits():
    blk = np.zeros(12, np.uint8)
    blk[0:2] = np.frombuffer(np.float16(1.0).tobytes(), np.uint8)
    blk[4:12] = 0x55
    out = o.gemm(o.TERNARY_1_58, np.ones((1, 32), np.float16), blk, 1)
    assert abs(float(out[0, 0])) <= 1e-4


def test_kat_unit_weights_give_k():
    # tests/test_bridge_basic.py:58-81,97-117: scale 1, Q4_0 nibble 9 / MLX nibble 1, X == 1  =>  Y == K
    K, N = 64, 8
    w = np.zeros((N * K // 32, 18), np.uint8); w[:, 1] = 0x3C; w[:, 2:] = 0x99
    assert np.all(o.gemm(o.Q4_0, np.ones((3, K), np.float16), w.reshape(-1), N) == K)
    w = np.zeros((N * K // 32, 20), np.uint8); w[:, 1] = 0x3C; w[:, 4:] = 0x11
    assert np.all(o.gemm(o.MLX_4BIT, np.ones((3, K), np.float16), w.reshape(-1), N) == K)


def test_block_sizes():
    # struct sizes pinned by test_tier1_feature_coverage.mm:258-261,... and tests/test_quant_registry.mm
    assert {f: o.BLOCK[f] for f in FORMATS} == {0: (32, 18), 1: (32, 20), 2: (256, 144), 3: (32, 12), 4: (256, 160),
                                                5: (256, 144), 7: (128, 34)}
    assert o.weight_bytes(o.Q4_0, 4096, 4096) == 4096 * 4096 // 32 * 18
    assert o.weight_bytes(o.Q4_K, 4096, 4096) == 4096 * 4096 // 256 * 144


def test_var_rate_mode_packing():
    # test_tier1_feature_coverage.mm:406-415
    W = o.RefLcg(1337).weights(o.VAR_RATE_AFFINE, 256, 4).reshape(-1, 160)
    for s in range(8):
        bits = 3 if s < 2 else (4 if s < 6 else 5)
        assert np.all((W[:, 20 + s] & 7) == bits) and np.all(((W[:, 20 + s] >> 3) & 3) == s % 3)


# ---- fixtures produced by the reference's verifier ----
@pytest.mark.parametrize("fmt", FORMATS)
def test_gemm_fixture(fmt):
    z = np.load(GOLD / "gemm_tier1.npz")
    M, K, N, H, D = 33, 512, 256, 4, 64
    g = o.RefLcg(1337)
    W = g.weights(fmt, K, N)
    st_w = g.state
    X = g.activations(M, K)
    assert np.array_equal(W, z[f"W{fmt}"]), "weight generator differs from the reference's"
    assert np.array_equal(X.view(np.uint16), z[f"X{fmt}"]), "activation generator differs from the reference's"
    assert [st_w, g.state] == [int(v) for v in z[f"state{fmt}"]]
    assert np.array_equal(o.gemm(fmt, X, W, N).view(np.uint16), z[f"Y{fmt}"])
    assert np.array_equal(o.gemm(fmt, X, W, N, True, H, D).view(np.uint16), z[f"Yh{fmt}"])


def test_q8_and_attention_fixture():
    z = np.load(GOLD / "attention_q8.npz")
    Q, K, V = h(z["Q"]), h(z["K"]), h(z["V"])
    g = o.RefLcg(2026)
    assert np.array_equal(g.activations(*Q.shape).view(np.uint16), z["Q"])
    assert np.array_equal(o.quantize_q8_0(K), z["Kq"]) and np.array_equal(o.quantize_q8_0(V), z["Vq"])
    Kd = o.dequantize_q8_0(z["Kq"], K.shape)
    Vd = o.dequantize_q8_0(z["Vq"], V.shape)
    assert np.array_equal(Kd.view(np.uint16), z["Kd"]) and np.array_equal(Vd.view(np.uint16), z["Vd"])
    assert np.array_equal(o.attention(Q, Kd, Vd, 0.125).view(np.uint16), z["O"])


def test_swiglu_fixture():
    z = np.load(GOLD / "swiglu_brick3.npz")
    A = h(z["A"])
    M, K = A.shape
    F = z["Out"].shape[1]
    g = o.RefLcg(2026)
    assert np.array_equal(g.brick3_activations(M, K).view(np.uint16), z["A"])
    assert np.array_equal(g.q4_0_bench(K, F), z["Wg"]) and np.array_equal(g.q4_0_bench(K, F), z["Wu"])
    assert np.array_equal(o.swiglu_fused(o.Q4_0, A, z["Wg"], z["Wu"], F).view(np.uint16), z["Out"])


def test_layer_fixture():
    # The reference layer accumulates in fp32 and keeps Q, K, V in fp32; the oracle accumulates in double
    # and rounds Q, K, V to fp16 like the device path, so agreement is to a few fp16 ulps, not bit-exact.
    z = np.load(GOLD / "layer_q4_0.npz")
    X = h(z["X"])
    ws = [z[f"W{i}"] for i in range(7)]
    Y = o.layer(o.Q4_0, X, *ws, H=4, Hkv=4, D=64, F=512, attn_scale=0.125)
    ref = h(z["Y"]).astype(np.float64)
    assert np.abs(Y.astype(np.float64) - ref).max() <= 2e-3


def test_q8_0_edge_blocks():
    x = np.zeros(96, np.float16)
    x[32:64] = np.float16(6e-8)          # smallest subnormal: scale rounds to a tiny fp16
    x[64] = np.float16(65504); x[65] = np.float16(-65504)
    q = o.quantize_q8_0(x).reshape(3, 34)
    assert np.all(q[0] == 0)
    assert q[2, 2:].view(np.int8)[0] == 127 and q[2, 2:].view(np.int8)[1] == -127
    back = o.dequantize_q8_0(q.reshape(-1), (96,))
    assert np.all(np.isfinite(back.astype(np.float32)[:64]))


# ---- extension layouts agree with the reference layouts they restate ----
def test_mlx_g64_matches_aos_when_groups_repeat():
    rng = np.random.default_rng(3)
    K, N = 128, 5
    W64 = o.baseline_weights(o.MLX_4BIT_G64, K, N, rng)
    dq = o.dequant_matrix(o.MLX_4BIT_G64, W64, N, K)
    qs = W64[: N * K // 2].view(np.uint32).reshape(N, K // 8)
    sc = W64[N * K // 2: N * K // 2 + N * (K // 64) * 2].view(np.float16).reshape(N, K // 64).astype(np.float64)
    bi = W64[N * K // 2 + N * (K // 64) * 2:].view(np.float16).reshape(N, K // 64).astype(np.float64)
    for n in range(N):
        for k in range(K):
            q = (int(qs[n, k // 8]) >> (4 * (k % 8))) & 15
            assert dq[n, k] == q * sc[n, k // 64] + bi[n, k // 64]


def test_mlx_planar_matches_aos():
    """The planar group-32 layout of the reference's layer benchmarks holds the same weights as its 20-byte blocks
    (bench_all_scales.mm:62-95 against quant_router.h:41-45): same values, same sizes as mlx_4bit_buffer_size()."""
    rng = np.random.default_rng(8)
    for K, N in ((64, 5), (96, 3), (256, 4)):            # 96 x 3: nine blocks, both side planes need padding
        Wa = o.baseline_weights(o.MLX_4BIT, K, N, rng)
        Wp = o.mlx_aos_to_planar(Wa, K, N)
        nb = N * K // 32
        scales_off = (nb * 16 + 15) & ~15
        assert Wp.size == ((scales_off + nb * 2 + 15) & ~15) + nb * 2 == o.weight_bytes(o.MLX_4BIT_PLANAR, K, N)
        assert np.array_equal(o.dequant_matrix(o.MLX_4BIT_PLANAR, Wp, N, K), o.dequant_matrix(o.MLX_4BIT, Wa, N, K))
        X = rng.standard_normal((3, K)).astype(np.float16)
        assert np.array_equal(o.gemm(o.MLX_4BIT_PLANAR, X, Wp, N), o.gemm(o.MLX_4BIT, X, Wa, N))


def test_ternary_row_matches_blocks_with_equal_scales():
    rng = np.random.default_rng(4)
    K, N = 64, 6
    Wr = o.baseline_weights(o.TERNARY_ROW, K, N, rng)
    words = Wr[: N * K // 4].view(np.uint32).reshape(N, K // 16)
    rs = Wr[N * K // 4:].view(np.float16)
    blocks = np.zeros((N, K // 32, 12), np.uint8)
    for n in range(N):
        for b in range(K // 32):
            blocks[n, b, 0:2] = np.frombuffer(rs[n].tobytes(), np.uint8)
            blocks[n, b, 4:12] = words[n, 2 * b: 2 * b + 2].view(np.uint8)
    a = o.dequant_matrix(o.TERNARY_ROW, Wr, N, K)
    b = o.dequant_matrix(o.TERNARY_1_58, blocks.reshape(-1), N, K)
    assert np.array_equal(a, b)


# ---- the reference's verifier itself, where it has been built ----
needs_ref = pytest.mark.skipif(o.ref_lib() is None, reason="oracle/_ref not built (reference checkout absent)")


@needs_ref
@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("shape", [(1, 256, 8), (5, 512, 40), (17, 1024, 24)])
def test_gemm_bit_exact_vs_reference_build(fmt, shape):
    M, K, N = shape
    g = o.RefLcg(99 + fmt)
    W = g.weights(fmt, K, N)
    X = g.activations(M, K)
    assert np.array_equal(o.gemm(fmt, X, W, N).view(np.uint16), o.ref_gemm(fmt, X, W, N).view(np.uint16))


@needs_ref
def test_var_rate_all_modes_vs_reference_build():
    K, N, M = 512, 16, 4
    g = o.RefLcg(5)
    W = g.weights(o.VAR_RATE_AFFINE, K, N).reshape(-1, 160).copy()
    rng = np.random.default_rng(0)
    W[:, 20:28] = ((rng.integers(0, 4, (W.shape[0], 8)) << 3) | rng.choice([3, 4, 5], (W.shape[0], 8))).astype(np.uint8)
    X = g.activations(M, K)
    a = o.gemm(o.VAR_RATE_AFFINE, X, W.reshape(-1), N)
    b = o.ref_gemm(o.VAR_RATE_AFFINE, X, W.reshape(-1), N)
    assert np.array_equal(a.view(np.uint16), b.view(np.uint16))
