"""Projection GEMM parity on the GPU, through the C ABI, against the CPU oracle.

Test plan follows the reference's: tier-1 parity at 1/128 for every format at the M boundary set
(tests/e2e/test_tier1_feature_coverage.mm:122-223), unit-weight known answers and shape/error probes
of the bridge (tests/test_bridge_basic.py, tests/redteam_bridge.py:274-471), then the benchmark shapes."""
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle as o
from gpu_util import TOL, check, dev, device_weight_gold, run_gemm

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden"
BRIDGE_FORMATS = (o.Q4_0, o.MLX_4BIT, o.Q4_K, o.TERNARY_1_58, o.VAR_RATE_AFFINE, o.EXL3)


@pytest.mark.parametrize("fmt", BRIDGE_FORMATS)
@pytest.mark.parametrize("M", [33, 127, 128, 129, 512])
def test_tier1_parity(bridge, fmt, M):
    K, N = 512, 256
    g = o.RefLcg(1337)
    W = g.weights(fmt, K, N)
    X = g.activations(M, K)
    Y = run_gemm(bridge, fmt, X, W, N)
    diff = np.abs(Y.astype(np.float64) - o.gemm_f64(fmt, X, W, N))
    assert diff.max() <= TOL, f"max-abs {diff.max()}"


@pytest.mark.parametrize("fmt", BRIDGE_FORMATS)
def test_golden_fixture_and_direct_head(bridge, fmt):
    z = np.load(GOLD / "gemm_tier1.npz")
    X = z[f"X{fmt}"].view(np.float16)
    W = z[f"W{fmt}"]
    Y = run_gemm(bridge, fmt, X, W, 256)
    assert np.abs(Y.astype(np.float32) - z[f"Y{fmt}"].view(np.float16).astype(np.float32)).max() <= TOL
    Yh = run_gemm(bridge, fmt, X, W, 256, layout=1, H=4, D=64)
    assert np.abs(Yh.astype(np.float32) - z[f"Yh{fmt}"].view(np.float16).astype(np.float32)).max() <= TOL
    # the head-major result is the standard result re-laid out, bit for bit
    assert np.array_equal(Yh.view(np.uint16), Y.reshape(33, 4, 64).transpose(1, 0, 2).copy().view(np.uint16))


@pytest.mark.parametrize("fmt", [o.Q4_0, o.MLX_4BIT, o.TERNARY_1_58, o.Q4_K])
@pytest.mark.parametrize("shape", [(33, 64, 64), (64, 64, 64), (128, 128, 128), (33, 256, 256), (1, 512, 128)])
def test_unit_weights_give_k(bridge, pkg, fmt, shape):
    from m4_prefill_engine_b200.modules import unit_weights
    M, K, N = shape
    if fmt == o.Q4_K and K % 256:
        pytest.skip("super-block format needs K % 256 == 0")
    W = unit_weights(fmt, K, N).numpy()
    Y = run_gemm(bridge, fmt, np.ones((M, K), np.float16), W, N)
    assert np.all(Y == np.float16(K))


def test_error_codes(bridge):
    L = bridge.lib
    X = torch.zeros(64 * 256, dtype=torch.float16, device="cuda")
    W = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    Y = torch.zeros(64 * 256, dtype=torch.float16, device="cuda")
    xp, wp, yp = X.data_ptr(), W.data_ptr(), Y.data_ptr()
    xb, wb, yb = X.numel() * 2, W.numel(), Y.numel() * 2
    call = L.m4_bridge_dispatch_gemm
    assert call(None, xb, wp, wb, yp, yb, 0, 4, 64, 64) == -2
    assert call(xp + 1, xb - 1, wp, wb, yp, yb, 0, 4, 64, 64) == -2          # odd fp16 pointer
    for bad in (-1, 6, 999, -999):
        assert call(xp, xb, wp, wb, yp, yb, bad, 4, 64, 64) == -3
    assert call(xp, xb, wp, wb, yp, yb, 0, 0, 64, 64) == -4
    assert call(xp, xb, wp, wb, yp, yb, 0, 4, 48, 64) == -4                  # K % 32
    for sb in (2, 4, 5):
        assert call(xp, xb, wp, wb, yp, yb, sb, 4, 128, 64) == -4            # K % 256 for super-blocks
    assert call(xp, 4 * 64 * 2 - 2, wp, wb, yp, yb, 0, 4, 64, 64) == -2      # X too small
    assert call(xp, xb, wp, 64 * 2 * 18 - 1, yp, yb, 0, 4, 64, 64) == -2     # W too small
    assert call(xp, xb, wp, wb, yp, 4 * 64 * 2 - 2, 0, 4, 64, 64) == -2      # Y too small
    assert call(xp, xb, wp, wb, yp, yb, 0, 4, 64, 64) == 0
    with pytest.raises(RuntimeError, match="status code -3"):
        bridge.dispatch_gemm(X, W, Y, 6, 4, 64, 64)
    bridge.synchronize()


@pytest.mark.parametrize("shape", [(5, 64, 33), (9, 64, 65), (33, 256, 33), (70, 512, 65), (3, 96, 10), (40, 288, 130)])
def test_ragged_shapes(bridge, shape):
    M, K, N = shape
    g = o.RefLcg(5)
    W = g.weights(o.Q4_0, K, N)
    X = g.activations(M, K)
    Y = run_gemm(bridge, o.Q4_0, X, W, N)
    assert np.abs(Y.astype(np.float64) - o.gemm_f64(o.Q4_0, X, W, N)).max() <= TOL


def test_every_format_on_the_fallback_kernel(bridge):
    M, K, N = 17, 512, 40
    for fmt in BRIDGE_FORMATS + (o.PRISM_Q2_0,):
        g = o.RefLcg(8)
        W = g.weights(fmt, K, N)
        X = g.activations(M, K)
        bridge.lib.b200_bridge_force_generic(1)
        try:
            Y = run_gemm(bridge, fmt, X, W, N, ex=True)
        finally:
            bridge.lib.b200_bridge_force_generic(0)
        assert np.abs(Y.astype(np.float64) - o.gemm_f64(fmt, X, W, N)).max() <= TOL


@pytest.mark.parametrize("fmt", [o.MLX_4BIT_G64, o.TERNARY_ROW, o.MLX_4BIT_PLANAR])
@pytest.mark.parametrize("shape", [(33, 512, 96), (1, 4096, 200), (129, 4096, 1000), (300, 1024, 130), (40, 192, 70)])
def test_extension_layouts(bridge, fmt, shape):
    """Planar layouts 100 / 101 / 102: tensor-core path (K % 256 == 0; the K = 4096 cases split K and cut ragged
    row and token tiles) and the CUDA-core path (K = 192), which must agree with each other as well."""
    M, K, N = shape
    X, W = o.baseline_inputs(fmt, M, K, N, 3)
    gold = o.gemm_f64(fmt, X, W, N)
    Y = run_gemm(bridge, fmt, X, W, N, ex=True)
    check(Y, gold, f"fmt {fmt} {shape}")
    bridge.lib.b200_bridge_force_generic(1)
    try:
        Yg = run_gemm(bridge, fmt, X, W, N, ex=True)
    finally:
        bridge.lib.b200_bridge_force_generic(0)
    check(Yg, gold, f"fmt {fmt} {shape} generic")


@pytest.mark.parametrize("fmt", [o.MLX_4BIT_G64, o.TERNARY_ROW, o.MLX_4BIT_PLANAR])
def test_extension_layouts_swiglu(bridge, fmt):
    from gpu_util import check_swiglu
    from test_swiglu_attention_gpu import run_swiglu
    M, K, F = 130, 512, 300
    X, Wg = o.baseline_inputs(fmt, M, K, F, 8)
    _, Wu = o.baseline_inputs(fmt, M, K, F, 9)
    X = (X.astype(np.float32) * 0.25).astype(np.float16)
    out = run_swiglu(bridge, fmt, X, Wg, Wu, F)
    check_swiglu(out, o.gemm_f64(fmt, X, Wg, F), o.gemm_f64(fmt, X, Wu, F), f"swiglu fmt {fmt}")


def test_host_pointers_and_gemv(bridge):
    K, N = 512, 256
    g = o.RefLcg(3)
    W = g.weights(o.Q4_0, K, N)
    X = g.activations(33, K)
    a = run_gemm(bridge, o.Q4_0, X, W, N)
    b = run_gemm(bridge, o.Q4_0, X, W, N, host=True)           # pageable host memory in and out
    assert np.array_equal(a.view(np.uint16), b.view(np.uint16))
    Wt = torch.from_numpy(W)
    assert bridge.register_weights(Wt) == 0                     # resident copy keyed by the host pointer
    Yh = torch.zeros(33, N, dtype=torch.float16)
    bridge.dispatch_gemm(torch.from_numpy(X), Wt, Yh, o.Q4_0, 33, K, N)
    bridge.synchronize()
    assert np.array_equal(Yh.numpy().view(np.uint16), a.view(np.uint16))
    assert bridge.lib.b200_bridge_unregister_weights(Wt.data_ptr()) == 0
    y = torch.zeros(N, dtype=torch.float16, device="cuda")
    bridge.dispatch_gemv(dev(X[0]), dev(W), y, o.Q4_0, K, N)
    bridge.synchronize()
    assert np.abs(y.cpu().numpy().astype(np.float64) - o.gemm_f64(o.Q4_0, X[:1], W, N)[0]).max() <= TOL


@pytest.mark.parametrize("fmt", [o.Q4_0, o.Q4_K])
@pytest.mark.parametrize("layout", [0, 1])
def test_grouped_projections(bridge, fmt, layout):
    """Three projections of the same activations in one launch (Q, K, V): bit-identical to separate dispatches."""
    import ctypes
    M, K, D = 2048, 512, 128
    Ns = [1536, 512, 384]          # 19 weight tiles x 8 token tiles = 152 tiles: above the SM count, no K split
    g = o.RefLcg(44)
    Ws = [g.weights(fmt, K, n) for n in Ns]
    X = (g.activations(M, K).astype(np.float32) * 0.5).astype(np.float16)
    Xd = dev(X)
    Wd = [dev(w) for w in Ws]
    shape = lambda n: (n // D, M, D) if layout else (M, n)
    Yg = [torch.full(shape(n), float("nan"), dtype=torch.float16, device="cuda") for n in Ns]
    vp = ctypes.c_void_p
    rc = bridge.lib.b200_bridge_dispatch_gemm_grouped(Xd.data_ptr(), (vp * 3)(*[w.data_ptr() for w in Wd]),
                                                      (vp * 3)(*[y.data_ptr() for y in Yg]), (ctypes.c_uint32 * 3)(*Ns), 3, fmt, M, K,
                                                      layout, D)
    assert rc == 0
    bridge.synchronize()
    assert bridge.device_error() == 0
    for n, w, y in zip(Ns, Ws, Yg):
        ref = run_gemm(bridge, fmt, X, w, n, layout=layout, H=n // D if layout else 0, D=D if layout else 0)
        assert np.array_equal(y.cpu().numpy().view(np.uint16), ref.view(np.uint16))
    gold = o.gemm_f64(fmt, X[:64], Ws[2], Ns[2])
    got = Yg[2].cpu().numpy()
    got = got.transpose(1, 0, 2).reshape(M, Ns[2]) if layout else got
    check(got[:64], gold, "grouped vs oracle")
    # few tokens and a K long enough to split: the grouped launch splits K like a single projection would (partial tiles
    # of all three matrices meet in the scratch buffer) and still agrees with separate dispatches bit for bit
    K2, M2 = 1024, 64
    Xs = (g.activations(M2, K2).astype(np.float32) * 0.5).astype(np.float16)
    Ws2 = [g.weights(fmt, K2, n) for n in Ns]
    Xd2, Wd2 = dev(Xs), [dev(w) for w in Ws2]
    Y2 = [torch.full(((n // D, M2, D) if layout else (M2, n)), float("nan"), dtype=torch.float16, device="cuda") for n in Ns]
    assert bridge.lib.b200_bridge_dispatch_gemm_grouped(Xd2.data_ptr(), (vp * 3)(*[w.data_ptr() for w in Wd2]),
                                                        (vp * 3)(*[y.data_ptr() for y in Y2]), (ctypes.c_uint32 * 3)(*Ns), 3, fmt, M2, K2,
                                                        layout, D) == 0
    bridge.synchronize()
    assert bridge.device_error() == 0
    bridge.lib.b200_bridge_enable_small_kernel(0)       # single projections of this size default to the cluster kernel, which sums
    try:                                                # the K splits in another order: compare with the persistent kernel's split
        for n, w, y in zip(Ns, Ws2, Y2):
            ref = run_gemm(bridge, fmt, Xs, w, n, layout=layout, H=n // D if layout else 0, D=D if layout else 0)
            assert np.array_equal(y.cpu().numpy().view(np.uint16), ref.view(np.uint16))
    finally:
        bridge.lib.b200_bridge_enable_small_kernel(1)
    got = Y2[1].cpu().numpy()
    got = got.transpose(1, 0, 2).reshape(M2, Ns[1]) if layout else got
    check(got, o.gemm_f64(fmt, Xs, Ws2[1], Ns[1]), "grouped split-K vs oracle")


def test_host_buffers_pipeline_in_order(bridge):
    """Host buffers are staged on separate copy streams (upload of call i+1 overlaps download of call i); calls
    that hand results to each other through host memory without a synchronize must still see them in order."""
    K = N = 512
    M = 64
    g = o.RefLcg(9)
    W = g.weights(o.Q4_0, K, N)
    Wd = dev(W)
    Xs = [(g.activations(M, K).astype(np.float32) * 0.5).astype(np.float16) for _ in range(6)]
    want = [run_gemm(bridge, o.Q4_0, x, W, N) for x in Xs]
    # 1. a burst of independent calls on alternating pinned buffers, one synchronize at the end
    Xp = [torch.from_numpy(x).pin_memory() for x in Xs]
    Yp = [torch.zeros(M, N, dtype=torch.float16).pin_memory() for _ in Xs]
    for x, y in zip(Xp, Yp):
        bridge.dispatch_gemm(x, Wd, y, o.Q4_0, M, K, N)
    bridge.synchronize()
    for y, w in zip(Yp, want):
        assert np.array_equal(y.numpy().view(np.uint16), w.view(np.uint16))
    # 2. a chain through host memory: the second call reads the buffer the first one writes
    h1 = torch.zeros(M, N, dtype=torch.float16).pin_memory()
    h2 = torch.zeros(M, N, dtype=torch.float16).pin_memory()
    for rep in range(3):
        bridge.dispatch_gemm(Xp[rep], Wd, h1, o.Q4_0, M, K, N)
        bridge.dispatch_gemm(h1, Wd, h2, o.Q4_0, M, K, N)
        bridge.synchronize()
        assert np.array_equal(h1.numpy().view(np.uint16), want[rep].view(np.uint16))
        chained = run_gemm(bridge, o.Q4_0, want[rep], W, N)
        assert np.array_equal(h2.numpy().view(np.uint16), chained.view(np.uint16))
    # 3. the same buffer reused as output by back-to-back calls: the last writer wins
    for x in Xp[:4]:
        bridge.dispatch_gemm(x, Wd, h1, o.Q4_0, M, K, N)
    bridge.synchronize()
    assert np.array_equal(h1.numpy().view(np.uint16), want[3].view(np.uint16))


@pytest.mark.parametrize("fmt", [o.Q4_0, o.MLX_4BIT, o.Q4_K, o.TERNARY_1_58, o.VAR_RATE_AFFINE, o.EXL3, o.MLX_4BIT_G64,
                                 o.TERNARY_ROW, o.MLX_4BIT_PLANAR])
@pytest.mark.parametrize("M", [1, 2, 3, 4])
def test_few_token_path(bridge, fmt, M):
    """A single token runs on the CUDA-core streaming kernel (one lane per 256-element chunk of a weight row): 16
    chunks per row (two rows per warp), 56 chunks per row (lanes loop), 1 chunk per row (32 rows per warp).  Two to
    four tokens take the tensor-core path at the same shapes."""
    for K, N in ((4096, 1000), (14336, 200), (256, 130)):
        X, W = o.baseline_inputs(fmt, M, K, N, 30 + M)
        check(run_gemm(bridge, fmt, X, W, N, ex=True), o.gemm_f64(fmt, X, W, N), f"fmt {fmt} M {M} K {K}")


@pytest.mark.parametrize("fmt", [o.Q4_0, o.TERNARY_1_58])
def test_residual_unsplit_shape(bridge, fmt):
    """Residual projections that do not split K (the residual is prefetched two batches ahead in the epilogue):
    ragged token and row tiles, several tiles per CTA."""
    M, K, N = 1000, 512, 9000            # 4 token tiles x 71 row tiles = 284 work items on 148 CTAs
    g = o.RefLcg(12)
    W = g.weights(fmt, K, N)
    X = (g.activations(M, K).astype(np.float32) * 0.5).astype(np.float16)
    R = g.activations(M, N)
    Y = run_gemm(bridge, fmt, X, W, N, residual=R)
    rows = np.r_[0:40, 250:262, 990:1000]
    check(Y[rows], o.gemm_f64(fmt, X[rows], W, N) + R[rows].astype(np.float64), f"residual fmt {fmt}")
    plain = run_gemm(bridge, fmt, X, W, N)
    want = (plain.astype(np.float32) + R.astype(np.float32))
    assert np.abs(Y.astype(np.float32) - want).max() <= 2 * np.spacing(np.abs(want).max().astype(np.float16)).astype(np.float32)


def test_residual_epilogue(bridge):
    M, K, N = 130, 512, 256
    g = o.RefLcg(4)
    W = g.weights(o.Q4_0, K, N)
    X = g.activations(M, K)
    R = g.activations(M, N)
    Y = run_gemm(bridge, o.Q4_0, X, W, N, residual=R)
    gold = o.gemm_f64(o.Q4_0, X, W, N) + R.astype(np.float64)
    assert np.abs(Y.astype(np.float64) - gold).max() <= TOL


# ---- benchmark shapes (K = N = 4096; the value distributions the benchmark contract names) ----
ALL_CODECS = [o.Q4_0, o.MLX_4BIT, o.Q4_K, o.TERNARY_1_58, o.VAR_RATE_AFFINE, o.EXL3, o.PRISM_Q2_0, o.MLX_4BIT_G64, o.TERNARY_ROW,
              o.MLX_4BIT_PLANAR]


@pytest.mark.parametrize("shape", [(33, 1024, 256), (127, 2048, 130), (129, 1024, 65), (512, 3072, 300), (2, 4096, 200)])
def test_prism_q2_0_tensor_core_path(bridge, shape):
    """Prism Q2_0 (34-byte blocks of 128 two-bit codes, code 3 = +2d; the reference's quant_router_gemm_prism_q2_0_64x64,
    quant_router_kernels.metal:726-747) on the tcgen05 path: packed stages of 1024 elements, so K % 1024 == 0 here; the
    reference's own generator (codes 0..3 uniform) and tolerance, ragged row and token tiles, split K, and agreement with
    the CUDA-core kernel, which serves the other K."""
    M, K, N = shape
    g = o.RefLcg(1337)
    W = g.weights(o.PRISM_Q2_0, K, N)
    X = g.activations(M, K)
    gold = o.gemm_f64(o.PRISM_Q2_0, X, W, N)
    Y = run_gemm(bridge, o.PRISM_Q2_0, X, W, N, ex=True)
    assert np.abs(Y.astype(np.float64) - gold).max() <= TOL
    check(Y, gold, f"prism q2_0 {shape}", dev_gold=device_weight_gold(o.PRISM_Q2_0, X, W, N))
    bridge.lib.b200_bridge_force_generic(1)
    try:
        Yg = run_gemm(bridge, o.PRISM_Q2_0, X, W, N, ex=True)
    finally:
        bridge.lib.b200_bridge_force_generic(0)
    assert np.abs(Yg.astype(np.float64) - gold).max() <= TOL
    Yh = run_gemm(bridge, o.PRISM_Q2_0, X, W, N if N % 64 else N, ex=True) if N % 64 else \
        run_gemm(bridge, o.PRISM_Q2_0, X, W, N, layout=1, H=N // 64, D=64)
    if N % 64 == 0:          # head-major output is the standard output re-laid out, bit for bit
        assert np.array_equal(Yh.view(np.uint16), Y.reshape(M, N // 64, 64).transpose(1, 0, 2).copy().view(np.uint16))


@pytest.mark.parametrize("fmt", ALL_CODECS)
@pytest.mark.parametrize("M", [33, 128, 129])
def test_8b_projection_small_m(bridge, fmt, M):
    K = N = 4096
    X, W = o.baseline_inputs(fmt, M, K, N, 100 + M)
    Y = run_gemm(bridge, fmt, X, W, N, ex=fmt > 5)
    check(Y, o.gemm_f64(fmt, X, W, N), f"projection fmt {fmt} M={M} K=N=4096", dev_gold=device_weight_gold(fmt, X, W, N))


def sampled_rows(M):
    """Both ragged ends of every 256-token tile plus 40 random rows."""
    return np.unique(np.concatenate([np.arange(0, M, 256), np.arange(255, M, 256), np.random.default_rng(0).integers(0, M, 40)]))


@pytest.mark.parametrize("fmt", ALL_CODECS)
def test_8b_projection_m2048(bridge, fmt):
    """Full size, every codec of the tensor-core path: sampled token rows (including both ragged ends of every
    256-token tile) against the oracle, and against the gold built from the kernel's exact fp16 weights under the
    strict criterion; plus two size-independent properties: runs are bit-reproducible, and permuting token rows
    permutes output rows bit for bit (each output is an independent K-ordered sum)."""
    M, K, N = 2048, 4096, 4096
    X, W = o.baseline_inputs(fmt, M, K, N, 7)
    Y = run_gemm(bridge, fmt, X, W, N, ex=fmt > 5)
    rows = sampled_rows(M)
    check(Y[rows], o.gemm_f64(fmt, X[rows], W, N), f"projection fmt {fmt} M=2048 K=N=4096", dev_gold=device_weight_gold(fmt, X[rows], W, N))
    assert np.array_equal(Y.view(np.uint16), run_gemm(bridge, fmt, X, W, N, ex=fmt > 5).view(np.uint16))
    perm = np.random.default_rng(1).permutation(M)
    Yp = run_gemm(bridge, fmt, X[perm], W, N, ex=fmt > 5)
    assert np.array_equal(Yp.view(np.uint16), Y[perm].view(np.uint16))


@pytest.mark.parametrize("fmt", [o.Q4_0, o.MLX_4BIT_PLANAR, o.TERNARY_ROW, o.PRISM_Q2_0])
def test_cta_pair_launch_is_bit_identical(bridge, fmt):
    """Launches with token tiles of 128 to 256 rows, no K split and an even number of weight tiles run as CTA pairs (one 256-row MMA
    over two SMs, operands handed over between the two CTAs): the same products in the same order as with one CTA per MMA,
    so the outputs must agree bit for bit -- plain, with a fused residual, head-major, and with a ragged last token tile."""
    L = bridge.lib
    M, K, N, D = 2000, 1024, 1536, 128          # 8 token tiles (the last one ragged) x 12 weight tiles: above the SM count, no K split
    X, W = o.baseline_inputs(fmt, M, K, N, 21)
    R = (np.random.default_rng(3).standard_normal((M, N)) * 0.5).astype(np.float16)
    outs = {}
    for pair in (1, 0):
        L.b200_bridge_enable_pair_kernel(pair)
        try:
            a = run_gemm(bridge, fmt, X, W, N, ex=True)
            used = L.b200_bridge_last_launch_pair()
            b = run_gemm(bridge, fmt, X, W, N, residual=R)
            c = run_gemm(bridge, fmt, X, W, N, layout=1, H=N // D, D=D)
        finally:
            L.b200_bridge_enable_pair_kernel(1)
        assert (used > 0) == bool(pair)
        outs[pair] = (a, b, c)
    for x, y in zip(outs[0], outs[1]):
        assert np.array_equal(x.view(np.uint16), y.view(np.uint16))
    gold = o.gemm_f64(fmt, X, W, N)
    check(outs[1][0], gold, f"CTA pairs fmt {fmt} M={M}", dev_gold=device_weight_gold(fmt, X, W, N))
    check(outs[1][1], gold + R.astype(np.float64), f"CTA pairs fmt {fmt} M={M} + residual")
    # narrower token tiles (7 of 224 rows) pair up as well; an odd number of weight tiles keeps one CTA per MMA
    X2, W2 = o.baseline_inputs(fmt, 1560, K, 2048, 22)
    check(run_gemm(bridge, fmt, X2, W2, 2048, ex=True), o.gemm_f64(fmt, X2, W2, 2048), f"CTA pairs fmt {fmt} M=1560")
    assert L.b200_bridge_last_launch_pair() > 0
    X3, W3 = o.baseline_inputs(fmt, 2048, K, 2432, 23)
    check(run_gemm(bridge, fmt, X3, W3, 2432, ex=True), o.gemm_f64(fmt, X3, W3, 2432), f"fmt {fmt} 19 weight tiles")
    assert L.b200_bridge_last_launch_pair() == 0


@pytest.mark.parametrize("fmt", ALL_CODECS)
def test_few_token_kernels_agree(bridge, fmt):
    """The cluster kernel (weights unpacked into tensor memory, K split over a thread-block cluster, partial tiles summed by
    the cluster's CTAs out of the L2-resident scratch) against the persistent kernel (split-K through a scratch buffer) on the same inputs: both
    within tolerance of the oracle, and of each other within the fp32 summation-order difference (one fp16 ulp)."""
    K, N = 4096, 1000 if fmt != o.PRISM_Q2_0 else 1024
    for M in (5, 33, 100, 128):
        X, W = o.baseline_inputs(fmt, M, K, N, 60 + M)
        gold = o.gemm_f64(fmt, X, W, N)
        Ya = run_gemm(bridge, fmt, X, W, N, ex=True)
        bridge.lib.b200_bridge_enable_small_kernel(0)
        try:
            Yb = run_gemm(bridge, fmt, X, W, N, ex=True)
        finally:
            bridge.lib.b200_bridge_enable_small_kernel(1)
        rf = 2.0 if fmt == o.VAR_RATE_AFFINE else 1.0      # three fp16 roundings per weight in that codec (see gpu_util.tolerance)
        check(Ya, gold, f"few-token cluster kernel fmt {fmt} M={M}", dev_gold=device_weight_gold(fmt, X, W, N), rms_factor=rf)
        check(Yb, gold, f"few-token persistent kernel fmt {fmt} M={M}", rms_factor=rf)
        ulp = np.spacing(np.abs(gold).astype(np.float16)).astype(np.float32)
        assert np.all(np.abs(Ya.astype(np.float32) - Yb.astype(np.float32)) <= np.maximum(2 * ulp, TOL / 4)), f"fmt {fmt} M={M}"
    # head-major output and a fused residual on the cluster kernel
    M, D = 70, 64
    X, W = o.baseline_inputs(fmt, M, K, 1024, 9)
    Y = run_gemm(bridge, fmt, X, W, 1024, ex=True)
    Yh = run_gemm(bridge, fmt, X, W, 1024, layout=1, H=1024 // D, D=D)
    assert np.array_equal(Yh.view(np.uint16), Y.reshape(M, 1024 // D, D).transpose(1, 0, 2).copy().view(np.uint16))
    R = o.RefLcg(4).activations(M, 1024)
    Yr = run_gemm(bridge, fmt, X, W, 1024, residual=R)
    check(Yr, o.gemm_f64(fmt, X, W, 1024) + R.astype(np.float64), f"few-token residual fmt {fmt}")


def test_1b_reference_config_q4_0(bridge):
    # the CPU-reference configuration: M=33, K=N=2048, d ~ U(0.005, 0.02), X ~ N(0,1)
    X, W = o.baseline_inputs(o.Q4_0, 33, 2048, 2048, 42)
    check(run_gemm(bridge, o.Q4_0, X, W, 2048), o.gemm_f64(o.Q4_0, X, W, 2048), "config 1: q4_0 M=33 K=N=2048",
          dev_gold=device_weight_gold(o.Q4_0, X, W, 2048))


@pytest.mark.parametrize("fmt", [o.TERNARY_1_58, o.TERNARY_ROW])
@pytest.mark.parametrize("M", [128, 2048])
def test_ternary_n14336(bridge, fmt, M):
    """The ternary up-projection shape (K=4096, N=14336) at both token counts, both ternary layouts; at M=2048 sampled
    token rows.  Column shards of this projection are independent: rows [r*N/8, (r+1)*N/8) of the packed matrix give
    columns of the same range of Y bit for bit (what the N-sharded multi-GPU run relies on)."""
    K, N = 4096, 14336
    X, W = o.baseline_inputs(fmt, M, K, N, 9)
    Y = run_gemm(bridge, fmt, X, W, N, ex=fmt > 5)
    rows = np.arange(M) if M <= 128 else sampled_rows(M)
    check(Y[rows], o.gemm_f64(fmt, X[rows], W, N), f"ternary fmt {fmt} M={M} N=14336", dev_gold=device_weight_gold(fmt, X[rows], W, N))
    from m4_prefill_engine_b200.layer import shard_rows_any
    for r in (0, 5):
        Ws = shard_rows_any(W, fmt, K, N, r, 8)
        Ys = run_gemm(bridge, fmt, X, Ws, N // 8, ex=fmt > 5)
        whole = Y[:, r * (N // 8):(r + 1) * (N // 8)]
        if M >= 2048:        # same plan (no K split) for the shard and the whole matrix: the same bits
            assert np.array_equal(Ys.view(np.uint16), whole.view(np.uint16))
        else:                # few tokens: the narrow shard splits K (fp32 partial sums added in split order), the whole matrix does not
            assert np.abs(Ys.astype(np.float32) - whole.astype(np.float32)).max() <= np.spacing(np.float16(np.abs(whole).max())).astype(np.float32)
