"""Decoder layer and the Linear wrapper on the GPU against the oracle's layer gold
(bench_8b_engine.mm:376-705 verifies its pipeline against cpu_reference_prefill_layer the same way)."""
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle as o
from gpu_util import PARITY_REPORT, TOL, dev, parity_stats

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden"


SHRINK = {o.MLX_4BIT: 0.06, o.Q4_K: 0.03, o.TERNARY_1_58: 1.0}


def layer_weights(fmt, K, H, Hkv, D, F, seed=1337):
    g = o.RefLcg(seed)
    shapes = {"q": (H * D, K), "k": (Hkv * D, K), "v": (Hkv * D, K), "o": (K, H * D), "gate": (F, K), "up": (F, K), "down": (K, F)}
    if fmt == o.Q4_0:   # the reference layer's own scale range (bench_8b_engine.mm:44-53)
        return {n: g.q4_0_bench(k, r, 0.003, 0.0003) for n, (r, k) in shapes.items()}, g
    # other formats: the reference's generator ranges, with the fp16 scale fields shrunk so that a whole
    # layer (two residual blocks deep) stays far inside the fp16 range
    out = {}
    for n, (r, k) in shapes.items():
        be, bb = o.BLOCK[fmt]
        blocks = g.weights(fmt, k, r).reshape(-1, bb)
        nfields = 1 if fmt == o.TERNARY_1_58 else 2          # d (and bias / dmin)
        hdr = blocks[:, :2 * nfields].copy().view(np.float16).astype(np.float32) * SHRINK[fmt]
        blocks[:, :2 * nfields] = hdr.astype(np.float16).view(np.uint8)
        out[n] = blocks.reshape(-1)
    return out, g


def layer_gold_rows(X, w, n1, n2, rows, H, Hkv, D, F, eps, theta):
    """The oracle's Llama-style layer (Q4_0, RMSNorm, RoPE, Q8_0 KV) for selected token rows only: keys and values of
    every token (they are needed by late queries), then per selected row the query projection, attention over keys
    0..row, O projection + residual, and the MLP block, with the fp16 roundings of o.layer (oracle.cpp, orc_layer)."""
    M, K = X.shape
    fmt, scale = o.Q4_0, D ** -0.5
    xn = o.rmsnorm(X, n1, eps)
    kv = []
    for name in ("k", "v"):
        t = o.gemm(fmt, xn, w[name], Hkv * D, direct_head=True, H=Hkv, D=D)
        if name == "k":
            t = o.rope(t, theta, 0)
        kv.append(o.dequantize_q8_0(o.quantize_q8_0(t), t.shape))
    out = np.empty((len(rows), K), np.float16)
    for i, r in enumerate(rows):
        q = o.rope(o.gemm(fmt, xn[r:r + 1], w["q"], H * D, direct_head=True, H=H, D=D), theta, r)
        a = o.attention(q, kv[0][:, :r + 1], kv[1][:, :r + 1], scale, pos0=r, tokens_major=True)
        x_mid = (X[r:r + 1].astype(np.float64) + o.gemm_f64(fmt, a, w["o"], K)).astype(np.float16)
        act = o.swiglu_fused(fmt, o.rmsnorm(x_mid, n2, eps), w["gate"], w["up"], F)
        out[i] = (x_mid.astype(np.float64) + o.gemm_f64(fmt, act, w["down"], K)).astype(np.float16)[0]
    return out


def run_layer(pkg, cfg_kwargs, X, w, norms=None, host_io=False, fused_kv=False):
    from m4_prefill_engine_b200.layer import TransformerLayerConfig, TransformerLayerCoordinator
    cfg = TransformerLayerConfig(**cfg_kwargs)
    layer = TransformerLayerCoordinator(cfg)
    assert layer.initialize_pipelines()
    layer.set_fused_kv_epilogue(fused_kv)
    wd = {k: dev(v) for k, v in w.items()}
    keep = []
    if norms is not None:
        keep = [dev(norms[0]), dev(norms[1])]
        layer.set_norm_weights(*keep)
    Xd = torch.from_numpy(X) if host_io else dev(X)
    Yd = torch.zeros(X.shape, dtype=torch.float16, device="cpu" if host_io else "cuda")
    layer.forward(Xd, wd["q"], wd["k"], wd["v"], wd["o"], wd["gate"], wd["up"], wd["down"], Yd)
    layer.bridge.synchronize()
    assert layer.bridge.device_error() == 0
    n = layer.kernels_per_forward()
    layer.close()
    return Yd.cpu().numpy(), n


def test_layer_reference_fixture(bridge, pkg):
    z = np.load(GOLD / "layer_q4_0.npz")
    X = z["X"].view(np.float16)
    w = dict(zip(("q", "k", "v", "o", "gate", "up", "down"), (z[f"W{i}"] for i in range(7))))
    Y, n = run_layer(pkg, dict(M=24, K=256, H=4, D=64, N_mlp=512, attn_scale=0.125), X, w)
    # the reference's pipeline bench passes at 0.05 against this gold (bench_8b_engine.mm:694)
    assert np.abs(Y.astype(np.float32) - z["Y"].view(np.float16).astype(np.float32)).max() <= TOL
    assert n in (5, 7)   # q+k+v (one grouped launch where the shape fills the GPU, else three), attention, o(+residual), swiglu, down(+residual): residual adds and transposes are fused away


@pytest.mark.parametrize("fmt", [o.Q4_0, o.MLX_4BIT, o.Q4_K, o.TERNARY_1_58])
@pytest.mark.parametrize("M", [33, 129])
def test_layer_reference_semantics(bridge, pkg, fmt, M):
    K, H, D, F = 512, 8, 64, 768
    w, g = layer_weights(fmt, K, H, H, D, F)
    X = g.activations(M, K)
    Y, _ = run_layer(pkg, dict(M=M, K=K, H=H, D=D, N_mlp=F, attn_scale=D ** -0.5, weight_format=fmt), X, w)
    gold = o.layer(fmt, X, w["q"], w["k"], w["v"], w["o"], w["gate"], w["up"], w["down"], H, H, D, F, D ** -0.5)
    diff = np.abs(Y.astype(np.float64) - gold.astype(np.float64))
    rms = float(np.sqrt(np.mean(gold.astype(np.float64) ** 2)))
    assert diff.max() <= max(TOL, 2.0 ** -7 * rms), f"max-abs {diff.max()} rms {rms}"


@pytest.mark.parametrize("M", [129, 600])
def test_layer_mlx_planar_weights(bridge, pkg, M):
    """The layer on the planar group-32 MLX layout of the reference's layer benchmarks (bench_all_scales.mm:62-95,
    kernels gemm_mma_mlx_4bit_64x64 / qkv_head_gemm_mma_mlx_4bit_64x64 / swiglu_mma_mlx_4bit_dual_simd): the same
    weights as 20-byte blocks and as three planes give the oracle's layer within tolerance, and each other closely
    (the two codecs produce the same fp16 weights; the K-split plans of the launches may differ)."""
    K, H, D, F = 512, 8, 64, 768
    w, g = layer_weights(o.MLX_4BIT, K, H, H, D, F)
    shapes = {"q": (H * D, K), "k": (H * D, K), "v": (H * D, K), "o": (K, H * D), "gate": (F, K), "up": (F, K), "down": (K, F)}
    wp = {n: o.mlx_aos_to_planar(w[n], k, r) for n, (r, k) in shapes.items()}
    X = g.activations(M, K)
    kw = dict(M=M, K=K, H=H, D=D, N_mlp=F, attn_scale=D ** -0.5)
    Ya, _ = run_layer(pkg, dict(kw, weight_format=o.MLX_4BIT), X, w)
    Yp, _ = run_layer(pkg, dict(kw, weight_format=o.MLX_4BIT_PLANAR), X, wp)
    gold = o.layer(o.MLX_4BIT_PLANAR, X, wp["q"], wp["k"], wp["v"], wp["o"], wp["gate"], wp["up"], wp["down"], H, H, D, F, D ** -0.5)
    assert np.array_equal(gold, o.layer(o.MLX_4BIT, X, w["q"], w["k"], w["v"], w["o"], w["gate"], w["up"], w["down"], H, H, D, F, D ** -0.5))
    rms = float(np.sqrt(np.mean(gold.astype(np.float64) ** 2)))
    for Y, what in ((Ya, "blocks"), (Yp, "planes")):
        diff = np.abs(Y.astype(np.float64) - gold.astype(np.float64))
        PARITY_REPORT.append(parity_stats(Y, gold.astype(np.float64), f"layer mlx {what} M={M}"))
        assert diff.max() <= max(TOL, 2.0 ** -7 * rms), f"{what}: max-abs {diff.max()} rms {rms}"
    assert np.abs(Ya.astype(np.float64) - Yp.astype(np.float64)).max() <= max(TOL, 2.0 ** -7 * rms) / 2


@pytest.mark.parametrize("host_io", [False, True])
def test_layer_llama_style(bridge, pkg, host_io):
    """RMSNorm + grouped-query attention + rotary embedding + Q8_0 KV, the benchmark's layer (small shape)."""
    M, K, H, Hkv, D, F = 100, 512, 4, 2, 128, 1024
    w, g = layer_weights(o.Q4_0, K, H, Hkv, D, F)
    X = g.activations(M, K)
    rng = np.random.default_rng(1)
    n1 = (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float16)
    n2 = (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float16)
    kw = dict(M=M, K=K, H=H, D=D, N_mlp=F, attn_scale=D ** -0.5, num_kv_heads=Hkv, rms_eps=1e-5, rope_theta=500000.0, kv_q8_0=True)
    Y, _ = run_layer(pkg, kw, X, w, (n1, n2), host_io=host_io)
    gold = o.layer(o.Q4_0, X, w["q"], w["k"], w["v"], w["o"], w["gate"], w["up"], w["down"], H, Hkv, D, F, D ** -0.5,
                   rms_eps=1e-5, norm1=n1, norm2=n2, rope_theta=500000.0, kv_q8=True)
    diff = np.abs(Y.astype(np.float64) - gold.astype(np.float64))
    assert diff.max() <= 2 * TOL, f"max-abs {diff.max()}"


def test_layer_8b_full_size(bridge, pkg):
    """The benchmark's layer at its full size (M=2048, K=4096, 32/8 heads, D=128, F=14336, Q4_0): grouped Q/K/V launch,
    tensor-memory attention over 16 key tiles, residual epilogues.  Checked through two size-independent properties:
    a causal layer's first rows depend on the first tokens only, so rows [0, 48) must match the oracle's layer run on
    48 tokens; and changing the tokens from 1500 on must leave every earlier output row bit-identical."""
    M, K, H, Hkv, D, F = 2048, 4096, 32, 8, 128, 14336
    rng = np.random.default_rng(7)

    def q4_0(rows, cols):                     # the reference layer's scale range (bench_8b_engine.mm:44-53)
        nb = rows * cols // 32
        W = rng.integers(0, 256, (nb, 18), dtype=np.uint8)
        W[:, 0:2] = rng.uniform(0.0003, 0.0033, nb).astype(np.float16).view(np.uint8).reshape(-1, 2)
        return W.reshape(-1)
    w = {"q": q4_0(H * D, K), "k": q4_0(Hkv * D, K), "v": q4_0(Hkv * D, K), "o": q4_0(K, H * D), "gate": q4_0(F, K), "up": q4_0(F, K),
         "down": q4_0(K, F)}
    X = (rng.standard_normal((M, K), dtype=np.float32) * 0.35).astype(np.float16)
    n1 = (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float16)
    n2 = (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float16)
    kw = dict(M=M, K=K, H=H, D=D, N_mlp=F, attn_scale=D ** -0.5, num_kv_heads=Hkv, rms_eps=1e-5, rope_theta=500000.0, kv_q8_0=True)
    Y, n = run_layer(pkg, kw, X, w, (n1, n2))
    # rmsnorm; Q+K+V; rotary embedding + Q8_0 K/V (and K, V as the cache gives them back); attention; O; residual + rmsnorm;
    # gate/up; down + residual
    assert n == 8 and np.all(np.isfinite(Y.astype(np.float32)))
    Yf, nf = run_layer(pkg, kw, X, w, (n1, n2), fused_kv=True)         # the same work inside the Q+K+V projection's epilogue
    assert nf == 8 and np.array_equal(Y.view(np.uint16), Yf.view(np.uint16))
    R = 48
    gold = o.layer(o.Q4_0, X[:R], w["q"], w["k"], w["v"], w["o"], w["gate"], w["up"], w["down"], H, Hkv, D, F, D ** -0.5,
                   rms_eps=1e-5, norm1=n1, norm2=n2, rope_theta=500000.0, kv_q8=True)
    diff = np.abs(Y[:R].astype(np.float64) - gold.astype(np.float64))
    assert diff.max() <= 2 * TOL, f"max-abs {diff.max()}"
    PARITY_REPORT.append(parity_stats(Y[:R], gold.astype(np.float64), "8B layer M=2048, rows [0,48)"))
    # late rows: query positions that attend over up to 16 key tiles, each checked against the oracle run for that
    # row over the full key/value cache
    late = [2047, 2046, 1920, 1793, 1500, 1279, 1024, 1023, 777, 512, 300, 255, 129, 128, 127, 64]
    gold_late = layer_gold_rows(X, w, n1, n2, late, H, Hkv, D, F, 1e-5, 500000.0)
    dl = np.abs(Y[late].astype(np.float64) - gold_late.astype(np.float64))
    PARITY_REPORT.append(parity_stats(Y[late], gold_late.astype(np.float64), "8B layer M=2048, 16 late rows"))
    assert dl.max() <= 2 * TOL, f"late rows: max-abs {dl.max()} at row {late[int(dl.max(axis=1).argmax())]}"
    X2 = X.copy()
    X2[1500:] = (rng.standard_normal((M - 1500, K), dtype=np.float32) * 0.35).astype(np.float16)
    Y2, _ = run_layer(pkg, kw, X2, w, (n1, n2))
    assert np.array_equal(Y[:1500].view(np.uint16), Y2[:1500].view(np.uint16))
    assert not np.array_equal(Y[1500:].view(np.uint16), Y2[1500:].view(np.uint16))


def test_rmsnorm_and_rope_ops(bridge):
    L = bridge.lib
    import ctypes
    g = o.RefLcg(12)
    X = g.activations(37, 512)
    wt = (1.0 + 0.2 * np.random.default_rng(2).standard_normal(512)).astype(np.float16)
    Xd, wd = dev(X), dev(wt)
    Yd = torch.zeros_like(Xd)
    assert L.b200_bridge_rmsnorm(Xd.data_ptr(), wd.data_ptr(), Yd.data_ptr(), 37, 512, ctypes.c_float(1e-5)) == 0
    bridge.synchronize()
    gold = o.rmsnorm(X, wt, 1e-5).astype(np.float32)
    assert np.abs(Yd.cpu().numpy().astype(np.float32) - gold).max() <= 2e-3     # two fp16 roundings, values ~3
    Q = g.activations(3, 50, 128)
    Qd = dev(Q)
    assert L.b200_bridge_rope(Qd.data_ptr(), 3, 50, 128, ctypes.c_float(500000.0), 7) == 0
    bridge.synchronize()
    assert np.abs(Qd.cpu().numpy().astype(np.float32) - o.rope(Q, 500000.0, 7).astype(np.float32)).max() <= 2e-3


def test_layer_tensor_parallel_emulated_on_one_gpu(bridge, pkg):
    """Two tensor-parallel ranks emulated one after the other on a single GPU: the all-reduce hook of each
    rank adds the other rank's partial sums, which were captured in an earlier pass.  Three passes make
    both reductions consistent; the result must match the single-GPU layer and the oracle."""
    from m4_prefill_engine_b200.layer import TransformerLayerConfig, TransformerLayerCoordinator, shard_layer_weights
    M, K, H, Hkv, D, F, tp = 70, 512, 4, 2, 128, 1024, 2
    w, g = layer_weights(o.Q4_0, K, H, Hkv, D, F)
    X = g.activations(M, K)
    base = dict(M=M, K=K, H=H, D=D, N_mlp=F, attn_scale=D ** -0.5, num_kv_heads=Hkv, kv_q8_0=True, rope_theta=10000.0)
    single, _ = run_layer(pkg, base, X, w)
    stream = torch.cuda.ExternalStream(bridge.lib.b200_bridge_stream())
    cfg = TransformerLayerConfig(**base, tp_size=tp)
    Xd = dev(X)
    stash = [[None, None] for _ in range(tp)]       # stash[rank][call] = that rank's partial sums
    outs = [None] * tp
    for _pass in range(3):
        new_stash = [[None, None] for _ in range(tp)]
        for r in range(tp):
            sw = {k: dev(v) for k, v in shard_layer_weights(o.Q4_0, w, cfg, r, tp).items()}
            layer = TransformerLayerCoordinator(cfg)
            calls = {"n": 0}

            def hook(ptr, count, r=r, calls=calls, new_stash=new_stash):
                class Raw:
                    __cuda_array_interface__ = {"shape": (count,), "typestr": "<f4", "data": (ptr, False), "version": 3}
                t = torch.as_tensor(Raw(), device="cuda")
                with torch.cuda.stream(stream):
                    new_stash[r][calls["n"]] = t.clone()
                    other = stash[1 - r][calls["n"]]
                    if other is not None:
                        t.add_(other)
                calls["n"] += 1
            layer.set_allreduce(hook)
            Yd = torch.zeros_like(Xd)
            layer.forward(Xd, sw["q"], sw["k"], sw["v"], sw["o"], sw["gate"], sw["up"], sw["down"], Yd)
            bridge.synchronize()
            outs[r] = Yd.cpu().numpy()
            layer.close()
        stash = new_stash
    assert np.array_equal(outs[0].view(np.uint16), outs[1].view(np.uint16))       # both ranks hold the same result
    assert np.abs(outs[0].astype(np.float32) - single.astype(np.float32)).max() <= 2e-3
    gold = o.layer(o.Q4_0, X, w["q"], w["k"], w["v"], w["o"], w["gate"], w["up"], w["down"], H, Hkv, D, F, D ** -0.5,
                   rope_theta=10000.0, kv_q8=True)
    assert np.abs(outs[0].astype(np.float64) - gold.astype(np.float64)).max() <= 2 * TOL


def test_linear_wrapper(bridge, pkg):
    from m4_prefill_engine_b200.modules import M4QuantizedLinear
    K, N = 512, 192
    g = o.RefLcg(6)
    W = g.weights(o.Q4_0, K, N)
    lin = M4QuantizedLinear.from_quantized(W, "q4_0", K, N)
    x = torch.from_numpy(g.activations(2, 3, 5, K)).cuda()
    y = lin(x)
    assert y.shape == (2, 3, 5, N) and y.dtype == torch.float16
    gold = o.gemm_f64(o.Q4_0, x.reshape(-1, K).cpu().numpy(), W, N).reshape(2, 3, 5, N)
    assert np.abs(y.cpu().numpy().astype(np.float64) - gold).max() <= TOL
    assert lin(torch.zeros(0, K, device="cuda")).shape == (0, N)                     # empty input: no bridge call
    assert lin(torch.zeros(4, 0, K)).shape == (4, 0, N)
    y1 = lin(x[0, 0, 0].float())                                                     # 1-D, non-fp16 -> cast, GEMV
    assert y1.shape == (N,) and np.abs(y1.cpu().numpy().astype(np.float64) - gold[0, 0, 0]).max() <= TOL
    with pytest.raises(ValueError):
        lin(torch.zeros(3, K + 32, device="cuda"))
    lin.init_synthetic_weights()
    assert torch.all(lin(torch.ones(7, K, device="cuda")) == K)
    yc = lin(torch.ones(2, K), check_finite=True)                                    # host input, tripwire on
    assert torch.all(yc.cpu() == K)
