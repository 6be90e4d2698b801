"""Fused SwiGLU, Q8_0 KV compression and causal attention on the GPU against the oracle
(brick3_swiglu_bench.mm:268-426 and brick4_attn_bench.mm:216-328 verify the same way)."""
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle as o
from gpu_util import TOL, cfloat, check, check_swiglu, dev, run_gemm

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden"


def run_swiglu(br, fmt, X, Wg, Wu, F):
    M, K = X.shape
    out = torch.full((M, F), float("nan"), dtype=torch.float16, device="cuda")
    br.dispatch_swiglu(dev(X), dev(Wg), dev(Wu), out, fmt, M, K, F)
    br.synchronize()
    assert br.device_error() == 0
    return out.cpu().numpy()


def test_swiglu_brick3_fixture(bridge):
    z = np.load(GOLD / "swiglu_brick3.npz")
    A = z["A"].view(np.float16)
    out = run_swiglu(bridge, o.Q4_0, A, z["Wg"], z["Wu"], z["Out"].shape[1])
    gold = z["Out"].view(np.float16).astype(np.float64)
    # the reference's bench passes its fused kernels at 0.05 on this distribution (brick3_swiglu_bench.mm:419)
    assert np.abs(out.astype(np.float64) - gold).max() <= 0.05
    check(out, gold, "brick3 fixture")


@pytest.mark.parametrize("fmt", [o.Q4_0, o.MLX_4BIT, o.Q4_K, o.TERNARY_1_58, o.VAR_RATE_AFFINE, o.EXL3])
@pytest.mark.parametrize("M", [33, 128, 129, 300])
def test_swiglu_formats(bridge, fmt, M):
    K, F = 512, 384
    g = o.RefLcg(2026)
    Wg = g.weights(fmt, K, F)
    Wu = g.weights(fmt, K, F)
    X = g.activations(M, K)
    out = run_swiglu(bridge, fmt, X, Wg, Wu, F)
    check_swiglu(out, o.gemm_f64(fmt, X, Wg, F), o.gemm_f64(fmt, X, Wu, F), f"swiglu fmt {fmt} M {M}")
    gold = o.swiglu_fused(fmt, X, Wg, Wu, F).astype(np.float64)       # the fused gold agrees with the product of golds
    assert np.abs(out.astype(np.float64) - gold).max() <= 0.05 * max(1.0, float(np.abs(gold).max()) / 8)


def test_swiglu_equals_two_gemms(bridge):
    # split form: silu(gate) * up computed from two separate projections (cpu_gold_reference.h:499-511)
    from gpu_util import run_gemm
    M, K, F = 64, 512, 256
    g = o.RefLcg(11)
    Wg = g.weights(o.Q4_0, K, F); Wu = g.weights(o.Q4_0, K, F); X = g.activations(M, K)
    fused = run_swiglu(bridge, o.Q4_0, X, Wg, Wu, F)
    split = o.swiglu_elementwise(run_gemm(bridge, o.Q4_0, X, Wg, F), run_gemm(bridge, o.Q4_0, X, Wu, F))
    assert np.abs(fused.astype(np.float32) - split.astype(np.float32)).max() <= 2 * TOL


def test_swiglu_8b_q4k_sampled(bridge):
    """Benchmark shape K=4096 -> F=14336, Q4_K, M=2048: sampled rows against the oracle.  Inputs are scaled
    (X ~ N(0,1) * 0.05) so that silu(g)*u stays inside the fp16 range with these weight magnitudes."""
    M, K, F = 2048, 4096, 14336
    rng = np.random.default_rng(5)
    X = (rng.standard_normal((M, K), dtype=np.float32) * 0.05).astype(np.float16)
    Wg = o.baseline_weights(o.Q4_K, K, F, rng)
    Wu = o.baseline_weights(o.Q4_K, K, F, rng)
    out = run_swiglu(bridge, o.Q4_K, X, Wg, Wu, F)
    rows = np.array([0, 127, 128, 1000, 2047])
    check_swiglu(out[rows], o.gemm_f64(o.Q4_K, X[rows], Wg, F), o.gemm_f64(o.Q4_K, X[rows], Wu, F), "8B swiglu")


# ---- Q8_0 KV ----
def test_quantize_kv_bit_exact(bridge):
    L = bridge.lib
    z = np.load(GOLD / "attention_q8.npz")
    for name, qname in (("K", "Kq"), ("V", "Vq")):
        x = z[name].view(np.float16)
        xd = dev(x)
        qd = torch.zeros(x.size // 32 * 34, dtype=torch.uint8, device="cuda")
        assert L.b200_bridge_quantize_kv_q8_0(xd.data_ptr(), x.size * 2, qd.data_ptr(), qd.numel(), x.size) == 0
        bridge.synchronize()
        assert np.array_equal(qd.cpu().numpy(), z[qname])
    g = o.RefLcg(9)
    x = g.activations(5000 * 32)
    x[:64] = 0
    x[64:96] = np.float16(6e-8)
    x[100] = np.float16(65504)
    x[200:232] = np.float16(-1.0)
    xd = dev(x)
    qd = torch.zeros(x.size // 32 * 34, dtype=torch.uint8, device="cuda")
    assert L.b200_bridge_quantize_kv_q8_0(xd.data_ptr(), x.size * 2, qd.data_ptr(), qd.numel(), x.size) == 0
    dd = torch.zeros(x.size, dtype=torch.float16, device="cuda")
    assert L.b200_bridge_dequantize_q8_0(qd.data_ptr(), qd.numel(), dd.data_ptr(), x.size * 2, x.size) == 0
    bridge.synchronize()
    gq = o.quantize_q8_0(x)
    assert np.array_equal(qd.cpu().numpy(), gq)
    assert np.array_equal(dd.cpu().numpy().view(np.uint16), o.dequantize_q8_0(gq, x.shape).view(np.uint16))
    assert L.b200_bridge_quantize_kv_q8_0(xd.data_ptr(), x.size * 2, qd.data_ptr(), qd.numel(), 33) == -4


def run_attn(br, Q, K, V, scale, Hkv, Mkv, pos0=0, tokens_major=False, kv_fp16=False):
    Hq, M, D = Q.shape
    shape = (M, Hq * D) if tokens_major else (Hq, M, D)
    O = torch.full(shape, float("nan"), dtype=torch.float16, device="cuda")
    Kd, Vd, Qd = dev(K), dev(V), dev(Q)
    rc = br.lib.b200_bridge_dispatch_attention_q8kv(Qd.data_ptr(), Kd.data_ptr(), Vd.data_ptr(), O.data_ptr(), Hq, Hkv, M, Mkv, D,
                                                    cfloat(scale), pos0, int(tokens_major), int(kv_fp16))
    assert rc == 0
    br.synchronize()
    return O.cpu().numpy()


def test_attention_fixture(bridge):
    z = np.load(GOLD / "attention_q8.npz")
    Q = z["Q"].view(np.float16)
    O = run_attn(bridge, Q, z["Kq"], z["Vq"], 0.125, Q.shape[0], Q.shape[1])
    assert np.abs(O.astype(np.float32) - z["O"].view(np.float16).astype(np.float32)).max() <= TOL


@pytest.mark.parametrize("case", [
    dict(Hq=4, Hkv=4, M=64, D=64), dict(Hq=4, Hkv=4, M=96, D=64), dict(Hq=4, Hkv=4, M=33, D=128),
    dict(Hq=8, Hkv=2, M=129, D=128), dict(Hq=8, Hkv=2, M=200, D=128, tokens_major=True),
    dict(Hq=3, Hkv=3, M=1, D=64), dict(Hq=4, Hkv=1, M=100, D=128, kv_fp16=True), dict(Hq=4, Hkv=4, M=64, D=64, kv_fp16=True),
    dict(Hq=4, Hkv=2, M=31, D=128, Mkv=95, pos0=64), dict(Hq=32, Hkv=8, M=512, D=128),
    dict(Hq=8, Hkv=1, M=77, D=64), dict(Hq=16, Hkv=2, M=130, D=128, tokens_major=True), dict(Hq=6, Hkv=2, M=90, D=128),
    dict(Hq=2, Hkv=2, M=300, D=128, kv_fp16=True), dict(Hq=8, Hkv=4, M=257, D=64, Mkv=300, pos0=43),
])
def test_attention_cases(bridge, case):
    Hq, Hkv, M, D = case["Hq"], case["Hkv"], case["M"], case["D"]
    Mkv, pos0 = case.get("Mkv", M), case.get("pos0", 0)
    tm, f16 = case.get("tokens_major", False), case.get("kv_fp16", False)
    g = o.RefLcg(2026)
    Q = g.activations(Hq, M, D); K = g.activations(Hkv, Mkv, D); V = g.activations(Hkv, Mkv, D)
    scale = float(D) ** -0.5
    if f16:
        gold = o.attention(Q, K, V, scale, pos0, tm)
        O = run_attn(bridge, Q, K, V, scale, Hkv, Mkv, pos0, tm, True)
    else:
        Kq, Vq = o.quantize_q8_0(K), o.quantize_q8_0(V)
        gold = o.attention(Q, o.dequantize_q8_0(Kq, K.shape), o.dequantize_q8_0(Vq, V.shape), scale, pos0, tm)
        O = run_attn(bridge, Q, Kq, Vq, scale, Hkv, Mkv, pos0, tm, False)
    assert np.all(np.isfinite(O.astype(np.float32)))
    assert np.abs(O.astype(np.float64) - gold.astype(np.float64)).max() <= TOL


def test_attention_tensor_memory_kernel_long(bridge):
    """Head dim 128 over a Q8_0 cache runs on the tcgen05 / tensor-memory kernel: several 128-key tiles, ragged last
    tile, a position offset, grouped heads; against the oracle and against the warp-level MMA kernel."""
    Hq, Hkv, M, Mkv, D, pos0 = 8, 2, 700, 1000, 128, 300
    g = o.RefLcg(77)
    Q = g.activations(Hq, M, D); K = g.activations(Hkv, Mkv, D); V = g.activations(Hkv, Mkv, D)
    Kq, Vq = o.quantize_q8_0(K), o.quantize_q8_0(V)
    gold = o.attention(Q, o.dequantize_q8_0(Kq, K.shape), o.dequantize_q8_0(Vq, V.shape), D ** -0.5, pos0, True)
    a = run_attn(bridge, Q, Kq, Vq, D ** -0.5, Hkv, Mkv, pos0, True)
    assert np.abs(a.astype(np.float64) - gold.astype(np.float64)).max() <= TOL
    bridge.lib.b200_bridge_force_legacy_attention(1)
    try:
        b = run_attn(bridge, Q, Kq, Vq, D ** -0.5, Hkv, Mkv, pos0, True)
    finally:
        bridge.lib.b200_bridge_force_legacy_attention(0)
    assert np.abs(b.astype(np.float64) - gold.astype(np.float64)).max() <= TOL
    assert np.abs(a.astype(np.float32) - b.astype(np.float32)).max() <= 2e-3
    # the kernel that unpacks the Q8_0 tiles itself, with V transposed in shared memory (K-major operand, hook 2) and in
    # its natural [key][d] form (MN-major operand, hook 3): the same products in the same order.  The default (cache
    # dequantised once, tiles through TMA) moves a row's reference maximum only for jumps above 2^8 and evaluates part of
    # the exponentials as a polynomial, so it agrees with them to rounding, not bit for bit.
    outs = {}
    for hook in (2, 3):
        bridge.lib.b200_bridge_force_legacy_attention(hook)
        try:
            outs[hook] = run_attn(bridge, Q, Kq, Vq, D ** -0.5, Hkv, Mkv, pos0, True)
        finally:
            bridge.lib.b200_bridge_force_legacy_attention(0)
    assert np.array_equal(outs[2].view(np.uint16), outs[3].view(np.uint16))
    assert np.abs(a.astype(np.float32) - outs[3].astype(np.float32)).max() <= 2e-3
    assert bridge.device_error() == 0


def test_attention_unaligned_cache(bridge):
    """K and V caches that start on an odd 2-byte boundary (a view into a larger buffer) take the piecewise copy path."""
    Hq, Hkv, M, D = 4, 2, 260, 128
    g = o.RefLcg(78)
    Q = g.activations(Hq, M, D); K = g.activations(Hkv, M, D); V = g.activations(Hkv, M, D)
    Kq, Vq = o.quantize_q8_0(K), o.quantize_q8_0(V)
    gold = o.attention(Q, o.dequantize_q8_0(Kq, K.shape), o.dequantize_q8_0(Vq, V.shape), D ** -0.5, 0, False)
    for shift in (2, 6, 10):
        Kb = torch.zeros(Kq.size + 32, dtype=torch.uint8, device="cuda"); Vb = torch.zeros(Vq.size + 32, dtype=torch.uint8, device="cuda")
        Kb[shift:shift + Kq.size] = dev(Kq); Vb[shift:shift + Vq.size] = dev(Vq)
        Qd = dev(Q)
        O = torch.full((Hq, M, D), float("nan"), dtype=torch.float16, device="cuda")
        rc = bridge.lib.b200_bridge_dispatch_attention_q8kv(Qd.data_ptr(), Kb.data_ptr() + shift, Vb.data_ptr() + shift, O.data_ptr(),
                                                            Hq, Hkv, M, M, D, cfloat(D ** -0.5), 0, 0, 0)
        assert rc == 0
        bridge.synchronize()
        assert np.abs(O.cpu().numpy().astype(np.float64) - gold.astype(np.float64)).max() <= TOL, f"shift {shift}"
    assert bridge.device_error() == 0


def test_attention_causal_isolation(bridge):
    # changing token t leaves every output before t unchanged (tests/redteam_engine.py:303-352)
    H, M, D, t = 4, 150, 128, 97
    g = o.RefLcg(31)
    Q = g.activations(H, M, D); K = g.activations(H, M, D); V = g.activations(H, M, D)
    a = run_attn(bridge, Q, o.quantize_q8_0(K), o.quantize_q8_0(V), D ** -0.5, H, M)
    K2, V2, Q2 = K.copy(), V.copy(), Q.copy()
    K2[:, t:] += np.float16(0.5); V2[:, t:] -= np.float16(0.25); Q2[:, t:] *= np.float16(2)
    b = run_attn(bridge, Q2, o.quantize_q8_0(K2), o.quantize_q8_0(V2), D ** -0.5, H, M)
    assert np.array_equal(a[:, :t].view(np.uint16), b[:, :t].view(np.uint16))
    assert not np.array_equal(a[:, t:].view(np.uint16), b[:, t:].view(np.uint16))


def test_attention_chunked_prefill_consistency(bridge):
    # prefill n tokens == prefill n-1 then one more at offset n-1 (tests/redteam_engine.py:355-400, diff <= 1e-3)
    H, M, D = 4, 130, 128
    g = o.RefLcg(32)
    Q = g.activations(H, M, D); K = g.activations(H, M, D); V = g.activations(H, M, D)
    Kq, Vq = o.quantize_q8_0(K), o.quantize_q8_0(V)
    full = run_attn(bridge, Q, Kq, Vq, D ** -0.5, H, M)
    last = run_attn(bridge, np.ascontiguousarray(Q[:, M - 1:]), Kq, Vq, D ** -0.5, H, M, pos0=M - 1)
    assert np.abs(full[:, M - 1:].astype(np.float32) - last.astype(np.float32)).max() <= 1e-3


@pytest.mark.parametrize("D,Hq,Hkv", [(128, 8, 2), (64, 8, 8)])
@pytest.mark.parametrize("fmt", [o.Q4_0, o.Q4_K])
def test_fused_qkv_epilogue_is_bit_exact(bridge, fmt, D, Hq, Hkv):
    """Rotary embedding and Q8_0 compression fused into the Q/K/V projection's epilogue, written straight into a Q8_0
    cache at a token offset (chunked prefill): the cache bytes and Q equal, bit for bit, what the unfused path gives --
    head-major projections, then b200_bridge_rope, then the Q8_0 quantiser, whose arithmetic is the reference's
    quantize_kv_to_q8_0 (unified_8b_kernels.metal:118-145) and which is itself pinned bit-exact against the reference.
    Then attention over past + present from that cache matches the oracle."""
    import ctypes
    L = bridge.lib
    M1, M2, K = 512, 300, 512                  # two chunks; K = 512 is two packed chunks, which the planner never splits
    theta, scale = 10000.0, D ** -0.5
    g = o.RefLcg(77)
    Wq, Wk, Wv = g.weights(fmt, K, Hq * D), g.weights(fmt, K, Hkv * D), g.weights(fmt, K, Hkv * D)
    shrink = 0.05 if fmt == o.Q4_K else 1.0
    Xall = (g.activations(M1 + M2, K).astype(np.float32) * shrink).astype(np.float16)
    Mt = M1 + M2
    nblk = Hkv * Mt * (D // 32)
    Kc = torch.zeros(nblk * 34, dtype=torch.uint8, device="cuda")
    Vc = torch.zeros(nblk * 34, dtype=torch.uint8, device="cuda")
    Wd = [dev(w) for w in (Wq, Wk, Wv)]
    Kref = np.zeros((Hkv, Mt, (D // 32) * 34), np.uint8)
    Vref = np.zeros_like(Kref)
    outs = []
    for pos0, M in ((0, M1), (M1, M2)):
        X = Xall[pos0:pos0 + M]
        Xd = dev(X)
        Qf = torch.full((Hq, M, D), float("nan"), dtype=torch.float16, device="cuda")
        rc = L.b200_bridge_dispatch_qkv_fused(Xd.data_ptr(), Wd[0].data_ptr(), Wd[1].data_ptr(), Wd[2].data_ptr(), Qf.data_ptr(), Kc.data_ptr(),
                                              Vc.data_ptr(), fmt, M, K, Hq, Hkv, D, cfloat(theta), pos0, 1, Mt)
        assert rc == 0
        # unfused: three head-major projections, rope on Q and K, quantiser on K and V
        Qu = dev(run_gemm(bridge, fmt, X, Wq, Hq * D, layout=1, H=Hq, D=D))
        Ku = dev(run_gemm(bridge, fmt, X, Wk, Hkv * D, layout=1, H=Hkv, D=D))
        Vu = dev(run_gemm(bridge, fmt, X, Wv, Hkv * D, layout=1, H=Hkv, D=D))
        assert L.b200_bridge_rope(Qu.data_ptr(), Hq, M, D, cfloat(theta), pos0) == 0
        assert L.b200_bridge_rope(Ku.data_ptr(), Hkv, M, D, cfloat(theta), pos0) == 0
        n = Hkv * M * D
        Kq = torch.zeros(n // 32 * 34, dtype=torch.uint8, device="cuda")
        Vq = torch.zeros_like(Kq)
        assert L.b200_bridge_quantize_kv_q8_0(Ku.data_ptr(), n * 2, Kq.data_ptr(), Kq.numel(), n) == 0
        assert L.b200_bridge_quantize_kv_q8_0(Vu.data_ptr(), n * 2, Vq.data_ptr(), Vq.numel(), n) == 0
        bridge.synchronize()
        assert bridge.device_error() == 0
        assert torch.equal(Qf, Qu)
        Kref[:, pos0:pos0 + M] = Kq.cpu().numpy().reshape(Hkv, M, -1)
        Vref[:, pos0:pos0 + M] = Vq.cpu().numpy().reshape(Hkv, M, -1)
        # the oracle's rope and quantiser on the same fp16 projections agree with the device's to the last bit of Q8_0
        assert np.array_equal(o.quantize_q8_0(Vu.cpu().numpy()).reshape(Hkv, M, -1), Vref[:, pos0:pos0 + M])
        outs.append(Qf)
    assert np.array_equal(Kc.cpu().numpy().reshape(Hkv, Mt, -1), Kref)
    assert np.array_equal(Vc.cpu().numpy().reshape(Hkv, Mt, -1), Vref)
    # attention of the second chunk over the whole cache (past + present)
    O = torch.zeros(Hq, M2, D, dtype=torch.float16, device="cuda")
    assert L.b200_bridge_dispatch_attention_q8kv(outs[1].data_ptr(), Kc.data_ptr(), Vc.data_ptr(), O.data_ptr(), Hq, Hkv, M2, Mt, D,
                                                 cfloat(scale), M1, 0, 0) == 0
    bridge.synchronize()
    Kd = o.dequantize_q8_0(Kc.cpu().numpy(), (Hkv, Mt, D))
    Vd = o.dequantize_q8_0(Vc.cpu().numpy(), (Hkv, Mt, D))
    gold = o.attention(outs[1].cpu().numpy(), Kd, Vd, scale, pos0=M1)
    assert np.abs(O.cpu().numpy().astype(np.float32) - gold.astype(np.float32)).max() <= 2e-3 * max(1.0, float(np.abs(gold.astype(np.float32)).max()))
    # few tokens and a long K: the planner splits K, which the fused epilogue does not do -- refused, the caller runs the
    # unfused sequence
    K2 = 2048
    Wz = [torch.zeros(L.b200_bridge_weight_bytes(fmt, K2, n), dtype=torch.uint8, device="cuda") for n in (Hq * D, Hkv * D, Hkv * D)]
    Xs = torch.zeros(33, K2, dtype=torch.float16, device="cuda")
    Qs = torch.zeros(Hq, 33, D, dtype=torch.float16, device="cuda")
    assert L.b200_bridge_dispatch_qkv_fused(Xs.data_ptr(), Wz[0].data_ptr(), Wz[1].data_ptr(), Wz[2].data_ptr(), Qs.data_ptr(), Kc.data_ptr(),
                                            Vc.data_ptr(), fmt, 33, K2, Hq, Hkv, D, cfloat(theta), 0, 1, Mt) == -4
