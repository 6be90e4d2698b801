"""Generates tests/golden/*.npz from the reference's own CPU verifier.

Run in a checkout where the reference sources are available (oracle/build.py builds
oracle/_ref/libm4ref.so from them):  python tests/golden/make_golden.py
Every array is produced by the reference code itself -- its seeded generators
(tests/e2e/test_common.h:253-427, brick3/brick4/bench_8b generators) and its golds -- so the
fixtures pin the oracle restatement on machines that do not have the reference.
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
import oracle as o  # noqa: E402

OUT = Path(__file__).resolve().parent


def main():
    r = o.ref_lib()
    assert r is not None, "reference checkout not available: cannot regenerate fixtures"
    # --- GEMM golds, all seven formats, tier-1 shape (tests/e2e/test_tier1_feature_coverage.mm:177-223) ---
    M, K, N, H, D = 33, 512, 256, 4, 64
    gemm = {}
    for fmt in (0, 1, 2, 3, 4, 5, 7):
        be, bb = o.BLOCK[fmt]
        W = np.empty(N * (K // be) * bb, dtype=np.uint8)
        st = r.ref_gen_weights(1337, fmt, o._ptr(W), N * (K // be))
        X = np.empty((M, K), dtype=np.float16)
        st2 = r.ref_gen_activations(st, o._ptr(X), X.size)
        Y = np.empty((M, N), dtype=np.float16)
        assert r.ref_gemm(fmt, o._ptr(X), o._ptr(W), o._ptr(Y), M, N, K, 0, 0, 0) == 0
        Yh = np.empty((H, M, D), dtype=np.float16)
        assert r.ref_gemm(fmt, o._ptr(X), o._ptr(W), o._ptr(Yh), M, N, K, 1, H, D) == 0
        gemm[f"W{fmt}"] = W
        gemm[f"X{fmt}"] = X.view(np.uint16)
        gemm[f"Y{fmt}"] = Y.view(np.uint16)
        gemm[f"Yh{fmt}"] = Yh.view(np.uint16)
        gemm[f"state{fmt}"] = np.array([st, st2], dtype=np.uint64)
    np.savez_compressed(OUT / "gemm_tier1.npz", **gemm)

    # --- Q8_0 quantiser + attention gold (brick4_attn_bench.mm:37-119) ---
    Hh, Mm, Dd = 2, 80, 64
    Q = np.empty((Hh, Mm, Dd), np.float16); Kk = np.empty_like(Q); V = np.empty_like(Q)
    st = r.ref_gen_activations(2026, o._ptr(Q), Q.size)
    st = r.ref_gen_activations(st, o._ptr(Kk), Kk.size)
    r.ref_gen_activations(st, o._ptr(V), V.size)
    Kq = np.empty(Kk.size // 32 * 34, dtype=np.uint8); Vq = np.empty_like(Kq)
    r.ref_quantize_q8_0(o._ptr(Kk), o._ptr(Kq), Kk.size); r.ref_quantize_q8_0(o._ptr(V), o._ptr(Vq), V.size)
    Kd = np.empty_like(Kk); Vd = np.empty_like(V)
    r.ref_dequantize_q8_0(o._ptr(Kq), o._ptr(Kd), Kk.size); r.ref_dequantize_q8_0(o._ptr(Vq), o._ptr(Vd), V.size)
    O = np.empty_like(Q)
    r.ref_brick4_attention(o._ptr(Q), o._ptr(Kd), o._ptr(Vd), o._ptr(O), Hh, Mm, Dd, 0.125)
    np.savez_compressed(OUT / "attention_q8.npz", Q=Q.view(np.uint16), K=Kk.view(np.uint16), V=V.view(np.uint16), Kq=Kq, Vq=Vq,
                        Kd=Kd.view(np.uint16), Vd=Vd.view(np.uint16), O=O.view(np.uint16))

    # --- fused SwiGLU gold with its own generator (brick3_swiglu_bench.mm:23-99) ---
    M3, F3, K3 = 20, 96, 256
    A = np.empty((M3, K3), np.float16); Wg = np.empty(F3 * (K3 // 32) * 18, np.uint8); Wu = np.empty_like(Wg)
    Out = np.empty((M3, F3), np.float16)
    r.ref_brick3_swiglu(2026, o._ptr(A), o._ptr(Wg), o._ptr(Wu), o._ptr(Out), M3, F3, K3, 1)
    np.savez_compressed(OUT / "swiglu_brick3.npz", A=A.view(np.uint16), Wg=Wg, Wu=Wu, Out=Out.view(np.uint16))

    # --- layer gold (bench_8b_engine.mm:44-225), small shape ---
    M4, K4, H4, D4, F4 = 24, 256, 4, 64, 512
    st = 1337
    ws = []
    for n, k in ((H4 * D4, K4), (H4 * D4, K4), (H4 * D4, K4), (K4, H4 * D4), (F4, K4), (F4, K4), (K4, F4)):
        w = np.empty(n * (k // 32) * 18, np.uint8)
        st = r.ref_layer_gen_q4_0(st, o._ptr(w), n * (k // 32), 0.003)
        ws.append(w)
    X = np.empty((M4, K4), np.float16)
    r.ref_gen_activations(st, o._ptr(X), X.size)
    Y = np.empty_like(X)
    r.ref_layer(o._ptr(X), *[o._ptr(w) for w in ws], o._ptr(Y), M4, K4, H4, D4, F4, 0.125)
    np.savez_compressed(OUT / "layer_q4_0.npz", X=X.view(np.uint16), Y=Y.view(np.uint16),
                        **{f"W{i}": w for i, w in enumerate(ws)})
    print("fixtures written to", OUT)


if __name__ == "__main__":
    main()
