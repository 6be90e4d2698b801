"""Multi-layer model loop (embedding, L decoder layers, final RMSNorm, lm_head) on the GPU against the oracle composed
the same way: the reference's TransformerModel.__call__ (src/engine/model.py:340-368) with use_cache=False."""
import numpy as np
import pytest
import torch

import oracle as o
from gpu_util import PARITY_REPORT, TOL, dev, parity_stats

pytestmark = pytest.mark.gpu


def small_model(pkg, fmt, L, M, K, H, Hkv, D, F, V, seed=3):
    from m4_prefill_engine_b200.model import EngineConfig, TransformerModel
    cfg = EngineConfig(num_layers=L, hidden_dim=K, num_q_heads=H, num_kv_heads=Hkv, head_dim=D, intermediate_dim=F, vocab_size=V,
                       rope_theta=10000.0, weight_format=fmt, max_context_length=4096)
    g = o.RefLcg(seed)
    rng = np.random.default_rng(seed)
    shapes = {"q": (H * D, K), "k": (Hkv * D, K), "v": (Hkv * D, K), "o": (K, H * D), "gate": (F, K), "up": (F, K), "down": (K, F)}
    layers = []
    for _ in range(L):
        w = {n: g.q4_0_bench(k, r, 0.003, 0.0003) for n, (r, k) in shapes.items()}
        n1 = (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float16)
        n2 = (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float16)
        layers.append((w, n1, n2))
    emb = (rng.standard_normal((V, K)) * 0.35).astype(np.float16)
    fn = (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float16)
    head = g.q4_0_bench(K, V, 0.003, 0.0003)
    model = TransformerModel(cfg, M)
    model.set_embedding(dev(emb))
    for i, (w, n1, n2) in enumerate(layers):
        model.set_layer(i, {k: dev(v) for k, v in w.items()}, dev(n1), dev(n2))
    model.set_head(dev(fn), dev(head))
    return cfg, model, layers, emb, fn, head


def oracle_model(cfg, layers, emb, fn, head, tokens):
    h = emb[np.asarray(tokens)]
    for w, n1, n2 in layers:
        h = o.layer(o.Q4_0, h, w["q"], w["k"], w["v"], w["o"], w["gate"], w["up"], w["down"], cfg.num_q_heads, cfg.num_kv_heads,
                    cfg.head_dim, cfg.intermediate_dim, cfg.scale, rms_eps=cfg.norm_eps, norm1=n1, norm2=n2, rope_theta=cfg.rope_theta,
                    kv_q8=True)
    return h, o.gemm_f64(o.Q4_0, o.rmsnorm(h, fn, cfg.norm_eps), head, cfg.vocab_size)


@pytest.mark.parametrize("M", [40, 300])
def test_model_prefill_matches_oracle(bridge, pkg, M):
    L, K, H, Hkv, D, F, V = 3, 256, 4, 2, 64, 512, 640
    cfg, model, layers, emb, fn, head = small_model(pkg, o.Q4_0, L, M, K, H, Hkv, D, F, V)
    tokens = np.random.default_rng(1).integers(0, V, M).astype(np.int32)
    hidden = torch.zeros(M, K, dtype=torch.float16, device="cuda")
    logits = model.forward(torch.from_numpy(tokens), hidden=hidden)           # host token ids
    bridge.synchronize()
    assert bridge.device_error() == 0
    gold_h, gold_logits = oracle_model(cfg, layers, emb, fn, head, tokens)
    dh = np.abs(hidden.cpu().numpy().astype(np.float64) - gold_h.astype(np.float64))
    assert dh.max() <= 3 * TOL, f"hidden state after {L} layers: max-abs {dh.max()}"
    got = logits.cpu().numpy()
    PARITY_REPORT.append(parity_stats(got, gold_logits, f"model logits L={L} M={M} vocab={V}"))
    rms = float(np.sqrt(np.mean(gold_logits ** 2)))
    assert np.abs(got.astype(np.float64) - gold_logits).max() <= max(3 * TOL, 2.0 ** -6 * rms)
    # device token ids give the same bits; a second call on the same buffers too
    l2 = model.forward(torch.from_numpy(tokens).cuda())
    bridge.synchronize()
    assert torch.equal(l2, logits)
    assert model.kernels_per_forward() >= 2 + 5 * L
    model.close()


def test_model_rejects_bad_tokens_and_shapes(bridge, pkg):
    from m4_prefill_engine_b200.model import EngineConfig, TransformerModel
    L, M, K, H, Hkv, D, F, V = 1, 33, 256, 4, 2, 64, 512, 128
    cfg, model, *_ = small_model(pkg, o.Q4_0, L, M, K, H, Hkv, D, F, V)
    good = np.zeros(M, np.int32)
    for bad_id in (-1, V, 10 ** 6):
        t = good.copy(); t[7] = bad_id
        with pytest.raises(IndexError):                         # the reference's Embedding raises the same (model.py:60-63)
            model.forward(torch.from_numpy(t))
    with pytest.raises(ValueError):
        model.forward(torch.zeros(M + 1, dtype=torch.int32))
    # ids that are already on the device cannot be checked by the host: the gather kernel reports 401 and reads nothing
    # outside the table
    t = good.copy(); t[3] = V + 5
    out = model.forward(torch.from_numpy(t).cuda())
    bridge.synchronize()
    assert bridge.device_error() == 401
    assert bool(torch.isfinite(out.float()).all().item())
    assert bridge.lib.b200_bridge_clear_device_error() == 0
    model.forward(torch.from_numpy(good))
    bridge.synchronize()
    assert bridge.device_error() == 0
    model.close()
    with pytest.raises(ValueError):
        EngineConfig(num_q_heads=6, num_kv_heads=4)
    with pytest.raises(ValueError):
        EngineConfig(activation="geglu")
    with pytest.raises(ValueError):
        TransformerModel(EngineConfig(max_context_length=64), 65)
