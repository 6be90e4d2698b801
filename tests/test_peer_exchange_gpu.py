"""Tensor-parallel reduction over peer memory: the fused reduce-scatter epilogue of the row-split projection, the
owner's reduce + residual + broadcast, and the wait for every rank's rows.

On one GPU the ranks of a group are emulated phase by phase on the bridge's single stream (all scatters, then all
reductions, then all waits), the "peer" buffers being ordinary local allocations: every flag a kernel waits for has
been raised by a kernel that ran before it, so nothing waits on a later launch.  The two-process run over real IPC
mappings is in test_tp_nccl_gpu.py."""
import ctypes

import numpy as np
import pytest
import torch

import oracle as o
from gpu_util import check, dev

pytestmark = pytest.mark.gpu


def _arr(xs):
    return (ctypes.c_void_p * len(xs))(*[int(x) for x in xs])


@pytest.mark.parametrize("world,fmt", [(2, o.Q4_0), (4, o.Q4_0), (8, o.Q4_0), (2, o.Q4_K), (2, o.TERNARY_1_58)])
def test_scatter_reduce_broadcast_emulated_ranks(bridge, pkg, world, fmt):
    from m4_prefill_engine_b200.layer import _bind_layer, shard_cols
    L = bridge.lib
    _bind_layer(L)
    M, K_total, N = 256 * world, 1024 * world, 384           # rows per rank = 256 (one token tile)
    g = o.RefLcg(5 + world)
    W = g.weights(fmt, K_total, N)
    X = (g.activations(M, K_total).astype(np.float32) * 0.5).astype(np.float16)
    R = g.activations(M, N)
    gold = o.gemm_f64(fmt, X, W, N) + R.astype(np.float64)
    k_loc = K_total // world
    Xs = [dev(np.ascontiguousarray(X[:, r * k_loc:(r + 1) * k_loc])) for r in range(world)]
    Ws = [dev(shard_cols(W, fmt, K_total, N, r, world)) for r in range(world)]
    Rd = dev(R)
    rows = M // world
    recv = [torch.full((world, rows, N), float("nan"), dtype=torch.float32, device="cuda") for _ in range(world)]
    out = [torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda") for _ in range(world)]
    flags = [torch.zeros(16, dtype=torch.int32, device="cuda") for _ in range(world)]
    torch.cuda.synchronize()
    recv_p, out_p, flag_p = _arr([t.data_ptr() for t in recv]), _arr([t.data_ptr() for t in out]), _arr([t.data_ptr() for t in flags])
    for epoch in (1, 2):                                       # twice: the flags only grow, buffers are reused
        for r in range(world):
            assert L.b200_peer_gemm_scatter(Xs[r].data_ptr(), Ws[r].data_ptr(), fmt, M, k_loc, N, r, world, recv_p, flag_p, epoch) == 0
        for r in range(world):
            assert L.b200_peer_reduce_broadcast(r, world, recv_p, out_p, flag_p, epoch, Rd.data_ptr(), M, N) == 0
        for r in range(world):
            assert L.b200_peer_wait_rows(r, world, flag_p, epoch) == 0
        bridge.synchronize()
        assert bridge.device_error() == 0
        for r in range(world):
            assert flags[r].cpu().tolist() == [epoch] * world + [0] * (8 - world) + [epoch] * world + [0] * (8 - world)
            check(out[r].cpu().numpy(), gold, f"rank {r} world {world} fmt {fmt}")
        assert all(torch.equal(out[0], out[r]) for r in range(1, world))     # every rank holds the same bits


@pytest.mark.parametrize("partial_fp16", [False, True])
@pytest.mark.parametrize("world", [2, 8])
def test_reduction_with_fused_rmsnorm_emulated_ranks(bridge, pkg, world, partial_fp16):
    """Row-sharded residual stream: the owner of a row adds the partial rows and the residual, keeps the fp16 sum for
    itself and sends rmsnorm(sum) * w to every rank.  Ranks emulated phase by phase on one GPU; several token tiles per
    rank, so the rotated owner order of the scatter epilogue (rank r sends to r+1 first, to itself last) is exercised."""
    from m4_prefill_engine_b200.layer import _bind_layer, shard_cols
    L = bridge.lib
    _bind_layer(L)
    L.b200_peer_set_partial_fp16.argtypes = [ctypes.c_int]
    L.b200_peer_set_partial_fp16.restype = None
    fmt = o.Q4_0
    M, K_total, N = 512 * world, 256 * world, 1024           # two token tiles per rank, eight weight tiles
    g = o.RefLcg(40 + world)
    W = g.weights(fmt, K_total, N)
    X = (g.activations(M, K_total).astype(np.float32) * 0.5).astype(np.float16)
    R = g.activations(M, N)
    wn = (1.0 + 0.1 * np.random.default_rng(3).standard_normal(N)).astype(np.float16)
    gold_mid = (o.gemm_f64(fmt, X, W, N) + R.astype(np.float64))
    k_loc = K_total // world
    Xs = [dev(np.ascontiguousarray(X[:, r * k_loc:(r + 1) * k_loc])) for r in range(world)]
    Ws = [dev(shard_cols(W, fmt, K_total, N, r, world)) for r in range(world)]
    Rd, wd = dev(R), dev(wn)
    rows = M // world
    recv = [torch.full((world, rows, N), float("nan"), dtype=torch.float32, device="cuda") for _ in range(world)]
    out = [torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda") for _ in range(world)]
    keep = [torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda") for _ in range(world)]
    flags = [torch.zeros(16, dtype=torch.int32, device="cuda") for _ in range(world)]
    torch.cuda.synchronize()
    recv_p, out_p, flag_p = _arr([t.data_ptr() for t in recv]), _arr([t.data_ptr() for t in out]), _arr([t.data_ptr() for t in flags])
    for epoch in (1, 2):
        L.b200_peer_set_partial_fp16(int(partial_fp16))      # partial sums as fp16 in the (fp32-sized) receive buffers, or as fp32
        try:
            for r in range(world):
                assert L.b200_peer_gemm_scatter(Xs[r].data_ptr(), Ws[r].data_ptr(), fmt, M, k_loc, N, r, world, recv_p, flag_p, epoch) == 0
            for r in range(world):
                assert L.b200_peer_reduce_norm_broadcast(r, world, recv_p, out_p, flag_p, epoch, Rd.data_ptr(), M, N, wd.data_ptr(),
                                                         ctypes.c_float(1e-5), keep[r].data_ptr()) == 0
            for r in range(world):
                assert L.b200_peer_wait_rows(r, world, flag_p, epoch) == 0
        finally:
            L.b200_peer_set_partial_fp16(0)
        bridge.synchronize()
        assert bridge.device_error() == 0
        mid = np.concatenate([keep[r][r * rows:(r + 1) * rows].cpu().numpy() for r in range(world)])    # each rank kept its own rows
        check(mid, gold_mid, f"kept rows, world {world}")
        want = o.rmsnorm(mid, wn, 1e-5)                        # the normalisation of exactly the rows that were kept
        got = out[0].cpu().numpy()
        assert np.abs(got.astype(np.float32) - want.astype(np.float32)).max() <= 2 * np.spacing(np.float16(np.abs(want).max())).astype(np.float32)
        assert all(torch.equal(out[0], out[r]) for r in range(1, world))
        for r in range(world):                                 # nothing outside a rank's own rows was written to its keep buffer
            other = torch.cat([keep[r][:r * rows], keep[r][(r + 1) * rows:]])
            assert bool(torch.isnan(other).all().item())


def test_scatter_rejects_unsupported_shapes(bridge, pkg):
    from m4_prefill_engine_b200.layer import _bind_layer
    L = bridge.lib
    _bind_layer(L)
    K, N = 512, 256
    W = dev(o.RefLcg(1).weights(o.Q4_0, K, N))
    buf = torch.zeros(1 << 20, dtype=torch.float32, device="cuda")
    fl = torch.zeros(16, dtype=torch.int32, device="cuda")
    p2 = _arr([buf.data_ptr()] * 2)
    f2 = _arr([fl.data_ptr()] * 2)
    X = torch.zeros(200, K, dtype=torch.float16, device="cuda")
    # 100 rows per rank is not a whole number of token tiles; K = 96 has no tensor-core path: both refused, nothing runs
    assert L.b200_peer_gemm_scatter(X.data_ptr(), W.data_ptr(), o.Q4_0, 200, K, N, 0, 2, p2, f2, 1) == -4
    X2 = torch.zeros(512, 96, dtype=torch.float16, device="cuda")
    assert L.b200_peer_gemm_scatter(X2.data_ptr(), W.data_ptr(), o.Q4_0, 512, 96, N, 0, 2, p2, f2, 1) == -4
    bridge.synchronize()
    assert int(fl.sum().item()) == 0


def test_wait_runs_out_and_reports(bridge, pkg):
    """Failure detection without a fault: a rank waits for rows that no peer will ever write (a flag nothing sets),
    with the wait limit lowered to 50 ms.  The kernel gives up, the host reads error 302, the waits that follow return
    at once, and after clearing the error word the same context runs a projection correctly."""
    import time
    from m4_prefill_engine_b200.layer import _bind_layer
    L = bridge.lib
    _bind_layer(L)
    L.b200_peer_set_wait_limit_ms.argtypes = [ctypes.c_uint]
    L.b200_peer_set_wait_limit_ms.restype = None
    flags = [torch.zeros(16, dtype=torch.int32, device="cuda") for _ in range(2)]
    fp = _arr([f.data_ptr() for f in flags])
    assert bridge.device_error() == 0
    L.b200_peer_set_wait_limit_ms(50)
    try:
        t0 = time.perf_counter()
        assert L.b200_peer_wait_rows(0, 2, fp, 7) == 0          # enqueues; nobody ever raises epoch 7
        bridge.synchronize()
        dt = time.perf_counter() - t0
        assert bridge.device_error() == 302
        assert 0.02 < dt < 5.0
        t0 = time.perf_counter()
        for _ in range(5):                                       # a wait that already failed is not repeated
            assert L.b200_peer_wait_rows(0, 2, fp, 7) == 0
        bridge.synchronize()
        assert time.perf_counter() - t0 < 0.05 * 5
        # the arrival side: a reduction whose sources never arrive reports 301 and writes nothing
        assert L.b200_bridge_clear_device_error() == 0
        assert bridge.device_error() == 0
        M, K = 512, 256
        recv = [torch.zeros(2, M // 2, K, dtype=torch.float32, device="cuda") for _ in range(2)]
        out = [torch.full((M, K), 3.0, dtype=torch.float16, device="cuda") for _ in range(2)]
        res = torch.zeros(M, K, dtype=torch.float16, device="cuda")
        assert L.b200_peer_reduce_broadcast(0, 2, _arr([t.data_ptr() for t in recv]), _arr([t.data_ptr() for t in out]), fp, 9,
                                            res.data_ptr(), M, K) == 0
        bridge.synchronize()
        assert bridge.device_error() == 301
        assert float(out[0].min().item()) == 3.0 and float(out[1].min().item()) == 3.0
    finally:
        L.b200_peer_set_wait_limit_ms(0)
        assert L.b200_bridge_clear_device_error() == 0
    # the context is intact: an ordinary projection still matches the oracle
    from gpu_util import run_gemm
    X, W = o.baseline_inputs(o.Q4_0, 33, 512, 128, 3)
    check(run_gemm(bridge, o.Q4_0, X, W, 128), o.gemm_f64(o.Q4_0, X, W, 128), "after a timed-out wait")
    assert bridge.device_error() == 0
