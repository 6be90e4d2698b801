"""The allocation-free GEMM entry point against the regular one.

Some callers of this library may not allocate device memory while they run: the application that
hosts them has handed all remaining GPU memory to its own pool (so a cudaMalloc inside the library
could fail, or stall the host while the driver synchronises the device), or they sit in a
latency-critical loop where that synchronisation is not allowed.  For them
`b200_bridge_gemm_scratch_static` runs the few-token projection with its split-K scratch in a fixed
device array that is part of the library image.  It must give the same answer as
`m4_bridge_dispatch_gemm`, call after call, although the array keeps the previous call's contents.
This file is collected last so that a failure here cannot hide one elsewhere.
"""
import numpy as np
import pytest
import torch

import oracle as o
from gpu_util import TOL, check, dev

pytestmark = pytest.mark.gpu


def _call(br, fn, Xd, Wd, Yd, fmt, M, K, N):
    rc = fn(Xd.data_ptr(), Xd.numel() * 2, Wd.data_ptr(), Wd.numel(), Yd.data_ptr(), Yd.numel() * 2, fmt, M, K, N)
    br.synchronize()
    return rc


@pytest.fixture(params=[1, 0], ids=["cluster-kernel", "split-k-scratch"])
def few_token_path(request, bridge):
    """Few-token shapes run on the cluster kernel by default (no scratch at all); with it switched off they take the
    persistent kernel, whose split-K scratch is what this entry point keeps in the static array."""
    bridge.lib.b200_bridge_enable_small_kernel(request.param)
    yield request.param
    bridge.lib.b200_bridge_enable_small_kernel(1)


def test_static_scratch_matches_regular_entry_point(bridge, few_token_path):
    L = bridge.lib
    K = N = 4096
    first = None
    # two calls in a row on different inputs and different split shapes: the second sees the first's leftovers
    for M, fmt, seed in ((33, o.Q4_0, 1), (129, o.MLX_4BIT, 2), (33, o.Q4_0, 1)):
        X, W = o.baseline_inputs(fmt, M, K, N, seed)
        Xd, Wd = dev(X), dev(W)
        Y_ref = torch.zeros(M, N, dtype=torch.float16, device="cuda")
        Y_new = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
        assert _call(bridge, L.m4_bridge_dispatch_gemm, Xd, Wd, Y_ref, fmt, M, K, N) == 0
        assert _call(bridge, L.b200_bridge_gemm_scratch_static, Xd, Wd, Y_new, fmt, M, K, N) == 0
        assert bridge.device_error() == 0
        a, b = Y_ref.cpu().numpy(), Y_new.cpu().numpy()
        assert np.all(np.isfinite(b.astype(np.float32)))
        assert np.abs(a.astype(np.float32) - b.astype(np.float32)).max() <= TOL
        check(b, o.gemm_f64(fmt, X, W, N), f"static-scratch GEMM M={M} fmt={fmt}")
        if first is None:
            first = b.copy()
    assert np.array_equal(first.view(np.uint16), b.view(np.uint16))      # same inputs again: same bits


def test_static_scratch_calls_leave_device_memory_alone(bridge, few_token_path):
    """What the entry point is for: from the second call on (the first one may still make the driver load code), a
    call changes the amount of free device memory by nothing, whatever the split shape -- the regular entry point, by
    contrast, grows its scratch on demand.  cudaMemGetInfo is read straight from the runtime, with no torch
    allocation between the readings."""
    import ctypes
    L = bridge.lib
    rt = ctypes.CDLL("libcudart.so.12")
    K = N = 4096
    sets = []
    for M, fmt, seed in ((33, o.Q4_0, 1), (129, o.MLX_4BIT, 2), (65, o.Q4_K, 3)):
        X, W = o.baseline_inputs(fmt, M, K, N, seed)
        sets.append((dev(X), dev(W), torch.zeros(M, N, dtype=torch.float16, device="cuda"), fmt, M))
    torch.cuda.synchronize()

    def free_bytes():
        f, t = ctypes.c_size_t(), ctypes.c_size_t()
        assert rt.cudaMemGetInfo(ctypes.byref(f), ctypes.byref(t)) == 0
        return f.value
    for Xd, Wd, Yd, fmt, M in sets:                        # first round: warm
        assert _call(bridge, L.b200_bridge_gemm_scratch_static, Xd, Wd, Yd, fmt, M, K, N) == 0
    before = free_bytes()
    for _ in range(3):
        for Xd, Wd, Yd, fmt, M in sets:
            assert _call(bridge, L.b200_bridge_gemm_scratch_static, Xd, Wd, Yd, fmt, M, K, N) == 0
            assert free_bytes() == before
    assert bridge.device_error() == 0


def test_static_scratch_limits(bridge):
    L = bridge.lib
    K, N = 4096, 2048
    X = torch.zeros(512, K, dtype=torch.float16, device="cuda")
    W = torch.zeros(N * (K // 32) * 18, dtype=torch.uint8, device="cuda")
    Y = torch.zeros(512, N, dtype=torch.float16, device="cuda")
    # 512 tokens x 2048 outputs are 32 tiles, split four ways: 4 Mi floats of scratch, over the 3 Mi limit
    assert _call(bridge, L.b200_bridge_gemm_scratch_static, X, W, Y, 0, 512, K, N) == -7
    assert b"static array holds" in L.b200_bridge_last_error_string()
    # host memory would have to be staged, which needs an allocation: refused
    Xh = torch.zeros(33, K, dtype=torch.float16)
    assert L.b200_bridge_gemm_scratch_static(Xh.data_ptr(), Xh.numel() * 2, W.data_ptr(), W.numel(), Y.data_ptr(), Y.numel() * 2,
                                             0, 33, K, N) == -2
    assert _call(bridge, L.b200_bridge_gemm_scratch_static, X, W, Y, 9, 33, K, N) == -3
    # a launch with enough tiles to fill the GPU does not split K, needs no scratch and is accepted
    Xb = torch.zeros(2048, K, dtype=torch.float16, device="cuda")
    Yb = torch.zeros(2048, N, dtype=torch.float16, device="cuda")
    assert _call(bridge, L.b200_bridge_gemm_scratch_static, Xb, W, Yb, 0, 2048, K, N) == 0
