"""GGUF ingest: container parsing, PrismML Q2_0 extraction and layer streaming, on synthetic files built here (the
reference tests its loader the same way: tests/test_gguf_loader.mm:45-330, tests/test_gguf_layer_streamer.mm), plus one
GPU test that runs projections on weights served from a file."""
import struct

import numpy as np
import pytest

import oracle as o


@pytest.fixture(scope="module")
def gguf(pkg, lib_path):
    from m4_prefill_engine_b200 import gguf as g
    return g


def prism_payload(K, N, scale):
    """The reference fixture's pattern (tests/test_gguf_loader.mm:107-127): byte i of a block holds codes (i, i+1, i+2, i+3) mod 4."""
    nb = K * N // 128
    blk = np.zeros((nb, 34), np.uint8)
    blk[:, 0:2] = np.frombuffer(np.float16(scale).tobytes(), np.uint8)
    i = np.arange(32)
    blk[:, 2:] = ((i % 4) | (((i + 1) % 4) << 2) | (((i + 2) % 4) << 4) | (((i + 3) % 4) << 6)).astype(np.uint8)
    return blk.reshape(-1)


def test_rejects_bad_magic_truncation_and_versions(gguf):
    K, N = 256, 128
    good = gguf.write_gguf([("model.layers.0.mlp.gate.weight", (K, N), gguf.GGML_PRISM_Q2_0, prism_payload(K, N, 0.05))],
                           {"general.architecture": "prism", "prism.block_count": 16})
    ld = gguf.GGUFLoader()
    assert ld.parse_from_buffer(good)
    assert not ld.parse_from_buffer(b"BAD!" + good[4:]) and not ld.is_open()
    assert "magic" in ld.last_error()
    assert not ld.parse_from_buffer(good[:20])                        # shorter than the header
    assert not ld.parse_from_buffer(good[:60])                        # metadata table cut off
    for v in (1, 4, 99):
        assert not ld.parse_from_buffer(good[:4] + struct.pack("<I", v) + good[8:])
    huge = good[:8] + struct.pack("<QQ", 2 ** 60, 3) + good[24:]      # implausible tensor count must not allocate
    assert not ld.parse_from_buffer(huge)
    # an array whose declared length exceeds the bytes left is refused without reserving memory for it
    arr = b"GGUF" + struct.pack("<IQQ", 3, 0, 1) + struct.pack("<Q", 1) + b"k" + struct.pack("<IIQ", 9, 4, 2 ** 40)
    assert not ld.parse_from_buffer(arr + b"\0" * 64)
    assert ld.parse_from_buffer(good[:4] + struct.pack("<I", 2) + good[8:]) and ld.version() == 2


@pytest.mark.parametrize("alignment", [32, 64, 4096])
def test_parse_metadata_directory_and_q2_0_extraction(gguf, tmp_path, alignment):
    K, N, scale = 256, 128, 0.05
    payload = prism_payload(K, N, scale)
    data = gguf.write_gguf([("model.layers.0.mlp.gate.weight", (K, N), gguf.GGML_PRISM_Q2_0, payload)],
                           {"general.architecture": "prism", "prism.block_count": 16}, alignment=alignment)
    ld = gguf.GGUFLoader()
    assert ld.parse_from_buffer(data) and ld.is_open()
    assert (ld.version(), ld.tensor_count(), ld.metadata_count(), ld.alignment()) == (3, 1, 3, alignment)
    assert ld.get_string_metadata("general.architecture") == "prism"
    assert ld.get_uint_metadata("general.alignment") == alignment and ld.get_uint_metadata("prism.block_count") == 16
    assert ld.has_metadata("prism.block_count") and not ld.has_metadata("no.such.key")
    assert ld.get_uint_metadata("no.such.key", 7) == 7 and ld.get_string_metadata("prism.block_count", "x") == "x"
    assert ld.tensor_data_offset() % alignment == 0
    info = ld.get_tensor_info("model.layers.0.mlp.gate.weight")
    assert info["n_dims"] == 2 and info["dims"] == [K, N] and info["type"] == 100 and info["size_bytes"] == K * N // 128 * 34
    assert info["file_offset"] == ld.tensor_data_offset() and info["format"] == o.PRISM_Q2_0
    assert ld.tensor_names() == ["model.layers.0.mlp.gate.weight"]
    assert ld.get_tensor_info("missing") is None and ld.get_tensor_raw_data("missing") is None and ld.extract_q2_0_tensor("missing") is None
    raw = ld.get_tensor_raw_data("model.layers.0.mlp.gate.weight")
    assert np.array_equal(raw, payload)
    blocks, k, n = ld.extract_q2_0_tensor("model.layers.0.mlp.gate.weight")
    assert (k, n) == (K, N) and blocks.shape == (K * N // 128, 34) and np.array_equal(blocks.reshape(-1), payload)
    # the extracted blocks decode to (code - 1) * scale with code 3 -> +2 * scale (the reference test's check, :235-277)
    W = o.dequant_matrix(o.PRISM_Q2_0, blocks.reshape(-1), N, K)
    codes = (np.arange(K) // 4 % 32 + np.arange(K) % 4) % 4
    assert np.array_equal(W[0], (codes - 1) * float(np.float16(scale)))
    assert (codes == 3).any()
    # the same file from disk through the memory map
    path = tmp_path / "m.gguf"
    path.write_bytes(data)
    disk = gguf.GGUFLoader()
    assert disk.open(str(path)) and disk.tensor_count() == 1
    b2, _, _ = disk.extract_q2_0_tensor("model.layers.0.mlp.gate.weight")
    assert np.array_equal(b2, blocks)
    assert not gguf.GGUFLoader().open(str(tmp_path / "absent.gguf"))


def test_q2_0_extraction_refusals(gguf):
    K, N = 256, 4
    payload = prism_payload(K, N, 0.02)
    # element count not a multiple of 128; blocks that leave the file; a tensor without dimensions
    odd = gguf.write_gguf([("w", (100, 3), gguf.GGML_PRISM_Q2_0, payload[:34 * 3])])
    ld = gguf.GGUFLoader()
    assert ld.parse_from_buffer(odd) and ld.extract_q2_0_tensor("w") is None
    short = gguf.write_gguf([("w", (K, N), gguf.GGML_PRISM_Q2_0, payload)])
    assert ld.parse_from_buffer(short[:-40]) and ld.extract_q2_0_tensor("w") is None and ld.get_tensor_raw_data("w") is None
    nodims = gguf.write_gguf([("w", (), gguf.GGML_PRISM_Q2_0, payload)])
    assert ld.parse_from_buffer(nodims) and ld.extract_q2_0_tensor("w") is None


def model_file(gguf, tmp_path, layers=4, K=256, N=128):
    rng = np.random.default_rng(0)
    tensors = [("token_embd.weight", (K, 64), gguf.GGML_F16, rng.integers(0, 256, K * 64 * 2, dtype=np.uint8)),
               ("output_norm.weight", (K,), gguf.GGML_F32, rng.integers(0, 256, K * 4, dtype=np.uint8))]
    weights = {}
    for l in range(layers):
        for part, ty, fmt in (("attn_q", gguf.GGML_Q4_0, o.Q4_0), ("ffn_gate", gguf.GGML_PRISM_Q2_0, o.PRISM_Q2_0)):
            w = o.RefLcg(100 + 7 * l + ty).weights(fmt, K, N)
            name = f"blk.{l}.{part}.weight" if l % 2 else f"model.layers.{l}.{part}.weight"
            tensors.append((name, (K, N), ty, w))
            weights[name] = (fmt, w)
    path = tmp_path / "model.gguf"
    path.write_bytes(gguf.write_gguf(tensors, {"general.architecture": "llama"}))
    return path, weights, sum(int(t[3].size) for t in tensors), K * 64 * 2 + K * 4


def test_layer_streamer_on_host(gguf, tmp_path):
    """Grouping by layer index, LRU residency accounting and refusals, without a GPU (upload=False)."""
    S = gguf.GGUFLayerStreamer
    assert S.parse_layer_index("model.layers.12.mlp.up.weight") == 12 and S.parse_layer_index("blk.3.attn_q.weight") == 3
    for shared in ("token_embd.weight", "model.layers.x.w", "model.layers.5", "blk..w", "layers.1.w"):
        assert S.parse_layer_index(shared) == -1
    path, weights, total, shared = model_file(gguf, tmp_path)
    st = S()
    assert st.open(str(path), resident_layer_count=2, upload=False)
    assert st.num_layers() == 4 and st.total_model_bytes() == total and st.shared_bytes() == shared
    assert st.current_resident_bytes() == shared                     # shared tensors are resident from the start
    assert st.tensor_data("token_embd.weight") is not None
    assert st.tensor_data("model.layers.0.attn_q.weight") is None   # layer 0 not acquired yet
    per_layer = (total - shared) // 4
    assert st.acquire_layer(0) and st.is_resident(0) and st.is_resident(1)       # the next layer is requested along with it
    assert st.current_resident_bytes() == shared + 2 * per_layer
    assert st.acquire_layer(1) and st.acquire_layer(2)
    assert st.is_resident(2) and st.is_resident(3) and not st.is_resident(0) and not st.is_resident(1)
    assert st.current_resident_bytes() == shared + 2 * per_layer and st.peak_resident_bytes() <= shared + 3 * per_layer
    assert st.tensor_data("model.layers.0.attn_q.weight") is None and st.tensor_data("model.layers.2.attn_q.weight") is not None
    assert st.acquire_layer(3) and st.acquire_layer(0) and st.is_resident(0)
    assert not st.acquire_layer(9) and not st.acquire_layer(-1)
    st.close()
    assert not S().open(str(tmp_path / "absent.gguf"))


@pytest.mark.gpu
def test_projection_on_weights_served_from_a_file(gguf, tmp_path, bridge):
    """Q4_0 and Prism Q2_0 tensors go from the file to the device through the streamer (two layers resident) and straight
    into the projection kernels: the payload layouts are the kernels' layouts, nothing is repacked."""
    import torch
    from gpu_util import TOL
    K, N, M = 1024, 256, 40
    path, weights, _, _ = model_file(gguf, tmp_path, layers=3, K=K, N=N)
    st = gguf.GGUFLayerStreamer()
    assert st.open(str(path), resident_layer_count=2, upload=True)
    X = o.RefLcg(5).activations(M, K)
    Xd = torch.from_numpy(X).cuda()
    for l in range(3):
        assert st.acquire_layer(l)
        for name, (fmt, w) in weights.items():
            if st.parse_layer_index(name) != l:
                continue
            p = st.tensor_data(name)
            assert p is not None
            Y = torch.zeros(M, N, dtype=torch.float16, device="cuda")
            rc = bridge.lib.b200_bridge_dispatch_gemm_ex(Xd.data_ptr(), M * K * 2, p, w.size, Y.data_ptr(), M * N * 2, fmt, M, K, N, 0, 0, 0, None, 0)
            assert rc == 0
            bridge.synchronize()
            assert np.abs(Y.cpu().numpy().astype(np.float64) - o.gemm_f64(fmt, X, w, N)).max() <= TOL, name
    assert not st.is_resident(0) and st.is_resident(2)
    assert bridge.device_error() == 0
    st.close()
