"""Tensor-parallel decoder layer on 2, 4 and 8 GPUs (each skipped where fewer are visible), with the row-split
projections reduced either by NCCL or by the fused exchange over peer memory: every rank must hold the same output,
and it must match the CPU oracle's layer.  One process per GPU, 127.0.0.1 rendezvous."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

WORKER = r'''
import os, sys, numpy as np, torch, torch.distributed as dist
root = sys.argv[1]; sys.path.insert(0, root); sys.path.insert(0, os.path.join(root, "tests"))
import oracle as o
from __graft_entry__ import load_package
load_package()
from m4_prefill_engine_b200.bridge import B200Bridge
from m4_prefill_engine_b200.layer import (PeerExchange, TransformerLayerConfig, TransformerLayerCoordinator, shard_layer_weights,
                                           torch_allreduce_hook)
rank, world, mode = int(sys.argv[3]), int(sys.argv[4]), sys.argv[5]
torch.cuda.set_device(rank)
os.environ["NCCL_NVLS_ENABLE"] = "0"
dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{sys.argv[2]}", rank=rank, world_size=world,
                        device_id=torch.device("cuda", rank))
br = B200Bridge.get_instance(); assert br.init()
# whole heads per rank at 8 ranks; F / world and H * D / world multiples of 256 (the row-split projections' K);
# the fused exchange wants M / world to be a multiple of the 256-token tile
M, K, H, Hkv, D, F = (70 if mode == "nccl" else 256 * world), 512, 16, 8, 128, 2048
g = o.RefLcg(1337)
shapes = {"q": (H * D, K), "k": (Hkv * D, K), "v": (Hkv * D, K), "o": (K, H * D), "gate": (F, K), "up": (F, K), "down": (K, F)}
w = {n: g.q4_0_bench(k, r, 0.003, 0.0003) for n, (r, k) in shapes.items()}
X = g.activations(M, K)
cfg = TransformerLayerConfig(M=M, K=K, H=H, D=D, N_mlp=F, attn_scale=D ** -0.5, num_kv_heads=Hkv, kv_q8_0=True,
                             rope_theta=10000.0, tp_size=world)
sw = {k: torch.from_numpy(v).cuda() for k, v in shard_layer_weights(o.Q4_0, w, cfg, rank, world).items()}
layer = TransformerLayerCoordinator(cfg, br)
px = None
if mode == "nccl":
    layer.set_allreduce(torch_allreduce_hook(br))
else:
    px = PeerExchange.setup(layer)          # IPC mappings of the other rank's buffers
    assert px is not None, "peer mappings not available"
Xd = torch.from_numpy(X).cuda(); Yd = torch.zeros_like(Xd)
for _ in range(3):
    layer.forward(Xd, sw["q"], sw["k"], sw["v"], sw["o"], sw["gate"], sw["up"], sw["down"], Yd)
if px is not None:
    # a second layer on the same exchange buffers (the layers of a model share one exchange)
    layer2 = TransformerLayerCoordinator(cfg, br)
    layer2.attach_peer_exchange(px)
    Y2 = torch.zeros_like(Xd)
    layer2.forward(Xd, sw["q"], sw["k"], sw["v"], sw["o"], sw["gate"], sw["up"], sw["down"], Y2)
    layer.forward(Xd, sw["q"], sw["k"], sw["v"], sw["o"], sw["gate"], sw["up"], sw["down"], Yd)
    br.synchronize()
    assert torch.equal(Y2, Yd), "second layer on the shared exchange disagrees"
    layer2.close()
br.synchronize(); torch.cuda.synchronize()
assert br.device_error() == 0
Y = Yd.cpu().numpy()
gold = o.layer(o.Q4_0, X, w["q"], w["k"], w["v"], w["o"], w["gate"], w["up"], w["down"], H, Hkv, D, F, D ** -0.5,
               rope_theta=10000.0, kv_q8=True)
diff = float(np.abs(Y.astype(np.float64) - gold.astype(np.float64)).max())
assert diff <= 2 * 0.0078125, diff
other = [torch.zeros_like(Yd) for _ in range(world)]
dist.all_gather(other, Yd)
assert all(torch.equal(other[0], t) for t in other), "ranks disagree"
dist.barrier()
layer.close()
if px is not None:
    px.close()
dist.barrier(); dist.destroy_process_group()
print("rank", rank, "ok maxdiff", diff)
'''


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("mode", ["nccl", "peer"])
def test_layer_tp(tmp_path, mode, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    script = tmp_path / "tp_worker.py"
    script.write_text(WORKER)
    port = 29600 + (os.getpid() % 300) + (0 if mode == "nccl" else 301) + 700 * (world // 4)
    procs = [subprocess.Popen([sys.executable, str(script), str(ROOT), str(port), str(r), str(world), mode], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = []
    for p in procs:
        try:
            outs.append(p.communicate(timeout=300)[0])
        except subprocess.TimeoutExpired:
            p.kill()
            outs.append("timeout")
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
