"""KV-head-sharded prefill on two GPUs against the unsharded strategy (needs >= 2 CUDA devices)."""
import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _worker(rank, world, port, ret, peer_store):
    sys.path.insert(0, ROOT)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    from kascade_b200 import EfficientKascadeStrategy, _native as nat
    from kascade_b200.strategy import shard_kv_heads
    from tests.cases import SMALL_RAGGED as c, make_inputs
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world, device_id=dev)

    class M:
        num_key_value_groups = c.H // c.G

    full = EfficientKascadeStrategy(list(c.anchors), "x/y", k=c.pct, tile_size=c.tile, rolling_prefill=c.rolling,
                                    head_mapping=c.head_mapping(), register=False)
    part = EfficientKascadeStrategy(list(c.anchors), "x/y", k=c.pct, tile_size=c.tile, rolling_prefill=c.rolling,
                                    head_mapping=c.head_mapping(), register=False, shard=(rank, world),
                                    peer_store=peer_store)
    heads = shard_kv_heads(c.G, rank, world)
    hg = c.H // c.G
    qh = [g * hg + i for g in heads for i in range(hg)]
    worst = 0.0
    for layer in range(c.layers):
        q, k, v = (x.to(dev, torch.float16) for x in make_inputs(c, layer))
        m = M()
        m.layer_idx = layer
        ref, _ = full.attention_forward(m, q, k, v, None, c.D ** -0.5)                 # [B,L,H,D]
        out, _ = part.attention_forward(m, q[:, qh].contiguous(), k[:, heads].contiguous(), v[:, heads].contiguous(),
                                        None, c.D ** -0.5)
        part.wait_gathers()
        torch.cuda.synchronize()
        worst = max(worst, (out.float() - ref[:, :, qh].float()).abs().max().item())
        gathered = part.gathered_out
        if peer_store:                                                                  # [B,L,H,D], written by both ranks' kernels
            whole = gathered
        else:                                                                           # [world,B,L,H/world,D]
            whole = torch.cat([gathered[r] for r in range(world)], dim=2)
        worst = max(worst, (whole.float() - ref.float()).abs().max().item())
    ret[rank] = (worst, nat.read_status())
    dist.destroy_process_group()


@pytest.mark.parametrize("peer_store", [False, True], ids=["all_gather", "peer_store"])
def test_sharded_prefill_matches_unsharded(peer_store):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    port = 29600 + (os.getpid() % 1000) + (500 if peer_store else 0)
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, ret, peer_store), nprocs=world, join=True)
    for r in range(world):
        worst, status = ret[r]
        assert status == 0
        assert worst == 0.0, f"rank {r}: sharded output differs from unsharded by {worst}"
