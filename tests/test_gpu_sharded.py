"""KV-head-sharded prefill on two GPUs against the unsharded strategy (needs >= 2 CUDA devices)."""
import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _worker(rank, world, port, ret, exchange):
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
                                    exchange=exchange)
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
        if gathered.dim() == 4:                                                         # [B,L,H,D], filled by both ranks
            whole = gathered
        else:                                                                           # rank-major [world,B,L,H/world,D]
            whole = torch.cat([gathered[r] for r in range(world)], dim=2)
        worst = max(worst, (whole.float() - ref.float()).abs().max().item())
    ret[rank] = (worst, nat.read_status())
    dist.destroy_process_group()


@pytest.mark.parametrize("exchange", ["nccl", "peer_store", "push", "push_slices", "multicast"])
def test_sharded_prefill_matches_unsharded(exchange):
    """Outputs of every layer, gathered by an NCCL all-gather, by the kernels' own peer stores (plain or multicast), or
    by copy-engine pushes on side streams (pitched or contiguous slices), equal the unsharded strategy's bit for bit."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    port = 29600 + (os.getpid() % 1000) + {"nccl": 0, "peer_store": 500, "push": 1000, "multicast": 1500, "push_slices": 2000}[exchange]
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, ret, exchange), nprocs=world, join=True)
    for r in range(world):
        worst, status = ret[r]
        assert status == 0
        assert worst == 0.0, f"rank {r}: sharded output differs from unsharded by {worst}"


def test_call_with_tensors_of_another_device_than_the_current_one():
    """The wrappers make the tensors' GPU current for the call: a host thread whose current device is 0 can
    run the kernels on tensors that live on device 1, and each device keeps its own init state."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from kascade_b200 import _native as nat
    g = torch.Generator().manual_seed(8)
    q = (torch.randn(1, 160, 8, 128, generator=g) / 128 ** 0.5).half()
    k = (torch.randn(1, 160, 2, 128, generator=g) / 128 ** 0.5).half()
    v = torch.randn(1, 160, 2, 128, generator=g).half()
    outs = []
    torch.cuda.set_device(0)
    for dev in ("cuda:1", "cuda:0"):
        out = torch.empty(1, 160, 8, 128, dtype=torch.float16, device=dev)
        nat.prefill_dense(q.to(dev), k.to(dev), v.to(dev), 128 ** -0.5, out, None)
        assert torch.cuda.current_device() == 0
        torch.cuda.synchronize(dev)
        outs.append(out.cpu())
        assert nat.read_status(dev) == 0
    assert torch.equal(outs[0], outs[1])
    ref = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2).float(), k.transpose(1, 2).float(),
                                                           v.transpose(1, 2).float(), is_causal=True, enable_gqa=True)
    assert (outs[0].float() - ref.transpose(1, 2)).abs().max().item() < 2e-3
