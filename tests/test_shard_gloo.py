"""World-size-2 gloo test of the head-sharded prefill plumbing (CPU): the all-gathered index rows and the
sharded head maps must make every local reuse head read exactly the row the unsharded layer reads."""
import os
import sys

import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from kascade_b200.strategy import gather_index_rows, shard_head_map, shard_kv_heads
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    G, T, K = 8, 5, 7
    g = torch.Generator().manual_seed(0)
    full_idx = torch.randint(0, 1000, (1, G, T, K), generator=g, dtype=torch.int32)
    full_cnt = torch.randint(0, K + 1, (1, G, T), generator=g, dtype=torch.int32)
    mapping = [7, 1, 5, 6, 3, 3, 3, 3]
    mine = shard_kv_heads(G, rank, world)
    idx, cnt = gather_index_rows(full_idx[:, mine].contiguous(), full_cnt[:, mine].contiguous())
    ok = torch.equal(idx, full_idx) and torch.equal(cnt, full_cnt)
    local_map = shard_head_map(mapping, rank, world)
    for gl, g_global in enumerate(mine):               # local head gl reads gathered row local_map[gl]
        ok = ok and torch.equal(idx[0, local_map[gl]], full_idx[0, mapping[g_global]])
    ret[rank] = bool(ok)
    dist.destroy_process_group()


def test_gather_index_rows_world2():
    world = 2
    port = 29500 + (os.getpid() % 2000)
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert dict(ret) == {0: True, 1: True}
