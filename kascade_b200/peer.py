"""Buffers that every GPU of a single-node job can write into (head-sharded prefill).

`alloc_peer_buffers` gives each rank `copies` local fp16 tensors of the same shape plus, for every copy,
the device addresses under which ALL ranks' tensors are mapped into this process, so that a kernel
running here can store into its peers' memory over NVLink (plain stores; nothing here uses multicast).
Two mechanisms, tried in this order: torch's symmetric memory, then CUDA IPC handles exchanged with
`all_gather_object`.  There is no fallback beyond that: if neither works the call raises.
"""
from __future__ import annotations

from typing import List, Tuple

import torch
import torch.distributed as dist


class PeerBuffers:
    def __init__(self, tensors: List[torch.Tensor], pointers: List[List[int]], how: str, keep=None, multicast=None):
        self.tensors = tensors            # this rank's buffers, one per copy
        self.pointers = pointers          # [copy][rank] -> device address valid in this process
        self.how = how                    # "symmetric_memory" or "cuda_ipc"
        self._keep = keep                 # handles / mapped tensors that must stay alive
        self.multicast = multicast        # [copy] -> NVLink multicast address of the buffer (0 / None: not available)

    def fanout_pointers(self, copy: int, rank: int) -> List[int]:
        """Own buffer first, then the peers starting with rank + 1 (ranks stagger their targets)."""
        world = len(self.pointers[copy])
        return [self.pointers[copy][(rank + i) % world] for i in range(world)]


def _via_symmetric_memory(shape, dtype, device, copies, group) -> PeerBuffers:
    import torch.distributed._symmetric_memory as symm
    tensors, pointers, keep, mc = [], [], [], []
    for _ in range(copies):
        t = symm.empty(*shape, dtype=dtype, device=device)
        hdl = symm.rendezvous(t, group=group)
        tensors.append(t)
        pointers.append([int(p) for p in hdl.buffer_ptrs])
        mc.append(int(getattr(hdl, "multicast_ptr", 0) or 0))
        keep.append(hdl)
    return PeerBuffers(tensors, pointers, "symmetric_memory", keep, mc)


def _via_cuda_ipc(shape, dtype, device, copies, group) -> PeerBuffers:
    from torch.multiprocessing.reductions import reduce_tensor
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    tensors, pointers, keep = [], [], []
    for _ in range(copies):
        t = torch.empty(*shape, dtype=dtype, device=device)
        fn, args = reduce_tensor(t)
        gathered = [None] * world
        dist.all_gather_object(gathered, (fn, args), group=group)
        ptrs = []
        for r, (f, a) in enumerate(gathered):
            if r == rank:
                ptrs.append(t.data_ptr())
                continue
            peer = f(*a)                                   # maps the peer's allocation into this process
            # one element in each direction makes torch enable peer access between the two devices
            probe = torch.empty(1, dtype=dtype, device=device)
            probe.copy_(peer.view(-1)[:1])
            keep.append(peer)
            ptrs.append(peer.data_ptr())
        tensors.append(t)
        pointers.append(ptrs)
    torch.cuda.synchronize(device)
    dist.barrier(group=group)
    return PeerBuffers(tensors, pointers, "cuda_ipc", keep)


def alloc_peer_buffers(shape: Tuple[int, ...], dtype, device, copies: int = 2, group=None) -> PeerBuffers:
    if group is None:
        group = dist.group.WORLD
    errors = []
    for how in (_via_symmetric_memory, _via_cuda_ipc):
        try:
            ok = torch.ones(1, dtype=torch.int32, device=device)
            try:
                bufs = how(shape, dtype, device, copies, group)
            except Exception as e:                         # noqa: BLE001 - reported below if every way fails
                errors.append(f"{how.__name__}: {type(e).__name__}: {e}")
                ok.zero_()
                bufs = None
            # all ranks must agree on the mechanism
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
            if int(ok.item()) == 1:
                return bufs
        except Exception as e:                             # noqa: BLE001
            errors.append(f"{how.__name__}: {type(e).__name__}: {e}")
    raise RuntimeError("no way to map peer GPU memory in this job: " + "; ".join(errors))
