"""Host side of the Kascade hot path: the ``efficient_kascade`` attention strategy.

Mirrors the plugin interface of the reference (strategies/Strategy.py:8-27,
strategies/EfficientKascadeStrategy.py:16-168): same constructor arguments, the same
``attention_forward(module, query, key, value, attention_mask, scaling, dropout, **kw)`` hook that
HF attention modules call once per layer in layer order, the same ``register_attention`` into the
HF registries and the same ``.npy`` head-mapping lookup (strategies/KascadeStrategy.py:174-183).
All arithmetic runs in libkascade_b200.so through :mod:`kascade_b200._native`; PyTorch only owns
device memory and the stream.

Selection semantics follow the reference's PyTorch ``KascadeStrategy`` (the parity oracle):
budget ``min(max(128, int(k/100*Lk)), Lk) - tile_size`` (strategies/KascadeStrategy.py:127-129),
rolling prefill budgets ``max(128, k*tile_start//100)`` (:134-139), keys at or after a tile's
first query are never candidates (:83), layer 0 dense (:99).  Index rows are stored per query tile
([B, G, T, k], as in strategies/EfficientKascadeStrategy.py:82-84) in ascending key order with an
explicit count per row.
"""
from __future__ import annotations

import math
import os
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from . import _native as nat

__all__ = ["Strategy", "EfficientKascadeStrategy", "topk_budget", "shard_kv_heads", "shard_head_map",
           "gather_index_rows"]


def shard_kv_heads(num_kv_heads: int, rank: int, world: int) -> List[int]:
    """KV heads owned by `rank` when a layer's heads are split evenly over `world` GPUs."""
    if num_kv_heads % world:
        raise ValueError(f"{num_kv_heads} KV heads do not divide over {world} ranks")
    per = num_kv_heads // world
    return list(range(rank * per, (rank + 1) * per))


def shard_head_map(mapping_row: Sequence[int], rank: int, world: int) -> List[int]:
    """The head-mapping entries of the local KV heads.  Values stay GLOBAL anchor-head ids: a reuse
    head may map to an anchor head that another rank computed, which is why the anchors' index rows
    are all-gathered (`gather_index_rows`)."""
    return [int(mapping_row[g]) for g in shard_kv_heads(len(mapping_row), rank, world)]


def gather_index_rows(local_idx: torch.Tensor, local_count: torch.Tensor, group=None):
    """All-gather the anchor index rows of every rank's KV heads.

    local_idx [1, Gl, T, k], local_count [1, Gl, T]  ->  ([1, G, T, k], [1, G, T]) with heads in rank
    order (batch 1: the gathered buffers are then exactly the [B, G, T, k] layout the kernels index).
    Works on NCCL (GPU) and gloo (CPU tests)."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    if local_idx.shape[0] != 1:
        raise NotImplementedError("head-sharded prefill supports batch 1")
    _, gl, T, k = local_idx.shape
    idx = torch.empty((1, world * gl, T, k), dtype=local_idx.dtype, device=local_idx.device)
    cnt = torch.empty((1, world * gl, T), dtype=local_count.dtype, device=local_count.device)
    dist.all_gather_into_tensor(idx.view(world, -1), local_idx.reshape(1, -1).contiguous(), group=group)
    dist.all_gather_into_tensor(cnt.view(world, -1), local_count.reshape(1, -1).contiguous(), group=group)
    return idx, cnt


def topk_budget(pct: float, lk: int, tile_size: int) -> int:
    """strategies/KascadeStrategy.py:127-129."""
    k = min(max(128, int((pct / 100) * lk)), lk)
    if tile_size > 1:
        k -= tile_size
    return k


class Strategy:
    """strategies/Strategy.py:8-27: a named attention function that registers itself."""

    def __init__(self, name: str):
        self.name = name
        self.register_attention()

    def register_attention(self):
        pass

    def attention_forward(self, module, query, key, value, attention_mask, scaling, dropout=0.0, **kwargs):
        pass


class EfficientKascadeStrategy(Strategy):
    """Drop-in for the reference's ``EfficientKascadeStrategy``.

    Extra keyword arguments (not in the reference) are keyword-only: ``head_mapping`` passes the
    ``[num_layers][G]`` table directly instead of reading the ``.npy`` file, ``register`` skips the
    HF registration (for use without transformers), ``shard=(rank, world)`` makes this instance
    compute only its slice of the KV heads of every prefill layer (batch 1): the caller passes the
    local heads' q/k/v, anchor index rows are all-gathered over torch.distributed, and the per-head
    outputs of every layer are all-gathered into ``self.gathered_out`` ([world, B, L, H/world, D]).
    ``exchange`` picks how the sharded outputs travel:

    * ``"nccl"`` (default): an asynchronous ``all_gather_into_tensor`` per layer;
    * ``"peer_store"`` (or ``peer_store=True``): no collective, the prefill kernels store their rows straight
      into every rank's [B, L, H, D] buffer over NVLink (best on two GPUs, where a layer's compute time
      exceeds its link time);
    * ``"push"``: the kernel writes this rank's heads into its own [B, L, H, D] buffer and the copy engines
      push that slice into the peers' buffers on side streams while the next layers' kernels run (best
      from four GPUs on, where a reuse layer's link time exceeds its compute time);
    * ``"push_slices"``: like ``"push"``, but the buffers are rank-major ([world, B, L, H/world, D], the layout of
      ``"nccl"``): a rank's slice is one contiguous piece, which the copy engines move at the full link rate (a
      pitched copy of 1-2 KB rows reaches about 60 % of it), and a deeper ring (12 buffers) lets the copies of
      the short reuse layers lag behind the kernels;
    * ``"multicast"``: the kernel stores every row once to an NVLink multicast address (NVLS) and the NVSwitch
      delivers it to all ranks: a rank's egress is its own slice instead of (ranks - 1) copies of it.  Needs
      symmetric memory with a multicast mapping; falls back to ``"peer_store"`` where there is none.

    In the peer-mapped modes ``gathered_out`` is a buffer of a small ring (``copies``), complete
    once ``wait_gathers()`` has returned on every rank.  The buffer of layer n is written again by layer
    n + copies (and by the peers' kernels or copies of that layer): a consumer that reads every layer's
    ``gathered_out`` must call ``wait_gathers()`` after every layer, on all ranks, before it reads."""

    def __init__(self, recompute_layers: List[int], model_name: str, k=1, tile_size=1, rolling_prefill=False,
                 block_size=12288, *, head_mapping: Optional[Sequence[Sequence[int]]] = None,
                 register: bool = True, shard: Optional[tuple] = None, peer_store: bool = False,
                 exchange: Optional[str] = None, copies: Optional[int] = None):
        if recompute_layers is None:
            raise ValueError("recompute_layers cannot be None for EfficientKascadeStrategy")
        if not (0 <= k <= 100):
            raise AssertionError(f"Invalid k: {k}. It should be between 0 and 100%.")
        if tile_size != nat.TILE:
            # the reference only ships kernels for tile_size 32 (README.md:74)
            raise ValueError(f"tile_size must be {nat.TILE}, got {tile_size}")
        self.k = k
        self.tile_size = tile_size
        self.rolling_prefill = rolling_prefill
        self._block_size = block_size          # accepted for signature parity; the kernels tile on their own
        self.recompute_layers = list(recompute_layers)
        self._heads, self._groups, self._dim = 32, 8, nat.HEAD_DIM
        self._head_mapping = [list(map(int, r)) for r in head_mapping] if head_mapping is not None \
            else self.get_head_mapping(model_name)
        self._register = register
        self._shard = tuple(shard) if shard is not None else None
        if exchange is None:
            exchange = "peer_store" if peer_store else "nccl"
        if exchange not in ("nccl", "peer_store", "push", "push_slices", "multicast"):
            raise ValueError(f"exchange must be 'nccl', 'peer_store', 'push', 'push_slices' or 'multicast', got {exchange!r}")
        sharded = self._shard is not None and self._shard[1] > 1
        self._exchange = exchange if sharded else "nccl"
        self._peer_store = self._exchange in ("peer_store", "push", "push_slices", "multicast")   # outputs live in peer-mapped buffers
        self._copies = int(copies) if copies else {"push": 4, "push_slices": 12}.get(self._exchange, 2)
        self._peer = None                       # kascade_b200.peer.PeerBuffers, allocated at the first prefill
        self._peer_copy = 0
        self._push = None                       # push mode: streams, events and plans
        self._checked_device = None
        self.gathered_out: Optional[torch.Tensor] = None
        self._pending = []
        # cross-layer state written by anchor layers (strategies/KascadeStrategy.py:95,133)
        self._tile_idx: Optional[torch.Tensor] = None       # prefill [B,G,T,k]
        self._tile_count: Optional[torch.Tensor] = None     # prefill [B,G,T]
        self._dec_idx: Optional[torch.Tensor] = None        # decode  [B,G,k]
        self._dec_count: Optional[torch.Tensor] = None      # decode  [B,G]
        self._dec_kmax = 0
        self._map_dev: Dict[tuple, torch.Tensor] = {}
        self._buf: Dict[str, torch.Tensor] = {}
        super().__init__("efficient_kascade")

    # ------------------------------------------------------------------------------------------
    def get_head_mapping(self, model_name: str):
        """strategies/KascadeStrategy.py:174-183 (path relative to the working directory)."""
        try:
            base = model_name.split("/")[-1]
            path = f"./results/head_mappings/{base}_layers_{'_'.join(map(str, self.recompute_layers))}.npy"
            return np.load(path).tolist()
        except Exception:
            raise ValueError(f"Head mapping file not found for model {model_name} with layers {self.recompute_layers}.")

    def register_attention(self):
        """strategies/EfficientKascadeStrategy.py:163-168."""
        if not getattr(self, "_register", True):
            return
        from transformers.masking_utils import ALL_MASK_ATTENTION_FUNCTIONS
        from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS

        def _fwd(module, query, key, value, attention_mask, scaling, dropout=0.0, **kwargs):
            return self.attention_forward(module, query, key, value, attention_mask, scaling, dropout=dropout, **kwargs)

        ALL_MASK_ATTENTION_FUNCTIONS.register(self.name, ALL_MASK_ATTENTION_FUNCTIONS["sdpa"])
        ALL_ATTENTION_FUNCTIONS.register(self.name, _fwd)

    def check_status(self, device=None):
        """Raise ``KascadeNativeError`` if a kernel gave up a bounded device-side wait since the last check
        (its outputs are then invalid).  Synchronises the device.  Called by this class at the first layer of
        every prompt, in ``wait_gathers()`` and wherever it has to synchronise anyway; a host that wants to
        know right after a forward calls it itself."""
        nat.check_status(device, "in an efficient_kascade prefill")

    def exchange_description(self) -> str:
        if self._shard is None or self._shard[1] == 1:
            return "single GPU"
        how = f" ({self._peer.how})" if self._peer is not None else ""
        return {"nccl": "outputs all-gathered by NCCL",
                "peer_store": "outputs stored into the peers by the kernel epilogue" + how,
                "push": f"outputs pushed to the peers by the copy engines on side streams, {self._copies} buffers" + how,
                "push_slices": f"contiguous rank-major slices pushed to the peers by the copy engines on side streams, "
                               f"{self._copies} buffers" + how,
                "multicast": "outputs stored once to an NVLink multicast address by the kernel epilogue (NVLS)" + how,
                }[self._exchange]

    def is_anchor(self, layer_idx: int) -> bool:
        return layer_idx == 0 or layer_idx in self.recompute_layers

    # ------------------------------------------------------------------------------------------
    def _scratch(self, name: str, shape, dtype, device) -> torch.Tensor:
        """Grow-only cache of device buffers, so steady-state calls allocate nothing."""
        n = int(math.prod(shape))
        buf = self._buf.get(name)
        if buf is None or buf.numel() < n or buf.dtype != dtype or buf.device != device:
            buf = torch.empty(max(n, 1), dtype=dtype, device=device)
            self._buf[name] = buf
        return buf[:n].view(*shape)

    def _mapping(self, layer_idx: int, device) -> torch.Tensor:
        key = (layer_idx, device)
        m = self._map_dev.get(key)
        if m is None:
            row = self._head_mapping[layer_idx]
            if self._shard is not None:
                row = shard_head_map(row, *self._shard)
            m = torch.tensor(row, dtype=torch.int32, device=device)
            self._map_dev[key] = m
        return m

    @staticmethod
    def _token_major(x: torch.Tensor) -> torch.Tensor:
        """[B, heads, L, D] -> a [B, L, heads, D] view with D contiguous and 16-byte aligned strides."""
        y = x.transpose(1, 2)
        if y.stride(3) != 1 or any(s % 8 for s in y.stride()[:3]) or y.data_ptr() % 16:
            y = y.contiguous()
        return y

    # ------------------------------------------------------------------------------------------
    def attention_forward(self, module, query, key, value, attention_mask, scaling, dropout=0.0, **kwargs):
        """query [B,H,Lq,D], key/value [B,G,Lk,D] -> (out [B,Lq,H,D], None).

        The reference (strategies/EfficientKascadeStrategy.py:126-161) never reads the mask: prompts are
        causal and unpadded, a decode step attends to the whole cache.  Here the mask is read for one
        thing only, padding of a batch (leading / trailing key positions that no query may see): the kernels
        then get every sequence's first row and length and treat it as if it had been run alone."""
        if query.dtype not in nat.DTYPES or key.dtype != query.dtype or value.dtype != query.dtype:
            raise nat.KascadeNativeError(f"efficient_kascade takes fp16 or bf16 q / k / v of one type; got {query.dtype}, "
                                         f"{key.dtype}, {value.dtype}")
        B, H, Lq, D = query.shape
        G, Lk = key.shape[1], key.shape[2]
        layer = int(module.layer_idx)
        pad = self._padding(attention_mask, B, Lk) if self._shard is None else None
        if pad is not None:
            if Lq == 1:
                return self._decode_padded(pad, module, query, key, value, scaling), None
            if Lq != Lk:
                raise NotImplementedError("prefill expects the whole prompt (Lq == Lk); chunked prefill is not supported")
            starts, lens = pad
            dev = query.device
            rg = (torch.tensor(starts, dtype=torch.int32, device=dev), torch.tensor(lens, dtype=torch.int32, device=dev), lens)
            q, k, v = self._token_major(query), self._token_major(key), self._token_major(value)
            return self._prefill(layer, q, k, v, scaling, ragged=rg), None
        if Lq == 1:
            kv = nat.kv_layout_contiguous(*self._cache_views(key, value))
            seq_lens = self._scratch("seq_lens_full", (B,), torch.int32, query.device)
            seq_lens.fill_(Lk)
            dense = Lk <= 128                      # strategies/EfficientKascadeStrategy.py:137-140
            out = self._decode(layer, query[:, :, 0], kv, seq_lens, Lk, scaling, G, dense_only=dense)
            return out.unsqueeze(1), None
        if Lq != Lk:
            raise NotImplementedError("prefill expects the whole prompt (Lq == Lk); chunked prefill is not supported")
        if layer == 0:
            # a tile-prefill kernel that gave up a bounded wait leaves a status word behind, and every later
            # one returns at entry while it is set: find out before the next prompt is queued behind it
            self.check_status(query.device)
        q, k, v = self._token_major(query), self._token_major(key), self._token_major(value)
        if Lk <= 128:
            out = torch.empty(B, Lq, H, D, dtype=query.dtype, device=query.device)
            nat.prefill_dense(q, k, v, scaling, out, None)
            return out, None
        return self._prefill(layer, q, k, v, scaling), None

    # -- padded batches ---------------------------------------------------------------------------
    def _padding(self, attention_mask, B: int, Lk: int):
        """(first row, length) of every sequence if the batch is padded, read from the key columns that the mask
        lets the LAST query row see (left padding hides a prefix, right padding a suffix), or None for a batch
        without padding.  HF hands the same mask tensor to every layer of a forward, so the (synchronising) look at
        it happens once per forward."""
        if attention_mask is None or attention_mask.dim() != 4 or attention_mask.shape[0] != B \
                or attention_mask.shape[-1] != Lk:
            return None
        ref = getattr(self, "_pad_ref", None)
        if ref is None or ref() is not attention_mask or self._pad_version != attention_mask._version:
            import weakref
            last = attention_mask[:, 0, -1, :]                                    # [B, Lk]
            seen = last if last.dtype == torch.bool else last == 0
            n_seen = seen.sum(-1)
            first = torch.where(n_seen > 0, seen.to(torch.int32).argmax(-1), torch.zeros_like(n_seen))
            both = torch.stack([first, n_seen]).tolist()
            if attention_mask.is_cuda:
                self.check_status(attention_mask.device)                          # the host has just synchronised
            starts, lens = [int(x) for x in both[0]], [int(x) for x in both[1]]
            self._pad_ref, self._pad_version = weakref.ref(attention_mask), attention_mask._version
            self._pads = None if all(n == Lk for n in lens) else (starts, lens)
        return self._pads

    def _decode_padded(self, pad, module, query, key, value, scaling) -> torch.Tensor:
        """One decode step of a padded batch, every kernel launched once: the cache rows of sequence b are
        starts[b] .. starts[b] + lens[b] - 1, described to the decode kernels as a block table with one-token pages
        (logical position -> cache row), so index rows, budgets and lengths are those of the unpadded sequences."""
        starts, lens = pad
        B, H, Lq, D = query.shape
        G, Lk = key.shape[1], key.shape[2]
        dev = query.device
        max_len = max(lens)
        if max_len == 0:
            return torch.zeros(B, Lq, H, D, dtype=query.dtype, device=dev)
        cached = getattr(self, "_pad_rows", None)
        if cached is None or cached[0] is not pad or cached[1].device != dev:
            first = torch.tensor(starts, dtype=torch.int32, device=dev)
            rows = (first[:, None] + torch.arange(Lk, dtype=torch.int32, device=dev)[None, :]).clamp_(max=Lk - 1)
            cached = self._pad_rows = (pad, rows.contiguous(), torch.tensor(lens, dtype=torch.int32, device=dev))
        key, value = self._cache_views(key, value)
        kv = nat.kv_layout_rows(key, value, cached[1])
        out = self._decode(int(module.layer_idx), query[:, :, 0], kv, cached[2], max_len, scaling, G,
                           dense_only=max_len <= 128,              # strategies/EfficientKascadeStrategy.py:137-140
                           mean_len=max(sum(lens) / len(lens), 1.0))
        return out.unsqueeze(1)

    @staticmethod
    def _cache_views(key, value):
        if key.stride(3) != 1 or any(s % 8 for s in key.stride()[:3]) or key.stride() != value.stride():
            key, value = key.contiguous(), value.contiguous()
        return key, value

    # -- prefill -----------------------------------------------------------------------------------
    def _prefill(self, layer: int, q, k, v, scaling, ragged=None) -> torch.Tensor:
        """q [B,L,H,D], k / v [B,L,G,D] token-major views.  `ragged` = (first rows [B] int32, lengths [B] int32 on
        the device, lengths on the host): a padded batch, every kernel still launched once; rows outside a sequence
        come back as zeros."""
        B, L, H, D = q.shape
        G = k.shape[2]
        dev = q.device
        T = -(-L // self.tile_size)
        self._out_dtype = q.dtype
        fan = self._next_fanout(B, L, H, D, dev) if self._peer_store else None      # None: not in use (or not available)
        rg = nat.ragged(ragged[0], ragged[1]) if ragged is not None else None
        if self._exchange == "push_slices" and self._peer_store:
            fan, out = None, self.gathered_out[self._shard[0]]      # this rank's contiguous [B, L, H/world, D] slot
            if rg is not None:
                out.zero_()
        elif fan is not None:
            out = None
        elif rg is not None:
            out = torch.zeros(B, L, H, D, dtype=q.dtype, device=dev)
        else:
            out = torch.empty(B, L, H, D, dtype=q.dtype, device=dev)
        if self.is_anchor(layer):
            kk = topk_budget(self.k, L, self.tile_size) if ragged is None else \
                max(1, max(topk_budget(self.k, n, self.tile_size) for n in ragged[2]))
            lse2 = self._scratch("lse2", (B, L, H), torch.float32, dev)
            if layer == 0 and fan is not None:
                nat.prefill_dense(q, k, v, scaling, None, lse2, fanout=fan)
            else:
                nat.prefill_dense(q, k, v if layer == 0 else None, scaling, out if layer == 0 else None, lse2, ragged=rg)
            stride = -(-L // 128) * 128
            pooled = self._scratch("pooled", (B, G, T, stride), torch.float32, dev)
            nat.prefill_pool_scores(q, k, lse2, scaling, pooled, ragged=rg)
            n_valid = self._scratch("n_valid", (B, G, T), torch.int32, dev)
            k_row = self._scratch("k_row", (B, G, T), torch.int32, dev)
            if ragged is None:
                nat.prefill_budgets(n_valid, k_row, B, G, T, kk, self.k, self.rolling_prefill and L > 128)
            else:
                nat.prefill_budgets_ragged(n_valid, k_row, ragged[1], B, G, T, kk, self.k, self.rolling_prefill)
            self._tile_idx = self._scratch("tile_idx", (B, G, T, max(kk, 1)), torch.int32, dev)
            self._tile_count = self._scratch("tile_count", (B, G, T), torch.int32, dev)
            nat.topk_select(pooled, n_valid, k_row, kk, self._tile_idx, self._tile_count, n_cols=L)
            if self._shard is not None:
                self._tile_idx, self._tile_count = gather_index_rows(self._tile_idx, self._tile_count)
            if layer == 0:
                return self._publish(out)
            head_map = self._mapping(layer, dev) if self._shard is not None else None
        else:
            if self._tile_idx is None:
                raise RuntimeError("reuse layer called before any anchor layer")
            head_map = self._mapping(layer, dev)
        nat.prefill_sparse(q, k, v, self._tile_idx, self._tile_count, head_map, scaling, out, fanout=fan, ragged=rg)
        return self._publish(out)

    def _publish(self, out: torch.Tensor) -> torch.Tensor:
        """Head-sharded runs: start the exchange of this layer's per-head outputs (asynchronous) and return
        the local slice."""
        if self._shard is None:
            return out
        if self._peer_store:
            full = self.gathered_out
            rank, world = self._shard
            if self._exchange == "push_slices":
                piece = full[rank].numel() * full.element_size()
                c = self._peer_copy
                nat.peer_push(self._push["plans"][c], full, rank * piece, world * piece, piece, 1, self._push["ready"][c])
                return full[rank]
            h = full.shape[2] // world
            if self._exchange == "push":
                # the kernel has written this rank's heads into its own buffer; the copy engines carry the
                # slice to the peers while the next layers run
                B, L, H, D = full.shape
                c = self._peer_copy
                nat.peer_push(self._push["plans"][c], full, rank * h * D * 2, H * D * 2, h * D * 2, B * L,
                              self._push["ready"][c])
            return full[:, :, rank * h:(rank + 1) * h]
        import torch.distributed as dist
        world = self._shard[1]
        self._pending = [w for w in self._pending if not w[0].is_completed()]
        buf = torch.empty((world,) + tuple(out.shape), dtype=out.dtype, device=out.device)
        work = dist.all_gather_into_tensor(buf.view(world, -1), out.view(1, -1), async_op=True)
        self._pending.append((work, buf, out))
        self.gathered_out = buf
        return out

    def wait_gathers(self, check_status: bool = False):
        """Block the current stream until every rank's outputs started so far have arrived.  With
        ``check_status`` the device status word is read too (that synchronises the host)."""
        if self._peer_store:
            if self._peer is not None:
                import torch.distributed as dist
                if self._push is not None:                 # this rank's own copies first
                    nat.stream_wait_events([e for evs in self._push["done"] for e in evs])
                # stream-ordered after this rank's kernels and copies; completes once every rank has got here
                dist.all_reduce(self._scratch("peer_sync", (1,), torch.int32, self._peer.tensors[0].device))
        else:
            for work, _, _ in self._pending:
                work.wait()
            self._pending = []
        if check_status:
            self.check_status()

    def _next_fanout(self, B: int, L: int, H: int, D: int, dev):
        """Peer-mapped output buffers: the [B, L, H_total, D] buffer of this layer (a ring of `copies`) as a
        kb200_out_fanout — every rank's buffer in peer-store mode, this rank's own buffer in push mode."""
        rank, world = self._shard
        shape = (world, B, L, H, D) if self._exchange == "push_slices" else (B, L, H * world, D)
        if self._peer is None or tuple(self._peer.tensors[0].shape) != shape or self._peer.tensors[0].dtype != self._out_dtype:
            from .peer import alloc_peer_buffers
            try:
                self._peer = alloc_peer_buffers(shape, self._out_dtype, dev, copies=self._copies)
            except RuntimeError as e:
                # no peer mapping in this job (every rank gets here together): keep the sharded prefill
                # running with the NCCL all-gather of the outputs
                import warnings
                warnings.warn(f"exchange '{self._exchange}' disabled, outputs are all-gathered with NCCL instead: {e}")
                self._peer_store, self._exchange = False, "nccl"
                return None
            n = self._copies
            if self._exchange == "multicast" and not (self._peer.multicast and all(self._peer.multicast)):
                import warnings
                warnings.warn("no NVLink multicast mapping for the output buffers: exchange 'multicast' -> 'peer_store'")
                self._exchange = "peer_store"
            if self._exchange == "multicast":
                self._peer_fans = [nat.out_fanout([self._peer.multicast[c]], H * world, rank * H, multicast=True)
                                   for c in range(n)]
            elif self._exchange in ("push", "push_slices"):
                self._peer_fans = [nat.out_fanout([self._peer.pointers[c][rank]], H * world, rank * H) for c in range(n)]
                streams = [torch.cuda.Stream(device=dev) for _ in range(world - 1)]
                done = [[torch.cuda.Event() for _ in range(world - 1)] for _ in range(n)]
                ready = [torch.cuda.Event() for _ in range(n)]
                plans = [nat.push_plan(self._peer.fanout_pointers(c, rank)[1:], streams, done[c]) for c in range(n)]
                self._push = {"streams": streams, "done": done, "ready": ready, "plans": plans}
            else:
                self._peer_fans = [nat.out_fanout(self._peer.fanout_pointers(c, rank), H * world, rank * H)
                                   for c in range(n)]
        self._peer_copy = (self._peer_copy + 1) % self._copies
        if self._push is not None:
            # the copies that still read this buffer (layer n - copies) must have finished
            nat.stream_wait_events(self._push["done"][self._peer_copy])
        self.gathered_out = self._peer.tensors[self._peer_copy]
        return self._peer_fans[self._peer_copy]

    # -- decode ------------------------------------------------------------------------------------
    def _decode_budgets(self, seq_lens: torch.Tensor, max_len: int):
        """Per-sequence key budgets on the device (no sync): the reference formula for a cache of
        seq_lens[b] keys; sequences of at most 128 keys attend to everything."""
        lens = seq_lens.to(torch.float64)
        kk = torch.clamp(torch.floor((self.k / 100) * lens), min=128.0)
        kk = torch.minimum(kk, lens) - self.tile_size
        kk = torch.where(lens <= 128, lens, kk).to(torch.int32)
        # rows are as long as the largest per-sequence budget: the reference formula at max_len, and the
        # "at most 128 keys: attend to everything" rule for the short sequences of a mixed batch
        kmax = max_len if max_len <= 128 else max(topk_budget(self.k, max_len, self.tile_size), 128)
        return kk, max(kmax, 1)

    @staticmethod
    def _splits(B: int, G: int, keys_max: int, raggedness: float, dev) -> int:
        """Splits per (sequence, KV head).  The library's own choice assumes sequences of one length; in a batch whose
        longest sequence is `raggedness` times the mean the CTAs of the long ones would set the kernel's time, so
        they are cut until the longest CTA is about the batch's work divided by three CTAs per SM (measured on
        batches of 32-128 sequences of 4k-65k tokens: 10-19 % faster at 32 and 64 sequences, no change at 128)."""
        s = nat.decode_default_splits(B, G, keys_max)
        if raggedness > 1.25:
            slots = 3 * torch.cuda.get_device_properties(dev).multi_processor_count
            want = -(-int(raggedness * slots) // max(B * G, 1))
            s = max(s, min(want, max(keys_max // 256, 1), 32))
        return s

    def _decode(self, layer: int, q, kv, seq_lens, max_len: int, scaling, G: int, dense_only=False,
                mean_len: Optional[float] = None) -> torch.Tensor:
        B, H, D = q.shape
        dev = q.device
        if q.stride(2) != 1 or q.stride(0) % 2 or q.stride(1) % 2:
            q = q.contiguous()
        out = torch.empty(B, H, D, dtype=q.dtype, device=dev)
        ragged = float(max_len) / mean_len if mean_len else 1.0
        splits_a = self._splits(B, G, max_len, ragged, dev)
        if dense_only or self.is_anchor(layer):
            stride = -(-max_len // 4) * 4
            logits = self._scratch("dec_logits", (B, H, stride), torch.float32, dev)
            pooled = self._scratch("dec_pooled", (B, G, stride), torch.float32, dev)
            lse2 = self._scratch("dec_lse2", (B, H), torch.float32, dev)
            ws = self._scratch("dec_ws", (nat.load().kb200_decode_workspace_bytes(B, H, splits_a),), torch.uint8, dev)
            want_out = dense_only or layer == 0
            nat.decode_anchor_paged(q, kv, seq_lens, max_len, scaling, logits, pooled, out if want_out else None,
                                    lse2, ws, splits_a)
            if dense_only:
                return out
            k_row, kmax = self._decode_budgets(seq_lens, max_len)
            self._dec_kmax = kmax
            self._dec_idx = self._scratch("dec_idx", (B, G, kmax), torch.int32, dev)
            self._dec_count = self._scratch("dec_count", (B, G), torch.int32, dev)
            n_valid = seq_lens.view(B, 1).expand(B, G).contiguous()
            k_rows = k_row.view(B, 1).expand(B, G).contiguous()
            nat.topk_select(pooled, n_valid, k_rows, kmax, self._dec_idx, self._dec_count, n_cols=max_len)
            if layer == 0:
                return out
            head_map = None
        else:
            if self._dec_idx is None:
                raise RuntimeError("reuse layer called before any anchor layer")
            head_map = self._mapping(layer, dev)
        kmax = self._dec_kmax
        splits = self._splits(B, G, kmax, ragged, dev)
        ws = self._scratch("dec_ws_s", (nat.load().kb200_decode_workspace_bytes(B, H, splits),), torch.uint8, dev)
        nat.decode_sparse_paged(q, kv, self._dec_idx, self._dec_count, kmax, head_map, scaling, out, None, ws, splits)
        return out

    @staticmethod
    def append_kv(key_new, value_new, key_cache, value_cache, block_table, start_pos, n_new=None, *, query=None,
                  q_norm_weight=None, k_norm_weight=None, norm_eps: float = 1e-6, inv_freq=None,
                  rope_scale: float = 1.0, k_scale=None, v_scale=None):
        """Prefill -> decode hand-off: write the new tokens' K / V rows (key_new / value_new [B,T,G,D] views,
        positions start_pos[b] + t) into the paged cache the decode kernels read, in one kernel; with
        `inv_freq` (the model's rotary table) and / or the norm weights the rows (and `query` [B,T,H,D], returned
        transformed) are normalised and rotated on the way, as the Hugging Face module would have done; into an FP8
        (e4m3) cache, with `k_scale` / `v_scale` [num_pages, G] fp32, the rows are stored as value / scale.
        The reference has no counterpart (it receives rotated tensors and copies them per call,
        strategies/EfficientKascadeStrategy.py:144-150)."""
        kv = nat.kv_layout_paged(key_cache, value_cache, block_table, k_scale, v_scale)
        q_out = torch.empty_like(query, memory_format=torch.contiguous_format) if query is not None else None
        nat.kv_write(query, q_out, key_new, value_new, start_pos, n_new, kv, q_norm_weight, k_norm_weight, norm_eps,
                     inv_freq, rope_scale)
        return q_out

    def paged_decode_forward(self, layer_idx: int, query, key_cache, value_cache, block_table, seq_lens, scaling,
                             max_seq_len: Optional[int] = None, k_scale=None, v_scale=None,
                             mean_seq_len: Optional[float] = None) -> torch.Tensor:
        """Paged-attention backend entry: query [B,H,D] fp16 / bf16, key/value cache
        [num_pages, page_size, G, D] of the same type, block_table [B, max_pages] int32, seq_lens [B] int32
        -> out [B,H,D].  An FP8 (e4m3) cache comes with k_scale / v_scale [num_pages, G] fp32 and takes fp16
        queries.  `mean_seq_len` is a hint of the host for batches of very different lengths (the work is then cut
        into more, smaller pieces); results do not depend on it beyond summation order.  The reference has no paged kernel (README.md:135); the nearest
        signature is kernels/flash_decoding/reuse_kascade_gqa_decode_with_kvcache.py:160-171."""
        if max_seq_len is None:
            max_seq_len = int(seq_lens.max().item())
        kv = nat.kv_layout_paged(key_cache, value_cache, block_table, k_scale, v_scale)
        return self._decode(int(layer_idx), query, kv, seq_lens, int(max_seq_len), scaling, key_cache.shape[2],
                            mean_len=mean_seq_len)
