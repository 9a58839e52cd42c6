"""The similarity statistic behind anchor selection and head mappings, computed on the GPU by the library's own
kernels, without ever holding ``[Lq, Lk]`` attention weights.

The reference's statistics runner (runners/stats_runner.py:155-168, ``_similarity_layer``) gathers, from the
materialised post-softmax weights of layer j (pooled per KV head), the mass that falls on the Top-k keys of
(layer i, head h1) and divides it by the mass on layer j's own Top-k keys, both plus the mass on the query's own
tile.  A mass of that kind is a ratio of two softmax normalisers::

    sum_{key in S} softmax(s)[key] = sum_{key in S} exp(s_key) / sum_{all keys} exp(s_key) = exp(lse_S - lse_all)

and both normalisers are what the prefill kernels already produce: ``kb200_prefill_dense`` (lse-only pass) gives
``lse_all`` of every (query, head), and ``kb200_prefill_sparse`` attends to exactly "index row ++ own tile" and
returns the lse of that set - with ``head_map`` it takes the index rows of any other KV head.  So the statistic of a
layer pair costs G sparse passes (one per rotation of the heads) and no quadratic memory: a 32 768-token prompt of
a 32-layer model needs 528 x 8 passes of ~1.2 ms.

The index rows are the ones the efficient strategy itself would use (tile-level rows from the pooled scores,
rolling budgets), i.e. the statistic is evaluated on the sets that will be reused.  Feed
:class:`DeviceSimilarityAccumulator` one prompt at a time, layer by layer, and hand ``average()`` to
``kascade_b200.head_mapping.select_layers``.
"""
from __future__ import annotations

from typing import List

import torch

from . import _native as nat
from .strategy import topk_budget

__all__ = ["DeviceSimilarityAccumulator"]


class DeviceSimilarityAccumulator:
    """Drop-in for ``head_mapping.SimilarityAccumulator`` fed with activations instead of weights and indices.

    ``add_layer(q, k, scaling)``: q ``[1, L, H, D]``, k ``[1, L, G, D]`` token-major fp16 / bf16 CUDA tensors (rotated,
    as the attention sees them), once per layer in layer order; ``end_prompt()``; ``average()`` ->
    ``[layers, layers, G, G]`` with ``sim[i, j, h2, h1]`` for ``i <= j`` (runners/stats_runner.py:28-40, 84-96,
    127-131)."""

    def __init__(self, num_layers: int, heads: int = 8, k: float = 10, tile_size: int = 32, rolling_prefill: bool = True,
                 reduce: str = "amin"):
        if tile_size != nat.TILE:
            raise ValueError(f"tile_size must be {nat.TILE}, got {tile_size}")
        if reduce not in ("amin", "mean"):
            raise ValueError(f"reduce must be 'amin' or 'mean', got {reduce!r}")
        self.num_layers, self.heads, self.k, self.tile, self.rolling, self.reduce = \
            num_layers, heads, k, tile_size, rolling_prefill, reduce
        self.sim = None
        self.prompts = 0
        self._layers: List[tuple] = []

    # ------------------------------------------------------------------------------------------------
    def add_layer(self, q: torch.Tensor, k: torch.Tensor, scaling: float):
        B, L, H, D = q.shape
        G = k.shape[2]
        if B != 1 or G != self.heads or H != G * nat.GROUP_SIZE:
            raise ValueError(f"expected q [1, L, {self.heads * nat.GROUP_SIZE}, D] and k [1, L, {self.heads}, D]")
        dev = q.device
        T = -(-L // self.tile)
        lse_all = torch.empty(B, L, H, dtype=torch.float32, device=dev)
        nat.prefill_dense(q, k, None, scaling, None, lse_all)                       # lse-only pass
        stride = -(-L // 128) * 128
        pooled = torch.empty(B, G, T, stride, dtype=torch.float32, device=dev)
        nat.prefill_pool_scores(q, k, lse_all, scaling, pooled)
        kk = topk_budget(self.k, L, self.tile)
        n_valid = torch.empty(B, G, T, dtype=torch.int32, device=dev)
        k_row = torch.empty(B, G, T, dtype=torch.int32, device=dev)
        nat.prefill_budgets(n_valid, k_row, B, G, T, kk, self.k, self.rolling and L > 128)
        idx = torch.empty(B, G, T, max(kk, 1), dtype=torch.int32, device=dev)
        count = torch.empty(B, G, T, dtype=torch.int32, device=dev)
        nat.topk_select(pooled, n_valid, k_row, kk, idx, count, n_cols=L)
        self._layers.append((q, k, float(scaling), lse_all, idx, count))

    def _mass(self, layer: tuple, idx, count, head_map) -> torch.Tensor:
        """[L, G]: per query and KV head, the attention mass of `layer` on (index rows of the mapped head ++ own tile),
        summed over the KV head's query heads."""
        q, k, scaling, lse_all, _, _ = layer
        B, L, H, _ = q.shape
        out = torch.empty_like(q, memory_format=torch.contiguous_format)
        lse_set = torch.empty(B, L, H, dtype=torch.float32, device=q.device)
        nat.prefill_sparse(q, k, k, idx, count, head_map, scaling, out, lse_set)    # V is irrelevant here: K stands in
        return torch.exp2(lse_set - lse_all).view(L, self.heads, nat.GROUP_SIZE).sum(-1)

    def end_prompt(self):
        if len(self._layers) != self.num_layers:
            raise ValueError(f"{len(self._layers)} layers recorded, {self.num_layers} expected")
        G, dev = self.heads, self._layers[0][0].device
        if self.sim is None:
            self.sim = torch.zeros(self.num_layers, self.num_layers, G, G, dtype=torch.float32, device=dev)
        maps = [((torch.arange(G, device=dev) + s) % G).to(torch.int32) for s in range(G)]
        heads = torch.arange(G, device=dev)
        for j, layer_j in enumerate(self._layers):
            own = self._mass(layer_j, layer_j[4], layer_j[5], maps[0])             # on its own rows
            for i in range(j + 1):
                _, _, _, _, idx_i, count_i = self._layers[i]
                for s in range(G):
                    ratio = self._mass(layer_j, idx_i, count_i, maps[s]) / own      # [L, G2], h1 = (h2 + s) % G
                    red = ratio.amin(0) if self.reduce == "amin" else ratio.mean(0)
                    self.sim[i, j, heads, maps[s].long()] += red
        self._layers = []
        self.prompts += 1

    def average(self) -> torch.Tensor:
        if self.prompts == 0:
            raise ValueError("no prompt recorded")
        return self.sim / self.prompts
