"""Anchor-layer selection and head mappings: the producer of the ``.npy`` file the strategy loads.

The reference derives, from attention statistics of a calibration run, (1) which layers recompute
their Top-k index rows ("anchors", called pivots there) and (2) for every other layer, which KV head
of its anchor each of its KV heads should borrow rows from.  It does this at the end of its
statistics runner (runners/stats_runner.py: ``_similarity_layer`` :155-168, ``_process_select_layers``
:183-197, ``_pick_k_layers`` :291-331, ``_get_pivot_score`` :333-339, ``_find_head_mappings``
:341-352) and writes ``./results/head_mappings/<model>_layers_<a>_<b>_....npy`` (int32 ``[layers, G]``),
the file ``EfficientKascadeStrategy.get_head_mapping`` reads.

This module restates that host logic on plain tensors so that a mapping can be produced for a new model
without the reference's runner stack: feed per-layer statistics to :class:`SimilarityAccumulator` (or
bring a ready ``[layers, layers, G, G]`` similarity tensor), then :func:`select_layers`.

Conventions (as in the reference): ``sim[i, j, h2, h1]`` = how much of the attention mass that head
``h2`` of layer ``j`` puts on ITS OWN Top-k keys it would keep with the Top-k keys of head ``h1`` of
layer ``i`` (``i <= j``).
"""
from __future__ import annotations

import math
import os
from typing import Dict, Iterable, List, Optional, Sequence

import numpy as np
import torch

__all__ = ["similarity_layer", "SimilarityAccumulator", "layer_similarity", "pick_k_layers", "pivot_score",
           "find_head_mappings", "select_layers", "save_head_mapping"]


def similarity_layer(indices_1: torch.Tensor, indices_2: torch.Tensor, attn_weights_2: torch.Tensor,
                     last_tile_attn_2: Optional[torch.Tensor] = None, reduce: str = "amin") -> torch.Tensor:
    """runners/stats_runner.py:155-168.

    indices_1 / indices_2 [B, G, Lq, k] int64: Top-k key positions of layers 1 and 2; attn_weights_2
    [B, G, Lq, Lk]: post-softmax weights of layer 2 (pooled per KV head); last_tile_attn_2 [B, G, Lq]: mass on
    the query's own tile, which every variant attends to anyway (zeros if None).  Returns ``[G2, G1]``: over
    the queries, the minimum (``reduce="amin"``, used for layer selection) or mean of
    ``(mass of layer 2 on layer 1's keys + own tile) / (mass of layer 2 on its own keys + own tile)``.
    Batch 1, as in the reference (its own-tile term is broadcast along the first head axis)."""
    B, heads, Lq, _ = indices_1.shape
    if last_tile_attn_2 is None:
        last_tile_attn_2 = attn_weights_2.new_zeros(B, heads, Lq)
    denom = torch.gather(attn_weights_2, -1, indices_2)                                   # [B, G2, Lq, k]
    w2 = attn_weights_2.unsqueeze(2).expand(-1, -1, heads, -1, -1)                        # [B, G2, G1, Lq, Lk]
    idx1 = indices_1.unsqueeze(1).expand(-1, heads, -1, -1, -1)                           # [B, G2, G1, Lq, k]
    num = torch.gather(w2, -1, idx1)
    den = denom.unsqueeze(2).expand(-1, -1, heads, -1, -1)
    weighted = (num.sum(-1) + last_tile_attn_2) / (den.sum(-1) + last_tile_attn_2)        # [B, G2, G1, Lq]
    if reduce == "amin":
        sim = weighted.amin(-1)
    elif reduce == "mean":
        sim = weighted.mean(-1)
    else:
        raise ValueError(f"reduce must be 'amin' or 'mean', got {reduce!r}")
    return sim[0]


class SimilarityAccumulator:
    """Running sum of the pairwise layer / head similarities over calibration prompts
    (runners/stats_runner.py:28-40, 127-131, 84-96).  Per prompt: ``add_layer`` once per layer in layer
    order, then ``end_prompt``; ``average()`` gives the ``[layers, layers, G, G]`` tensor (upper triangle)."""

    def __init__(self, num_layers: int, heads: int, reduce: str = "amin", device="cpu"):
        self.num_layers, self.heads, self.reduce = num_layers, heads, reduce
        self.sim = torch.zeros(num_layers, num_layers, heads, heads, dtype=torch.float32, device=device)
        self.prompts = 0
        self._layers: List[tuple] = []

    def add_layer(self, indices: torch.Tensor, attn_weights: torch.Tensor, last_tile_attn: Optional[torch.Tensor] = None):
        self._layers.append((indices, attn_weights, last_tile_attn))

    def end_prompt(self):
        if len(self._layers) != self.num_layers:
            raise ValueError(f"{len(self._layers)} layers recorded, {self.num_layers} expected")
        for i in range(self.num_layers):
            for j in range(i, self.num_layers):
                idx_j, w_j, last_j = self._layers[j]
                self.sim[i, j] += similarity_layer(self._layers[i][0], idx_j, w_j, last_j, self.reduce).to(self.sim)
        self._layers = []
        self.prompts += 1

    def average(self) -> torch.Tensor:
        if self.prompts == 0:
            raise ValueError("no prompt recorded")
        return self.sim / self.prompts


def layer_similarity(sim_avg: torch.Tensor, importance: Optional[torch.Tensor] = None) -> np.ndarray:
    """runners/stats_runner.py:186-187: best-matching anchor head per head, averaged over the heads, weighted by
    the importance of the reusing layer (column)."""
    layer_sim = sim_avg.amax(dim=-1).mean(dim=-1)
    if importance is not None:
        layer_sim = layer_sim * importance.unsqueeze(0).to(layer_sim.device)
    return layer_sim.cpu().numpy()


def pick_k_layers(sim, K: int) -> List[int]:
    """runners/stats_runner.py:291-331: the K anchors (the first is layer 0) that maximise
    ``sum_j sim[anchor(j)][j]``, anchor(j) = the last anchor <= j, by dynamic programming over (anchors used,
    layers covered).  The sum over a segment is kept as a running sum in the reference's left-to-right order,
    so values (and therefore ties, which go to the smallest split point) come out as there; the cost drops
    from O(K N^3) to O(K N^2)."""
    N = len(sim)
    # seg[l][i] = sim[l][l+1] + ... + sim[l][i-1], accumulated left to right
    seg = [[0] * (N + 1) for _ in range(N)]
    for l in range(N):
        run = 0
        for i in range(l + 1, N + 1):
            seg[l][i] = run
            if i < N:
                run = run + sim[l][i]
    V = [[-math.inf] * (N + 1) for _ in range(K + 1)]
    path = [[-1] * (N + 1) for _ in range(K + 1)]
    V[0][0] = sim[0][0]
    for k in range(1, K + 1):
        for i in range(N + 1):
            best_val, best_l = -math.inf, -1
            for l in range(i):
                val = V[k - 1][l] + seg[l][i] + sim[l][l]
                if val > best_val:
                    best_val, best_l = val, l
            V[k][i], path[k][i] = best_val, best_l
    cur, pivots = N, []
    for k in range(K, 0, -1):
        cur = path[k][cur]
        pivots.append(cur)
    pivots.reverse()
    return pivots


def pivot_score(sim, pivots_with_end: Sequence[int]):
    """runners/stats_runner.py:333-339: (sum, min) of the similarities a choice of anchors realises; the list
    ends with the number of layers."""
    scores = []
    for left, right in zip(pivots_with_end[:-1], pivots_with_end[1:]):
        scores += [round(sim[left][j], 3) for j in range(left, right)]       # in the elements' own precision
    return sum(scores), min(scores)


def find_head_mappings(sim_avg: torch.Tensor, pivots_with_end: Sequence[int]) -> List[List[int]]:
    """runners/stats_runner.py:341-352: for every layer, per KV head, the anchor KV head with the highest
    similarity (first maximum); rows of anchor layers map onto themselves through the same arg-max."""
    num_layers = sim_avg.shape[0]
    pattern = [0] * num_layers
    for i in range(1, len(pivots_with_end)):
        for j in range(pivots_with_end[i - 1], pivots_with_end[i]):
            pattern[j] = pivots_with_end[i - 1]
    head_mat = sim_avg[pattern, list(range(num_layers)), ...]                              # [layers, G(layer), G(anchor)]
    return head_mat.max(dim=-1).indices.cpu().to(torch.int32).tolist()


def select_layers(sim_avg: torch.Tensor, importance: Optional[torch.Tensor] = None,
                  counts: Iterable[int] = (3, 4, 5, 6, 7, 8)) -> Dict[tuple, List[List[int]]]:
    """runners/stats_runner.py:183-197: for each anchor count, the best anchors and their head mapping."""
    num_layers = sim_avg.shape[0]
    layer_sim = layer_similarity(sim_avg, importance)
    out = {}
    for k in counts:
        pivots = pick_k_layers(layer_sim, k)
        out[tuple(pivots)] = find_head_mappings(sim_avg, pivots + [num_layers])
    return out


def save_head_mapping(model_name: str, pivots: Sequence[int], mapping: Sequence[Sequence[int]], root: str = ".") -> str:
    """Writes the file ``EfficientKascadeStrategy.get_head_mapping`` reads (strategies/KascadeStrategy.py:174-183;
    written at runners/stats_runner.py:184,197): int32 ``[layers, G]``."""
    base = model_name.split("/")[-1]
    folder = os.path.join(root, "results", "head_mappings")
    os.makedirs(folder, exist_ok=True)
    path = os.path.join(folder, f"{base}_layers_{'_'.join(map(str, pivots))}.npy")
    np.save(path, np.array(mapping, dtype=np.int32))
    return path
