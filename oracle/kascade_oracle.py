"""CPU oracle for the Kascade sparse-attention path (TEST INFRASTRUCTURE ONLY).

This module restates, in plain fp32 torch-on-CPU arithmetic, what the reference's PyTorch
``KascadeStrategy`` computes for the anchor / reuse, prefill / decode cases.  It exists only so
that tests, the smoke check and the CPU-baseline leg of the benchmark have something to compare the
CUDA kernels with; the product path never imports it.

Parity status: pinned.  ``tests/golden/*.npz`` were produced by executing the reference's own
``KascadeStrategy`` (strategies/KascadeStrategy.py) on seeded inputs (generator script:
``tests/golden/make_golden.py``); ``tests/test_oracle_golden.py`` checks this restatement against
them.  The reference itself ships no golden vectors for this path.

Conventions
-----------
* ``q``  : [B, H, Lq, D]   ``k``/``v`` : [B, G, Lk, D]   (the HF attention layout the reference's
  ``attention_forward`` receives, strategies/KascadeStrategy.py:115-124).
* outputs: [B, Lq, H, D]  (strategies/KascadeStrategy.py:111).
* index rows are kept **per query tile** ([B, G, T, k]) — the reference stores the same row
  repeated for each of the tile's queries (strategies/KascadeStrategy.py:90-95).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

__all__ = [
    "topk_budget", "rolling_budget", "pooled_scores_prefill", "pooled_scores_decode",
    "KascadeOracle", "allowed_mask_prefill", "sparse_prefill_output", "sparse_decode_output",
    "band_check", "clean_index_row",
]


# --------------------------------------------------------------------------------------------
# budgets
# --------------------------------------------------------------------------------------------
def topk_budget(pct: float, lk: int, tile_size: int) -> int:
    """Number of keys an anchor layer selects.

    strategies/KascadeStrategy.py:127-129: ``min(max(128, int(pct/100*Lk)), Lk)`` and, when
    tiling is on, minus one tile (the tile's own keys are always attended).
    """
    k = min(max(128, int((pct / 100) * lk)), lk)
    if tile_size > 1:
        k -= tile_size
    return k


def rolling_budget(pct: float, tile_start: int) -> int:
    """Entries of the sorted Top-k list a tile keeps under rolling prefill.

    strategies/KascadeStrategy.py:134-139: ``((pct * tile_start) // 100).clamp(min=128)``;
    list positions at or beyond this number are overwritten with ``Lk-1``.
    """
    return max(128, int((pct * tile_start) // 100))


# --------------------------------------------------------------------------------------------
# pooled post-softmax scores
# --------------------------------------------------------------------------------------------
def _causal_probs(q_blk: torch.Tensor, k_rep: torch.Tensor, scaling: float, q0: int) -> torch.Tensor:
    """softmax over keys ``j <= i`` of the scaled logits, fp32.

    strategies/KascadeStrategy.py:36,68-70 and attention_utils.py:6-22 (subtract the row maximum,
    exponentiate, divide by the sum)."""
    lq, lk = q_blk.shape[-2], k_rep.shape[-2]
    s = torch.matmul(q_blk, k_rep.transpose(2, 3)).float() * scaling
    qi = torch.arange(q0, q0 + lq).view(-1, 1)
    kj = torch.arange(lk).view(1, -1)
    s = s.masked_fill(kj > qi, float("-inf"))
    s = s - s.amax(dim=-1, keepdim=True)
    p = s.exp_()
    return p / p.sum(dim=-1, keepdim=True)


def pooled_scores_prefill(q, k, scaling, tile_size, row_block: int = 1024, return_probs=False):
    """Per (batch, KV head, query tile) sum of post-softmax probabilities.

    strategies/KascadeStrategy.py:72-83: sum the probabilities of the query heads that share a
    KV head, then of the ``tile_size`` queries of a tile (a short last tile is zero-padded), and
    zero every key at or after the tile's first query.  Returns fp32 [B, G, T, Lk]."""
    B, H, L, D = q.shape
    G = k.shape[1]
    hg = H // G
    T = math.ceil(L / tile_size)
    k_rep = k.repeat_interleave(hg, dim=1)
    pooled = torch.zeros(B, G, T, k.shape[2], dtype=torch.float32)
    row_block = max(tile_size, (row_block // tile_size) * tile_size)
    probs = [] if return_probs else None
    for q0 in range(0, L, row_block):
        q1 = min(q0 + row_block, L)
        p = _causal_probs(q[:, :, q0:q1], k_rep, scaling, q0)            # [B,H,n,Lk]
        if return_probs:
            probs.append(p)
        n = q1 - q0
        pg = p.view(B, G, hg, n, -1).sum(dim=2)                          # heads first (…:75)
        nt = math.ceil(n / tile_size)
        if nt * tile_size != n:
            pg = torch.cat([pg, pg.new_zeros(B, G, nt * tile_size - n, pg.shape[-1])], dim=2)
        pooled[:, :, q0 // tile_size: q0 // tile_size + nt] = pg.view(B, G, nt, tile_size, -1).sum(dim=3)
    starts = torch.arange(T) * tile_size
    pooled *= (torch.arange(k.shape[2]).view(1, -1) < starts.view(-1, 1)).to(pooled.dtype)
    if return_probs:
        return pooled, torch.cat(probs, dim=2)
    return pooled


def pooled_scores_decode(q, k, scaling):
    """Decode step: [B, G, Lk] sum over the group's query heads of softmax(q·K^T·scaling).

    strategies/KascadeStrategy.py:70,75 with Lq == 1 (no tiles, mask all zeros)."""
    B, H, _, D = q.shape
    G = k.shape[1]
    hg = H // G
    s = torch.einsum("bghd,bgld->bghl", q.view(B, G, hg, D).float(), k.float()) * scaling
    s = s - s.amax(dim=-1, keepdim=True)
    p = s.exp_()
    p = p / p.sum(dim=-1, keepdim=True)
    return p.sum(dim=2), p.view(B, H, -1)


# --------------------------------------------------------------------------------------------
# sparse attention given index rows
# --------------------------------------------------------------------------------------------
def allowed_mask_prefill(idx_rows: torch.Tensor, L: int, tile_size: int) -> torch.Tensor:
    """Boolean [B, G, L, L]: which keys each query may attend to in a sparse prefill layer.

    strategies/KascadeStrategy.py:56-68: a query attends to the keys listed in its tile's index
    row that are not in its future, plus the keys from the first query of its tile up to itself.
    ``idx_rows`` is [B, G, T, k] (any order, duplicates and out-of-window entries allowed)."""
    B, G, T, _ = idx_rows.shape
    sel = torch.zeros(B, G, T, L, dtype=torch.bool)
    sel.scatter_(3, idx_rows.long().clamp(0, L - 1), True)
    sel = sel.repeat_interleave(tile_size, dim=2)[:, :, :L]
    qi = torch.arange(L).view(-1, 1)
    kj = torch.arange(L).view(1, -1)
    local = kj >= (qi // tile_size) * tile_size
    causal = kj <= qi
    return (sel | local) & causal


def sparse_prefill_output(q, k, v, idx_rows, scaling, tile_size, row_block: int = 1024):
    """softmax restricted to ``allowed_mask_prefill`` times V; returns [B, L, H, D] fp32.

    strategies/KascadeStrategy.py:56-70,110-111 (reuse layers) and :99-108 (anchor layers > 0,
    where zeroing the other probabilities and renormalising equals a softmax over the kept set)."""
    B, H, L, D = q.shape
    G = k.shape[1]
    hg = H // G
    out = torch.empty(B, L, H, D, dtype=torch.float32)
    allowed = allowed_mask_prefill(idx_rows, L, tile_size)               # [B,G,L,L]
    for q0 in range(0, L, row_block):
        q1 = min(q0 + row_block, L)
        s = torch.einsum("bghqd,bgkd->bghqk", q[:, :, q0:q1].reshape(B, G, hg, q1 - q0, D).float(),
                         k.float()) * scaling
        s = s.masked_fill(~allowed[:, :, None, q0:q1], float("-inf"))
        p = torch.softmax(s, dim=-1)
        o = torch.einsum("bghqk,bgkd->bghqd", p, v.float())
        out[:, q0:q1] = o.reshape(B, H, q1 - q0, D).transpose(1, 2)
    return out


def sparse_decode_output(q, k, v, idx_rows, scaling):
    """Decode step over an explicit key set: idx_rows [B, G, k] -> [B, 1, H, D] fp32.

    strategies/KascadeStrategy.py:56-67 with Lq == 1: every logit is replaced by the minimum
    except at the listed keys (no local window)."""
    B, H, _, D = q.shape
    G = k.shape[1]
    hg = H // G
    Lk = k.shape[2]
    sel = torch.zeros(B, G, Lk, dtype=torch.bool).scatter_(2, idx_rows.long(), True)
    s = torch.einsum("bghd,bgld->bghl", q.view(B, G, hg, D).float(), k.float()) * scaling
    s = s.masked_fill(~sel[:, :, None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = torch.einsum("bghl,bgld->bghd", p, v.float())
    return o.reshape(B, 1, H, D)


# --------------------------------------------------------------------------------------------
# the strategy, restated
# --------------------------------------------------------------------------------------------
@dataclass
class KascadeOracle:
    """Stateful restatement of ``KascadeStrategy`` (strategies/KascadeStrategy.py:11-183).

    Call :meth:`attention_forward` once per layer, in layer order starting at 0, exactly like the
    HF decoder does with the reference strategy."""

    recompute_layers: Sequence[int]
    head_mapping: Sequence[Sequence[int]]        # [num_layers][G]; anchor rows are the identity
    k: float = 10
    tile_size: int = 32
    rolling_prefill: bool = True
    row_block: int = 1024
    # state written by anchor layers (strategies/KascadeStrategy.py:95,133)
    index_rows: Optional[torch.Tensor] = field(default=None, repr=False)   # [B,G,T,k] or [B,G,1,k]
    pooled: Optional[torch.Tensor] = field(default=None, repr=False)       # last anchor's scores
    probs: Optional[torch.Tensor] = field(default=None, repr=False)

    def is_anchor(self, layer_idx: int) -> bool:
        # strategies/KascadeStrategy.py:55-56,72-73
        return layer_idx == 0 or layer_idx in self.recompute_layers

    def attention_forward(self, layer_idx: int, q, k, v, scaling: float) -> torch.Tensor:
        B, H, Lq, D = q.shape
        Lk = k.shape[2]
        kk = topk_budget(self.k, Lk, self.tile_size)
        if Lq == 1:
            return self._decode(layer_idx, q, k, v, scaling, kk)
        assert Lq == Lk, "prefill expects the whole prompt (queries == keys)"
        assert Lq > self.tile_size
        return self._prefill(layer_idx, q, k, v, scaling, kk)

    # -- prefill ------------------------------------------------------------------------------
    def _prefill(self, layer_idx, q, k, v, scaling, kk):
        B, H, L, D = q.shape
        G = k.shape[1]
        ts = self.tile_size
        if self.is_anchor(layer_idx):
            keep_p = layer_idx == 0
            res = pooled_scores_prefill(q, k, scaling, ts, self.row_block, return_probs=keep_p)
            pooled, probs = res if keep_p else (res, None)
            idx = torch.topk(pooled, kk, dim=-1).indices                  # :84, descending order
            if self.rolling_prefill and L > 128:                          # :85-89,134
                T = pooled.shape[2]
                budgets = torch.tensor([rolling_budget(self.k, t * ts) for t in range(T)])
                idx = idx.masked_fill(torch.arange(kk).view(1, -1) >= budgets.view(-1, 1), L - 1)
            self.index_rows = idx.to(torch.int32)
            self.pooled = pooled
            if layer_idx == 0:                                            # dense output, :99
                vv = v.repeat_interleave(H // G, dim=1).float()
                return torch.matmul(probs, vv).transpose(1, 2).contiguous()
            rows = self.index_rows
        else:
            rows = self.index_rows[:, list(self.head_mapping[layer_idx])]  # :58
        return sparse_prefill_output(q, k, v, rows, scaling, ts, self.row_block)

    # -- decode -------------------------------------------------------------------------------
    def _decode(self, layer_idx, q, k, v, scaling, kk):
        B, H, _, D = q.shape
        G = k.shape[1]
        if self.is_anchor(layer_idx):
            pooled, probs = pooled_scores_decode(q, k, scaling)
            idx = torch.topk(pooled, kk, dim=-1).indices                  # :96
            self.index_rows = idx.to(torch.int32).unsqueeze(2)            # [B,G,1,k]
            self.pooled = pooled
            if layer_idx == 0:
                vv = v.repeat_interleave(H // G, dim=1).float()
                return torch.einsum("bhl,bhld->bhd", probs, vv).view(B, 1, H, D)
            rows = self.index_rows[:, :, 0]
        else:
            rows = self.index_rows[:, list(self.head_mapping[layer_idx]), 0]
        return sparse_decode_output(q, k, v, rows, scaling)


# --------------------------------------------------------------------------------------------
# comparison helpers used by the parity tests
# --------------------------------------------------------------------------------------------
def clean_index_row(row, tile_start: int) -> List[int]:
    """The keys of an oracle index row that matter for a prefill tile: strictly before the tile,
    without duplicates, ascending.  Everything else in the row (zero-score picks of early tiles,
    the ``Lk-1`` rolling filler) is either masked by causality or already inside the tile's local
    window (strategies/KascadeStrategy.py:59-68)."""
    return sorted({int(j) for j in row if 0 <= int(j) < tile_start})


def band_check(scores: torch.Tensor, chosen: Sequence[int], k: int, n_valid: int, rel: float = 2.0 ** -10):
    """Tie-band comparison of one selected index set against the exact Top-k of ``scores``.

    ``scores`` is the oracle's pooled score row, ``n_valid`` the number of candidate keys (keys
    ``>= n_valid`` are not candidates), ``chosen`` the set under test, ``k`` the budget.  Passing
    means: ``min(k, n_valid)`` distinct candidates were chosen, every candidate scoring above the
    k-th largest score by more than one fp16 ulp (relative ``rel``) is chosen, and none scoring
    below it by more than that is.  Returns (ok, message)."""
    chosen = [int(c) for c in chosen]
    want = min(k, n_valid)
    if len(set(chosen)) != len(chosen):
        return False, "duplicate indices"
    if len(chosen) != want:
        return False, f"selected {len(chosen)} keys, expected {want}"
    if any(c < 0 or c >= n_valid for c in chosen):
        return False, "index outside the candidate range"
    if want == n_valid or want == 0:
        return True, "all candidates"
    row = scores[:n_valid].double()
    tau = torch.topk(row, want).values[-1].item()
    hi, lo = tau * (1 + rel), tau * (1 - rel)
    mask = torch.zeros(n_valid, dtype=torch.bool)
    mask[torch.tensor(chosen, dtype=torch.long)] = True
    must = row > hi
    never = row < lo
    if bool((must & ~mask).any()):
        j = int((must & ~mask).nonzero()[0])
        return False, f"key {j} (score {row[j]:.6e} > band top {hi:.6e}) not selected"
    if bool((never & mask).any()):
        j = int((never & mask).nonzero()[0])
        return False, f"key {j} (score {row[j]:.6e} < band bottom {lo:.6e}) selected"
    return True, "ok"
