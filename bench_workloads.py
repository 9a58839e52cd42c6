"""Seeded synthetic workloads with the shapes and value distributions of the benchmark
configurations (Llama-3.1-8B attention shapes).  No dataset is involved: the reference's own kernel
benchmarks also run on random tensors (scripts/benchmark_prefill.py, scripts/benchmark_decode.py).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence, Tuple

import torch

LLAMA_ANCHORS = (0, 2, 8, 13, 14)
QWEN3_ANCHORS = (0, 3, 9, 17, 25)          # the long-prompt configuration (36 layers, QK-norm)


@dataclass
class PrefillWorkload:
    """Prefill attention stack: batch 1, causal, 32 query / 8 KV heads, head_dim 128, fp16."""
    seq_len: int = 32768
    layers: int = 32
    anchors: Tuple[int, ...] = LLAMA_ANCHORS
    H: int = 32
    G: int = 8
    D: int = 128
    pct: float = 10
    tile: int = 32
    rolling: bool = True
    B: int = 1
    qk_norm: bool = False             # RMS-normalise the rows of Q and K (unit gain), as Qwen3 does per head

    def head_mapping(self, seed: int = 1234) -> List[List[int]]:
        g = torch.Generator().manual_seed(seed)
        rows = []
        for layer in range(self.layers):
            if layer == 0 or layer in self.anchors:
                rows.append(list(range(self.G)))
            else:
                rows.append(torch.randint(0, self.G, (self.G,), generator=g).tolist())
        return rows

    def layer_inputs(self, layer: int, device, heads: Sequence[int] = None):
        """q [B,L,H,D], k, v [B,L,G,D] fp16 token-major: N(0,1)/sqrt(D), plus per KV head 1 % of the key
        positions shifted by 2.5 along a unit direction that every query carries with weight 0.5."""
        gen = torch.Generator(device=device).manual_seed(layer)
        B, L, H, G, D = self.B, self.seq_len, self.H, self.G, self.D
        q = torch.randn(B, L, H, D, generator=gen, device=device) / D ** 0.5
        k = torch.randn(B, L, G, D, generator=gen, device=device) / D ** 0.5
        v = torch.randn(B, L, G, D, generator=gen, device=device) / D ** 0.5
        u = torch.randn(D, generator=gen, device=device)
        u /= u.norm()
        n_hot = max(1, L // 100)
        for g in range(G):
            pos = torch.randperm(L, generator=gen, device=device)[:n_hot]
            k[:, pos, g] += 2.5 * u
        q += 0.5 * u
        if self.qk_norm:
            q *= torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + 1e-6)
            k *= torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + 1e-6)
        q, k, v = q.half(), k.half(), v.half()
        if heads is not None:                       # a KV-head shard: its KV heads and their query heads
            hg = H // G
            qh = [g * hg + i for g in heads for i in range(hg)]
            q, k, v = q[:, :, qh].contiguous(), k[:, :, list(heads)].contiguous(), v[:, :, list(heads)].contiguous()
        return q, k, v

    # ---- algorithmic work (per layer, whole batch, all heads) -----------------------------------
    def flops_qk_causal(self) -> float:
        return 2.0 * self.B * self.H * self.D * self.seq_len * self.seq_len / 2

    def flops_dense(self) -> float:
        return 2 * self.flops_qk_causal()

    def sparse_keys_per_tile(self) -> List[int]:
        from kascade_b200.strategy import topk_budget
        kk = topk_budget(self.pct, self.seq_len, self.tile)
        out = []
        for t in range(-(-self.seq_len // self.tile)):
            start = t * self.tile
            kt = min(kk, max(128, int(self.pct * start // 100))) if self.rolling else kk
            out.append(min(kt, start) + self.tile)
        return out

    def flops_sparse(self) -> float:
        rows = self.tile * (self.H // self.G)
        return sum(4.0 * rows * self.D * n for n in self.sparse_keys_per_tile()) * self.G * self.B

    def flops_stack(self) -> float:
        n_anchor = len([a for a in self.anchors if a != 0])
        n_reuse = self.layers - n_anchor - 1
        layer0 = self.flops_dense() + self.flops_qk_causal()
        anchor = 2 * self.flops_qk_causal() + self.flops_sparse()
        return layer0 + n_anchor * anchor + n_reuse * self.flops_sparse()


@dataclass
class DecodeWorkload:
    """Paged sparse decode: every sequence at the same context, 16-token pages, seeded random page
    permutation, one new token per sequence per step."""
    batch: int = 64
    context: int = 32768
    layers: int = 32
    anchors: Tuple[int, ...] = LLAMA_ANCHORS
    H: int = 32
    G: int = 8
    D: int = 128
    pct: float = 10
    page: int = 16
    distinct_caches: int = 4          # layer caches held in HBM and cycled over the 32 layers
    contexts: Sequence[int] = None    # per-sequence contexts (ragged batch); None: every sequence at `context`
    reserve: int = 0                  # tokens of page room behind every sequence (for tokens generated later)

    def seq_lens(self) -> List[int]:
        return [self.context] * self.batch if self.contexts is None else [int(c) for c in self.contexts]

    @staticmethod
    def ragged(batch_total: int = 256, lo: int = 4096, hi: int = 65536, seed: int = 0, rank: int = 0, world: int = 1,
               **kw) -> "DecodeWorkload":
        """The long-reasoning decode configuration: contexts uniform in [lo, hi] from `seed`, batch-sharded."""
        lens = torch.randint(lo, hi + 1, (batch_total,), generator=torch.Generator().manual_seed(seed)).tolist()
        mine = lens[rank::world]
        return DecodeWorkload(batch=len(mine), context=max(mine), contexts=mine, **kw)

    def head_mapping(self, seed: int = 4321) -> List[List[int]]:
        return PrefillWorkload(layers=self.layers, anchors=self.anchors, G=self.G).head_mapping(seed)

    def make_cache(self, idx: int, device):
        """(k_cache, v_cache [pages, 16, G, D] fp16, block_table [B, pages_per_seq] int32)."""
        gen = torch.Generator(device=device).manual_seed(1000 + idx)
        pps = -(-(self.context + self.reserve) // self.page)
        per_seq = [-(-(n + self.reserve) // self.page) for n in self.seq_lens()]
        n_pages = sum(per_seq)
        shape = (n_pages, self.page, self.G, self.D)
        k = torch.empty(shape, dtype=torch.float16, device=device)
        v = torch.empty(shape, dtype=torch.float16, device=device)
        chunk = max(1, n_pages // 16)
        for s in range(0, n_pages, chunk):               # bounded fp32 temporaries
            e = min(n_pages, s + chunk)
            k[s:e] = (torch.randn((e - s,) + shape[1:], generator=gen, device=device) / self.D ** 0.5).half()
            v[s:e] = (torch.randn((e - s,) + shape[1:], generator=gen, device=device) / self.D ** 0.5).half()
        cpu_gen = torch.Generator().manual_seed(2000 + idx)
        perm = torch.randperm(n_pages, generator=cpu_gen).to(torch.int32)
        table = torch.zeros(self.batch, pps, dtype=torch.int32)
        o = 0
        for b, n in enumerate(per_seq):
            table[b, :n] = perm[o:o + n]
            o += n
        table = table.to(device)
        # sink keys at positions 0..3 of every sequence (K += 3 N(0,1))
        first = table[:, 0].long()
        k[first, :4] += (3 * torch.randn(self.batch, 4, self.G, self.D, generator=gen, device=device)).half()
        return k, v, table

    def query(self, layer: int, device):
        gen = torch.Generator(device=device).manual_seed(5000 + layer)
        return (torch.randn(self.batch, self.H, self.D, generator=gen, device=device) / self.D ** 0.5).half()

    def budget(self) -> int:
        from kascade_b200.strategy import topk_budget
        return topk_budget(self.pct, self.context, 32)

    # ---- algorithmic bytes per layer kind ---------------------------------------------------------
    def bytes_reuse(self) -> float:
        from kascade_b200.strategy import topk_budget
        keys = sum(topk_budget(self.pct, n, 32) for n in self.seq_lens())
        return self.G * keys * (2 * self.D * 2 + 4) + 2 * self.batch * self.H * self.D * 2

    def bytes_dense_k(self) -> float:
        return self.G * sum(self.seq_lens()) * self.D * 2

    def bytes_step(self) -> float:
        n_anchor = len([a for a in self.anchors if a != 0])
        n_reuse = self.layers - n_anchor - 1
        return 2 * self.bytes_dense_k() + n_anchor * (self.bytes_dense_k() + self.bytes_reuse()) + n_reuse * self.bytes_reuse()

    def bytes_dense_step(self) -> float:
        return self.layers * 2 * self.bytes_dense_k()
