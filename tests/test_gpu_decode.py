"""Paged decode kernels against the CPU oracle (GPU)."""
import numpy as np
import os
import pytest
import torch

from oracle.kascade_oracle import (KascadeOracle, band_check, pooled_scores_decode, sparse_decode_output,
                                   topk_budget)
from tests.cases import CASES, CFG1, SMALL_ROLL, decode_inputs
from tests.gpu_util import assert_close, paged_from_contiguous

pytestmark = pytest.mark.gpu
LOG2E = 1.4426950408889634


def _sparse(q, k, v, rows, counts, head_map, scale, paged=True, splits=0, page_size=16):
    """q [B,H,1,D], k/v [B,G,L,D] fp32 cpu (fp16-representable); rows [B,G,kmax] int32."""
    from kascade_b200 import _native as nat
    dev = torch.device("cuda")
    B, H, _, D = q.shape
    qd = q[:, :, 0].to(dev, torch.float16).contiguous()
    kd, vd = k.to(dev, torch.float16), v.to(dev, torch.float16)
    if paged:
        kc, vc, bt = paged_from_contiguous(kd, vd, page_size=page_size, seed=7)
        kv = nat.kv_layout_paged(kc, vc, bt)
    else:
        kd, vd = kd.contiguous(), vd.contiguous()
        kv = nat.kv_layout_contiguous(kd, vd)
    out = torch.full((B, H, D), 7.0, dtype=torch.float16, device=dev)
    lse = torch.zeros(B, H, dtype=torch.float32, device=dev)
    kmax = rows.shape[-1]
    s = splits if splits else nat.decode_default_splits(B, k.shape[1], kmax)
    ws = nat.decode_workspace(B, H, max(s, 1), dev)
    nat.decode_sparse_paged(qd, kv, rows.to(dev).contiguous(), None if counts is None else counts.to(dev),
                            kmax, None if head_map is None else torch.tensor(head_map, dtype=torch.int32, device=dev),
                            scale, out, lse, ws, splits)
    torch.cuda.synchronize()
    return out.cpu(), lse.cpu()


@pytest.mark.parametrize("case", [CFG1, SMALL_ROLL], ids=lambda c: c.name)
@pytest.mark.parametrize("paged", [True, False], ids=["paged", "contiguous"])
def test_sparse_decode_golden_rows(case, paged, golden_dir):
    """Reuse-layer decode with the reference's own index rows teacher-forced, against the reference's
    output stored in the golden file."""
    c = case
    gold = np.load(os.path.join(golden_dir, f"{c.name}.npz"))
    hm = c.head_mapping()
    layer = 1
    q, k, v = decode_inputs(c, layer)
    rows = torch.from_numpy(gold["decode_idx_0"])                   # [B,G,k] anchor rows of layer 0
    out, _ = _sparse(q, k, v, rows, None, hm[layer], c.D ** -0.5, paged=paged)
    ref = torch.from_numpy(gold[f"decode_out_{layer}"])[:, 0]       # [B,H,D]
    assert_close(out, ref, what=f"{c.name} decode reuse layer")


@pytest.mark.parametrize("splits", [1, 2, 5, 16])
@pytest.mark.parametrize("kcount", [1, 15, 16, 17, 300, 1000])
def test_sparse_decode_ragged_counts_and_splits(splits, kcount):
    g = torch.Generator().manual_seed(splits * 100 + kcount)
    B, G, H, L, D = 3, 2, 8, 1500, 128
    q = (torch.randn(B, H, 1, D, generator=g) / D ** 0.5).half().float()
    k = (torch.randn(B, G, L, D, generator=g)).half().float()
    v = (torch.randn(B, G, L, D, generator=g)).half().float()
    kmax = 1000
    rows = torch.stack([torch.stack([torch.randperm(L, generator=g)[:kmax] for _ in range(G)]) for _ in range(B)]).int()
    counts = torch.tensor([[kcount, max(kcount // 2, 0)], [0, kcount], [min(kmax, kcount + 3), kcount]], dtype=torch.int32)
    out, lse = _sparse(q, k, v, rows, counts, [1, 0], 0.3, paged=True, splits=splits)
    # reference: the per-(b,g) key set is row head_map[g] truncated to its count
    for b in range(B):
        for gg in range(G):
            src = [1, 0][gg]
            n = int(counts[b, src])
            hs = slice(gg * 4, gg * 4 + 4)
            if n == 0:
                assert float(out[b, hs].abs().max()) == 0.0
                continue
            ref = sparse_decode_output(q[b:b + 1, hs], k[b:b + 1, gg:gg + 1], v[b:b + 1, gg:gg + 1],
                                       rows[b:b + 1, src:src + 1, :n], 0.3)[0, 0]
            assert_close(out[b, hs], ref, what=f"b{b} g{gg} n{n} splits{splits}")
            kk = k[b, gg, rows[b, src, :n].long()]
            s = (q[b, hs, 0] @ kk.t()) * 0.3 * LOG2E
            ref_lse = torch.logsumexp(s * np.log(2.0), -1) / np.log(2.0)
            assert (lse[b, hs] - ref_lse).abs().max() < 1e-3


@pytest.mark.parametrize("with_v", [True, False], ids=["layer0", "anchor"])
@pytest.mark.parametrize("splits", [0, 1, 3])
def test_anchor_decode_dense(with_v, splits):
    from kascade_b200 import _native as nat
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(17)
    B, G, H, D = 3, 2, 8, 128
    lens = [1037, 16, 700]
    L = max(lens)
    q = (torch.randn(B, H, 1, D, generator=g) / D ** 0.5).half().float()
    k = (torch.randn(B, G, L, D, generator=g) * 1.5).half().float()
    v = (torch.randn(B, G, L, D, generator=g)).half().float()
    scale = D ** -0.5
    kc, vc, bt = paged_from_contiguous(k.to(dev, torch.float16), v.to(dev, torch.float16), seed=3)
    kv = nat.kv_layout_paged(kc, vc if with_v else None, bt)
    stride = (L + 3) // 4 * 4
    logits = torch.zeros(B, H, stride, dtype=torch.float32, device=dev)
    pooled = torch.full((B, G, stride), -1.0, dtype=torch.float32, device=dev)
    out = torch.zeros(B, H, D, dtype=torch.float16, device=dev) if with_v else None
    lse = torch.zeros(B, H, dtype=torch.float32, device=dev)
    s = splits if splits else nat.decode_default_splits(B, G, L)
    ws = nat.decode_workspace(B, H, max(s, 1), dev)
    nat.decode_anchor_paged(q[:, :, 0].to(dev, torch.float16).contiguous(), kv,
                            torch.tensor(lens, dtype=torch.int32, device=dev), L, scale, logits, pooled, out, lse,
                            ws, splits)
    torch.cuda.synchronize()
    for b, n in enumerate(lens):
        ref_pool, ref_p = pooled_scores_decode(q[b:b + 1], k[b:b + 1, :, :n], scale)
        got = pooled[b, :, :n].cpu()
        rel = ((got - ref_pool[0]).abs() / ref_pool[0]).max().item()
        assert rel < 2e-4, f"pooled scores b{b}: rel err {rel}"
        assert (pooled[b, :, n:].cpu() == -1.0).all(), "entries beyond the sequence must not be written"
        if with_v:
            ref_o = torch.einsum("hl,hld->hd", ref_p[0], v[b, :, :n].repeat_interleave(4, 0))
            assert_close(out[b], ref_o, what=f"dense decode b{b}")


@pytest.mark.parametrize("case", [CFG1, SMALL_ROLL], ids=lambda c: c.name)
def test_anchor_decode_topk_band(case):
    """decode anchor: logits -> pooled -> radix select, index sets checked with the tie-band rule."""
    from kascade_b200 import _native as nat
    dev = torch.device("cuda")
    c = case
    q, k, v = decode_inputs(c, 0)
    L = k.shape[2]
    scale = c.D ** -0.5
    kc, vc, bt = paged_from_contiguous(k.to(dev, torch.float16), v.to(dev, torch.float16), seed=5)
    kv = nat.kv_layout_paged(kc, vc, bt)
    stride = (L + 3) // 4 * 4
    logits = torch.empty(c.B, c.H, stride, dtype=torch.float32, device=dev)
    pooled = torch.empty(c.B, c.G, stride, dtype=torch.float32, device=dev)
    out = torch.empty(c.B, c.H, c.D, dtype=torch.float16, device=dev)
    lse = torch.empty(c.B, c.H, dtype=torch.float32, device=dev)
    ws = nat.decode_workspace(c.B, c.H, 32, dev)
    nat.decode_anchor_paged(q[:, :, 0].to(dev, torch.float16).contiguous(), kv,
                            torch.full((c.B,), L, dtype=torch.int32, device=dev), L, scale, logits, pooled, out, lse, ws)
    kk = topk_budget(c.pct, L, c.tile)
    idx = torch.empty(c.B, c.G, kk, dtype=torch.int32, device=dev)
    cnt = torch.empty(c.B, c.G, dtype=torch.int32, device=dev)
    nat.topk_select(pooled, None, None, kk, idx, cnt, n_cols=L)
    torch.cuda.synchronize()
    ref_pool, _ = pooled_scores_decode(q, k, scale)
    idx = idx.cpu()
    assert (cnt.cpu() == kk).all()
    for b in range(c.B):
        for g in range(c.G):
            ok, msg = band_check(ref_pool[b, g], idx[b, g].tolist(), kk, L)
            assert ok, f"b{b} g{g}: {msg}"


def test_decode_step_replays_from_a_cuda_graph():
    """A whole decode step (anchor and reuse layers through the strategy's paged entry) captured into a
    CUDA graph gives the same outputs as the eager step, also after the cache content changed: the
    library allocates nothing, never synchronises and keeps no host-side state per call."""
    from kascade_b200 import EfficientKascadeStrategy
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(23)
    B, G, H, D, L, layers = 4, 8, 32, 128, 3000, 4
    anchors = [0, 2]
    hm = [list(range(G)), [3, 3, 0, 7, 1, 6, 2, 5], list(range(G)), [1, 0, 3, 2, 5, 4, 7, 6]]
    strat = EfficientKascadeStrategy(anchors, "x/y", k=10, tile_size=32, rolling_prefill=True, head_mapping=hm,
                                     register=False)
    k = torch.randn(B, G, L, D, generator=g).half().to(dev)
    v = torch.randn(B, G, L, D, generator=g).half().to(dev)
    kc, vc, bt = paged_from_contiguous(k, v, seed=9)
    qs = [(torch.randn(B, H, D, generator=g) / D ** 0.5).half().to(dev) for _ in range(layers)]
    seq_lens = torch.tensor([L, L - 17, 2048, 1500], dtype=torch.int32, device=dev)
    outs = [torch.zeros(B, H, D, dtype=torch.float16, device=dev) for _ in range(layers)]

    def step():
        for l in range(layers):
            outs[l].copy_(strat.paged_decode_forward(l, qs[l], kc, vc, bt, seq_lens, D ** -0.5, L))

    step()                                        # allocates every scratch buffer
    torch.cuda.synchronize()
    eager = [o.clone() for o in outs]
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for o in outs:
        o.zero_()
    graph.replay()
    torch.cuda.synchronize()
    for l in range(layers):
        assert torch.equal(outs[l], eager[l]), f"layer {l}: graph replay differs from the eager step"
    # new cache content and queries, same addresses: the replay must follow the data
    kc.mul_(0.5)
    for q in qs:
        q.neg_()
    step()
    torch.cuda.synchronize()
    eager2 = [o.clone() for o in outs]
    graph.replay()
    torch.cuda.synchronize()
    for l in range(layers):
        assert torch.equal(outs[l], eager2[l]), f"layer {l}: graph replay did not pick up the new cache content"
    from kascade_b200 import _native as nat
    assert nat.read_status() == 0


def test_mixed_batch_short_sequences_attend_to_everything():
    """A ragged paged batch that mixes contexts of at most 128 keys with longer ones: the short sequences
    attend to all their keys (strategies/EfficientKascadeStrategy.py:137-140 runs dense attention for them),
    also when the budget of the longest sequence (10 % of 1000 -> 96 keys) is smaller than their length.
    Every sequence must come out as when it is decoded alone."""
    from kascade_b200 import EfficientKascadeStrategy
    g = torch.Generator().manual_seed(42)
    G, H, D, page = 2, 8, 128, 16
    lens = [100, 128, 1000, 129]
    B, Lmax = len(lens), max(lens)
    hm = [[0, 1], [1, 0]]
    scale = D ** -0.5
    k = (torch.randn(B, G, Lmax, D, generator=g) / D ** 0.5).half().cuda()
    v = torch.randn(B, G, Lmax, D, generator=g).half().cuda()
    kc, vc, bt = paged_from_contiguous(k, v, page_size=page, seed=3)
    seq_lens = torch.tensor(lens, dtype=torch.int32, device="cuda")
    qs = [(torch.randn(B, H, D, generator=g) / D ** 0.5).half().cuda() for _ in range(2)]

    def run(batch_rows):
        strat = EfficientKascadeStrategy([0], "x/y", k=10, tile_size=32, head_mapping=hm, register=False)
        sl = seq_lens[batch_rows].contiguous()
        outs = [strat.paged_decode_forward(layer, qs[layer][batch_rows].contiguous(), kc, vc, bt[batch_rows].contiguous(),
                                           sl, scale, int(sl.max().item())).clone() for layer in (0, 1)]
        return outs, strat._dec_count.clone()

    whole, counts = run(list(range(B)))
    torch.cuda.synchronize()
    assert counts[:, 0].tolist() == [100, 128, 96, 96], counts.tolist()
    for b in range(B):
        alone, _ = run([b])
        for layer in (0, 1):
            # (not bit-wise: the split count, hence the summation order, depends on the batch)
            assert_close(whole[layer][b], alone[layer][0], atol=1e-3, rtol=5e-3,
                         what=f"sequence {b} (len {lens[b]}), layer {layer}: in the batch vs alone")
    # the short sequences equal dense attention over all their keys
    for b in (0, 1):
        kb, vb = k[b, :, :lens[b]].float(), v[b, :, :lens[b]].float()
        qb = qs[1][b].float().view(G, 4, D)
        # reuse layer 1 maps KV head g to the rows of anchor head hm[1][g] but reads its OWN keys: all of them here
        p = torch.softmax(torch.einsum("ghd,gld->ghl", qb, kb) * scale, -1)
        ref = torch.einsum("ghl,gld->ghd", p, vb).reshape(H, D)
        assert_close(whole[1][b], ref, what=f"short sequence {b} against dense attention")
