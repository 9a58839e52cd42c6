"""Tile prefill kernels (tcgen05) against the CPU oracle and the reference's golden vectors (GPU)."""
import os

import numpy as np
import pytest
import torch

from oracle.kascade_oracle import (KascadeOracle, band_check, clean_index_row, pooled_scores_prefill,
                                   rolling_budget, sparse_prefill_output, topk_budget)
from tests.cases import CASES, CFG1, SMALL_RAGGED, SMALL_ROLL, make_inputs
from tests.gpu_util import assert_close

pytestmark = pytest.mark.gpu
LOG2E = 1.4426950408889634


def _dev(x):
    return x.to("cuda", torch.float16)


def _status_ok():
    from kascade_b200 import _native as nat
    st = nat.read_status()
    assert st == 0, f"a kernel gave up a bounded wait (code {st})"


def _dense_ref(q, k, v, scaling):
    B, H, L, D = q.shape
    G = k.shape[1]
    kk = k.repeat_interleave(H // G, 1)
    vv = v.repeat_interleave(H // G, 1)
    s = (q @ kk.transpose(2, 3)).float() * scaling
    s = s.masked_fill(torch.ones(L, L, dtype=torch.bool).triu(1), float("-inf"))
    lse2 = torch.logsumexp(s, -1) * LOG2E
    return (torch.softmax(s, -1) @ vv).transpose(1, 2), lse2.transpose(1, 2)      # [B,L,H,D], [B,L,H]


@pytest.mark.parametrize("case", [SMALL_RAGGED, SMALL_ROLL, CFG1], ids=lambda c: c.name)
def test_dense_prefill_and_lse(case):
    from kascade_b200 import _native as nat
    c = case
    q, k, v = make_inputs(c, 0)
    ref_o, ref_lse = _dense_ref(q, k, v, c.D ** -0.5)
    qd, kd, vd = (_dev(x).transpose(1, 2) for x in (q, k, v))          # token-major views
    out = torch.zeros(c.B, c.L, c.H, c.D, dtype=torch.float16, device="cuda")
    lse = torch.zeros(c.B, c.L, c.H, dtype=torch.float32, device="cuda")
    nat.prefill_dense(qd, kd, vd, c.D ** -0.5, out, lse)
    _status_ok()
    assert_close(out, ref_o, what=f"{c.name} dense prefill")
    assert (lse.cpu() - ref_lse).abs().max() < 1e-3
    lse_only = torch.zeros_like(lse)
    nat.prefill_dense(qd, kd, None, c.D ** -0.5, None, lse_only)
    _status_ok()
    assert (lse_only.cpu() - ref_lse).abs().max() < 1e-3


@pytest.mark.parametrize("case", [SMALL_RAGGED, SMALL_ROLL, CFG1], ids=lambda c: c.name)
def test_pooled_scores(case):
    from kascade_b200 import _native as nat
    c = case
    q, k, v = make_inputs(c, 0)
    ref = pooled_scores_prefill(q, k, c.D ** -0.5, c.tile)               # [B,G,T,L], zeros at j >= tile start
    _, ref_lse = _dense_ref(q, k, v, c.D ** -0.5)
    qd, kd = (_dev(x).transpose(1, 2) for x in (q, k))
    T = -(-c.L // c.tile)
    stride = -(-c.L // 128) * 128
    pooled = torch.full((c.B, c.G, T, stride), -1.0, dtype=torch.float32, device="cuda")
    nat.prefill_pool_scores(qd, kd, ref_lse.contiguous().cuda(), c.D ** -0.5, pooled)
    _status_ok()
    got = pooled.cpu()
    for t in range(T):
        n = t * c.tile
        if n:
            rel = ((got[:, :, t, :n] - ref[:, :, t, :n]).abs() / ref[:, :, t, :n]).max().item()
            assert rel < 5e-4, f"tile {t}: rel err {rel}"
        assert (got[:, :, t, n:] == -1.0).all(), f"tile {t}: wrote at or beyond the tile start"


def _golden_rows(gold, c, layer):
    """The reference's index rows of anchor `layer`, converted to the kernel's layout: per tile the
    keys strictly before the tile, ascending, with a count (everything else in a reference row is
    causally masked or inside the tile's own window)."""
    ref_rows = torch.from_numpy(gold[f"prefill_idx_{layer}"])
    B, G, T, kk = ref_rows.shape
    idx = torch.zeros(B, G, T, kk, dtype=torch.int32)
    cnt = torch.zeros(B, G, T, dtype=torch.int32)
    for b in range(B):
        for g in range(G):
            for t in range(T):
                keep = clean_index_row(ref_rows[b, g, t].tolist(), t * c.tile)
                cnt[b, g, t] = len(keep)
                idx[b, g, t, :len(keep)] = torch.tensor(keep, dtype=torch.int32)
    return idx, cnt


@pytest.mark.parametrize("case", CASES, ids=lambda c: c.name)
def test_sparse_prefill_teacher_forced(case, golden_dir):
    """Reuse layers (and anchors > 0) with the reference's own rows, against the reference's outputs."""
    from kascade_b200 import _native as nat
    c = case
    gold = np.load(os.path.join(golden_dir, f"{c.name}.npz"))
    hm = c.head_mapping()
    qsel = torch.from_numpy(gold["sampled_queries"].astype(np.int64))
    anchor_rows = None
    for layer in range(c.layers):
        is_anchor = layer == 0 or layer in c.anchors
        if is_anchor:
            anchor_rows = _golden_rows(gold, c, layer)
        if layer == 0:
            continue
        q, k, v = make_inputs(c, layer)
        qd, kd, vd = (_dev(x).transpose(1, 2) for x in (q, k, v))
        out = torch.zeros(c.B, c.L, c.H, c.D, dtype=torch.float16, device="cuda")
        head_map = None if is_anchor else torch.tensor(hm[layer], dtype=torch.int32, device="cuda")
        nat.prefill_sparse(qd, kd, vd, anchor_rows[0].cuda(), anchor_rows[1].cuda(), head_map, c.D ** -0.5, out)
        _status_ok()
        ref = torch.from_numpy(gold[f"prefill_out_{layer}"]).float()
        assert_close(out[:, qsel.cuda()], ref, what=f"{c.name} sparse prefill layer {layer}")


@pytest.mark.parametrize("case", CASES, ids=lambda c: c.name)
def test_strategy_prefill_end_to_end(case):
    """The whole strategy, free-running, like the reference is driven by HF: index sets must pass the
    tie-band rule against the oracle's pooled scores; outputs are compared with the oracle evaluated
    on the strategy's own index rows (so a legal boundary swap does not count as an error)."""
    from kascade_b200 import EfficientKascadeStrategy
    c = case
    strat = EfficientKascadeStrategy(list(c.anchors), "x/none", k=c.pct, tile_size=c.tile,
                                     rolling_prefill=c.rolling, head_mapping=c.head_mapping(), register=False)

    class M:
        pass

    scaling = c.D ** -0.5
    T = -(-c.L // c.tile)
    kk = topk_budget(c.pct, c.L, c.tile)
    rows = None
    for layer in range(c.layers):
        q, k, v = make_inputs(c, layer)
        m = M()
        m.layer_idx, m.num_key_value_groups = layer, c.H // c.G
        out, _ = strat.attention_forward(m, _dev(q), _dev(k), _dev(v), None, scaling)
        _status_ok()
        assert out.shape == (c.B, c.L, c.H, c.D)
        if strat.is_anchor(layer):
            idx, cnt = strat._tile_idx.cpu(), strat._tile_count.cpu()
            pooled = pooled_scores_prefill(q, k, scaling, c.tile)
            for b in range(c.B):
                for g in range(c.G):
                    for t in range(T):
                        budget = min(kk, rolling_budget(c.pct, t * c.tile)) if (c.rolling and c.L > 128) else kk
                        got = idx[b, g, t, :int(cnt[b, g, t])].tolist()
                        assert got == sorted(got)
                        ok, msg = band_check(pooled[b, g, t], got, budget, t * c.tile)
                        assert ok, f"layer {layer} (b{b} g{g} t{t}): {msg}"
            rows = torch.full((c.B, c.G, T, max(kk, 1)), c.L - 1, dtype=torch.int32)
            for b in range(c.B):
                for g in range(c.G):
                    for t in range(T):
                        n = int(cnt[b, g, t])
                        rows[b, g, t, :n] = idx[b, g, t, :n]
            if layer == 0:
                ref, _ = _dense_ref(q, k, v, scaling)
            else:
                ref = sparse_prefill_output(q, k, v, rows, scaling, c.tile)
        else:
            ref = sparse_prefill_output(q, k, v, rows[:, c.head_mapping()[layer]], scaling, c.tile)
        assert_close(out, ref, what=f"{c.name} strategy layer {layer}")


@pytest.mark.parametrize("direction", ["growing", "shrinking"])
def test_row_reference_moves_across_blocks(direction):
    """Scores whose maximum grows (or shrinks) by far more than 2^8 from one 128-key block to the next: the
    shared accumulator of the two softmax streams has to be rescaled on nearly every block (or never), with
    the reference handed from one stream to the other in block order."""
    from kascade_b200 import _native as nat
    g = torch.Generator().manual_seed(7)
    B, H, G, L, D = 1, 8, 2, 1024 + 32, 128
    u = torch.randn(D, generator=g)
    u = u / u.norm()
    q = (0.05 * torch.randn(B, H, L, D, generator=g) + 4.0 * u).half().float()
    ramp = (torch.arange(L) // 128).float()
    if direction == "shrinking":
        ramp = ramp.max() - ramp
    # logit of key j ~ 4 * ramp_j * 4 / sqrt(128) * ... : steps of about 12 in log2 units between blocks
    k = (0.05 * torch.randn(B, G, L, D, generator=g) + (2.1 * ramp)[None, None, :, None] * u).half().float()
    v = torch.randn(B, G, L, D, generator=g).half().float()
    scale = 1.0
    ref_o, ref_lse = _dense_ref(q, k, v, scale)
    qd, kd, vd = (_dev(x).transpose(1, 2) for x in (q, k, v))
    out = torch.zeros(B, L, H, D, dtype=torch.float16, device="cuda")
    lse = torch.zeros(B, L, H, dtype=torch.float32, device="cuda")
    nat.prefill_dense(qd, kd, vd, scale, out, lse)
    _status_ok()
    assert_close(out, ref_o, what=f"dense prefill, {direction} maxima")
    assert (lse.cpu() - ref_lse).abs().max() < 2e-3
    lse_only = torch.zeros_like(lse)
    nat.prefill_dense(qd, kd, None, scale, None, lse_only)
    assert (lse_only.cpu() - ref_lse).abs().max() < 2e-3
    # sparse path over all earlier keys (budget = everything): same result as dense
    T = -(-L // 32)
    idx = torch.arange(L, dtype=torch.int32).repeat(B, G, T, 1).contiguous().cuda()
    cnt = (torch.arange(T, dtype=torch.int32) * 32).repeat(B, G, 1).contiguous().cuda()
    sp = torch.zeros_like(out)
    nat.prefill_sparse(qd, kd, vd, idx, cnt, None, scale, sp)
    _status_ok()
    assert_close(sp, ref_o, what=f"sparse prefill over all keys, {direction} maxima")


def test_rejected_arguments_name_the_problem():
    """Bad calls return an error with a message (nothing is launched): fan-out limits, head ranges, strides."""
    from kascade_b200 import _native as nat
    dev = torch.device("cuda")
    B, L, H, G, D = 1, 64, 8, 2, 128
    q = torch.zeros(B, L, H, D, dtype=torch.float16, device=dev)
    k = torch.zeros(B, L, G, D, dtype=torch.float16, device=dev)
    out = torch.zeros(B, L, H, D, dtype=torch.float16, device=dev)
    with pytest.raises(nat.KascadeNativeError, match="1..8"):
        nat.out_fanout([out.data_ptr()] * 9, H, 0)
    fan = nat.out_fanout([out.data_ptr()], H, 4)                       # heads [4, 12) of an 8-head row
    with pytest.raises(nat.KascadeNativeError, match="do not fit"):
        nat.prefill_dense(q, k, k, 0.1, None, None, fanout=fan)
    fan = nat.out_fanout([out.data_ptr() + 2], H, 0)                   # misaligned
    with pytest.raises(nat.KascadeNativeError, match="aligned"):
        nat.prefill_dense(q, k, k, 0.1, None, None, fanout=fan)
    with pytest.raises(nat.KascadeNativeError, match="nothing to compute"):
        nat.prefill_dense(q, k, k, 0.1, None, None)
    with pytest.raises(nat.KascadeNativeError, match="query heads"):
        nat.prefill_dense(q[:, :, :6], k, k, 0.1, out[:, :, :6].contiguous(), None)
    idx = torch.zeros(B, G, 2, 4, dtype=torch.int32, device=dev)
    cnt = torch.zeros(B, G, 2, dtype=torch.int32, device=dev)
    with pytest.raises(nat.KascadeNativeError, match="head_map"):
        nat.prefill_sparse(q[:, :, :4], k[:, :, :1], k[:, :, :1], idx, cnt, None, 0.1, out[:, :, :4].contiguous())
    kc = torch.zeros(4, 12, G, D, dtype=torch.float16, device=dev)      # page size 12 is not a power of two
    bt = torch.zeros(B, 4, dtype=torch.int32, device=dev)
    with pytest.raises(nat.KascadeNativeError, match="power of two"):
        nat.kv_write(None, None, k, k, torch.zeros(B, dtype=torch.int32, device=dev), None, nat.kv_layout_paged(kc, kc, bt))
    assert nat.read_status() == 0
