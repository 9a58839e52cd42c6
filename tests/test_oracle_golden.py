"""The CPU oracle against vectors produced by the reference's own KascadeStrategy
(tests/golden/make_golden.py).  No GPU."""
import os

import numpy as np
import pytest
import torch

from oracle.kascade_oracle import (KascadeOracle, band_check, clean_index_row, rolling_budget,
                                   topk_budget)
from tests.cases import CASES, decode_inputs, input_checksum, make_inputs


def test_budgets():
    # strategies/KascadeStrategy.py:127-129 evaluated by hand
    assert topk_budget(10, 2048, 32) == 172
    assert topk_budget(10, 2049, 32) == 172
    assert topk_budget(10, 32768, 32) == 3244
    assert topk_budget(10, 200, 32) == 96
    assert topk_budget(50, 100, 32) == 68
    assert rolling_budget(10, 0) == 128 and rolling_budget(10, 1280) == 128
    assert rolling_budget(10, 32736) == 3273


@pytest.mark.parametrize("case", CASES, ids=lambda c: c.name)
def test_oracle_matches_reference(case, golden_dir):
    gold = np.load(os.path.join(golden_dir, f"{case.name}.npz"))
    c = case
    orc = KascadeOracle(recompute_layers=c.anchors, head_mapping=c.head_mapping(), k=c.pct,
                        tile_size=c.tile, rolling_prefill=c.rolling)
    assert np.array_equal(np.asarray(c.head_mapping(), dtype=np.int32), gold["head_mapping"])
    scaling = c.D ** -0.5
    qsel = torch.tensor(gold["sampled_queries"].astype(np.int64))
    cks = 0.0
    T = -(-c.L // c.tile)
    for layer in range(c.layers):
        q, k, v = make_inputs(c, layer)
        cks += input_checksum(q, k, v)
        anchor = orc.is_anchor(layer)
        if not anchor:
            # teacher-force the reference's rows so output parity is not clouded by legal swaps
            orc.index_rows = ref_rows
        out = orc.attention_forward(layer, q, k, v, scaling)
        if anchor:
            ref_rows = torch.from_numpy(gold[f"prefill_idx_{layer}"])
            kk = ref_rows.shape[-1]
            assert kk == topk_budget(c.pct, c.L, c.tile)
            # index sets: identical up to ties inside one fp16 ulp of the k-th score
            n_diff = 0
            for b in range(c.B):
                for g in range(c.G):
                    for t in range(T):
                        ts0 = t * c.tile
                        budget = min(kk, rolling_budget(c.pct, ts0)) if (c.rolling and c.L > 128) else kk
                        ref = clean_index_row(ref_rows[b, g, t].tolist(), ts0)
                        mine = clean_index_row(orc.index_rows[b, g, t].tolist(), ts0)
                        ok, msg = band_check(orc.pooled[b, g, t], ref, budget, ts0)
                        assert ok, f"reference row fails band check {(layer, b, g, t)}: {msg}"
                        ok, msg = band_check(orc.pooled[b, g, t], mine, budget, ts0)
                        assert ok, f"oracle row fails band check {(layer, b, g, t)}: {msg}"
                        n_diff += len(set(ref) ^ set(mine))
            assert n_diff <= 0.002 * c.B * c.G * T * kk, f"too many boundary swaps: {n_diff}"
            if layer > 0:
                # the anchor's own sparse output, recomputed with the reference's rows
                from oracle.kascade_oracle import sparse_prefill_output
                out = sparse_prefill_output(q, k, v, ref_rows, scaling, c.tile)
        ref_out = torch.from_numpy(gold[f"prefill_out_{layer}"]).float()
        d = (out[:, qsel] - ref_out).abs().max().item()
        assert d < 2e-4, f"prefill layer {layer}: max abs diff {d}"      # fp16 storage of the golden
    for layer in range(c.layers):
        q, k, v = decode_inputs(c, layer)
        cks += input_checksum(q, k, v)
        anchor = orc.is_anchor(layer)
        if not anchor:
            orc.index_rows = ref_rows
        out = orc.attention_forward(layer, q, k, v, scaling)
        if anchor:
            ref_rows = torch.from_numpy(gold[f"decode_idx_{layer}"]).unsqueeze(2)
            kk = ref_rows.shape[-1]
            assert kk == topk_budget(c.pct, c.L + 1, c.tile)
            for b in range(c.B):
                for g in range(c.G):
                    ok, msg = band_check(orc.pooled[b, g], ref_rows[b, g, 0].tolist(), kk, c.L + 1)
                    assert ok, msg
            if layer > 0:
                from oracle.kascade_oracle import sparse_decode_output
                out = sparse_decode_output(q, k, v, ref_rows[:, :, 0], scaling)
        d = (out - torch.from_numpy(gold[f"decode_out_{layer}"])).abs().max().item()
        assert d < 2e-6, f"decode layer {layer}: max abs diff {d}"
    assert abs(cks - float(gold["checksum"])) < 1e-6 * max(1.0, abs(cks)), "inputs differ from the golden run"
