"""bf16 activations and caches through the same kernels (GPU).  bf16 is Qwen3's native type; the reference ships
fp16 kernels only.  Inputs are bf16-representable, the checker is the fp32 oracle on the same values; probabilities
are rounded to bf16 (8 bits of mantissa) before the P.V product, so the output tolerance is wider than for fp16
(max-abs 1.5e-2 / rel 3e-2); index rows are held to the same tie-band rule, because the pooled scores are fp32."""
import pytest
import torch

from oracle.kascade_oracle import (band_check, pooled_scores_prefill, rolling_budget, sparse_decode_output,
                                   sparse_prefill_output, topk_budget)
from tests.gpu_util import assert_close, paged_from_contiguous

pytestmark = pytest.mark.gpu
TOL = dict(atol=1.5e-2, rtol=3e-2)


def _inputs(B, H, G, L, seed):
    g = torch.Generator().manual_seed(seed)
    D = 128
    q = (torch.randn(B, H, L, D, generator=g) / D ** 0.5).bfloat16()
    k = (torch.randn(B, G, L, D, generator=g) / D ** 0.5).bfloat16()
    v = (torch.randn(B, G, L, D, generator=g) / D ** 0.5).bfloat16()
    k[:, :, :4] += (3 * torch.randn(B, G, 4, D, generator=g)).bfloat16()
    return q, k, v


def test_bf16_strategy_prefill_and_decode():
    from kascade_b200 import EfficientKascadeStrategy, _native as nat
    B, H, G, L, tile, pct = 1, 8, 2, 700, 32, 30
    hm = [[0, 1], [1, 0], [0, 1]]
    strat = EfficientKascadeStrategy([0, 2], "x/y", k=pct, tile_size=tile, rolling_prefill=True, head_mapping=hm,
                                     register=False)

    class M:
        num_key_value_groups = H // G

    scaling = 128 ** -0.5
    T = -(-L // tile)
    kk = topk_budget(pct, L, tile)
    rows = None
    for layer in range(3):
        q, k, v = _inputs(B, H, G, L, 40 + layer)
        m = M()
        m.layer_idx = layer
        out, _ = strat.attention_forward(m, q.cuda(), k.cuda(), v.cuda(), None, scaling)
        assert out.dtype == torch.bfloat16 and out.shape == (B, L, H, 128)
        qf, kf, vf = q.float(), k.float(), v.float()
        if strat.is_anchor(layer):
            idx, cnt = strat._tile_idx.cpu(), strat._tile_count.cpu()
            pooled = pooled_scores_prefill(qf, kf, scaling, tile)
            rows = torch.full((B, G, T, max(kk, 1)), L - 1, dtype=torch.int32)
            for g in range(G):
                for t in range(T):
                    n = int(cnt[0, g, t])
                    got = idx[0, g, t, :n].tolist()
                    ok, msg = band_check(pooled[0, g, t], got, min(kk, rolling_budget(pct, t * tile)), t * tile)
                    assert ok, f"layer {layer} (g{g} t{t}): {msg}"
                    rows[0, g, t, :n] = idx[0, g, t, :n]
        if layer == 0:
            ref = torch.nn.functional.scaled_dot_product_attention(qf, kf, vf, is_causal=True, enable_gqa=True,
                                                                   scale=scaling).transpose(1, 2)
        else:
            ref = sparse_prefill_output(qf, kf, vf, rows if strat.is_anchor(layer) else rows[:, hm[layer]], scaling, tile)
        assert_close(out, ref, what=f"bf16 prefill layer {layer}", **TOL)
    # one paged decode step: anchor layer 0 selects, layer 1 reuses
    q, k, v = _inputs(B, H, G, L + 1, 50)
    kc, vc, bt = paged_from_contiguous(k.cuda(), v.cuda(), seed=3)
    assert kc.dtype == torch.bfloat16
    lens = torch.full((B,), L + 1, dtype=torch.int32, device="cuda")
    q1 = q[:, :, -1].cuda().contiguous()
    out0 = strat.paged_decode_forward(0, q1, kc, vc, bt, lens, scaling, L + 1)
    qf, kf, vf = q[:, :, -1:].float(), k.float(), v.float()
    ref0 = torch.nn.functional.scaled_dot_product_attention(qf, kf, vf, enable_gqa=True, scale=scaling)[:, :, 0]
    assert out0.dtype == torch.bfloat16
    assert_close(out0, ref0, what="bf16 dense decode", **TOL)
    drows = strat._dec_idx.cpu()[:, :, :int(strat._dec_count.cpu().max())]
    out1 = strat.paged_decode_forward(1, q1, kc, vc, bt, lens, scaling, L + 1)
    ref1 = sparse_decode_output(qf, kf, vf, drows[:, hm[1]], scaling)[:, 0]
    assert_close(out1, ref1, what="bf16 sparse decode", **TOL)
    assert nat.read_status() == 0


def test_mixed_or_unknown_dtypes_are_rejected():
    from kascade_b200 import _native as nat
    q = torch.zeros(1, 64, 8, 128, dtype=torch.bfloat16, device="cuda")
    k = torch.zeros(1, 64, 2, 128, dtype=torch.float16, device="cuda")
    out = torch.empty(1, 64, 8, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(nat.KascadeNativeError, match="same dtype"):
        nat.prefill_dense(q, k, k, 0.1, out, None)
    with pytest.raises(nat.KascadeNativeError, match="fp16 or bf16"):
        nat.prefill_dense(q.float(), k, k, 0.1, out, None)
    kb = k.bfloat16()                                      # bf16 rows into an fp16 cache: one type for all operands
    with pytest.raises(nat.KascadeNativeError, match="all be fp16 or all bf16"):
        nat.kv_write(None, None, kb, kb, torch.zeros(1, dtype=torch.int32, device="cuda"), None,
                     nat.kv_layout_contiguous(k.transpose(1, 2), k.transpose(1, 2)))
