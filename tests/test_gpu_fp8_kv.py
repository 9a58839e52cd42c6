"""Paged decode over an FP8 (e4m3) KV cache with one scale per (page, KV head) (GPU).  The checker is plain fp32
attention over the DEQUANTISED cache (stored value x scale): the kernels turn the stored bytes into fp16 exactly
and apply the scales in fp32, so the usual tolerance holds (max-abs 2e-3 / rel 1e-2).  The reference has no
quantised cache."""
import pytest
import torch

from oracle.kascade_oracle import band_check, pooled_scores_decode, sparse_decode_output, topk_budget
from tests.gpu_util import assert_close, paged_from_contiguous

pytestmark = pytest.mark.gpu


def _quantise(cache):
    """[pages, 16, G, D] fp16 -> (e4m3 cache, scales [pages, G] fp32), scale = amax / 448 per (page, head)."""
    amax = cache.float().abs().amax(dim=(1, 3)).clamp(min=1e-6)          # [pages, G]
    scale = amax / 448.0
    q8 = (cache.float() / scale[:, None, :, None]).to(torch.float8_e4m3fn)
    return q8, scale.contiguous()


def _dequant_contiguous(q8, scale, table, L):
    """Back to [B, G, L, D] fp32 through the block table."""
    deq = q8.float() * scale[:, None, :, None]                            # [pages, 16, G, D]
    B = table.shape[0]
    rows = deq[table.long()]                                              # [B, pages_per_seq, 16, G, D]
    return rows.reshape(B, -1, deq.shape[2], deq.shape[3])[:, :L].permute(0, 2, 1, 3).contiguous().cpu()


@pytest.mark.parametrize("raw_bytes", [False, True], ids=["float8_e4m3fn", "uint8"])
def test_fp8_cache_anchor_and_reuse_decode(raw_bytes):
    from kascade_b200 import EfficientKascadeStrategy, _native as nat
    g = torch.Generator().manual_seed(21)
    B, H, G, D, L, pct = 3, 8, 2, 128, 1500, 20
    k = (torch.randn(B, G, L, D, generator=g) / D ** 0.5 * (1 + torch.rand(B, G, L, 1, generator=g))).half().cuda()
    v = (torch.randn(B, G, L, D, generator=g) * (1 + 3 * torch.rand(B, G, 1, 1, generator=g))).half().cuda()
    k[:, :, :4] += 3 * torch.randn(B, G, 4, D, generator=g).half().cuda()
    kc, vc, bt = paged_from_contiguous(k, v, seed=9)
    k8, ks = _quantise(kc)
    v8, vs = _quantise(vc)
    kf, vf = _dequant_contiguous(k8, ks, bt, L), _dequant_contiguous(v8, vs, bt, L)
    if raw_bytes:
        k8, v8 = k8.view(torch.uint8), v8.view(torch.uint8)
    lens = torch.full((B,), L, dtype=torch.int32, device="cuda")
    hm = [[0, 1], [1, 0]]
    strat = EfficientKascadeStrategy([0], "x/y", k=pct, tile_size=32, head_mapping=hm, register=False)
    scaling = D ** -0.5
    qs = [(torch.randn(B, H, D, generator=g) / D ** 0.5).half().cuda() for _ in range(2)]
    # anchor layer 0: dense attention over the dequantised cache, index rows from its pooled scores
    out0 = strat.paged_decode_forward(0, qs[0], k8, v8, bt, lens, scaling, L, k_scale=ks, v_scale=vs)
    q0 = qs[0].float().cpu()[:, :, None]
    ref0 = torch.nn.functional.scaled_dot_product_attention(q0, kf, vf, enable_gqa=True, scale=scaling)[:, :, 0]
    assert out0.dtype == torch.float16
    assert_close(out0, ref0, what="FP8 cache, dense decode")
    pooled, _ = pooled_scores_decode(q0, kf, scaling)
    kk = topk_budget(pct, L, 32)
    cnt, idx = strat._dec_count.cpu(), strat._dec_idx.cpu()
    for b in range(B):
        for h in range(G):
            n = int(cnt[b, h])
            assert n == kk
            ok, msg = band_check(pooled[b, h], idx[b, h, :n].tolist(), kk, L)
            assert ok, f"FP8 cache, index row (b{b} g{h}): {msg}"
    # reuse layer 1 on those rows
    out1 = strat.paged_decode_forward(1, qs[1], k8, v8, bt, lens, scaling, L, k_scale=ks, v_scale=vs)
    rows = idx[:, :, :kk]
    ref1 = sparse_decode_output(qs[1].float().cpu()[:, :, None], kf, vf, rows[:, hm[1]], scaling)[:, 0]
    assert_close(out1, ref1, what="FP8 cache, sparse decode")
    assert nat.read_status() == 0


def test_fp8_cache_needs_scales_and_fp16_queries():
    from kascade_b200 import _native as nat
    kc = torch.zeros(4, 16, 2, 128, dtype=torch.uint8, device="cuda")
    bt = torch.zeros(1, 4, dtype=torch.int32, device="cuda")
    with pytest.raises(nat.KascadeNativeError, match="k_scale"):
        nat.kv_layout_paged(kc, kc, bt)
    sc = torch.ones(4, 2, dtype=torch.float32, device="cuda")
    kv = nat.kv_layout_paged(kc, kc, bt, sc, sc)
    q = torch.zeros(1, 8, 128, dtype=torch.bfloat16, device="cuda")
    out = torch.empty_like(q)
    rows = torch.zeros(1, 2, 16, dtype=torch.int32, device="cuda")
    with pytest.raises(nat.KascadeNativeError, match="fp16 q"):
        nat.decode_sparse_paged(q, kv, rows, None, 16, None, 0.1, out, None, None, 1)
