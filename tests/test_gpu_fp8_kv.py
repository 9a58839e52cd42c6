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


@pytest.mark.parametrize("with_norm", [False, True], ids=["llama", "qwen3_qknorm"])
def test_kv_write_quantises_into_an_fp8_cache(with_norm):
    """The append kernel with an FP8 cache: rotated (and normalised) rows are stored as value / scale of their page
    and KV head, saturating, round to nearest even - against the oracle's torch restatement.  V rows are pure
    quantisation of the inputs: bit-identical; K rows inherit the last-bit freedom of cos / sin."""
    from kascade_b200 import _native as nat
    from oracle.kv_write_oracle import kv_write as oracle_kv_write
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(31)
    B, T, H, G, D, page = 2, 21, 8, 2, 128, 16
    start, n_new = [5, 1000], [21, 9]
    q = torch.randn(B, T, H, D, generator=g).half()
    k = (2 * torch.randn(B, T, G, D, generator=g)).half()
    v = (3 * torch.randn(B, T, G, D, generator=g)).half()
    max_len = max(s + n for s, n in zip(start, n_new))
    pps = -(-max_len // page)
    n_pages = B * pps + 1
    table = torch.randperm(n_pages, generator=g)[: B * pps].view(B, pps).to(torch.int32)
    k8 = torch.zeros(n_pages, page, G, D, dtype=torch.float8_e4m3fn)
    v8 = torch.zeros(n_pages, page, G, D, dtype=torch.float8_e4m3fn)
    ks = (0.02 + 0.02 * torch.rand(n_pages, G, generator=g)).float()        # about amax / 448 of these rows
    vs = (0.03 + 0.02 * torch.rand(n_pages, G, generator=g)).float()
    ks[int(table[0, 0])] = 0.004                                            # two pages small enough to saturate
    vs[int(table[1, 1000 // page])] = 0.004
    inv_freq = 1.0 / (500000.0 ** (torch.arange(0, D, 2, dtype=torch.int64).float() / D))
    q_gain = (1 + 0.1 * torch.randn(D, generator=g)).half() if with_norm else None
    k_gain = (1 + 0.1 * torch.randn(D, generator=g)).half() if with_norm else None
    ref_k, ref_v = k8.clone(), v8.clone()
    oracle_kv_write(q, k, v, start, n_new, ref_k, ref_v, table, page, q_gain, k_gain, 1e-6, inv_freq, 1.0,
                    k_scale=ks, v_scale=vs)
    kd, vd, td = k8.to(dev), v8.to(dev), table.to(dev)
    ks_d, vs_d = ks.to(dev), vs.to(dev)                   # (the layout holds raw pointers: the tensors must stay alive)
    q_out = torch.empty(B, T, H, D, dtype=torch.float16, device=dev)
    nat.kv_write(q.to(dev), q_out, k.to(dev), v.to(dev), torch.tensor(start, dtype=torch.int32, device=dev),
                 torch.tensor(n_new, dtype=torch.int32, device=dev), nat.kv_layout_paged(kd, vd, td, ks_d, vs_d),
                 None if q_gain is None else q_gain.to(dev), None if k_gain is None else k_gain.to(dev), 1e-6,
                 inv_freq.to(dev), 1.0)
    torch.cuda.synchronize()
    assert torch.equal(vd.cpu().view(torch.uint8), ref_v.view(torch.uint8)), "V rows: pure quantisation, bit for bit"
    got, want = kd.cpu().view(torch.uint8), ref_k.view(torch.uint8)
    differ = got != want
    assert float(differ.float().mean()) < 0.01, f"{float(differ.float().mean()):.3%} of the K bytes differ"
    # where they differ it is by one step of the format
    gf, wf = kd.cpu().float(), ref_k.float()
    assert bool(((gf - wf).abs()[differ] <= 0.126 * wf.abs()[differ].clamp(min=2.0 ** -6)).all())
    assert bool((wf.abs() == 448.0).any()) and bool((ref_v.float().abs() == 448.0).any()), \
        "the case is meant to saturate somewhere"
