"""KV-cache write path (RMS norm + rotary embedding + paged append) against its CPU oracle (GPU)."""
import pytest
import torch

from oracle.kv_write_oracle import kv_write as oracle_kv_write

pytestmark = pytest.mark.gpu
D = 128


def _inv_freq(theta):
    return 1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.int64).float() / D))


def _close_fp16(got, want, what):
    """Equal up to the last bit of cos / sin in the storage type: the device's sincosf and the host's cos / sin may
    round a value differently now and then, which moves one of the two products (magnitude up to ~4 for N(0,1)
    inputs) by one unit in its last place, 2^-9 in fp16 (2^-6 in bf16); the sum can be much smaller than the
    products."""
    ulp = 2.0 ** -8 if got.dtype == torch.float16 else 2.0 ** -5
    got, want = got.float().cpu(), want.float().cpu()
    diff = (got - want).abs()
    bad = diff > ulp
    assert not bool(bad.any()), f"{what}: {int(bad.sum())} elements differ, max {diff.max().item():.3e}"
    frac = float((diff > 0).float().mean())
    assert frac < 0.02, f"{what}: {frac:.3%} of the elements are not bit-identical"


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
@pytest.mark.parametrize("with_norm", [False, True], ids=["llama", "qwen3_qknorm"])
@pytest.mark.parametrize("with_q", [True, False], ids=["q", "no_q"])
def test_kv_write_paged(with_norm, with_q, dtype):
    from kascade_b200 import _native as nat
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(3)
    B, T, H, G, page = 3, 37, 8, 2, 16
    start = [0, 70001, 4095]
    n_new = [37, 5, 20]
    q = torch.randn(B, T, H, D, generator=g).to(dtype)
    k = torch.randn(B, T, G, D, generator=g).to(dtype)
    v = torch.randn(B, T, G, D, generator=g).to(dtype)
    max_len = max(s + n for s, n in zip(start, n_new))
    pps = -(-max_len // page)
    n_pages = B * pps + 2
    block_table = torch.randperm(n_pages, generator=g)[: B * pps].view(B, pps).to(torch.int32)
    k_cache = torch.randn(n_pages, page, G, D, generator=g).to(dtype)
    v_cache = torch.randn(n_pages, page, G, D, generator=g).to(dtype)
    inv_freq = _inv_freq(500000.0)
    q_gain = (1 + 0.1 * torch.randn(D, generator=g)).to(dtype) if with_norm else None
    k_gain = (1 + 0.1 * torch.randn(D, generator=g)).to(dtype) if with_norm else None

    ref_kc, ref_vc = k_cache.clone(), v_cache.clone()
    ref_q = oracle_kv_write(q if with_q else None, k, v, start, n_new, ref_kc, ref_vc, block_table, page,
                            q_gain, k_gain, 1e-6, inv_freq, 1.0)

    kc, vc, bt = k_cache.to(dev), v_cache.to(dev), block_table.to(dev)
    q_out = torch.full((B, T, H, D), 9.0, dtype=dtype, device=dev)
    nat.kv_write(q.to(dev) if with_q else None, q_out if with_q else None, k.to(dev), v.to(dev),
                 torch.tensor(start, dtype=torch.int32, device=dev), torch.tensor(n_new, dtype=torch.int32, device=dev),
                 nat.kv_layout_paged(kc, vc, bt), None if q_gain is None else q_gain.to(dev),
                 None if k_gain is None else k_gain.to(dev), 1e-6, inv_freq.to(dev), 1.0)
    torch.cuda.synchronize()
    written = torch.zeros(n_pages, page, dtype=torch.bool)
    for b in range(B):
        for t in range(n_new[b]):
            p = start[b] + t
            written[int(block_table[b, p // page]), p % page] = True
    _close_fp16(kc.cpu()[written], ref_kc[written], "appended k rows")
    assert torch.equal(vc.cpu(), ref_vc), "v rows are copied bit for bit; nothing else in the cache may change"
    # slots that were not appended to are untouched
    assert torch.equal(kc.cpu()[~written], k_cache[~written])
    if with_q:
        for b in range(B):
            _close_fp16(q_out[b, : n_new[b]], ref_q[b, : n_new[b]], f"q of sequence {b}")
            assert bool((q_out[b, n_new[b]:] == 9.0).all()), "rows beyond a sequence's new tokens must not be written"


def test_kv_write_contiguous_cache_then_decode_reads_it():
    """Append one token to an HF-style contiguous cache [B, G, L, D] (no rotary, no norm) and let the dense
    decode kernel attend over the result: the cache layout written is the layout read."""
    from kascade_b200 import _native as nat
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(5)
    B, G, H, L = 2, 2, 8, 200
    cache_k = torch.zeros(B, G, L + 1, D, dtype=torch.float16, device=dev)
    cache_v = torch.zeros(B, G, L + 1, D, dtype=torch.float16, device=dev)
    k_all = torch.randn(B, L + 1, G, D, generator=g).half().to(dev)
    v_all = torch.randn(B, L + 1, G, D, generator=g).half().to(dev)
    kv = nat.kv_layout_contiguous(cache_k, cache_v)
    zero = torch.zeros(B, dtype=torch.int32, device=dev)
    nat.kv_write(None, None, k_all[:, :L], v_all[:, :L], zero, None, kv)                       # the prompt
    nat.kv_write(None, None, k_all[:, L:], v_all[:, L:], torch.full((B,), L, dtype=torch.int32, device=dev), None, kv)
    torch.cuda.synchronize()
    assert torch.equal(cache_k, k_all.transpose(1, 2)) and torch.equal(cache_v, v_all.transpose(1, 2))
    q = (torch.randn(B, H, D, generator=g) / D ** 0.5).half().to(dev)
    stride = -(-(L + 1) // 4) * 4
    logits = torch.empty(B, H, stride, dtype=torch.float32, device=dev)
    pooled = torch.empty(B, G, stride, dtype=torch.float32, device=dev)
    out = torch.empty(B, H, D, dtype=torch.float16, device=dev)
    lse = torch.empty(B, H, dtype=torch.float32, device=dev)
    ws = nat.decode_workspace(B, H, 4, dev)
    nat.decode_anchor_paged(q, kv, torch.full((B,), L + 1, dtype=torch.int32, device=dev), L + 1, D ** -0.5, logits,
                            pooled, out, lse, ws, 0)
    kk = k_all.transpose(1, 2).float().repeat_interleave(H // G, 1)
    vv = v_all.transpose(1, 2).float().repeat_interleave(H // G, 1)
    p = torch.softmax(torch.einsum("bhd,bhld->bhl", q.float(), kk) * D ** -0.5, -1)
    ref = torch.einsum("bhl,bhld->bhd", p, vv)
    assert (out.float() - ref).abs().max().item() < 2e-3


def test_prefill_to_paged_decode_hand_off():
    """The prompt's K / V rows are appended to a paged cache with `append_kv`, then a decode step appends its
    own row and attends through the block table: same outputs as the same strategy fed the contiguous
    Hugging Face cache."""
    from kascade_b200 import EfficientKascadeStrategy, _native as nat
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(21)
    B, H, G, L, page, layers = 2, 32, 8, 700, 16, 3
    hm = [list(range(G)), [3, 3, 0, 7, 1, 6, 2, 5], list(range(G))]

    def make():
        return EfficientKascadeStrategy([0, 2], "x/y", k=10, tile_size=32, rolling_prefill=True, head_mapping=hm,
                                        register=False)

    class M:
        num_key_value_groups = H // G

    pps = -(-(L + 1) // page)
    n_pages = B * pps + 3
    bt = torch.randperm(n_pages, generator=g)[: B * pps].view(B, pps).to(torch.int32).to(dev)
    paged, contig = make(), make()
    zero = torch.zeros(B, dtype=torch.int32, device=dev)
    full = torch.full((B,), L, dtype=torch.int32, device=dev)
    for l in range(layers):
        k = torch.randn(B, G, L + 1, D, generator=g).half().to(dev)                 # HF layout [B, G, L, D]
        v = torch.randn(B, G, L + 1, D, generator=g).half().to(dev)
        q = (torch.randn(B, H, 1, D, generator=g) / D ** 0.5).half().to(dev)
        kc = torch.zeros(n_pages, page, G, D, dtype=torch.float16, device=dev)
        vc = torch.zeros_like(kc)
        # prompt rows, then the decode token's row (token-major views of the HF tensors, no copies)
        paged.append_kv(k[:, :, :L].transpose(1, 2), v[:, :, :L].transpose(1, 2), kc, vc, bt, zero)
        paged.append_kv(k[:, :, L:].transpose(1, 2), v[:, :, L:].transpose(1, 2), kc, vc, bt, full)
        m = M()
        m.layer_idx = l
        want, _ = contig.attention_forward(m, q, k, v, None, D ** -0.5)             # [B, 1, H, D]
        got = paged.paged_decode_forward(l, q[:, :, 0], kc, vc, bt, full + 1, D ** -0.5, L + 1)
        assert torch.equal(got, want[:, 0]), f"layer {l}: paged decode differs from the contiguous cache"
    assert nat.read_status() == 0
