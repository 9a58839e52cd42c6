"""Top-k select against torch.topk / the tie-band rule (GPU)."""
import pytest
import torch

from oracle.kascade_oracle import band_check

pytestmark = pytest.mark.gpu


def _run(scores, n_valid, k_row, k_max):
    from kascade_b200 import _native as nat
    dev = torch.device("cuda")
    s = scores.to(dev).contiguous()
    rows = s.numel() // s.shape[-1]
    out = torch.full((rows, max(k_max, 1)), -7, dtype=torch.int32, device=dev)
    cnt = torch.full((rows,), -1, dtype=torch.int32, device=dev)
    nv = None if n_valid is None else n_valid.to(dev).to(torch.int32)
    kr = None if k_row is None else k_row.to(dev).to(torch.int32)
    nat.topk_select(s, nv, kr, k_max, out, cnt)
    torch.cuda.synchronize()
    return out.cpu(), cnt.cpu()


@pytest.mark.parametrize("n,k", [(4096, 300), (1000, 128), (33, 5), (4, 4), (8192, 1), (65536, 6000)])
def test_distinct_scores_exact(n, k):
    g = torch.Generator().manual_seed(n + k)
    rows = 7
    stride = (n + 3) // 4 * 4 + 8
    scores = torch.rand(rows, stride, generator=g)
    scores[:, n:] = 9.0                                   # beyond n_cols: must be ignored
    from kascade_b200 import _native as nat
    dev = torch.device("cuda")
    s = scores.to(dev)
    out = torch.full((rows, k), -7, dtype=torch.int32, device=dev)
    cnt = torch.zeros(rows, dtype=torch.int32, device=dev)
    nat.topk_select(s, None, None, k, out, cnt, n_cols=n)
    torch.cuda.synchronize()
    ref = torch.topk(scores[:, :n], k, dim=-1).indices.sort(-1).values
    assert torch.equal(cnt.cpu(), torch.full((rows,), k, dtype=torch.int32))
    assert torch.equal(out.cpu().long(), ref), "index sets differ / not ascending"


def test_ties_take_lowest_index_and_negative_values():
    n = 2048
    scores = torch.zeros(3, n)
    scores[0, 100:200] = 1.0                              # 100 ones, rest zero; k = 150 -> ones + first 50 zeros
    scores[1] = -torch.arange(n, dtype=torch.float32)     # strictly decreasing, negative
    scores[2] = 0.5                                       # all tied
    out, cnt = _run(scores, None, None, 150)
    exp0 = sorted(list(range(100, 200)) + list(range(0, 50)))
    assert out[0].tolist() == exp0
    assert out[1].tolist() == list(range(150))
    assert out[2].tolist() == list(range(150))
    assert cnt.tolist() == [150, 150, 150]


def test_row_dependent_budgets_and_valid_lengths():
    g = torch.Generator().manual_seed(5)
    rows, n = 64, 2048
    scores = torch.rand(rows, n, generator=g) ** 4
    n_valid = torch.arange(rows) * 32                     # tile starts, as in an anchor prefill layer
    k_row = torch.clamp((10 * n_valid) // 100, min=128)
    out, cnt = _run(scores, n_valid, k_row, 172)
    for r in range(rows):
        want = min(int(k_row[r]), 172, int(n_valid[r]))
        assert int(cnt[r]) == want
        got = out[r, :want].tolist()
        assert got == sorted(got)
        ok, msg = band_check(scores[r], got, min(int(k_row[r]), 172), int(n_valid[r]), rel=0.0)
        assert ok, f"row {r}: {msg}"
        assert (out[r, want:] == -7).all(), "entries beyond the count must stay untouched"


def test_clustered_post_softmax_like_scores():
    # near-uniform attention: thousands of candidates within a few ulps of each other
    g = torch.Generator().manual_seed(11)
    n, k = 32768, 3244
    base = torch.full((4, n), 1.0 / n)
    scores = base * (1 + 1e-3 * torch.randn(4, n, generator=g))
    out, cnt = _run(scores, None, None, k)
    for r in range(4):
        ok, msg = band_check(scores[r], out[r].tolist(), k, n, rel=0.0)
        assert ok, msg


def test_rows_the_sample_cannot_bracket():
    """Rows on which the sampled bracket must fail, so that the histogram passes over the whole row decide: half of
    a long row tied at the threshold (the candidate lists overflow), a threshold inside a run of equal values with
    k beyond the distinct part, a step distribution, and a long row with negative values only."""
    g = torch.Generator().manual_seed(17)
    n = 40000
    rows = torch.zeros(4, n)
    rows[0] = torch.where(torch.rand(n, generator=g) < 0.5, torch.tensor(0.25), torch.rand(n, generator=g) * 0.2)
    rows[0, :100] = torch.rand(100, generator=g) + 1.0                    # 100 distinct large values, ~20000 ties at 0.25
    rows[1] = 0.125                                                        # everything tied except a few
    rows[1, 1000:1010] = 3.0
    rows[2] = (torch.arange(n) % 7).float()                                # seven plateaus
    rows[3] = -torch.rand(n, generator=g) - 1.0
    k = 5000
    out, cnt = _run(rows, None, None, k)
    assert cnt.tolist() == [k] * 4
    for r in range(4):
        vals = rows[r]
        order = torch.sort(vals, descending=True, stable=True).indices     # ties: lowest index first
        tau = vals[order[k - 1]]
        above = (vals > tau).nonzero().flatten()
        at = (vals == tau).nonzero().flatten()[: k - above.numel()]
        want = torch.cat([above, at]).sort().values
        assert torch.equal(out[r].long(), want), f"row {r}"


@pytest.mark.parametrize("n,k", [(131072, 13000), (70000, 128), (4097, 4000), (4096, 4000), (100000, 99999)])
def test_long_rows_and_extreme_budgets(n, k):
    g = torch.Generator().manual_seed(n)
    from kascade_b200 import _native as nat
    dev = torch.device("cuda")
    stride = (n + 3) // 4 * 4 + 8
    scores = torch.exp(3 * torch.randn(3, stride, generator=g) - 6)        # heavy-tailed, like pooled attention mass
    scores[:, n:] = 1e9                                                    # beyond n_cols: must be ignored
    out = torch.full((3, k), -7, dtype=torch.int32, device=dev)
    cnt = torch.zeros(3, dtype=torch.int32, device=dev)
    nat.topk_select(scores.to(dev), None, None, k, out, cnt, n_cols=n)
    torch.cuda.synchronize()
    ref = torch.topk(scores[:, :n], k, dim=-1).indices.sort(-1).values
    assert cnt.tolist() == [k] * 3
    assert torch.equal(out.cpu().long(), ref)


def test_rejects_bad_arguments():
    from kascade_b200 import _native as nat
    dev = torch.device("cuda")
    s = torch.zeros(2, 10, device=dev)                    # row stride not a multiple of 4
    out = torch.zeros(2, 4, dtype=torch.int32, device=dev)
    with pytest.raises(nat.KascadeNativeError):
        nat.topk_select(s, None, None, 4, out, None)
