"""The similarity statistic computed by the library's kernels (ratio of softmax normalisers) against the same
statistic from materialised fp32 attention weights, the way runners/stats_runner.py:155-168 defines it."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _weights(q, k, scaling):
    """Post-softmax causal weights pooled per KV head: [G, L, L] fp32 (sum over the KV head's 4 query heads)."""
    L, H, D = q.shape[1], q.shape[2], q.shape[3]
    G = k.shape[2]
    qf, kf = q[0].float().transpose(0, 1), k[0].float().transpose(0, 1)               # [H,L,D], [G,L,D]
    s = torch.einsum("hld,hmd->hlm", qf, kf.repeat_interleave(H // G, 0)) * scaling
    s = s.masked_fill(torch.triu(torch.ones(L, L, dtype=torch.bool, device=q.device), 1), float("-inf"))
    return torch.softmax(s, -1).view(G, H // G, L, L).sum(1)


@pytest.mark.parametrize("reduce", ["amin", "mean"])
def test_device_similarity_matches_materialised_weights(reduce):
    from kascade_b200.calibrate import DeviceSimilarityAccumulator
    from kascade_b200.head_mapping import select_layers
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(21)
    layers, L, H, G, D, tile = 3, 416, 32, 8, 128, 32
    scaling = D ** -0.5
    acc = DeviceSimilarityAccumulator(layers, G, k=30, tile_size=tile, rolling_prefill=True, reduce=reduce)
    qs, ks = [], []
    base = torch.randn(1, L, G, D, generator=g)
    for l in range(layers):                                   # layers share part of their keys, so sets overlap
        k = (0.7 * base + 0.7 * torch.randn(1, L, G, D, generator=g)).half().to(dev)
        q = (2.5 * torch.randn(1, L, H, D, generator=g)).half().to(dev)
        qs.append(q); ks.append(k)
        acc.add_layer(q, k, scaling)
    recorded = [(lay[4].clone(), lay[5].clone()) for lay in acc._layers]
    acc.end_prompt()
    got = acc.average().cpu()

    T = -(-L // tile)
    rows = torch.arange(L, device=dev)
    tile_of = rows // tile
    want = torch.zeros(layers, layers, G, G)
    for j in range(layers):
        w = _weights(qs[j], ks[j], scaling)                                            # [G2, L, L]
        own_tile = (torch.arange(L, device=dev)[None, :] // tile == tile_of[:, None])  # [L, L] keys of the query's tile
        last = (w * own_tile).sum(-1)                                                  # [G2, L] (causal zeros beyond)

        def mass_on(idx, count, h1):
            sel = torch.zeros(T, L, dtype=torch.bool, device=dev)
            for t in range(T):
                n = int(count[0, h1, t])
                sel[t, idx[0, h1, t, :n].long()] = True
            return (w * sel[tile_of][None]).sum(-1)                                    # [G2, L]

        den = torch.stack([mass_on(*recorded[j], h2)[h2] for h2 in range(G)]) + last   # [G2, L]
        for i in range(j + 1):
            for h1 in range(G):
                ratio = (mass_on(*recorded[i], h1) + last) / den                       # [G2, L]
                want[i, j, :, h1] = (ratio.amin(-1) if reduce == "amin" else ratio.mean(-1)).cpu()
    upper = torch.triu(torch.ones(layers, layers, dtype=torch.bool))
    assert torch.allclose(got[upper], want[upper], atol=4e-3, rtol=0), (got[upper] - want[upper]).abs().max()
    for i in range(layers):                                                            # a layer against itself
        assert torch.allclose(torch.diagonal(got[i, i]), torch.ones(G), atol=1e-6)
    assert bool((got[~upper] == 0).all())
    picked = select_layers(acc.average(), counts=(2,))
    (pivots, mapping), = picked.items()
    assert pivots[0] == 0 and len(mapping) == layers and all(len(r) == G for r in mapping)
