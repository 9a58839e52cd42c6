"""Padded batches through the strategy (GPU): each sequence must come out exactly as if it had been run alone and
unpadded; padded query rows are zero; a padded prefill and a padded decode step launch every kernel once for the
whole batch.  The
reference ignores the mask altogether (strategies/EfficientKascadeStrategy.py:126-161), which is only right for
unpadded batches."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _mask(pads, L, Lq, dtype=torch.float16, as_bool=False, right=None):
    """HF-style mask [B,1,Lq,L]: causal, the first pads[b] key positions hidden and, with `right`, also the last
    right[b] ones."""
    B = len(pads)
    qpos = torch.arange(L - Lq, L)[:, None]
    kpos = torch.arange(L)[None, :]
    ok = (kpos <= qpos)[None].repeat(B, 1, 1)
    for b, pad in enumerate(pads):
        ok[b, :, :pad] = False
        if right is not None and right[b]:
            ok[b, :, L - right[b]:] = False
    if as_bool:
        return ok[:, None].cuda()
    m = torch.zeros(B, 1, Lq, L, dtype=dtype)
    m.masked_fill_(~ok[:, None], torch.finfo(dtype).min)
    return m.cuda()


@pytest.mark.parametrize("as_bool", [False, True], ids=["additive", "bool"])
def test_left_padded_batch_equals_separate_runs(as_bool):
    from kascade_b200 import EfficientKascadeStrategy, _native as nat
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(11)
    B, H, G, D, L, layers = 3, 32, 8, 128, 416, 3
    pads = [0, 77, 160]
    hm = [list(range(G)), [3, 3, 0, 7, 1, 6, 2, 5], list(range(G))]

    def make():
        return EfficientKascadeStrategy([0, 2], "x/y", k=25, tile_size=32, rolling_prefill=True, head_mapping=hm,
                                        register=False)

    class M:
        num_key_value_groups = H // G

    qs = [(torch.randn(B, H, L + 1, D, generator=g) / D ** 0.5).half().to(dev) for _ in range(layers)]
    ks = [torch.randn(B, G, L + 1, D, generator=g).half().to(dev) for _ in range(layers)]
    vs = [torch.randn(B, G, L + 1, D, generator=g).half().to(dev) for _ in range(layers)]
    batch = make()
    alone = [make() for _ in range(B)]
    mask_p = _mask(pads, L, L, as_bool=as_bool)
    mask_d = _mask(pads, L + 1, 1, as_bool=as_bool)
    for phase in ("prefill", "decode"):
        for l in range(layers):
            m = M()
            m.layer_idx = l
            if phase == "prefill":
                q, k, v, mask = qs[l][:, :, :L], ks[l][:, :, :L], vs[l][:, :, :L], mask_p
            else:
                q, k, v, mask = qs[l][:, :, L:], ks[l], vs[l], mask_d
            n0 = nat.launch_count
            got, _ = batch.attention_forward(m, q, k, v, mask, D ** -0.5)
            if phase == "prefill":                       # one launch per kernel kind for the whole padded batch
                assert nat.launch_count - n0 == {0: 4, 1: 1, 2: 5}[l], f"layer {l}: {nat.launch_count - n0} launches"
            else:                                        # and so does a padded decode step (no loop over sequences)
                assert nat.launch_count - n0 == {0: 3, 1: 1, 2: 4}[l], f"decode layer {l}: {nat.launch_count - n0} launches"
            for b, pad in enumerate(pads):
                qb = q[b:b + 1, :, pad:] if phase == "prefill" else q[b:b + 1]
                want, _ = alone[b].attention_forward(m, qb, k[b:b + 1, :, pad:], v[b:b + 1, :, pad:], None, D ** -0.5)
                if phase == "prefill":
                    assert torch.equal(got[b:b + 1, pad:], want), f"{phase} layer {l} sequence {b}"
                    assert bool((got[b, :pad] == 0).all()), "padded query rows must be zero"
                else:
                    assert torch.equal(got[b:b + 1], want), f"{phase} layer {l} sequence {b}"
    assert nat.read_status() == 0


def test_right_and_mixed_padding_equal_separate_runs():
    """Right padding (sequence at the start of its slot), left padding and a mix, lengths that are not multiples
    of the tile, one sequence of only 150 tokens: the prefill of the whole batch in one launch per kernel
    equals the separate unpadded runs bit for bit."""
    from kascade_b200 import EfficientKascadeStrategy, _native as nat
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(12)
    B, H, G, D, L, layers = 4, 32, 8, 128, 400, 3
    left, right = [0, 0, 50, 0], [0, 123, 31, 250]
    hm = [list(range(G)), [1, 0, 0, 7, 4, 6, 2, 5], list(range(G))]

    def make():
        return EfficientKascadeStrategy([0, 2], "x/y", k=30, tile_size=32, rolling_prefill=True, head_mapping=hm,
                                        register=False)

    class M:
        num_key_value_groups = H // G

    batch, alone = make(), [make() for _ in range(B)]
    mask = _mask(left, L, L, right=right)
    for l in range(layers):
        q = (torch.randn(B, H, L, D, generator=g) / D ** 0.5).half().to(dev)
        k = torch.randn(B, G, L, D, generator=g).half().to(dev)
        v = torch.randn(B, G, L, D, generator=g).half().to(dev)
        m = M()
        m.layer_idx = l
        got, _ = batch.attention_forward(m, q, k, v, mask, D ** -0.5)
        for b in range(B):
            lo, hi = left[b], L - right[b]
            want, _ = alone[b].attention_forward(m, q[b:b + 1, :, lo:hi], k[b:b + 1, :, lo:hi], v[b:b + 1, :, lo:hi], None,
                                                 D ** -0.5)
            assert torch.equal(got[b:b + 1, lo:hi], want), f"layer {l} sequence {b}"
            assert bool((got[b, :lo] == 0).all()) and bool((got[b, hi:] == 0).all()), "rows outside a sequence must be zero"
    assert nat.read_status() == 0


def test_unpadded_mask_takes_the_batched_path():
    from kascade_b200 import EfficientKascadeStrategy
    s = EfficientKascadeStrategy([0], "x/y", k=10, tile_size=32, head_mapping=[list(range(8))] * 2, register=False)
    assert s._padding(_mask([0, 0], 64, 64), 2, 64) is None
    assert s._padding(None, 2, 64) is None
    assert s._padding(_mask([0, 5], 64, 64), 2, 64) == ([0, 5], [64, 59])
    assert s._padding(_mask([0, 5], 64, 64, right=[10, 0]), 2, 64) == ([0, 5], [54, 59])
