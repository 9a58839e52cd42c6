"""Tensor-core path self-test: descriptor encodings of the tcgen05 layer against a plain product."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_umma_conventions():
    from kascade_b200 import _native as nat
    g = torch.Generator().manual_seed(3)
    a = (torch.randn(128, 128, generator=g) / 4).to(torch.float16).cuda()
    b = (torch.randn(128, 128, generator=g) / 4).to(torch.float16).cuda()
    out, status = nat.selftest_umma(a, b)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0], f"a bounded wait gave up: {status.tolist()}"
    af, bf = a.float(), b.float()
    refs = [af @ bf.t(), af @ bf, af @ bf.t(), af @ bf]
    names = ["SS K-major x K-major", "SS K-major x MN-major", "TS tmem x K-major", "TS tmem x MN-major"]
    errs = [(out[i] - refs[i]).abs().max().item() for i in range(4)]
    print("umma selftest max abs errors:", dict(zip(names, errs)))
    for n, e in zip(names, errs):
        assert e < 1e-3, f"{n}: max abs err {e}"


def test_bounded_wait_runs_out_and_is_reported():
    """The give-up path of the kernels' bounded waits, made to happen harmlessly: a CTA waits (limit 1 ms) on
    a barrier nobody arrives on.  It must give up, free its tensor memory, return and leave its code in the
    device status word; while the word is set the tile-prefill kernels return at entry and the strategy raises
    at its next check; reading the word clears it and everything works again."""
    from kascade_b200 import EfficientKascadeStrategy, _native as nat
    assert nat.read_status() == 0
    res = nat.selftest_wait_timeout("cuda", limit_ns=1_000_000, code=77)
    torch.cuda.synchronize()
    code, gave_up, ns = res.tolist()
    assert code == 77 and gave_up == 128, f"wait did not run out as expected: {res.tolist()}"
    assert 1_000_000 <= ns < 50_000_000, f"the wait took {ns} ns for a 1 ms limit"
    # the word is still set: a prefill launch returns at entry and writes nothing
    g = torch.Generator().manual_seed(5)
    q = (torch.randn(1, 160, 8, 128, generator=g) / 128 ** 0.5).half().cuda()
    k = (torch.randn(1, 160, 2, 128, generator=g) / 128 ** 0.5).half().cuda()
    v = torch.randn(1, 160, 2, 128, generator=g).half().cuda()
    out = torch.full((1, 160, 8, 128), 7.0, dtype=torch.float16, device="cuda")
    nat.prefill_dense(q, k, v, 128 ** -0.5, out, None)
    torch.cuda.synchronize()
    assert bool((out == 7.0).all()), "a prefill kernel ran although the status word was set"
    strat = EfficientKascadeStrategy([0], "x/y", k=10, tile_size=32, head_mapping=[[0, 1]], register=False)
    with pytest.raises(nat.KascadeNativeError, match="code 77"):
        strat.check_status()
    assert nat.read_status() == 0                       # cleared by the check
    nat.prefill_dense(q, k, v, 128 ** -0.5, out, None)
    torch.cuda.synchronize()
    ref = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2).float(), k.transpose(1, 2).float(),
                                                           v.transpose(1, 2).float(), is_causal=True, enable_gqa=True)
    assert (out.float() - ref.transpose(1, 2)).abs().max().item() < 2e-3
    assert nat.read_status() == 0


def test_tensor_map_descriptors_are_cached():
    """Descriptors are kept per (pointer, strides, extents): a second pass over the same buffers encodes none."""
    from kascade_b200 import _native as nat
    g = torch.Generator().manual_seed(6)
    q = (torch.randn(1, 256, 8, 128, generator=g) / 128 ** 0.5).half().cuda()
    k = (torch.randn(1, 256, 2, 128, generator=g) / 128 ** 0.5).half().cuda()
    v = torch.randn(1, 256, 2, 128, generator=g).half().cuda()
    out = torch.empty(1, 256, 8, 128, dtype=torch.float16, device="cuda")
    nat.prefill_dense(q, k, v, 128 ** -0.5, out, None)
    n1 = nat.tensor_map_encodes()
    first = out.clone()
    for _ in range(3):
        nat.prefill_dense(q, k, v, 128 ** -0.5, out, None)
    torch.cuda.synchronize()
    assert nat.tensor_map_encodes() == n1, "the same layout was encoded again"
    assert torch.equal(out, first)
    q2 = q.clone()                                        # another pointer: one more descriptor (q), k and v cached
    nat.prefill_dense(q2, k, v, 128 ** -0.5, out, None)
    assert nat.tensor_map_encodes() == n1 + 1
