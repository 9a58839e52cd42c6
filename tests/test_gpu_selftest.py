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
