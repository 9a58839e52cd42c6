"""Helpers shared by the GPU parity tests."""
import torch


def paged_from_contiguous(k, v, page_size=16, seed=0, extra_pages=3):
    """k, v [B,G,L,D] fp16 (cuda) -> (k_cache, v_cache [P,page,G,D], block_table [B,pages] int32) with a
    seeded random permutation of the physical pages."""
    B, G, L, D = k.shape
    npg = -(-L // page_size)
    total = B * npg + extra_pages
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(total, generator=g)[: B * npg].view(B, npg)
    k_cache = torch.randn(total, page_size, G, D, generator=g).to(k.dtype).to(k.device)
    v_cache = torch.randn(total, page_size, G, D, generator=g).to(k.dtype).to(k.device)
    pad = npg * page_size - L
    kp = torch.nn.functional.pad(k, (0, 0, 0, pad)).view(B, G, npg, page_size, D).permute(0, 2, 3, 1, 4)
    vp = torch.nn.functional.pad(v, (0, 0, 0, pad)).view(B, G, npg, page_size, D).permute(0, 2, 3, 1, 4)
    flat = perm.to(k.device).view(-1)
    k_cache[flat] = kp.reshape(B * npg, page_size, G, D)
    v_cache[flat] = vp.reshape(B * npg, page_size, G, D)
    return k_cache, v_cache, perm.to(torch.int32).to(k.device).contiguous()


def assert_close(got, ref, atol=2e-3, rtol=1e-2, what=""):
    """max-abs 2e-3 / rel 1e-2: the fp16-storage, fp32-accumulate tolerance of the parity contract."""
    got = got.float().cpu()
    ref = ref.float().cpu()
    diff = (got - ref).abs()
    bound = atol + rtol * ref.abs()
    bad = diff > bound
    assert not bool(bad.any()), (f"{what}: {int(bad.sum())} elements out of tolerance, max abs diff "
                                 f"{diff.max().item():.3e} (ref magnitude {ref.abs().max().item():.3e})")
    return diff.max().item()
