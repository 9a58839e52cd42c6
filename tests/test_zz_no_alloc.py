"""The allocation-free sparse-decode entry point against the regular one (GPU).

Some callers of the library cannot allocate device memory or pass a workspace (a server that gave all
HBM to its KV-cache pool, a plugin interface with inputs and outputs only).  For them
`kb200_decode_sparse_paged_noalloc` keeps its split partials in an array inside the library image.
This file checks, through the C ABI, that it returns what `kb200_decode_sparse_paged` returns — on two
calls in a row with different inputs, because every call reuses the same array and the second must
not see anything of the first — and that sizes beyond the built-in limit are rejected.  It is named so
that pytest collects it last."""
import pytest
import torch

from tests.gpu_util import assert_close, paged_from_contiguous

pytestmark = pytest.mark.gpu


def _problem(seed, B, G, L, kmax):
    g = torch.Generator().manual_seed(seed)
    H, D = 4 * G, 128
    q = (torch.randn(B, H, D, generator=g) / D ** 0.5).half().cuda()
    k = torch.randn(B, G, L, D, generator=g).half().cuda()
    v = torch.randn(B, G, L, D, generator=g).half().cuda()
    rows = torch.stack([torch.stack([torch.randperm(L, generator=g)[:kmax] for _ in range(G)]) for _ in range(B)])
    counts = torch.randint(kmax // 2, kmax + 1, (B, G), generator=g, dtype=torch.int32)
    head_map = torch.randint(0, G, (G,), generator=g, dtype=torch.int32)
    kc, vc, bt = paged_from_contiguous(k, v, seed=seed)
    return q, kc, vc, bt, rows.int().cuda().contiguous(), counts.cuda(), head_map.cuda()


def test_noalloc_matches_workspace_variant_twice_in_a_row():
    from kascade_b200 import _native as nat
    for call, (seed, splits) in enumerate([(101, 4), (202, 3)]):
        B, G, L, kmax = 4, 2, 3000, 1500
        q, kc, vc, bt, rows, counts, head_map = _problem(seed, B, G, L, kmax)
        kv = nat.kv_layout_paged(kc, vc, bt)
        H = 4 * G
        ref = torch.empty(B, H, 128, dtype=torch.float16, device="cuda")
        ref_lse = torch.empty(B, H, dtype=torch.float32, device="cuda")
        ws = nat.decode_workspace(B, H, splits, q.device)
        nat.decode_sparse_paged(q, kv, rows, counts, kmax, head_map, 0.25, ref, ref_lse, ws, splits)
        out = torch.full_like(ref, 9.0)
        lse = torch.zeros_like(ref_lse)
        nat.decode_sparse_paged_noalloc(q, kv, rows, counts, kmax, head_map, 0.25, out, lse, splits)
        torch.cuda.synchronize()
        assert_close(out, ref, what=f"no-alloc decode, call {call}")
        # with the same number of splits the two entry points run the same kernels on the same numbers
        assert torch.equal(out, ref), f"call {call}: outputs differ bit-wise at equal splits"
        assert torch.equal(lse, ref_lse), f"call {call}: lse differs bit-wise at equal splits"
        assert torch.isfinite(out.float()).all()


def test_noalloc_allocates_nothing_and_one_split_fits_any_batch():
    """A batch too large for two splits in the built-in array: the library's own choice (num_splits = 0) fits
    it, an explicit request for two splits is refused, one split needs no scratch and is accepted; the caching
    allocator's books do not move across the calls.  (On a 148-SM part the library's own choice is at most
    4 x 148 CTAs' worth of slots, so the "lower the choice until it fits" loop only matters on larger GPUs;
    kb200_decode_noalloc_splits exposes what it decides.)"""
    from kascade_b200 import _native as nat
    G, L, kmax = 2, 1100, 1024
    H = 4 * G
    B = 600                                            # 600 x 8 heads: 2 splits would need 9600 slots > 8192
    lib = nat.load()
    assert B * H * 2 > nat.NOALLOC_MAX_SLOTS
    chosen = lib.kb200_decode_noalloc_splits(B, H, G, kmax, 0)
    assert chosen >= 1 and (chosen == 1 or B * H * chosen <= nat.NOALLOC_MAX_SLOTS)
    assert chosen == 1, "600 x 2 CTAs already fill the GPU: one split expected"
    assert lib.kb200_decode_noalloc_splits(B, H, G, kmax, 2) == 0          # an explicit request is refused
    assert lib.kb200_decode_noalloc_splits(B, H, G, kmax, 1) == 1          # one split always fits
    q, kc, vc, bt, rows, counts, head_map = _problem(11, B, G, L, kmax)
    kv = nat.kv_layout_paged(kc, vc, bt)
    ref = torch.empty(B, H, 128, dtype=torch.float16, device="cuda")
    nat.decode_sparse_paged(q, kv, rows, counts, kmax, head_map, 0.25, ref, None, None, 1)
    out0 = torch.empty_like(ref)
    out1 = torch.empty_like(ref)
    nat.decode_sparse_paged_noalloc(q, kv, rows, counts, kmax, head_map, 0.25, out0, None, 0)   # warm: first call set-up
    torch.cuda.synchronize()
    before = (torch.cuda.memory_allocated(), torch.cuda.memory_reserved())
    n0 = nat.launch_count
    nat.decode_sparse_paged_noalloc(q, kv, rows, counts, kmax, head_map, 0.25, out0, None, 0)
    nat.decode_sparse_paged_noalloc(q, kv, rows, counts, kmax, head_map, 0.25, out1, None, 1)
    torch.cuda.synchronize()
    assert nat.launch_count - n0 == 2, "one kernel per call was expected (single split, no combine)"
    assert (torch.cuda.memory_allocated(), torch.cuda.memory_reserved()) == before
    assert torch.equal(out0, ref) and torch.equal(out1, ref)
    with pytest.raises(nat.KascadeNativeError, match="exceed the built-in scratch"):
        nat.decode_sparse_paged_noalloc(q, kv, rows, counts, kmax, head_map, 0.25, out1, None, 2)


def test_noalloc_default_splits_and_limit():
    from kascade_b200 import _native as nat
    B, G, L, kmax = 2, 2, 2000, 1200
    q, kc, vc, bt, rows, counts, head_map = _problem(7, B, G, L, kmax)
    kv = nat.kv_layout_paged(kc, vc, bt)
    H = 4 * G
    ref = torch.empty(B, H, 128, dtype=torch.float16, device="cuda")
    ws = nat.decode_workspace(B, H, 64, q.device)
    nat.decode_sparse_paged(q, kv, rows, counts, kmax, None, 0.25, ref, None, ws, 0)
    out = torch.empty_like(ref)
    nat.decode_sparse_paged_noalloc(q, kv, rows, counts, kmax, None, 0.25, out, None, 0)
    torch.cuda.synchronize()
    assert_close(out, ref, what="no-alloc decode, library-chosen splits")
    # beyond the built-in scratch: batch * heads * splits > NOALLOC_MAX_SLOTS must be refused, not truncated
    Bbig = nat.NOALLOC_MAX_SLOTS // (H * 2) + 1
    qbig = torch.zeros(Bbig, H, 128, dtype=torch.float16, device="cuda")
    rows_big = torch.zeros(Bbig, G, 16, dtype=torch.int32, device="cuda")
    bt_big = bt[:1].expand(Bbig, -1).contiguous()
    out_big = torch.empty(Bbig, H, 128, dtype=torch.float16, device="cuda")
    with pytest.raises(nat.KascadeNativeError, match="exceed the built-in scratch"):
        nat.decode_sparse_paged_noalloc(qbig, nat.kv_layout_paged(kc, vc, bt_big), rows_big, None, 16, None, 0.25,
                                        out_big, None, 2)
