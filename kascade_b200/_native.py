"""ctypes binding of libkascade_b200.so (the C ABI declared in include/kascade_b200.h).

The library is loaded from this package directory.  There is no fallback: if the shared object is
missing or a call is rejected, a ``KascadeNativeError`` is raised.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libkascade_b200.so")

HEAD_DIM = 128
GROUP_SIZE = 4
TILE = 32
FP16, BF16, FP8_E4M3 = 0, 1, 2        # KB200_FP16 / KB200_BF16 / KB200_FP8_E4M3
DTYPES = {torch.float16: FP16, torch.bfloat16: BF16}
FP8_TORCH = (torch.float8_e4m3fn, torch.uint8)   # an FP8 cache may be handed over as raw bytes

EXPORTS = [
    "kb200_init", "kb200_last_error", "kb200_abi_version", "kb200_topk_select",
    "kb200_decode_workspace_bytes", "kb200_decode_default_splits", "kb200_decode_sparse_paged",
    "kb200_decode_anchor_paged", "kb200_prefill_dense", "kb200_prefill_pool_scores",
    "kb200_prefill_sparse", "kb200_prefill_budgets", "kb200_selftest_umma", "kb200_read_status",
    "kb200_decode_sparse_paged_noalloc", "kb200_prefill_dense_fanout", "kb200_prefill_sparse_fanout",
    "kb200_kv_write", "kb200_prefill_dense_ragged", "kb200_prefill_pool_scores_ragged", "kb200_prefill_sparse_ragged",
    "kb200_prefill_budgets_ragged", "kb200_peer_push", "kb200_stream_wait_events", "kb200_selftest_wait_timeout", "kb200_tensor_map_encodes", "kb200_decode_noalloc_splits",
]


class KascadeNativeError(RuntimeError):
    pass


class KvLayout(C.Structure):
    _fields_ = [("k", C.c_void_p), ("v", C.c_void_p), ("stride_batch", C.c_int64),
                ("stride_page", C.c_int64), ("stride_token", C.c_int64), ("stride_head", C.c_int64),
                ("block_table", C.c_void_p), ("block_table_stride", C.c_int32),
                ("page_size", C.c_int32), ("dtype", C.c_int32),
                ("k_scale", C.c_void_p), ("v_scale", C.c_void_p), ("scale_stride_batch", C.c_int64),
                ("scale_stride_page", C.c_int64), ("scale_stride_head", C.c_int64)]


class ActLayout(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("stride_b", C.c_int64), ("stride_t", C.c_int64),
                ("stride_h", C.c_int64), ("dtype", C.c_int32)]


MAX_FANOUT = 8


class OutFanout(C.Structure):
    """kb200_out_fanout: the output rows of a call go into `count` buffers [B, L, total_heads, D]."""
    _fields_ = [("out", C.c_void_p * MAX_FANOUT), ("count", C.c_int32), ("total_heads", C.c_int32),
                ("head_offset", C.c_int32), ("multicast", C.c_int32)]


def out_fanout(pointers, total_heads: int, head_offset: int, multicast: bool = False) -> OutFanout:
    """pointers: device addresses (ints) of the [B, L, total_heads, D] fp16 buffers, own buffer first; with
    `multicast` a single NVLink multicast address that stands for the buffer on every GPU."""
    if not 1 <= len(pointers) <= MAX_FANOUT:
        raise KascadeNativeError(f"fan-out of {len(pointers)} outputs (1..{MAX_FANOUT} supported)")
    f = OutFanout()
    for i, ptr in enumerate(pointers):
        f.out[i] = int(ptr)
    f.count, f.total_heads, f.head_offset = len(pointers), int(total_heads), int(head_offset)
    f.multicast = 1 if multicast else 0
    if multicast and len(pointers) != 1:
        raise KascadeNativeError("a multicast fan-out takes exactly one address")
    return f


class Ragged(C.Structure):
    """kb200_ragged: per-sequence first row and length inside equally sized batch slots."""
    _fields_ = [("seq_start", C.c_void_p), ("seq_len", C.c_void_p)]


def ragged(seq_start: Optional[torch.Tensor], seq_len: torch.Tensor) -> Ragged:
    _want(seq_len, torch.int32, "seq_len")
    _want_opt(seq_start, torch.int32, "seq_start")
    return Ragged(0 if seq_start is None else seq_start.data_ptr(), seq_len.data_ptr())


class PushPlan(C.Structure):
    """kb200_push_plan: peers' buffers with one copy stream and one completion event per peer."""
    _fields_ = [("dst", C.c_void_p * MAX_FANOUT), ("stream", C.c_void_p * MAX_FANOUT),
                ("done_event", C.c_void_p * MAX_FANOUT), ("count", C.c_int32)]


_lib = None
_inited = set()
launch_count = 0          # kernels of this library launched so far by this process (host-side tally)


def _launched(n: int):
    global launch_count
    launch_count += n


def load() -> C.CDLL:
    """dlopen the library (no CUDA call is made)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise KascadeNativeError(
                f"{LIB_PATH} is missing: build it with `python -m kascade_b200.build` "
                "(there is no fallback implementation)")
        lib = C.CDLL(LIB_PATH)
        lib.kb200_last_error.restype = C.c_char_p
        lib.kb200_decode_workspace_bytes.restype = C.c_size_t
        lib.kb200_decode_workspace_bytes.argtypes = [C.c_int, C.c_int, C.c_int]
        lib.kb200_decode_default_splits.argtypes = [C.c_int, C.c_int, C.c_int]
        lib.kb200_init.argtypes = [C.c_int]
        vp, i64, i32, f32 = C.c_void_p, C.c_int64, C.c_int, C.c_float
        lib.kb200_topk_select.argtypes = [vp, i64, i32, vp, vp, i32, vp, i64, vp, i64, vp]
        lib.kb200_decode_sparse_paged.argtypes = [vp, i64, i64, C.POINTER(KvLayout), vp, i64, i64, vp,
                                                  i32, vp, f32, vp, vp, vp, C.c_size_t, i32, i32, i32,
                                                  i32, vp]
        lib.kb200_decode_sparse_paged_noalloc.argtypes = [vp, i64, i64, C.POINTER(KvLayout), vp, i64, i64, vp,
                                                          i32, vp, f32, vp, vp, i32, i32, i32, i32, vp]
        lib.kb200_decode_anchor_paged.argtypes = [vp, i64, i64, C.POINTER(KvLayout), vp, i32, f32, vp,
                                                  vp, i64, vp, vp, vp, C.c_size_t, i32, i32, i32, i32,
                                                  vp]
        AL = C.POINTER(ActLayout)
        lib.kb200_prefill_dense.argtypes = [AL, AL, AL, f32, vp, vp, i32, i32, i32, i32, vp]
        lib.kb200_prefill_pool_scores.argtypes = [AL, AL, vp, f32, vp, i64, i32, i32, i32, i32, vp]
        lib.kb200_prefill_sparse.argtypes = [AL, AL, AL, vp, i64, vp, vp, f32, vp, vp, i32, i32, i32,
                                             i32, i32, vp]
        FO = C.POINTER(OutFanout)
        lib.kb200_prefill_dense_fanout.argtypes = [AL, AL, AL, f32, FO, vp, i32, i32, i32, i32, vp]
        lib.kb200_prefill_sparse_fanout.argtypes = [AL, AL, AL, vp, i64, vp, vp, f32, FO, vp, i32, i32, i32,
                                                    i32, i32, vp]
        lib.kb200_prefill_budgets.argtypes = [vp, vp, i32, i32, i32, i32, f32, i32, vp]
        RG = C.POINTER(Ragged)
        lib.kb200_prefill_dense_ragged.argtypes = [AL, AL, AL, f32, vp, vp, RG, i32, i32, i32, i32, vp]
        lib.kb200_prefill_pool_scores_ragged.argtypes = [AL, AL, vp, f32, vp, i64, RG, i32, i32, i32, i32, vp]
        lib.kb200_prefill_sparse_ragged.argtypes = [AL, AL, AL, vp, i64, vp, vp, f32, vp, vp, RG, i32, i32, i32,
                                                    i32, i32, vp]
        lib.kb200_prefill_budgets_ragged.argtypes = [vp, vp, vp, i32, i32, i32, i32, f32, i32, vp]
        lib.kb200_kv_write.argtypes = [AL, vp, AL, AL, vp, vp, C.POINTER(KvLayout), vp, vp, f32, vp, f32, i32, i32,
                                       i32, i32, vp]
        lib.kb200_selftest_umma.argtypes = [vp, vp, vp, vp, vp]
        lib.kb200_peer_push.argtypes = [C.POINTER(PushPlan), vp, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, vp, vp]
        lib.kb200_stream_wait_events.argtypes = [vp, C.POINTER(C.c_void_p), i32]
        lib.kb200_selftest_wait_timeout.argtypes = [vp, C.c_uint64, i32, vp]
        lib.kb200_tensor_map_encodes.restype = C.c_longlong
        lib.kb200_tensor_map_encodes.argtypes = []
        lib.kb200_decode_noalloc_splits.argtypes = [i32, i32, i32, i32, i32]
        _lib = lib
    return _lib


def _check(rc: int, what: str):
    if rc != 0:
        raise KascadeNativeError(f"{what}: {load().kb200_last_error().decode()}")


def init(device: Optional[int] = None) -> C.CDLL:
    lib = load()
    if not torch.cuda.is_available():
        raise KascadeNativeError("kascade_b200 needs a CUDA device (sm_100a); none is visible")
    dev = torch.cuda.current_device() if device is None else int(device)
    if dev not in _inited:
        _check(lib.kb200_init(dev), "kb200_init")
        _inited.add(dev)
    return lib


def read_status(device=None) -> int:
    """Status word of `device` (default: the current one); 0 = every kernel ran to completion.  Reading
    clears it.  Synchronises the device."""
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    with torch.cuda.device(dev):
        out = C.c_int(0)
        _check(init(dev).kb200_read_status(C.byref(out)), "kb200_read_status")
    return out.value


def check_status(device=None, where: str = ""):
    """Raise if a kernel of this library gave up a bounded wait on `device` since the last check: its
    outputs (and those of every later tile-prefill launch, which return at entry while the word is set) are
    not valid.  Call it where the host synchronises anyway."""
    st = read_status(device)
    if st != 0:
        raise KascadeNativeError(f"a kernel gave up a bounded device-side wait (code {st}){' ' + where if where else ''}; "
                                 "outputs since the last status check are invalid")


def _on_device_of(arg_index: int):
    """Decorator: run the wrapped call with the GPU of its `arg_index`-th argument (a tensor) current.  The
    library launches on the current device, on the current stream of that device, and keeps its per-device
    state (kernel attributes, the built-in decode scratch) by it; without this a caller whose current device
    differs from the tensors' would launch on the wrong GPU."""
    def deco(fn):
        import functools

        @functools.wraps(fn)
        def wrapped(*args, **kwargs):
            t = args[arg_index]
            if not t.is_cuda:
                raise KascadeNativeError(f"{fn.__name__}: expected CUDA tensors, got one on {t.device}")
            if t.device.index == torch.cuda.current_device():
                return fn(*args, **kwargs)
            with torch.cuda.device(t.device):
                return fn(*args, **kwargs)
        return wrapped
    return deco


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> C.c_void_p:
    return C.c_void_p(0 if t is None else t.data_ptr())


def _want_opt(t: Optional[torch.Tensor], dtype, name: str):
    if t is not None:
        _want(t, dtype, name)


def _want(t: torch.Tensor, dtype, name: str):
    if t.dtype != dtype or not t.is_cuda:
        raise KascadeNativeError(f"{name}: expected a CUDA {dtype} tensor, got {t.dtype} on {t.device}")


def _half_code(t: torch.Tensor, name: str) -> int:
    """KB200_FP16 / KB200_BF16 of a CUDA fp16 or bf16 tensor."""
    if t.dtype not in DTYPES or not t.is_cuda:
        raise KascadeNativeError(f"{name}: expected a CUDA fp16 or bf16 tensor, got {t.dtype} on {t.device}")
    return DTYPES[t.dtype]


# ------------------------------------------------------------------------------------------------
@_on_device_of(0)
def topk_select(scores: torch.Tensor, n_valid: Optional[torch.Tensor], k_row: Optional[torch.Tensor],
                k_max: int, out_idx: torch.Tensor, out_count: Optional[torch.Tensor], n_cols: Optional[int] = None):
    """scores [..., row_stride] fp32 (last dim contiguous, rows equally spaced), out_idx [..., idx_stride]."""
    lib = init(scores.device.index)
    _want(scores, torch.float32, "scores")
    _want(out_idx, torch.int32, "out_idx")
    rows = scores.numel() // scores.shape[-1]
    assert scores.is_contiguous() and out_idx.is_contiguous()
    _check(lib.kb200_topk_select(_ptr(scores), scores.shape[-1], scores.shape[-1] if n_cols is None else n_cols,
                                 _ptr(n_valid), _ptr(k_row), k_max, _ptr(out_idx), out_idx.shape[-1],
                                 _ptr(out_count), rows, _stream()), "kb200_topk_select")
    _launched(1 if rows else 0)


@_on_device_of(0)
def prefill_budgets(n_valid, k_row, batch, groups, tiles, k_max, pct, rolling):
    lib = init(n_valid.device.index)
    _check(lib.kb200_prefill_budgets(_ptr(n_valid), _ptr(k_row), batch, groups, tiles, k_max, float(pct),
                                     int(bool(rolling)), _stream()), "kb200_prefill_budgets")
    _launched(1)


@_on_device_of(0)
def prefill_budgets_ragged(n_valid, k_row, seq_len, batch, groups, tiles, k_cap, pct, rolling):
    lib = init(n_valid.device.index)
    _want(seq_len, torch.int32, "seq_len")
    _check(lib.kb200_prefill_budgets_ragged(_ptr(n_valid), _ptr(k_row), _ptr(seq_len), batch, groups, tiles, k_cap,
                                            float(pct), int(bool(rolling)), _stream()), "kb200_prefill_budgets_ragged")
    _launched(1)


def _fp8_scales(k_scale, v_scale, need_v: bool):
    if k_scale is None or (need_v and v_scale is None):
        raise KascadeNativeError("an FP8 cache needs k_scale (and v_scale): one fp32 scale per (page, KV head)")
    _want(k_scale, torch.float32, "k_scale")
    _want_opt(v_scale, torch.float32, "v_scale")
    if v_scale is not None and (v_scale.shape != k_scale.shape or v_scale.stride() != k_scale.stride()):
        raise KascadeNativeError("k_scale and v_scale must have the same shape and strides")


def _holding(layout, *tensors):
    """The layouts carry raw device addresses: keep the tensors alive as long as the layout object is."""
    layout._keep = tuple(t for t in tensors if t is not None)
    return layout


def kv_layout_paged(k_cache: torch.Tensor, v_cache: Optional[torch.Tensor], block_table: torch.Tensor,
                    k_scale: Optional[torch.Tensor] = None, v_scale: Optional[torch.Tensor] = None) -> KvLayout:
    """vLLM-style cache [num_pages, page_size, G, D] and block table [B, max_pages] int32.  An FP8 cache
    (torch.float8_e4m3fn or raw uint8) comes with k_scale / v_scale [num_pages, G] fp32."""
    if k_cache.dtype in FP8_TORCH:
        assert k_cache.is_cuda and k_cache.dim() == 4 and k_cache.stride(3) == 1
        assert block_table.dtype == torch.int32 and block_table.stride(1) == 1
        if v_cache is not None:
            assert v_cache.shape == k_cache.shape and v_cache.stride() == k_cache.stride() and v_cache.dtype == k_cache.dtype
        _fp8_scales(k_scale, v_scale, v_cache is not None)
        assert k_scale.shape == (k_cache.shape[0], k_cache.shape[2])
        return _holding(KvLayout(k_cache.data_ptr(), 0 if v_cache is None else v_cache.data_ptr(), 0, k_cache.stride(0),
                                 k_cache.stride(1), k_cache.stride(2), block_table.data_ptr(), block_table.stride(0),
                                 k_cache.shape[1], FP8_E4M3, k_scale.data_ptr(),
                                 0 if v_scale is None else v_scale.data_ptr(), 0, k_scale.stride(0), k_scale.stride(1)),
                        k_cache, v_cache, block_table, k_scale, v_scale)
    code = _half_code(k_cache, "k_cache")
    assert k_cache.dim() == 4 and k_cache.stride(3) == 1
    assert block_table.dtype == torch.int32 and block_table.stride(1) == 1
    if v_cache is not None:
        assert v_cache.shape == k_cache.shape and v_cache.stride() == k_cache.stride() and v_cache.dtype == k_cache.dtype
    return _holding(KvLayout(k_cache.data_ptr(), 0 if v_cache is None else v_cache.data_ptr(), 0, k_cache.stride(0),
                             k_cache.stride(1), k_cache.stride(2), block_table.data_ptr(), block_table.stride(0),
                             k_cache.shape[1], code), k_cache, v_cache, block_table)


def kv_layout_contiguous(k: torch.Tensor, v: Optional[torch.Tensor], page_size: int = 16,
                         k_scale: Optional[torch.Tensor] = None, v_scale: Optional[torch.Tensor] = None) -> KvLayout:
    """HF cache view [B, G, L, D] (any batch / head / token strides, D contiguous).  An FP8 cache comes with
    k_scale / v_scale [B, G, ceil(L / page_size)] fp32."""
    if k.dtype in FP8_TORCH:
        assert k.is_cuda and k.dim() == 4 and k.stride(3) == 1
        if v is not None:
            assert v.shape == k.shape and v.stride() == k.stride() and v.dtype == k.dtype
        _fp8_scales(k_scale, v_scale, v is not None)
        assert k_scale.dim() == 3 and k_scale.shape[:2] == k.shape[:2]
        return _holding(KvLayout(k.data_ptr(), 0 if v is None else v.data_ptr(), k.stride(0), k.stride(2) * page_size,
                                 k.stride(2), k.stride(1), 0, 0, page_size, FP8_E4M3, k_scale.data_ptr(),
                                 0 if v_scale is None else v_scale.data_ptr(), k_scale.stride(0), k_scale.stride(2),
                                 k_scale.stride(1)), k, v, k_scale, v_scale)
    code = _half_code(k, "k")
    assert k.dim() == 4 and k.stride(3) == 1
    if v is not None:
        assert v.shape == k.shape and v.stride() == k.stride() and v.dtype == k.dtype
    return _holding(KvLayout(k.data_ptr(), 0 if v is None else v.data_ptr(), k.stride(0), k.stride(2) * page_size,
                             k.stride(2), k.stride(1), 0, 0, page_size, code), k, v)


def kv_layout_rows(k: torch.Tensor, v: Optional[torch.Tensor], row_table: torch.Tensor) -> KvLayout:
    """HF cache view [B, G, L, D] whose sequences do not start at row 0 (a padded batch): row_table [B, n] int32 gives
    the cache row of every logical position - a block table with one-token pages, which the decode kernels already
    know how to walk."""
    code = _half_code(k, "k")
    assert k.dim() == 4 and k.stride(3) == 1
    assert row_table.dtype == torch.int32 and row_table.dim() == 2 and row_table.stride(1) == 1
    if v is not None:
        assert v.shape == k.shape and v.stride() == k.stride() and v.dtype == k.dtype
    return _holding(KvLayout(k.data_ptr(), 0 if v is None else v.data_ptr(), k.stride(0), k.stride(2), k.stride(2),
                             k.stride(1), row_table.data_ptr(), row_table.stride(0), 1, code), k, v, row_table)


def decode_workspace(batch: int, heads: int, splits: int, device) -> torch.Tensor:
    n = load().kb200_decode_workspace_bytes(batch, heads, splits)
    return torch.empty(max(n, 16), dtype=torch.uint8, device=device)


def decode_default_splits(batch: int, groups: int, max_keys: int) -> int:
    init()
    return load().kb200_decode_default_splits(batch, groups, max_keys)


@_on_device_of(0)
def decode_sparse_paged(q, kv: KvLayout, topk_idx, topk_count, k_max, head_map, scale, out, lse2=None,
                        workspace=None, num_splits=0):
    """q [B,H,D] fp16; topk_idx [B,G,kstride] int32; out [B,H,D] fp16 contiguous."""
    lib = init(q.device.index)
    if _half_code(q, "q") != (FP16 if kv.dtype == FP8_E4M3 else kv.dtype):
        raise KascadeNativeError(f"q is {q.dtype} but the KV cache has dtype code {kv.dtype} (an FP8 cache takes fp16 q)")
    _want(out, q.dtype, "out")
    _want(topk_idx, torch.int32, "topk_idx")
    _want_opt(topk_count, torch.int32, "topk_count")
    _want_opt(head_map, torch.int32, "head_map")
    B, H, D = q.shape
    G = topk_idx.shape[1]
    assert D == HEAD_DIM and q.stride(2) == 1 and out.is_contiguous() and topk_idx.stride(2) == 1
    _check(lib.kb200_decode_sparse_paged(
        _ptr(q), q.stride(0), q.stride(1), C.byref(kv), _ptr(topk_idx), topk_idx.stride(0), topk_idx.stride(1),
        _ptr(topk_count), k_max, _ptr(head_map), float(scale), _ptr(out), _ptr(lse2), _ptr(workspace),
        0 if workspace is None else workspace.numel() * workspace.element_size(), B, H, G, num_splits, _stream()),
        "kb200_decode_sparse_paged")
    ns = num_splits if num_splits else lib.kb200_decode_default_splits(B, G, k_max)
    _launched(1 + (ns > 1))


NOALLOC_MAX_SLOTS = 8192


@_on_device_of(0)
def decode_sparse_paged_noalloc(q, kv: KvLayout, topk_idx, topk_count, k_max, head_map, scale, out, lse2=None,
                                num_splits=0):
    """Same result as decode_sparse_paged, for callers that cannot allocate or pass a workspace: the split
    partials live in a fixed array inside the library (batch * heads * splits <= NOALLOC_MAX_SLOTS).
    Calls that overlap on the GPU race on that array; the first call on a device belongs in set-up."""
    lib = init(q.device.index)
    if _half_code(q, "q") != (FP16 if kv.dtype == FP8_E4M3 else kv.dtype):
        raise KascadeNativeError(f"q is {q.dtype} but the KV cache has dtype code {kv.dtype} (an FP8 cache takes fp16 q)")
    _want(out, q.dtype, "out")
    _want(topk_idx, torch.int32, "topk_idx")
    _want_opt(topk_count, torch.int32, "topk_count")
    _want_opt(head_map, torch.int32, "head_map")
    B, H, D = q.shape
    G = topk_idx.shape[1]
    assert D == HEAD_DIM and q.stride(2) == 1 and out.is_contiguous() and topk_idx.stride(2) == 1
    _check(lib.kb200_decode_sparse_paged_noalloc(
        _ptr(q), q.stride(0), q.stride(1), C.byref(kv), _ptr(topk_idx), topk_idx.stride(0), topk_idx.stride(1),
        _ptr(topk_count), k_max, _ptr(head_map), float(scale), _ptr(out), _ptr(lse2), B, H, G, num_splits,
        _stream()), "kb200_decode_sparse_paged_noalloc")
    _launched(2 if lib.kb200_decode_noalloc_splits(B, H, G, k_max, num_splits) > 1 else 1)


@_on_device_of(0)
def decode_anchor_paged(q, kv: KvLayout, seq_lens, max_seq_len, scale, logits, pooled, out, lse2,
                        workspace=None, num_splits=0):
    """q [B,H,D]; logits [B,H,stride] fp32; pooled [B,G,stride] fp32; out [B,H,D] fp16 or None."""
    lib = init(q.device.index)
    if _half_code(q, "q") != (FP16 if kv.dtype == FP8_E4M3 else kv.dtype):
        raise KascadeNativeError(f"q is {q.dtype} but the KV cache has dtype code {kv.dtype} (an FP8 cache takes fp16 q)")
    _want_opt(out, q.dtype, "out")
    _want(logits, torch.float32, "logits")
    _want(pooled, torch.float32, "pooled")
    B, H, D = q.shape
    G = pooled.shape[1]
    assert logits.is_contiguous() and pooled.is_contiguous() and logits.shape[-1] == pooled.shape[-1]
    _check(lib.kb200_decode_anchor_paged(
        _ptr(q), q.stride(0), q.stride(1), C.byref(kv), _ptr(seq_lens), max_seq_len, float(scale), _ptr(logits),
        _ptr(pooled), logits.shape[-1], _ptr(out), _ptr(lse2), _ptr(workspace),
        0 if workspace is None else workspace.numel() * workspace.element_size(), B, H, G, num_splits, _stream()),
        "kb200_decode_anchor_paged")
    ns = num_splits if num_splits else lib.kb200_decode_default_splits(B, G, max_seq_len)
    _launched(2 + (ns > 1))


def act_layout(x: torch.Tensor) -> ActLayout:
    """x indexed [B, L, heads, D] (any strides, D contiguous)."""
    code = _half_code(x, "activation")
    assert x.dim() == 4 and x.stride(3) == 1 and x.shape[3] == HEAD_DIM
    return ActLayout(x.data_ptr(), x.stride(0), x.stride(1), x.stride(2), code)


@_on_device_of(0)
def prefill_dense(q, k, v, scale, out, lse2, fanout: Optional[OutFanout] = None, ragged: Optional[Ragged] = None):
    """q [B,L,H,D], k/v [B,L,G,D] (views allowed); out [B,L,H,D] fp16 contiguous or None; lse2 [B,L,H] fp32 or None.
    With `fanout` (see out_fanout) the rows go into several [B,L,total_heads,D] buffers instead of `out`; with
    `ragged` (see ragged()) every sequence has its own first row and length inside its slot of L rows."""
    lib = init(q.device.index)
    B, L, H, _ = q.shape
    G = k.shape[2]
    ql, kl = act_layout(q), act_layout(k)
    vl = act_layout(v) if v is not None else ActLayout(0, 0, 0, 0, 0)
    if ragged is not None:
        if out is not None:
            _want(out, q.dtype, "out")
            assert out.is_contiguous()
        _check(lib.kb200_prefill_dense_ragged(C.byref(ql), C.byref(kl), C.byref(vl), float(scale), _ptr(out), _ptr(lse2),
                                              C.byref(ragged), B, L, H, G, _stream()), "kb200_prefill_dense_ragged")
        _launched(1)
        return
    if fanout is not None:
        _check(lib.kb200_prefill_dense_fanout(C.byref(ql), C.byref(kl), C.byref(vl), float(scale), C.byref(fanout),
                                              _ptr(lse2), B, L, H, G, _stream()), "kb200_prefill_dense_fanout")
        _launched(1)
        return
    if out is not None:
        _want(out, q.dtype, "out")
        assert out.is_contiguous()
    _check(lib.kb200_prefill_dense(C.byref(ql), C.byref(kl), C.byref(vl), float(scale), _ptr(out), _ptr(lse2),
                                   B, L, H, G, _stream()), "kb200_prefill_dense")
    _launched(1)


@_on_device_of(0)
def prefill_pool_scores(q, k, lse2, scale, pooled, ragged: Optional[Ragged] = None):
    """pooled [B,G,T,row_stride] fp32 contiguous."""
    lib = init(q.device.index)
    B, L, H, _ = q.shape
    G = k.shape[2]
    ql, kl = act_layout(q), act_layout(k)
    _want(pooled, torch.float32, "pooled")
    _want(lse2, torch.float32, "lse2")
    assert pooled.is_contiguous() and lse2.is_contiguous()
    if ragged is not None:
        _check(lib.kb200_prefill_pool_scores_ragged(C.byref(ql), C.byref(kl), _ptr(lse2), float(scale), _ptr(pooled),
                                                    pooled.shape[-1], C.byref(ragged), B, L, H, G, _stream()),
               "kb200_prefill_pool_scores_ragged")
        _launched(1)
        return
    _check(lib.kb200_prefill_pool_scores(C.byref(ql), C.byref(kl), _ptr(lse2), float(scale), _ptr(pooled),
                                         pooled.shape[-1], B, L, H, G, _stream()), "kb200_prefill_pool_scores")
    _launched(1)


@_on_device_of(0)
def prefill_sparse(q, k, v, tile_idx, tile_count, head_map, scale, out, lse2=None, fanout: Optional[OutFanout] = None,
                   ragged: Optional[Ragged] = None):
    """tile_idx [B,G,T,kstride] int32, tile_count [B,G,T] int32, out [B,L,H,D] fp16 contiguous.
    With `fanout` (see out_fanout) the rows go into several [B,L,total_heads,D] buffers instead of `out`."""
    lib = init(q.device.index)
    B, L, H, _ = q.shape
    G = k.shape[2]
    ql, kl, vl = act_layout(q), act_layout(k), act_layout(v)
    _want(tile_idx, torch.int32, "tile_idx")
    _want(tile_count, torch.int32, "tile_count")
    _want_opt(head_map, torch.int32, "head_map")
    assert tile_idx.is_contiguous() and tile_count.is_contiguous()
    if fanout is not None:
        _check(lib.kb200_prefill_sparse_fanout(C.byref(ql), C.byref(kl), C.byref(vl), _ptr(tile_idx),
                                               tile_idx.shape[-1], _ptr(tile_count), _ptr(head_map), float(scale),
                                               C.byref(fanout), _ptr(lse2), B, L, H, G, tile_idx.shape[1],
                                               _stream()), "kb200_prefill_sparse_fanout")
        _launched(1)
        return
    _want(out, q.dtype, "out")
    assert out.is_contiguous()
    if ragged is not None:
        _check(lib.kb200_prefill_sparse_ragged(C.byref(ql), C.byref(kl), C.byref(vl), _ptr(tile_idx), tile_idx.shape[-1],
                                               _ptr(tile_count), _ptr(head_map), float(scale), _ptr(out), _ptr(lse2),
                                               C.byref(ragged), B, L, H, G, tile_idx.shape[1], _stream()),
               "kb200_prefill_sparse_ragged")
        _launched(1)
        return
    _check(lib.kb200_prefill_sparse(C.byref(ql), C.byref(kl), C.byref(vl), _ptr(tile_idx), tile_idx.shape[-1],
                                    _ptr(tile_count), _ptr(head_map), float(scale), _ptr(out), _ptr(lse2), B, L, H,
                                    G, tile_idx.shape[1], _stream()), "kb200_prefill_sparse")
    _launched(1)


@_on_device_of(2)
def kv_write(q_in, q_out, k_new, v_new, start_pos, n_new, kv: KvLayout, q_gain=None, k_gain=None, eps=1e-6,
             inv_freq=None, rope_scale=1.0):
    """q_in [B,T,H,D] (or None), k_new / v_new [B,T,G,D] views, all fp16 or all bf16 like the cache and the gains;
    start_pos [B] int32; n_new [B] int32 or None; kv: the cache to append to (kv_layout_paged /
    kv_layout_contiguous); inv_freq [D/2] fp32 or None."""
    lib = init(k_new.device.index)
    B, T, G, _ = k_new.shape
    kl, vl = act_layout(k_new), act_layout(v_new)
    ql = act_layout(q_in) if q_in is not None else ActLayout(0, 0, 0, 0, 0)
    H = q_in.shape[2] if q_in is not None else 0
    if q_in is not None:
        _want(q_out, k_new.dtype, "q_out")
        assert q_out.is_contiguous() and q_out.shape == q_in.shape
    _want(start_pos, torch.int32, "start_pos")
    _want_opt(n_new, torch.int32, "n_new")
    _want_opt(q_gain, k_new.dtype, "q_gain")
    _want_opt(k_gain, k_new.dtype, "k_gain")
    if inv_freq is not None:
        _want(inv_freq, torch.float32, "inv_freq")
        assert inv_freq.is_contiguous() and inv_freq.numel() == HEAD_DIM // 2
    _check(lib.kb200_kv_write(C.byref(ql), _ptr(q_out), C.byref(kl), C.byref(vl), _ptr(start_pos), _ptr(n_new),
                              C.byref(kv), _ptr(q_gain), _ptr(k_gain), float(eps), _ptr(inv_freq), float(rope_scale),
                              B, T, H, G, _stream()), "kb200_kv_write")
    _launched(1)


@_on_device_of(0)
def selftest_umma(a: torch.Tensor, b: torch.Tensor):
    lib = init(a.device.index)
    out = torch.zeros(4, 128, 128, dtype=torch.float32, device=a.device)
    status = torch.full((4,), -1, dtype=torch.int32, device=a.device)
    _check(lib.kb200_selftest_umma(_ptr(a), _ptr(b), _ptr(out), _ptr(status), _stream()), "kb200_selftest_umma")
    return out, status


def selftest_wait_timeout(device, limit_ns: int = 1_000_000, code: int = 77) -> torch.Tensor:
    """Runs the wait-that-runs-out selftest on `device`; returns [code, threads that gave up, elapsed ns].
    The device status word then holds `code` until read_status() / check_status() clears it."""
    result = torch.zeros(3, dtype=torch.int32, device=device)
    with torch.cuda.device(result.device):
        lib = init(result.device.index)
        _check(lib.kb200_selftest_wait_timeout(_ptr(result), int(limit_ns), int(code), _stream()),
               "kb200_selftest_wait_timeout")
    _launched(1)
    return result


def tensor_map_encodes() -> int:
    return int(load().kb200_tensor_map_encodes())


def _cuda_event(ev: torch.cuda.Event) -> int:
    """cudaEvent_t of a torch event (torch creates it lazily, at the first record)."""
    if not ev.cuda_event:
        ev.record()
    return int(ev.cuda_event)


def push_plan(dst_pointers, streams, done_events) -> PushPlan:
    """One entry per peer: device address of its buffer, a torch stream for the copy, a torch event."""
    if not (len(dst_pointers) == len(streams) == len(done_events)) or len(dst_pointers) > MAX_FANOUT:
        raise KascadeNativeError("push_plan: one stream and one event per peer, at most %d peers" % MAX_FANOUT)
    plan = PushPlan()
    for i, (ptr, st, ev) in enumerate(zip(dst_pointers, streams, done_events)):
        plan.dst[i], plan.stream[i], plan.done_event[i] = int(ptr), int(st.cuda_stream), _cuda_event(ev)
    plan.count = len(dst_pointers)
    return plan


def peer_push(plan: PushPlan, src: torch.Tensor, offset_bytes: int, pitch_bytes: int, width_bytes: int, rows: int,
              ready_event: torch.cuda.Event):
    """Copy the row slice [offset, offset + width) of every `pitch`-byte row of `src` into the peers' buffers with
    the copy engines, after everything queued on the current stream (see kb200_peer_push)."""
    with torch.cuda.device(src.device):
        _check(load().kb200_peer_push(C.byref(plan), _ptr(src), offset_bytes, pitch_bytes, width_bytes, rows,
                                      C.c_void_p(_cuda_event(ready_event)), _stream()), "kb200_peer_push")


def stream_wait_events(events):
    """Make the current stream wait for the given torch events (those already recorded)."""
    handles = [int(e.cuda_event) for e in events if e.cuda_event]
    if handles:
        arr = (C.c_void_p * len(handles))(*handles)
        _check(load().kb200_stream_wait_events(_stream(), arr, len(handles)), "kb200_stream_wait_events")
