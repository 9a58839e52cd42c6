"""Host-side logic and the C-ABI surface, without a GPU."""
import os
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from kascade_b200 import _native as nat
    lib = nat.load()                                   # dlopen only: no CUDA call
    header = open(os.path.join(ROOT, "include", "kascade_b200.h")).read()
    declared = sorted(set(re.findall(r"\b(kb200_[a-z0-9_]+)\s*\(", header)))
    assert len(declared) >= 14
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/kascade_b200.h but not exported"
    assert sorted(nat.EXPORTS) == [d for d in declared if d in nat.EXPORTS]
    assert set(declared) <= set(nat.EXPORTS), set(declared) - set(nat.EXPORTS)
    assert lib.kb200_abi_version() == 2          # 2: the layouts carry a dtype field (fp16 / bf16)
    assert lib.kb200_decode_workspace_bytes(64, 32, 2) == 64 * 32 * 2 * 130 * 4


def test_calls_fail_loudly_without_a_gpu():
    from kascade_b200 import _native as nat
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    with pytest.raises(nat.KascadeNativeError):
        nat.init()
    # the C side refuses to launch before kb200_init
    lib = nat.load()
    assert lib.kb200_topk_select(None, 0, 0, None, None, 0, None, 0, None, 0, None) != 0
    assert b"kb200_init" in lib.kb200_last_error()


def test_budget_matches_reference_formula():
    from kascade_b200 import topk_budget
    from oracle.kascade_oracle import topk_budget as oracle_budget
    for lk in (129, 200, 1280, 2048, 2049, 32768, 131072):
        for pct in (10, 20, 50):
            assert topk_budget(pct, lk, 32) == oracle_budget(pct, lk, 32)


def test_strategy_constructor_contract(tmp_path, monkeypatch):
    from kascade_b200 import EfficientKascadeStrategy
    monkeypatch.chdir(tmp_path)
    with pytest.raises(ValueError, match="Head mapping file not found"):
        EfficientKascadeStrategy([0, 2], "org/some-model", k=10, tile_size=32, register=False)
    os.makedirs("results/head_mappings")
    hm = np.stack([np.arange(8), np.zeros(8), np.arange(8), np.array([1, 1, 1, 1, 1, 1, 4, 1])]).astype(np.int32)
    np.save("results/head_mappings/some-model_layers_0_2.npy", hm)
    s = EfficientKascadeStrategy([0, 2], "org/some-model", k=10, tile_size=32, rolling_prefill=True, register=False)
    assert s.name == "efficient_kascade"
    assert s._head_mapping == hm.tolist()
    assert s.is_anchor(0) and s.is_anchor(2) and not s.is_anchor(1)
    with pytest.raises(ValueError):
        EfficientKascadeStrategy([0], "org/some-model", k=10, tile_size=16, register=False)
    with pytest.raises(AssertionError):
        EfficientKascadeStrategy([0], "org/some-model", k=101, tile_size=32, register=False)
    with pytest.raises(ValueError):
        EfficientKascadeStrategy(None, "org/some-model", k=10, tile_size=32, register=False)


def test_registers_in_hf_registries():
    from transformers.masking_utils import ALL_MASK_ATTENTION_FUNCTIONS
    from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS
    from kascade_b200 import EfficientKascadeStrategy
    s = EfficientKascadeStrategy([0], "x/y", k=10, tile_size=32, head_mapping=[list(range(8))] * 2)
    assert s.name in ALL_ATTENTION_FUNCTIONS.valid_keys()
    assert s.name in ALL_MASK_ATTENTION_FUNCTIONS.valid_keys()


def test_shard_helpers():
    from kascade_b200.strategy import shard_head_map, shard_kv_heads
    assert shard_kv_heads(8, 1, 4) == [2, 3]
    assert shard_head_map([7, 1, 5, 6, 3, 3, 3, 3], 3, 4) == [3, 3]
    assert shard_head_map([7, 1, 5, 6, 3, 3, 3, 3], 0, 2) == [7, 1, 5, 6]
    with pytest.raises(ValueError):
        shard_kv_heads(8, 0, 3)


def test_workload_accounting():
    from bench_workloads import DecodeWorkload, PrefillWorkload
    wl = PrefillWorkload()
    assert abs(wl.flops_dense() / 1e12 - 8.796) < 0.01
    assert abs(wl.flops_sparse() / 1e12 - 0.897) < 0.01
    assert abs(wl.flops_stack() / 1e12 - 76.2) < 0.2
    dw = DecodeWorkload()
    assert dw.budget() == 3244
    assert abs(dw.bytes_dense_k() / 1e9 - 4.295) < 0.01


def test_ragged_decode_workload_accounting():
    """The long-reasoning decode configuration: 256 seeded contexts in [4096, 65536], batch-sharded round-robin;
    algorithmic bytes are sums over the sequences (budgets follow the reference's formula per sequence)."""
    from kascade_b200.strategy import topk_budget
    from bench_workloads import DecodeWorkload
    whole = DecodeWorkload.ragged()
    assert whole.batch == 256 and min(whole.contexts) >= 4096 and max(whole.contexts) <= 65536
    assert whole.context == max(whole.contexts)
    parts = [DecodeWorkload.ragged(rank=r, world=4) for r in range(4)]
    assert sorted(sum((list(p.contexts) for p in parts), [])) == sorted(whole.contexts)
    assert abs(sum(p.bytes_step() for p in parts) - whole.bytes_step()) < 1e-6 * whole.bytes_step()
    keys = sum(topk_budget(10, n, 32) for n in whole.contexts)
    assert whole.bytes_reuse() == 8 * keys * (2 * 128 * 2 + 4) + 2 * 256 * 32 * 128 * 2
    uniform = DecodeWorkload()
    assert uniform.seq_lens() == [32768] * 64
    assert uniform.bytes_dense_k() == 64 * 8 * 32768 * 128 * 2


def test_long_prompt_workload_is_normalised():
    from bench_workloads import PrefillWorkload, QWEN3_ANCHORS
    wl = PrefillWorkload(seq_len=256, layers=36, anchors=QWEN3_ANCHORS, qk_norm=True)
    q, k, v = wl.layer_inputs(3, "cpu")
    rms_q = q.float().pow(2).mean(-1).sqrt()
    rms_k = k.float().pow(2).mean(-1).sqrt()
    assert (rms_q - 1).abs().max() < 5e-3 and (rms_k - 1).abs().max() < 5e-3
    hm = wl.head_mapping()
    assert len(hm) == 36 and all(hm[a] == list(range(8)) for a in QWEN3_ANCHORS)


def test_padding_is_read_from_the_last_mask_row():
    """Left / right / mixed padding of a batch, additive and boolean masks, from the key columns the last query row
    may see (host logic only: no kernel runs)."""
    import torch
    from kascade_b200 import EfficientKascadeStrategy
    s = EfficientKascadeStrategy([0], "x/y", k=10, tile_size=32, head_mapping=[list(range(8))] * 2, register=False)
    L = 48
    ok = torch.tril(torch.ones(L, L, dtype=torch.bool))[None].repeat(3, 1, 1)
    ok[1, :, :7] = False                       # 7 padded positions on the left
    ok[2, :, L - 5:] = False                   # 5 on the right
    ok[2, :, :2] = False                       # and 2 on the left
    additive = torch.zeros(3, 1, L, L).masked_fill_(~ok[:, None], torch.finfo(torch.float32).min)
    assert s._padding(additive, 3, L) == ([0, 7, 2], [48, 41, 41])
    assert s._padding(ok[:, None].clone(), 3, L) == ([0, 7, 2], [48, 41, 41])
    assert s._padding(torch.zeros(3, 1, L, L), 3, L) is None           # nothing hidden: the batched path
    assert s._padding(additive, 2, L) is None                          # not this batch's mask


def test_layout_helpers_refuse_host_tensors():
    import pytest
    import torch
    from kascade_b200 import _native as nat
    k = torch.zeros(2, 8, 40, 128, dtype=torch.float16)
    table = torch.zeros(2, 40, dtype=torch.int32)
    for make in (lambda: nat.kv_layout_rows(k, k.clone(), table), lambda: nat.kv_layout_contiguous(k, k.clone())):
        with pytest.raises(nat.KascadeNativeError, match="CUDA"):
            make()
