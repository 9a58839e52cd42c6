"""The strategy as a Hugging Face attention implementation (GPU): a small random-init Llama with the
benchmark's attention shape (32 query / 8 KV heads of 128) runs its prefill through `efficient_kascade`.
With k = 100 % every earlier key fits the budget, so the prefill must reproduce dense attention."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_llama_prefill_and_decode_through_the_registry():
    transformers = pytest.importorskip("transformers")
    from transformers import LlamaConfig, LlamaForCausalLM
    from kascade_b200 import EfficientKascadeStrategy, _native as nat
    torch.manual_seed(0)
    layers = 3
    cfg = LlamaConfig(hidden_size=4096, intermediate_size=512, num_hidden_layers=layers, num_attention_heads=32,
                      num_key_value_heads=8, head_dim=128, vocab_size=320, max_position_embeddings=4096,
                      attn_implementation="sdpa")
    model = LlamaForCausalLM(cfg).to("cuda", torch.float16).eval()
    ids = torch.randint(0, 320, (1, 480), device="cuda")
    with torch.no_grad():
        ref = model(ids, use_cache=True)
    strat = EfficientKascadeStrategy([0, 2], "x/y", k=100, tile_size=32, rolling_prefill=False,
                                     head_mapping=[list(range(8)), [3, 3, 0, 7, 1, 6, 2, 5], list(range(8))])
    model.config._attn_implementation = strat.name
    with torch.no_grad():
        got = model(ids, use_cache=True)
    assert nat.read_status() == 0
    assert nat.launch_count > 0, "the model did not go through the library"
    err = (got.logits.float() - ref.logits.float()).abs().max().item()
    scale = ref.logits.float().abs().max().item()
    assert err < 2e-2 * max(scale, 1.0), f"prefill logits differ from dense attention by {err} (scale {scale})"
    # one decode step on the cache the prefill produced: anchors select all but the 32 weakest keys, reuse layers
    # attend to exactly those keys, so the step stays close to dense attention
    nxt = torch.randint(0, 320, (1, 1), device="cuda")
    with torch.no_grad():
        step = model(nxt, past_key_values=got.past_key_values, use_cache=True)
        model.config._attn_implementation = "sdpa"
        step_ref = model(nxt, past_key_values=ref.past_key_values, use_cache=True)
    assert nat.read_status() == 0
    assert bool(torch.isfinite(step.logits).all())
    rel = (step.logits.float() - step_ref.logits.float()).abs().max().item() / max(step_ref.logits.float().abs().max().item(), 1.0)
    assert rel < 0.25, f"decode logits far from dense attention: {rel}"


def test_llama_left_padded_batch_through_the_registry():
    """Two prompts of different length, left-padded by the tokenizer convention (attention_mask of 0 / 1 per
    token): at k = 100 % the valid positions must reproduce dense attention with the same mask."""
    pytest.importorskip("transformers")
    from transformers import LlamaConfig, LlamaForCausalLM
    from kascade_b200 import EfficientKascadeStrategy, _native as nat
    torch.manual_seed(1)
    cfg = LlamaConfig(hidden_size=4096, intermediate_size=512, num_hidden_layers=2, num_attention_heads=32,
                      num_key_value_heads=8, head_dim=128, vocab_size=320, max_position_embeddings=4096,
                      attn_implementation="sdpa")
    model = LlamaForCausalLM(cfg).to("cuda", torch.float16).eval()
    # lengths that are multiples of the tile: only then does a 100 % budget (L - 32 keys) cover every tile's past
    L, pads = 352, [0, 128]
    ids = torch.randint(0, 320, (2, L), device="cuda")
    am = torch.ones(2, L, dtype=torch.long, device="cuda")
    for b, pad in enumerate(pads):
        am[b, :pad] = 0
    with torch.no_grad():
        ref = model(ids, attention_mask=am).logits
    strat = EfficientKascadeStrategy([0], "x/y", k=100, tile_size=32, rolling_prefill=False,
                                     head_mapping=[list(range(8)), [3, 3, 0, 7, 1, 6, 2, 5]])
    model.config._attn_implementation = strat.name
    n0 = nat.launch_count
    with torch.no_grad():
        got = model(ids, attention_mask=am).logits
    assert nat.launch_count > n0 and nat.read_status() == 0
    for b, pad in enumerate(pads):
        err = (got[b, pad:].float() - ref[b, pad:].float()).abs().max().item()
        scale = ref[b, pad:].float().abs().max().item()
        assert err < 2e-2 * max(scale, 1.0), f"sequence {b}: logits differ from dense attention by {err} (scale {scale})"


def test_llama_prefill_at_a_real_budget_against_the_oracle():
    """k = 10 %, rolling prefill, through the Hugging Face registry: the q / k / v that every attention module
    hands to the strategy are recorded, and each layer is then checked on the CPU — anchor layers' index rows by
    the tie-band rule against the oracle's pooled scores, every layer's output against the oracle evaluated on
    those inputs with the strategy's own rows (so a legal swap at the k-th score does not count)."""
    pytest.importorskip("transformers")
    from transformers import LlamaConfig, LlamaForCausalLM
    from kascade_b200 import EfficientKascadeStrategy, _native as nat
    from oracle.kascade_oracle import (band_check, pooled_scores_prefill, rolling_budget, sparse_prefill_output,
                                       topk_budget)
    from tests.gpu_util import assert_close
    torch.manual_seed(2)
    layers, L, tile, pct = 3, 1600, 32, 10
    cfg = LlamaConfig(hidden_size=1024, intermediate_size=256, num_hidden_layers=layers, num_attention_heads=8,
                      num_key_value_heads=2, head_dim=128, vocab_size=320, max_position_embeddings=4096,
                      attn_implementation="sdpa")
    model = LlamaForCausalLM(cfg).to("cuda", torch.float16).eval()
    hm = [[0, 1], [1, 1], [0, 1]]
    strat = EfficientKascadeStrategy([0, 2], "x/y", k=pct, tile_size=tile, rolling_prefill=True, head_mapping=hm)
    seen = {}
    inner = strat.attention_forward

    def recording(module, query, key, value, attention_mask, scaling, dropout=0.0, **kw):
        out, w = inner(module, query, key, value, attention_mask, scaling, dropout=dropout, **kw)
        idx = (strat._tile_idx.cpu().clone(), strat._tile_count.cpu().clone()) if strat.is_anchor(module.layer_idx) else None
        seen[int(module.layer_idx)] = (query.float().cpu(), key.float().cpu(), value.float().cpu(), float(scaling),
                                       out.float().cpu(), idx)
        return out, w

    strat.attention_forward = recording
    model.config._attn_implementation = strat.name
    ids = torch.randint(0, 320, (1, L), device="cuda")
    with torch.no_grad():
        model(ids)
    assert nat.read_status() == 0 and sorted(seen) == list(range(layers))
    T = -(-L // tile)
    kk = topk_budget(pct, L, tile)
    rows = None
    for layer in range(layers):
        q, k, v, scaling, out, idx = seen[layer]
        G = k.shape[1]
        if idx is not None:
            ti, tc = idx
            pooled = pooled_scores_prefill(q, k, scaling, tile)
            rows = torch.full((1, G, T, max(kk, 1)), L - 1, dtype=torch.int32)
            for g in range(G):
                for t in range(T):
                    n = int(tc[0, g, t])
                    got = ti[0, g, t, :n].tolist()
                    ok, msg = band_check(pooled[0, g, t], got, min(kk, rolling_budget(pct, t * tile)), t * tile)
                    assert ok, f"layer {layer} (g{g} t{t}): {msg}"
                    rows[0, g, t, :n] = ti[0, g, t, :n]
        if layer == 0:
            ref = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True,
                                                                   scale=scaling).transpose(1, 2)
        else:
            ref = sparse_prefill_output(q, k, v, rows[:, hm[layer]] if idx is None else rows, scaling, tile)
        assert_close(out, ref, what=f"HF layer {layer} at k = {pct} %")
