"""One generated step of the benchmark's decoder loop against the Hugging Face module path (GPU).

The long-reasoning decode benchmark drives the library directly: per layer `kb200_kv_write` rotates q / k and
appends the new K / V rows to a paged cache, then the Kascade paged decode attends.  Inside a Hugging Face model the
module rotates q / k itself, appends to its own contiguous cache and calls the registered strategy.  Both routes
must produce the same next-token logits from the same weights, prompt and cache."""
import pytest
import torch

from tests.gpu_util import paged_from_contiguous

pytestmark = pytest.mark.gpu


def test_decoder_step_equals_hf_module_path():
    pytest.importorskip("transformers")
    from transformers import LlamaConfig, LlamaForCausalLM
    from bench_decoder import KascadeLlamaDecoder
    from kascade_b200 import EfficientKascadeStrategy, _native as nat
    torch.manual_seed(3)
    layers, L, page = 3, 600, 16
    cfg = LlamaConfig(hidden_size=1024, intermediate_size=512, num_hidden_layers=layers, num_attention_heads=8,
                      num_key_value_heads=2, head_dim=128, vocab_size=320, max_position_embeddings=4096,
                      rope_parameters={"rope_theta": 500000.0, "rope_type": "default"}, attn_implementation="sdpa")
    model = LlamaForCausalLM(cfg).to("cuda", torch.float16).eval()
    anchors, hm = [0, 2], [[0, 1], [1, 0], [0, 1]]
    B = 2
    ids = torch.randint(0, 320, (B, L), device="cuda")
    nxt = torch.randint(0, 320, (B, 1), device="cuda")
    with torch.no_grad():
        pre = model(ids, use_cache=True)                                   # dense prefill: both routes start from this cache
    # the library route works on a paged copy of the prompt's cache, with page room for the new token
    paged, table = [], None
    for l in range(layers):
        k, v = pre.past_key_values.layers[l].keys, pre.past_key_values.layers[l].values      # [B, G, L, D]
        pad = torch.zeros(B, k.shape[1], page, k.shape[3], dtype=k.dtype, device=k.device)
        kc, vc, bt = paged_from_contiguous(torch.cat([k, pad], 2), torch.cat([v, pad], 2), page_size=page, seed=5)
        paged.append((kc, vc))
        table = bt                                                         # same seed -> same page layout for every layer
    dec = KascadeLlamaDecoder.from_hf(model, anchors, hm, topk_pct=25)
    seq_lens = torch.full((B,), L, dtype=torch.int32, device="cuda")
    with torch.no_grad():
        got_tok = dec.step(nxt[:, 0], lambda l: paged[l], table, seq_lens, L + 1)
    got = dec.last_logits.float()
    assert nat.read_status() == 0
    # the Hugging Face route: the registered strategy, one decode step on the module's own cache
    strat = EfficientKascadeStrategy(anchors, "x/y", k=25, tile_size=32, rolling_prefill=True, head_mapping=hm)
    model.config._attn_implementation = strat.name
    with torch.no_grad():
        ref = model(nxt, past_key_values=pre.past_key_values, use_cache=True).logits[:, 0].float()
    scale = ref.abs().max().item()
    err = (got - ref).abs().max().item()
    assert err < 2e-2 * max(scale, 1.0), f"logits of the two routes differ by {err} (scale {scale})"
    assert (got_tok == ref.argmax(-1)).float().mean().item() >= 0.5 or err < 1e-3 * max(scale, 1.0)
    # the appended rows are what the module wrote into its cache (rotation by the kernel vs by the module)
    for l in range(layers):
        k_hf = pre.past_key_values.layers[l].keys[:, :, L]                  # [B, G, D], written by the HF step above
        kc = paged[l][0]
        for b in range(B):
            pg = int(table[b, L // page])
            row = kc[pg, L % page]                                         # [G, D]
            assert (row.float() - k_hf[b].float()).abs().max().item() < 4e-3, f"layer {l}, sequence {b}: appended K row"
