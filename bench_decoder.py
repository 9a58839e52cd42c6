"""A Llama-architecture decoder around the Kascade decode path, for the long-reasoning decode benchmark.

The attention of every layer runs through the library: ``kb200_kv_write`` rotates q / k and appends the new
K / V rows to the paged cache in one kernel, ``EfficientKascadeStrategy.paged_decode_forward`` does the anchor /
reuse decode attention.  Everything else of the decoder (projections, SwiGLU, RMSNorm, embedding, LM head) is
plain ``torch`` — those layers are outside the path this repository implements; they are here so that the
benchmark can report generated tokens per second of a whole decoder step next to the attention time.

Weights are random (N(0, 0.02)) or copied from a Hugging Face ``LlamaForCausalLM`` (``from_hf``), which is how
the test checks one generated step of this loop against the Hugging Face module path.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch
import torch.nn.functional as F

from kascade_b200 import EfficientKascadeStrategy, _native as nat


@dataclass
class DecoderConfig:
    layers: int = 32
    hidden: int = 4096
    ffn: int = 14336
    heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    vocab: int = 128256
    rope_theta: float = 500000.0
    norm_eps: float = 1e-5
    anchors: Sequence[int] = (0, 2, 8, 13, 14)
    topk_pct: float = 10
    page: int = 16


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """LlamaRMSNorm: fp32 statistics, result rounded to the input type, then the gain."""
    v = x.float()
    v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)
    return weight * v.to(x.dtype)


class KascadeLlamaDecoder:
    """Decode-only Llama stack (one new token per sequence per step) over a paged KV cache."""

    def __init__(self, cfg: DecoderConfig, device, head_mapping: List[List[int]], seed: int = 0, init_std: float = 0.02,
                 with_vocab: bool = True):
        self.cfg, self.dev = cfg, device
        g = torch.Generator(device=device).manual_seed(seed)

        def w(*shape):
            return (torch.randn(*shape, generator=g, device=device, dtype=torch.float32) * init_std).half()

        c = cfg
        self.layers = []
        for _ in range(c.layers):
            self.layers.append({
                "qkv": w((c.heads + 2 * c.kv_heads) * c.head_dim, c.hidden),       # fused q, k, v projection
                "o": w(c.hidden, c.heads * c.head_dim),
                "gate_up": w(2 * c.ffn, c.hidden),
                "down": w(c.hidden, c.ffn),
                "ln1": torch.ones(c.hidden, dtype=torch.float16, device=device),
                "ln2": torch.ones(c.hidden, dtype=torch.float16, device=device),
            })
        self.norm = torch.ones(c.hidden, dtype=torch.float16, device=device)
        self.embed = w(c.vocab, c.hidden) if with_vocab else None                   # tied with the LM head
        self.inv_freq = (1.0 / (c.rope_theta ** (torch.arange(0, c.head_dim, 2, dtype=torch.float32) / c.head_dim))).to(device)
        self.strategy = EfficientKascadeStrategy(list(c.anchors), "bench/llama-decoder", k=c.topk_pct, tile_size=32,
                                                 rolling_prefill=True, head_mapping=head_mapping, register=False)

    @classmethod
    def from_hf(cls, model, anchors, head_mapping, topk_pct=10) -> "KascadeLlamaDecoder":
        """Same weights as a Hugging Face ``LlamaForCausalLM`` (fp16, on its device)."""
        hc = model.config
        cfg = DecoderConfig(layers=hc.num_hidden_layers, hidden=hc.hidden_size, ffn=hc.intermediate_size,
                            heads=hc.num_attention_heads, kv_heads=hc.num_key_value_heads, head_dim=hc.head_dim,
                            vocab=hc.vocab_size, rope_theta=float((getattr(hc, "rope_parameters", None) or {}).get("rope_theta", 0) or
                                                                  getattr(hc, "rope_theta", 10000.0)),
                            norm_eps=hc.rms_norm_eps, anchors=tuple(anchors), topk_pct=topk_pct)
        dev = next(model.parameters()).device
        self = cls(DecoderConfig(**{**cfg.__dict__, "layers": 0}), dev, head_mapping, with_vocab=False)
        self.cfg = cfg
        self.strategy = EfficientKascadeStrategy(list(anchors), "bench/llama-decoder", k=topk_pct, tile_size=32,
                                                 rolling_prefill=True, head_mapping=head_mapping, register=False)
        for lyr in model.model.layers:
            a, m = lyr.self_attn, lyr.mlp
            self.layers.append({
                "qkv": torch.cat([a.q_proj.weight, a.k_proj.weight, a.v_proj.weight], 0).detach().half().contiguous(),
                "o": a.o_proj.weight.detach().half().contiguous(),
                "gate_up": torch.cat([m.gate_proj.weight, m.up_proj.weight], 0).detach().half().contiguous(),
                "down": m.down_proj.weight.detach().half().contiguous(),
                "ln1": lyr.input_layernorm.weight.detach().half(), "ln2": lyr.post_attention_layernorm.weight.detach().half(),
            })
        self.norm = model.model.norm.weight.detach().half()
        self.embed = model.model.embed_tokens.weight.detach().half()
        self.lm_head = model.lm_head.weight.detach().half()
        self.inv_freq = model.model.rotary_emb.inv_freq.detach().float().to(dev).contiguous()
        return self

    # ------------------------------------------------------------------------------------------
    def attention(self, layer: int, q, k_new, v_new, caches, block_table, seq_lens, max_len: int):
        """q [B,H,D], k_new / v_new [B,G,D] (not rotated) at positions seq_lens[b]: rotate, append, attend."""
        c = self.cfg
        kc, vc = caches
        B = q.shape[0]
        kv = nat.kv_layout_paged(kc, vc, block_table)
        q_rot = torch.empty(B, 1, c.heads, c.head_dim, dtype=torch.float16, device=q.device)
        nat.kv_write(q.view(B, 1, c.heads, c.head_dim), q_rot, k_new.view(B, 1, c.kv_heads, c.head_dim),
                     v_new.view(B, 1, c.kv_heads, c.head_dim), seq_lens, None, kv, inv_freq=self.inv_freq)
        lens_after = self._lens_after
        return self.strategy.paged_decode_forward(layer, q_rot.view(B, c.heads, c.head_dim), kc, vc, block_table,
                                                  lens_after, c.head_dim ** -0.5, max_len, mean_seq_len=self.mean_len)

    def step(self, tokens_or_hidden, caches_of_layer, block_table, seq_lens, max_len: int, attention_only: bool = False):
        """One decode step for the whole batch.  seq_lens [B] int32 = cache lengths BEFORE the step (the position
        of the new token); the caller adds one afterwards.  Returns the next tokens [B] (or the hidden state if the
        decoder was built without a vocabulary)."""
        c = self.cfg
        x = F.embedding(tokens_or_hidden, self.embed) if tokens_or_hidden.dtype == torch.int64 else tokens_or_hidden
        B = x.shape[0]
        self._lens_after = seq_lens + 1
        nq, nk = c.heads * c.head_dim, c.kv_heads * c.head_dim
        for l, wts in enumerate(self.layers):
            if attention_only:                                  # the library's part of the step alone
                qkv = self._qkv_cache[l]
            else:
                qkv = F.linear(rms_norm(x, wts["ln1"], c.norm_eps), wts["qkv"])
                if self._qkv_cache is not None:
                    self._qkv_cache[l] = qkv
            q, k_new, v_new = qkv[:, :nq], qkv[:, nq:nq + nk], qkv[:, nq + nk:]
            att = self.attention(l, q.reshape(B, c.heads, c.head_dim), k_new.reshape(B, c.kv_heads, c.head_dim),
                                 v_new.reshape(B, c.kv_heads, c.head_dim), caches_of_layer(l), block_table, seq_lens, max_len)
            if attention_only:
                continue
            x = x + F.linear(att.view(B, nq), wts["o"])
            h = F.linear(rms_norm(x, wts["ln2"], c.norm_eps), wts["gate_up"])
            x = x + F.linear(F.silu(h[:, :c.ffn]) * h[:, c.ffn:], wts["down"])
        if attention_only:
            return None
        x = rms_norm(x, self.norm, c.norm_eps)
        head = getattr(self, "lm_head", None)
        if head is None:
            head = self.embed
        if head is None:
            return x
        self.last_logits = F.linear(x, head)
        return self.last_logits.argmax(-1)

    mean_len: Optional[float] = None      # the host's hint for batches of very different lengths (see paged_decode_forward)
    _qkv_cache: Optional[list] = None
    _lens_after: Optional[torch.Tensor] = None
