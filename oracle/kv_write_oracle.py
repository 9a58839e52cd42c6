"""CPU restatement of the KV-cache write path (test infrastructure only; never imported by the product path).

What is restated is what a Hugging Face Llama / Qwen3 attention module does to q and k before the
attention call, and what a paged cache does with the new rows:

* per-head RMS norm — transformers `LlamaRMSNorm.forward` / `Qwen3RMSNorm.forward`
  (models/llama/modeling_llama.py, class LlamaRMSNorm): fp32 `x * rsqrt(mean(x^2) + eps)`, cast back to
  the input dtype, times the gain;
* rotary embedding — `LlamaRotaryEmbedding.forward` (angles = position x inv_freq in fp32, cos / sin
  scaled and cast to the input dtype) and `apply_rotary_pos_emb` / `rotate_half`
  (`x * cos + cat(-x2, x1) * sin` in the input dtype);
* append — row of position p of sequence b goes to page `block_table[b, p // page]`, slot `p % page`
  (the vLLM-style layout `[pages, page, G, D]` the decode kernels read).

Parity pinned: tests/test_kv_write_cpu.py checks these functions against the installed `transformers`
modules themselves.  The reference (microsoft/kascade) has no kernel for this step: it receives the
rotated tensors from the Hugging Face module (strategies/EfficientKascadeStrategy.py:126-150).
"""
from __future__ import annotations

from typing import Optional

import torch


def rms_norm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    """x [..., D] fp16, gain [D] fp16 -> fp16."""
    xf = x.to(torch.float32)
    xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return gain * xf.to(x.dtype)


def rope_cos_sin(positions: torch.Tensor, inv_freq: torch.Tensor, scale: float, dtype) -> tuple:
    """positions [...] int, inv_freq [D/2] fp32 -> cos, sin [..., D] in `dtype`."""
    freqs = positions.to(torch.float32)[..., None] * inv_freq.to(torch.float32)
    emb = torch.cat((freqs, freqs), dim=-1)
    return (emb.cos() * scale).to(dtype), (emb.sin() * scale).to(dtype)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    d = x.shape[-1] // 2
    return torch.cat((-x[..., d:], x[..., :d]), dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [B, T, heads, D]; cos / sin [B, T, D]."""
    return (x * cos[:, :, None, :]) + (rotate_half(x) * sin[:, :, None, :])


def quantize_e4m3(x: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """x [..., G, D] (fp16 values), scale [..., G] fp32 -> e4m3 bytes of x / scale: fp32 division, clamped to the
    finite range of the format (+-448), rounded to nearest even."""
    y = (x.float() / scale[..., None].float()).clamp(-448.0, 448.0)
    return y.to(torch.float8_e4m3fn)


def kv_write(q: Optional[torch.Tensor], k: torch.Tensor, v: torch.Tensor, start_pos, n_new, k_cache, v_cache,
             block_table, page: int, q_gain=None, k_gain=None, eps: float = 1e-6, inv_freq=None, scale: float = 1.0,
             k_scale=None, v_scale=None):
    """q [B,T,H,D] or None, k / v [B,T,G,D] fp16 or bf16; caches [pages, page, G, D] are modified in place.
    With k_scale / v_scale [pages, G] fp32 the caches are e4m3 (torch.float8_e4m3fn) and a row is stored as
    value / scale of its page and KV head.  Returns the transformed q (or None)."""
    B, T = k.shape[:2]
    pos = torch.tensor(start_pos)[:, None] + torch.arange(T)[None, :]                   # [B, T]
    if k_gain is not None:
        k = rms_norm(k, k_gain, eps)
    if q is not None and q_gain is not None:
        q = rms_norm(q, q_gain, eps)
    if inv_freq is not None:
        cos, sin = rope_cos_sin(pos, inv_freq, scale, k.dtype)
        k = apply_rope(k, cos, sin)
        if q is not None:
            q = apply_rope(q, cos, sin)
    for b in range(B):
        n = T if n_new is None else int(n_new[b])
        for t in range(n):
            p = int(pos[b, t])
            phys = int(block_table[b, p // page])
            if k_scale is not None:
                k_cache[phys, p % page] = quantize_e4m3(k[b, t], k_scale[phys])
                v_cache[phys, p % page] = quantize_e4m3(v[b, t], v_scale[phys])
            else:
                k_cache[phys, p % page] = k[b, t]
                v_cache[phys, p % page] = v[b, t]
    return q
