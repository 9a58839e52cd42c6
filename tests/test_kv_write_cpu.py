"""The KV write-path oracle against the installed Hugging Face modules it restates (CPU)."""
import pytest
import torch

from oracle.kv_write_oracle import apply_rope, rms_norm, rope_cos_sin

llama = pytest.importorskip("transformers.models.llama.modeling_llama")


def _cfg(theta):
    from transformers import LlamaConfig
    cfg = LlamaConfig(hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                      max_position_embeddings=131072)
    try:
        cfg.rope_theta = theta
        if getattr(cfg, "rope_parameters", None) is not None:
            cfg.rope_parameters["rope_theta"] = theta
    except Exception:
        pass
    return cfg


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
@pytest.mark.parametrize("theta", [500000.0, 10000.0])
def test_rope_matches_transformers(theta, dtype):
    g = torch.Generator().manual_seed(0)
    B, T, H, G, D = 2, 5, 8, 2, 128
    q = torch.randn(B, T, H, D, generator=g).to(dtype)
    k = torch.randn(B, T, G, D, generator=g).to(dtype)
    pos = torch.tensor([[0, 1, 2, 70000, 131071], [5, 17, 4096, 32767, 99999]])
    rot = llama.LlamaRotaryEmbedding(config=_cfg(theta))
    cos_hf, sin_hf = rot(q, pos)                                                       # [B, T, D] in q's type
    cos, sin = rope_cos_sin(pos, rot.inv_freq, float(getattr(rot, "attention_scaling", 1.0)), dtype)
    assert torch.equal(cos, cos_hf) and torch.equal(sin, sin_hf)
    # transformers rotates [B, heads, T, D]
    q_hf, k_hf = llama.apply_rotary_pos_emb(q.transpose(1, 2), k.transpose(1, 2), cos_hf, sin_hf)
    assert torch.equal(apply_rope(q, cos, sin), q_hf.transpose(1, 2))
    assert torch.equal(apply_rope(k, cos, sin), k_hf.transpose(1, 2))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
def test_rms_norm_matches_transformers(dtype):
    g = torch.Generator().manual_seed(1)
    x = (torch.randn(3, 7, 4, 128, generator=g) * 2).to(dtype)
    norm = llama.LlamaRMSNorm(128, eps=1e-6).to(dtype)
    with torch.no_grad():
        norm.weight.copy_((1 + 0.1 * torch.randn(128, generator=g)).to(dtype))
        want = norm(x)
    assert torch.equal(rms_norm(x, norm.weight.data, 1e-6), want)
