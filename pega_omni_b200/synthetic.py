"""Random checkpoints of a talker architecture (no real weights are available offline).

Every matrix is bf16 ~ N(0, std) from a per-tensor seed derived from its checkpoint name; RMSNorm
gains are 1.0 so activations keep unit scale through the random stack. Tensor names are the
checkpoint names the reference loads (crates/omni-qwen3-tts/src/talker.rs:76-133,
crates/omni-qwen3/src/stack.rs:93-141).
"""
from __future__ import annotations

import zlib

import torch

from .config import StackConfig, TalkerConfig


def _stack_shapes(prefix: str, c: StackConfig):
    h, d = c.hidden_size, c.head_dim
    q, kv, i = c.num_attention_heads * d, c.num_key_value_heads * d, c.intermediate_size
    for l in range(c.num_hidden_layers):
        p = f"{prefix}.layers.{l}."
        yield p + "input_layernorm.weight", (h,)
        yield p + "self_attn.q_proj.weight", (q, h)
        yield p + "self_attn.k_proj.weight", (kv, h)
        yield p + "self_attn.v_proj.weight", (kv, h)
        yield p + "self_attn.q_norm.weight", (d,)
        yield p + "self_attn.k_norm.weight", (d,)
        yield p + "self_attn.o_proj.weight", (h, q)
        yield p + "post_attention_layernorm.weight", (h,)
        yield p + "mlp.gate_proj.weight", (i, h)
        yield p + "mlp.up_proj.weight", (i, h)
        yield p + "mlp.down_proj.weight", (h, i)
    yield f"{prefix}.norm.weight", (h,)


def tensor_shapes(cfg: TalkerConfig):
    t, p = cfg.talker, cfg.predictor
    h, ph = t.hidden_size, p.hidden_size
    yield "talker.model.text_embedding.weight", (cfg.text_vocab_size, h)
    yield "talker.model.codec_embedding.weight", (t.vocab_size, h)
    yield "talker.codec_head.weight", (t.vocab_size, h)
    yield "talker.text_projection.linear_fc1.weight", (h, h)
    yield "talker.text_projection.linear_fc1.bias", (h,)
    yield "talker.text_projection.linear_fc2.weight", (h, h)
    yield "talker.text_projection.linear_fc2.bias", (h,)
    yield "talker.code_predictor.small_to_mtp_projection.weight", (ph, h)
    yield "talker.code_predictor.small_to_mtp_projection.bias", (ph,)
    for g in range(cfg.num_code_groups - 1):
        yield f"talker.code_predictor.model.codec_embedding.{g}.weight", (p.vocab_size, h)
        yield f"talker.code_predictor.lm_head.{g}.weight", (p.vocab_size, ph)
    yield from _stack_shapes("talker.model", t)
    yield from _stack_shapes("talker.code_predictor.model", p)


def random_checkpoint(cfg: TalkerConfig, seed: int = 0, std: float = 0.02, device: str | torch.device = "cpu",
                      embed_std: float | None = None, head_std: float | None = None) -> dict[str, torch.Tensor]:
    """name -> bf16 tensor on `device`. Norm gains are ones; everything else N(0, std). `head_std` widens the
    output heads so logits are peaked like a trained model's instead of nearly flat."""
    device = torch.device(device)
    out: dict[str, torch.Tensor] = {}
    for name, shape in tensor_shapes(cfg):
        if name.endswith("norm.weight") or "layernorm" in name:
            out[name] = torch.ones(shape, dtype=torch.bfloat16, device=device)
            continue
        g = torch.Generator(device=device)
        g.manual_seed((zlib.crc32(name.encode()) ^ (seed * 0x9E3779B1)) & 0x7FFFFFFF)
        s = std
        if embed_std is not None and ("embedding" in name):
            s = embed_std
        if head_std is not None and ("codec_head" in name or "lm_head" in name):
            s = head_std
        n = 1
        for d in shape:
            n *= d
        # generate in f32 chunks to bound peak memory on large tables
        t = torch.empty(n, dtype=torch.bfloat16, device=device)
        step = 1 << 26
        for a in range(0, n, step):
            b = min(n, a + step)
            t[a:b] = (torch.randn(b - a, generator=g, device=device, dtype=torch.float32) * s).to(torch.bfloat16)
        out[name] = t.view(shape)
    return out
