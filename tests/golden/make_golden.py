"""Generates the golden vectors that pin the CPU oracle's decoder-stack arithmetic.

    python tests/golden/make_golden.py

Truth is the `transformers` Qwen3 model in f32 on CPU with random weights, the same model the
reference's own Higgs recorder uses as truth (tools/higgs_audio/golden.py:44-69). For each case the
script stores the inputs (checkpoint seed, prompt ids, forced codes) and Qwen3Model's final hidden
states; tests/test_oracle_golden.py replays the inputs through the oracle and compares. The
reference's real-checkpoint goldens need network and checkpoints and cannot be produced here.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from oracle.cpu import CpuOracle, bf16_round  # noqa: E402
from pega_omni_b200.config import presets  # noqa: E402
from pega_omni_b200.model import Draw, Prompt  # noqa: E402
from pega_omni_b200.synthetic import random_checkpoint  # noqa: E402


def hf_stack(cfg_stack, ck, prefix):
    from transformers import Qwen3Config, Qwen3Model
    c = cfg_stack
    kw = dict(hidden_size=c.hidden_size, intermediate_size=c.intermediate_size, num_hidden_layers=c.num_hidden_layers,
              num_attention_heads=c.num_attention_heads, num_key_value_heads=c.num_key_value_heads,
              head_dim=c.head_dim, rms_norm_eps=c.rms_norm_eps, vocab_size=32, attention_bias=False,
              max_position_embeddings=4096, use_sliding_window=False)
    try:
        conf = Qwen3Config(**kw, rope_parameters={"rope_type": "default", "rope_theta": c.rope_theta})
    except TypeError:
        conf = Qwen3Config(**kw, rope_theta=c.rope_theta)
    conf._attn_implementation = "eager"
    model = Qwen3Model(conf).float().eval()
    sd = {}
    for name, t in ck.items():
        if name.startswith(prefix + ".layers.") or name == prefix + ".norm.weight":
            sd[name[len(prefix) + 1:]] = t.float()
    sd["embed_tokens.weight"] = torch.zeros(32, c.hidden_size)
    missing, unexpected = model.load_state_dict(sd, strict=False)
    assert not [m for m in missing if "rotary" not in m], missing
    assert not unexpected, unexpected
    return model


def frame_embed(cfg, ck, pad_embed, frame):
    """pad + codec_emb[c0] + sum_g p_emb[g-1][c_g], f32 sum, one bf16 rounding (talker.cu:76-96)."""
    acc = pad_embed.astype(np.float32).copy()
    acc = acc + ck["talker.model.codec_embedding.weight"][frame[0]].float().numpy()
    for g in range(1, cfg.num_code_groups):
        acc = acc + ck[f"talker.code_predictor.model.codec_embedding.{g - 1}.weight"][frame[g]].float().numpy()
    return bf16_round(acc)


def make_case(name, preset, seed, prompt_lens, steps):
    cfg = presets[preset]()
    ck = random_checkpoint(cfg, seed=seed)
    rng = np.random.default_rng(seed + 1)
    oracle = CpuOracle(cfg, ck)
    hf = hf_stack(cfg.talker, ck, "talker.model")
    G = cfg.num_code_groups
    out = {"preset": preset, "seed": seed, "prompt_lens": np.asarray(prompt_lens), "steps": steps}
    prompts, sids = [], []
    for n in prompt_lens:
        prompts.append(Prompt(list(rng.integers(0, cfg.text_vocab_size, n)), list(rng.integers(-1, 64, n))))
        sids.append(oracle.open(n, steps + 1))
    forced = rng.integers(0, min(cfg.talker.vocab_size - cfg.control_tokens, cfg.predictor.vocab_size),
                          size=(steps + 1, len(prompt_lens), 16)).astype(np.int32)
    forced[:, :, G:] = 0
    out["text"] = np.concatenate([p.text for p in prompts]).astype(np.int32)
    out["codec"] = np.concatenate([p.codec for p in prompts]).astype(np.int32)
    out["forced"] = forced
    draws = [Draw([0.5] * 16, list(forced[0, s])) for s in range(len(sids))]
    oracle.start(sids, prompts, draws)
    embeds = oracle.embeds(sum(prompt_lens))  # the stack's input rows, as the oracle computed them
    pad = oracle.pad_embed()
    # HF truth: each sequence on its own, prompt then one row per decode step
    hidden = np.zeros((steps + 1, len(sids), cfg.talker.hidden_size), dtype=np.float32)
    at = 0
    with torch.no_grad():
        for s, n in enumerate(prompt_lens):
            rows = [embeds[at:at + n]]
            at += n
            for t in range(steps):
                rows.append(frame_embed(cfg, ck, pad, forced[t, s])[None])
            x = torch.from_numpy(np.concatenate(rows))[None]
            h = hf(inputs_embeds=x).last_hidden_state[0].numpy()
            hidden[0, s] = h[n - 1]
            for t in range(steps):
                hidden[t + 1, s] = h[n + t]
    out["hf_hidden"] = hidden
    # also record what the oracle itself produced when the vectors were made (drift detector)
    o_hidden = np.zeros_like(hidden)
    for s in range(len(sids)):
        o_hidden[0, s] = oracle.hidden(s)
    for t in range(steps):
        oracle.step(sids, [Draw([0.5] * 16, list(forced[t + 1, s])) for s in range(len(sids))])
        for s in range(len(sids)):
            o_hidden[t + 1, s] = oracle.hidden(s)
    out["oracle_hidden"] = o_hidden
    cos = [float(np.dot(a, b) / (np.linalg.norm(a) * np.linalg.norm(b)))
           for a, b in zip(hidden.reshape(-1, hidden.shape[-1]), o_hidden.reshape(-1, hidden.shape[-1]))]
    print(name, "min cosine oracle vs HF:", min(cos), "max abs:", float(np.abs(hidden - o_hidden).max()))
    np.savez_compressed(Path(__file__).resolve().parent / f"{name}.npz", **out)


if __name__ == "__main__":
    make_case("stack_hf_tiny128", "tiny128", 0, [5, 19, 33], 3)
    make_case("stack_hf_tiny64", "tiny64", 1, [7, 16], 2)
