"""The CPU oracle against the committed golden vectors (transformers' Qwen3Model in f32 as truth).

Thresholds follow the reference's own golden gates (crates/omni-qwen3-tts/tests/golden.rs:82-163:
logits cosine > 0.999); the oracle rounds every activation to bf16 like the GPU path, the truth is
f32, so element errors are bf16-sized.
"""
from pathlib import Path

import numpy as np
import pytest

from pega_omni_b200.config import presets
from pega_omni_b200.model import Draw, Prompt
from pega_omni_b200.synthetic import random_checkpoint

GOLDEN = Path(__file__).resolve().parent / "golden"


def cosine(a, b):
    return float(np.dot(a, b) / (np.linalg.norm(a) * np.linalg.norm(b)))


@pytest.mark.parametrize("name", ["stack_hf_tiny128", "stack_hf_tiny64"])
def test_oracle_matches_hf_qwen3(oracle_lib, name):
    g = np.load(GOLDEN / f"{name}.npz")
    cfg = presets[str(g["preset"])]()
    ck = random_checkpoint(cfg, seed=int(g["seed"]))
    o = oracle_lib.CpuOracle(cfg, ck)
    lens, steps, forced = [int(x) for x in g["prompt_lens"]], int(g["steps"]), g["forced"]
    prompts, sids, at = [], [], 0
    for n in lens:
        prompts.append(Prompt(list(g["text"][at:at + n]), list(g["codec"][at:at + n])))
        sids.append(o.open(n, steps + 1))
        at += n
    o.start(sids, prompts, [Draw([0.5] * 16, list(forced[0, s])) for s in range(len(sids))])
    got = np.zeros_like(g["hf_hidden"])
    for s in range(len(sids)):
        got[0, s] = o.hidden(s)
    for t in range(steps):
        codes = o.step(sids, [Draw([0.5] * 16, list(forced[t + 1, s])) for s in range(len(sids))])
        assert (codes == forced[t + 1]).all(), "teacher forcing must return the forced frame"
        for s in range(len(sids)):
            got[t + 1, s] = o.hidden(s)
    hf = g["hf_hidden"]
    for t in range(steps + 1):
        for s in range(len(sids)):
            assert cosine(got[t, s], hf[t, s]) > 0.9999, (t, s)
    assert np.abs(got - hf).max() < 0.05
    # the oracle has not drifted since the vectors were recorded (libm differences only)
    assert np.abs(got - g["oracle_hidden"]).max() < 2e-2
