"""Parity against the reference's own CUDA kernels replayed on the same GPU (oracle/ref_kernels.py).

The cubins are compiled from the reference checkout where it is present and travel with the repository; where they
are missing these tests skip. Two claims: (1) the fused sampler picks bit-identical token ids (and leaves a
bit-identical slot) for identical logits, uniforms and state; (2) teacher-forced logits of the whole tick agree
with the reference's kernels + cuBLAS: cosine >= 0.9999 and max-abs within two bf16 steps (see the comment at the gate)."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    from oracle import ref_kernels
    ref_kernels.build()
    if not ref_kernels.available():
        pytest.skip("reference cubins not built (no reference checkout on this machine)")
    return ref_kernels


def cosine(a, b):
    return float(np.dot(a, b) / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-30))


@pytest.mark.parametrize("vocab,group,temperature,top_k", [(3072, 0, 0.9, 50), (2048, 7, 0.9, 50), (2048, 2, 0.0, 50),
                                                            (3072, 0, 1.0, 0), (2048, 1, 0.7, 3)])
def test_sampler_bit_exact_against_reference_kernel(built_lib, ref, vocab, group, temperature, top_k):
    from pega_omni_b200.ops import Ops
    ops = Ops(0)
    rows = 64
    rng = np.random.default_rng(vocab * 31 + group)
    g = torch.Generator(device="cuda")
    g.manual_seed(5)
    logits = (torch.randn((rows, vocab), generator=g, device="cuda") * 2.5).to(torch.bfloat16)
    words = (vocab + 31) // 32
    stride = ((4 * (16 + words + (words & 1)) + 8 + 255) // 256) * 256
    state = np.zeros((rows, stride // 4), dtype=np.uint32)
    for s in range(rows):
        for t in rng.integers(0, 2048, 40):
            state[s, 16 + t // 32] |= np.uint32(1 << (t % 32))
    penalize = int(group == 0)
    lo, hi, exempt, min_frames = (vocab - 1024, vocab, 2150, 2) if penalize else (0, 0, -1, 0)
    dev = lambda a: torch.tensor(a, device="cuda")
    frames, lines = dev(rng.integers(0, 5, rows).astype(np.int32)), dev(np.arange(rows, dtype=np.int32))
    uniforms = dev(rng.random((rows, 16)).astype(np.float32))
    force = np.full((rows, 16), -1, dtype=np.int32)
    force[3, group] = 11
    force = dev(force)
    out = []
    for which in ("ours", "reference"):
        st = dev(state.view(np.int32).copy())
        codes = torch.full((rows, 16), -7, dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()
        if which == "ours":
            ops.sample(logits, temperature, top_k, 1.0, 1.05, lo, hi, exempt, min_frames, frames, uniforms, force, st,
                       lines, stride, penalize, 0, codes, group)
            ops.sync()
        else:
            mod = ref._Module(ref.OUT / "talker.cubin")
            p, i, f, l = ref._p, ref._i, ref._f, ref._l
            mod.launch("talker_sample", [rows], 1024,
                       [p(logits), i(vocab), f(temperature), i(top_k), f(1.05), i(lo), i(hi), i(exempt), i(min_frames),
                        p(frames), p(uniforms), p(force), p(st), p(lines), l(stride), i(penalize), p(codes), i(group)])
            torch.cuda.synchronize()
        out.append((codes.cpu().numpy(), st.cpu().numpy()))
    assert np.array_equal(out[0][0][:, group], out[1][0][:, group]), "token ids differ from the reference sampler"
    assert np.array_equal(out[0][1], out[1][1]), "slot state (last frame, repetition bitmap) differs"
    ops.close()


# "mid" (hidden 1024 / 512) is inside the reference's own shape limits (hidden a multiple of 256, stack.rs:101)
@pytest.mark.parametrize("preset,engine", [("mid", "tick"), ("mid", "ops")])
def test_teacher_forced_logits_match_reference_kernels(built_lib, ref, preset, engine):
    from pega_omni_b200.config import presets
    from pega_omni_b200.model import Draw, Limits, Model, Prompt
    from pega_omni_b200.synthetic import random_checkpoint
    cfg = presets[preset]()
    ck = random_checkpoint(cfg, seed=3, device="cuda")
    m = Model.load(0, ck, cfg, Limits(max_batch=8, max_tokens=256, kv_gib=0.02), tick_kernel=engine == "tick")
    rng = np.random.default_rng(12)
    lens, frames = [9, 33, 17, 26], 6
    prompts = [Prompt(list(rng.integers(0, cfg.text_vocab_size, n)), list(np.where(rng.random(n) < 0.3, 7, -1)))
               for n in lens]
    forced = rng.integers(0, 2048, size=(frames, len(lens), 16)).astype(np.int32)
    r = ref.RefTalker(cfg, ck, len(lens), max(lens) + frames + 2)
    seqs = [m.open(n, frames + 2) for n in lens]
    uniforms = np.full((len(lens), 16), 0.5, dtype=np.float32)
    worst_abs, worst_cos = 0.0, 1.0
    for t in range(frames):
        draws = [Draw([0.5] * 16, list(forced[t, s])) for s in range(len(lens))]
        if t == 0:
            ours = m.start(list(zip(seqs, prompts, draws))).codes
            theirs = r.start(prompts, uniforms, forced[t])
        else:
            ours = m.step(list(zip(seqs, draws))).codes
            theirs = r.step(uniforms, forced[t])
        assert np.array_equal(ours, theirs) and np.array_equal(ours, forced[t])
        for s in range(len(lens)):
            for a, b in [(m.talker_logits(s), r.talker_logits(s))] + list(zip(m.predictor_logits(s), r.predictor_logits(s))):
                worst_abs = max(worst_abs, float(np.abs(a - b).max()))
                worst_cos = min(worst_cos, cosine(a, b))
    # The reference's GEMMs are cuBLAS here (its own cuBLASLt configuration lives in an un-vendored runtime), ours
    # are tcgen05 tiles with a K split: two f32 summation orders. Observed worst difference 0.023 on logits of
    # magnitude 2..4, where one bf16 step is 0.0156; the gate is two such steps, plus the north-star's cosine.
    assert worst_abs <= 3.2e-2, worst_abs
    assert worst_cos >= 0.9999, worst_cos
    m.close()
