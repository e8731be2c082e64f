"""Known-answer tests of the oracle's token selection (crates/omni-qwen3-tts/kernels/talker.cu:108-293)
and a distribution check against the Hugging Face logits processors the kernel fuses."""
import numpy as np
import pytest


def fresh(vocab):
    return np.zeros(16, dtype=np.int32), np.zeros((vocab + 31) // 32, dtype=np.uint32)


def test_argmax_lowest_index_on_ties(oracle_lib):
    lg = np.zeros(3072, dtype=np.float32)
    lg[[7, 90, 1000]] = 3.0
    last, seen = fresh(3072)
    tok = oracle_lib.sample(lg, 0.0, 50, 1.0, 1.0, 0, 0, -1, 0, 5, 0.3, -1, last, seen, False, 3)
    assert tok == 7 and last[3] == 7 and not seen.any()


def test_forced_token_updates_state(oracle_lib):
    lg = np.random.default_rng(0).standard_normal(3072).astype(np.float32)
    last, seen = fresh(3072)
    tok = oracle_lib.sample(lg, 0.9, 50, 1.0, 1.05, 2048, 3072, 2150, 2, 9, 0.5, 1234, last, seen, True, 0)
    assert tok == 1234 and last[0] == 1234 and seen[1234 // 32] == 1 << (1234 % 32)


def test_suppression_and_end_token_gate(oracle_lib):
    lg = np.full(3072, -5.0, dtype=np.float32)
    lg[2150] = 50.0   # the end token dominates
    lg[2500] = 40.0   # a control token: never drawn
    lg[17] = 1.0
    for frame, want in ((0, 17), (1, 17), (2, 2150), (9, 2150)):
        last, seen = fresh(3072)
        tok = oracle_lib.sample(lg, 0.0, 50, 1.0, 1.0, 2048, 3072, 2150, 2, frame, 0.5, -1, last, seen, True, 0)
        assert tok == want, (frame, tok)


def test_repetition_penalty_sign_rule(oracle_lib):
    # positive logits are divided, negative multiplied (talker.cu:279)
    lg = np.array([2.0, 1.95] + [-30.0] * 62, dtype=np.float32)
    last, seen = fresh(64)
    seen[0] = 1  # token 0 was drawn before
    tok = oracle_lib.sample(lg, 0.0, 0, 1.0, 1.05, 0, 0, -1, 0, 5, 0.5, -1, last, seen, True, 0)
    assert tok == 1  # 2.0 / 1.05 < 1.95
    lg = np.array([-1.0, -1.04] + [-30.0] * 62, dtype=np.float32)
    last, seen = fresh(64)
    seen[0] = 1
    assert oracle_lib.sample(lg, 0.0, 0, 1.0, 1.05, 0, 0, -1, 0, 5, 0.5, -1, last, seen, True, 0) == 1


def test_top_k_keeps_ties_and_walks_vocabulary_order(oracle_lib):
    lg = np.full(2048, -20.0, dtype=np.float32)
    lg[[5, 900, 1500]] = [1.0, 1.0, 1.0]  # top_k = 2 but three tie at the threshold: all kept
    hits = set()
    for u in np.linspace(0.01, 0.99, 50):
        last, seen = fresh(2048)
        hits.add(oracle_lib.sample(lg, 1.0, 2, 1.0, 1.0, 0, 0, -1, 0, 5, float(u), -1, last, seen, False, 1))
    assert hits == {5, 900, 1500}
    # inverse CDF in vocabulary order: small u -> lowest kept index
    last, seen = fresh(2048)
    assert oracle_lib.sample(lg, 1.0, 2, 1.0, 1.0, 0, 0, -1, 0, 5, 0.0, -1, last, seen, False, 1) == 5
    last, seen = fresh(2048)
    assert oracle_lib.sample(lg, 1.0, 2, 1.0, 1.0, 0, 0, -1, 0, 5, 0.999999, -1, last, seen, False, 1) == 1500


def test_uniform_at_one_falls_back_to_last_kept(oracle_lib):
    lg = np.full(2048, -20.0, dtype=np.float32)
    lg[[3, 77]] = 2.0
    last, seen = fresh(2048)
    assert oracle_lib.sample(lg, 1.0, 2, 1.0, 1.0, 0, 0, -1, 0, 5, 1.0, -1, last, seen, False, 1) == 77


def test_distribution_matches_hf_processors(oracle_lib):
    torch = pytest.importorskip("torch")
    tfm = pytest.importorskip("transformers")
    rng = np.random.default_rng(3)
    vocab = 3072
    lg = (rng.standard_normal(vocab) * 2).astype(np.float32)
    lg = oracle_lib.bf16_round(lg)
    prev = rng.integers(0, 2048, 40)
    last0, seen0 = fresh(vocab)
    for t in prev:
        seen0[t // 32] |= np.uint32(1 << (t % 32))
    # HF chain: repetition penalty -> suppress -> temperature -> top-k -> softmax
    scores = torch.tensor(lg)[None]
    ids = torch.tensor(prev)[None]
    scores = tfm.RepetitionPenaltyLogitsProcessor(1.05)(ids, scores)
    suppress = [i for i in range(2048, vocab) if i != 2150]
    scores = tfm.SuppressTokensLogitsProcessor(suppress)(ids, scores)
    scores = tfm.TemperatureLogitsWarper(0.9)(ids, scores)
    scores = tfm.TopKLogitsWarper(50)(ids, scores)
    p = torch.softmax(scores, -1)[0].numpy()
    n = 20000
    counts = np.zeros(vocab)
    for i in range(n):
        last, seen = last0.copy(), seen0.copy()
        tok = oracle_lib.sample(lg, 0.9, 50, 1.0, 1.05, 2048, 3072, 2150, 2, 5, (i + 0.5) / n, -1, last, seen, True, 0)
        counts[tok] += 1
    assert set(np.nonzero(counts)[0]) <= set(np.nonzero(p)[0])
    assert np.abs(counts / n - p).max() < 2.5 / n + 1e-6


def test_philox_known_answer(oracle_lib):
    # Philox4x32-10 known-answer vector (Random123 kat_vectors): counter 0, key 0 -> first word 0x6627e8d5
    assert oracle_lib.philox_uniform(0, 0, 0) == np.float32((0x6627E8D5 >> 8) / 16777216.0)
    us = [oracle_lib.philox_uniform(7, f, g) for f in range(64) for g in range(16)]
    assert 0.0 <= min(us) and max(us) < 1.0 and abs(np.mean(us) - 0.5) < 0.05 and len(set(us)) > 1000
