"""CPU checks of the duplex (PersonaPlex) oracle: number formats, the draw, the token bookkeeping against the
reference's host specification, and the tick state machine."""
import numpy as np
import pytest

from oracle import duplex as O
from pega_omni_b200.duplex import PRESETS, Prompt, Step, random_checkpoint


def test_e4m3_known_values():
    # exact grid points, ties to even, saturation and the subnormal grid (E4M3: bias 7, 3 mantissa bits, max 448)
    x = np.array([0.0, 1.0, 1.0625, 1.1875, 448.0, 500.0, -1000.0, 2.0 ** -9, 2.0 ** -10, 0.017, 240.0, 17.0, 19.0],
                 np.float32)
    want = np.array([0.0, 1.0, 1.0, 1.25, 448.0, 448.0, -448.0, 2.0 ** -9, 0.0, 0.017578125, 240.0, 16.0, 20.0],
                    np.float32)
    assert np.array_equal(O.e4m3(x), want)


def test_e4m3_matches_torch_float8():
    torch = pytest.importorskip("torch")
    if not hasattr(torch, "float8_e4m3fn"):
        pytest.skip("no float8 in this torch")
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.normal(0, 100, 4000), rng.normal(0, 1, 4000), rng.normal(0, 0.01, 4000)]).astype(np.float32)
    x = np.clip(x, -448, 448)
    ref = torch.from_numpy(x).to(torch.float8_e4m3fn).to(torch.float32).numpy()
    assert np.array_equal(O.e4m3(x), ref)


def test_bf16_round_matches_torch():
    torch = pytest.importorskip("torch")
    x = np.random.default_rng(1).normal(0, 3, 10000).astype(np.float32)
    assert np.array_equal(O.bf16r(x), torch.from_numpy(x).to(torch.bfloat16).float().numpy())


def test_mix_is_the_32_bit_hash():
    # lm.cu:391-398 spelled out with Python integers
    def ref(x):
        x &= 0xFFFFFFFF
        x ^= x >> 16
        x = (x * 0x7FEB352D) & 0xFFFFFFFF
        x ^= x >> 15
        x = (x * 0x846CA68B) & 0xFFFFFFFF
        x ^= x >> 16
        return x
    xs = [0, 1, 2, 0xFFFFFFFF, 0x9E3779B9, 123456789]
    assert [int(v) for v in O.mix(np.array(xs, np.uint64))] == [ref(x) for x in xs]
    assert ref(0) == 0 and ref(1) != 1


def test_advance_is_the_host_specification():
    # crates/omni-personaplex/src/prompt.rs:167-183 restated independently, element by element
    rng = np.random.default_rng(2)
    for _ in range(200):
        row = list(rng.integers(0, 2048, 17))
        pending = list(rng.integers(0, 2048, 7))
        drawn = list(rng.integers(0, 2048, 9))
        caller = list(rng.integers(0, 2048, 8))
        nxt, pend, text, frame = O.advance(row, pending, drawn, caller)
        assert nxt[:9] == drawn and nxt[9] == caller[0] and nxt[10:] == pending
        assert pend == caller[1:]
        assert text == row[0] and frame[0] == row[1] and frame[1:] == drawn[2:]


def test_draw_forced_greedy_and_top_k():
    rng = np.random.default_rng(3)
    logits = O.bf16r(rng.normal(0, 2, 2048).astype(np.float32))
    assert O.sample(logits, 0.0, 0, 1, 2, 0) == int(np.argmax(logits))
    tied = logits.copy()
    tied[[5, 900]] = tied.max() + 1
    assert O.sample(tied, 0.0, 0, 1, 2, 0) == 5  # lowest index on ties
    kept_rank = np.argsort(-logits, kind="stable")[:25]
    floor = logits[kept_rank[-1]]
    for seed in range(50):
        tok = O.sample(logits, 0.8, 25, seed, seed * 7, 3)
        assert logits[tok] >= floor  # inside the top-k (ties kept)
    # different columns and seeds give different streams
    a = [O.sample(logits, 1.0, 250, s, 0, 1) for s in range(40)]
    b = [O.sample(logits, 1.0, 250, s, 0, 2) for s in range(40)]
    assert a != b and len(set(a)) > 5


def test_draw_follows_the_softmax():
    # Gumbel-max over top-k is a sample of softmax(logits / T) restricted to the top-k
    logits = O.bf16r(np.array([2.0, 1.0, 0.0, -1.0, -3.0, -9.0], np.float32))
    T, n = 0.7, 6000
    counts = np.zeros(6)
    for s in range(n):
        counts[O.sample(logits, T, 4, s, 99, 1)] += 1
    p = np.exp(logits[:4] / T)
    p /= p.sum()
    assert counts[4:].sum() == 0
    assert np.abs(counts[:4] / n - p).max() < 0.02


def _prompt(c, rng, steps):
    rows = rng.integers(0, c.card, (steps, 17)).astype(np.int32)
    rows[:, 0] = rng.integers(0, c.text_vocab, steps)
    rows[rng.random((steps, 17)) < 0.1] = -1
    first = rng.integers(0, c.card, 17)
    first[0] = rng.integers(0, c.text_vocab)
    return Prompt(rows, list(first), list(rng.integers(0, c.card, 7)))


def test_tick_state_machine_on_a_tiny_model():
    c = PRESETS["duplex-tiny"]
    ck = random_checkpoint(c, seed=0, head_std=0.2)
    orc = O.DuplexOracle(c, ck)
    rng = np.random.default_rng(4)
    sid = orc.open()
    prompt = _prompt(c, rng, 5)
    orc.start([(sid, prompt)])
    prev_row, prev_pending = list(prompt.first), list(prompt.pending)
    for t in range(4):
        caller = list(rng.integers(0, c.card, 8))
        em = orc.tick([(sid, Step(caller=caller, seed=t))])[0]
        drawn = list(orc.drawn[0])
        assert list(orc.rows[0]) == prev_row
        assert 0 <= drawn[0] < c.text_vocab and all(0 <= d < c.card for d in drawn[1:])
        nxt, pend, text, frame = O.advance(prev_row, prev_pending, drawn, caller)
        assert list(em) == [text] + frame
        prev_row, prev_pending = nxt, pend
    assert orc.sessions[sid]["pos"] == 9 and orc.sessions[sid]["frame"] == 4
    # same seeds, same draws
    orc2 = O.DuplexOracle(c, ck)
    sid2 = orc2.open()
    orc2.start([(sid2, prompt)])
    rng = np.random.default_rng(4)
    _prompt(c, rng, 5)
    caller = list(rng.integers(0, c.card, 8))
    orc2.tick([(sid2, Step(caller=caller, seed=0))])
    assert np.isfinite(orc2.text_logits).all() and np.isfinite(orc2.audio_logits).all()
