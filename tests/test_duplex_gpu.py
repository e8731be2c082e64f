"""Parity of the duplex (PersonaPlex) path on the GPU, through the C ABI, against the CPU oracle."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def cosine(a, b):
    a, b = a.astype(np.float64).ravel(), b.astype(np.float64).ravel()
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-30))


def make_prompt(c, rng, steps, voice_rows=0):
    from pega_omni_b200.duplex import Prompt
    rows = rng.integers(0, c.card, (steps, 17)).astype(np.int32)
    rows[:, 0] = rng.integers(0, c.text_vocab, steps)
    rows[rng.random((steps, 17)) < 0.1] = -1
    first = rng.integers(0, c.card, 17)
    first[0] = rng.integers(0, c.text_vocab)
    voice = None
    if voice_rows:
        voice = [int(rng.integers(0, voice_rows)) if p < 2 else -1 for p in range(steps)]
    return Prompt(rows, list(first), list(rng.integers(0, c.card, 7)), [-1] * 9, voice)


def forced_step(c, rng, seed=0):
    from pega_omni_b200.duplex import Step
    force = [int(rng.integers(0, c.text_vocab))] + [int(v) for v in rng.integers(0, c.card, 8)]
    return Step(force=force, caller=[int(v) for v in rng.integers(0, c.card, 8)], seed=seed)


@pytest.mark.parametrize("preset,sessions", [("duplex-tiny", 3), ("duplex-mid", 12)])
def test_teacher_forced_ticks_match_oracle(built_lib, preset, sessions):
    """Forced draws keep both sides on the same token path; logits of every tick (text and the eight codebooks) are
    compared. duplex-tiny runs past its 40-position context, so the ring wraps; 12 sessions take the tensor-core GEMM
    path, 3 the vector path."""
    from oracle.duplex import DuplexOracle
    from pega_omni_b200.duplex import PRESETS, Model, random_checkpoint
    c = PRESETS[preset]
    ck = random_checkpoint(c, seed=1, voice_rows=4, head_std=0.15)
    m = Model.load(0, ck, c, max_sessions=16, max_prefill=256)
    orc = DuplexOracle(c, ck)
    rng = np.random.default_rng(5)
    lens = [int(rng.integers(3, 14)) for _ in range(sessions)]
    prompts = [make_prompt(c, rng, n, voice_rows=4 if i % 2 == 0 else 0) for i, n in enumerate(lens)]
    gs = [m.open() for _ in prompts]
    os_ = [orc.open() for _ in prompts]
    m.start(list(zip(gs, prompts)))
    orc.start(list(zip(os_, prompts)))
    ticks = 34 if preset == "duplex-tiny" else 6
    worst_steps, worst_cos = 0.0, 1.0
    for t in range(ticks):
        steps = [forced_step(c, rng, seed=t * 100 + i) for i in range(sessions)]
        out = m.tick(list(zip(gs, steps)))
        want = orc.tick(list(zip(os_, steps)))
        assert np.array_equal(out.emitted, want), (t, out.emitted, want)
        for i in range(sessions):
            assert np.array_equal(m.input_row(i), orc.rows[i])
            assert np.array_equal(m.drawn(i), orc.drawn[i])
            for got, ref in ((m.text_logits(i), orc.text_logits[i]), (m.audio_logits(i), orc.audio_logits[i])):
                # in bf16 steps of the reference value (a step is 2^-7 of its binade; 1.6e-2 at |x| in [2, 4))
                step = np.exp2(np.floor(np.log2(np.maximum(np.abs(ref), 2.0))) - 7)
                worst_steps = max(worst_steps, float((np.abs(got - ref) / step).max()))
                worst_cos = min(worst_cos, cosine(got, ref))
    assert gs[0].pos == lens[0] + ticks and gs[0].frame == ticks
    # logits are stored as bf16 on both sides: two bf16 steps (3.2e-2 at |logit| < 4, the north-star's 2e-2 is
    # 1.25 steps there), with different f32 summation orders in the GEMMs and FP8 keys and values in between
    assert worst_steps <= 2.0, worst_steps
    assert worst_cos >= 0.9995, worst_cos
    m.close()


def test_draws_agree_with_oracle_on_the_same_logits(built_lib):
    """Free-running ticks: every draw of the GPU is the oracle's draw on the GPU's own logits (`__logf` against
    `logf` may move a near-tie: at most 1 in 100), and the first tick takes what the prompt fixed."""
    from oracle import duplex as O
    from pega_omni_b200.duplex import PRESETS, Model, Step, random_checkpoint
    c = PRESETS["duplex-tiny"]
    ck = random_checkpoint(c, seed=2, head_std=0.3)
    m = Model.load(0, ck, c, max_sessions=8, max_prefill=64)
    rng = np.random.default_rng(6)
    n = 8
    prompts = [make_prompt(c, rng, 4) for _ in range(n)]
    for p in prompts:
        p.first_force = [7, 3, -1, -1, -1, -1, -1, -1, -1]
    gs = [m.open() for _ in range(n)]
    m.start(list(zip(gs, prompts)))
    total = same = 0
    for t in range(6):
        steps = [Step(caller=[int(v) for v in rng.integers(0, c.card, 8)], seed=(t << 32) | (i + 1)) for i in range(n)]
        m.tick(list(zip(gs, steps)))
        for i in range(n):
            d = m.drawn(i)
            if t == 0:
                assert d[0] == 7 and d[1] == 3
            lo, hi = steps[i].seed & 0xFFFFFFFF, steps[i].seed >> 32
            want = [O.sample(m.text_logits(i), c.text_temperature, c.text_top_k, lo, hi, 0)] + \
                   [O.sample(m.audio_logits(i)[k], c.audio_temperature, c.audio_top_k, lo, hi, 1 + k) for k in range(8)]
            for k in range(9):
                if t == 0 and k < 2:
                    continue
                total += 1
                same += int(d[k] == want[k])
    assert same >= total * 0.99, (same, total)
    m.close()


def test_lockstep_sessions_are_bit_identical_and_batch_independent(built_lib):
    """The same prompt and seeds in two slots of one call give identical logits and draws; a session alone gives the
    same draws as inside a batch (rows do not mix)."""
    from pega_omni_b200.duplex import PRESETS, Model, Step, random_checkpoint
    c = PRESETS["duplex-tiny"]
    ck = random_checkpoint(c, seed=3, head_std=0.3)
    rng = np.random.default_rng(7)
    prompt = make_prompt(c, rng, 6)
    other = make_prompt(c, rng, 9)
    callers = [[int(v) for v in rng.integers(0, c.card, 8)] for _ in range(5)]
    m = Model.load(0, ck, c, max_sessions=4, max_prefill=64)
    a, b, x = m.open(), m.open(), m.open()
    m.start([(a, prompt), (x, other), (b, prompt)])
    batch = []
    for t in range(5):
        st = Step(caller=callers[t], seed=t + 11)
        out = m.tick([(a, st), (x, Step(caller=callers[t], seed=99)), (b, st)])
        assert np.array_equal(out.emitted[0], out.emitted[2])
        assert np.array_equal(m.text_logits(0), m.text_logits(2))
        assert np.array_equal(m.audio_logits(0), m.audio_logits(2))
        batch.append(out.emitted[0].copy())
    m.close()
    m = Model.load(0, ck, c, max_sessions=4, max_prefill=64)
    s = m.open()
    m.start([(s, prompt)])
    for t in range(5):
        out = m.tick([(s, Step(caller=callers[t], seed=t + 11))])
        assert np.array_equal(out.emitted[0], batch[t])
    m.close()


def test_leases_and_validation(built_lib):
    from pega_omni_b200.duplex import PRESETS, Model, Step, random_checkpoint
    from pega_omni_b200.model import Denied, OmniError
    c = PRESETS["duplex-tiny"]
    ck = random_checkpoint(c, seed=4)
    m = Model.load(0, ck, c, max_sessions=2, max_prefill=16)
    rng = np.random.default_rng(8)
    a, b = m.open(), m.open()
    with pytest.raises(Denied) as e:
        m.open()
    assert e.value.kind == "busy"
    with pytest.raises(OmniError):  # not started
        m.tick([(a, Step())])
    with pytest.raises(OmniError):  # prompt longer than the ring leaves no room (model.rs:276)
        m.start([(a, make_prompt(c, rng, c.context))])
    with pytest.raises(OmniError):  # more rows than max_prefill
        m.start([(a, make_prompt(c, rng, 10)), (b, make_prompt(c, rng, 10))])
    bad = make_prompt(c, rng, 3)
    bad.rows[1, 4] = c.card + 5  # outside the table: the device error word, not an out-of-bounds read
    with pytest.raises(OmniError) as e2:
        m.start([(a, bad)])
    assert e2.value.status == -3
    m.release(b)
    b2 = m.open()  # the lease is free again, and the model is still usable after the device error
    m.start([(b2, make_prompt(c, rng, 4))])
    out = m.tick([(b2, Step(seed=5))])
    assert out.emitted.shape == (1, 9)
    with pytest.raises(OmniError):  # started twice
        m.start([(b2, make_prompt(c, rng, 4))])
    missing = dict(ck)
    del missing["d.l1.gate_out"]
    with pytest.raises(OmniError) as e3:
        Model.load(0, missing, c, max_sessions=2)
    assert e3.value.status == -4
    m.close()


def test_prefix_cache_copies_instead_of_prefilling(built_lib):
    """`warm_prefix` / `is_cached` / `start` (model.rs:243-370): a prompt is prefilled once into the cache; every
    session started with the same rows gets the cached keys and values copied into its ring, so sessions with the same
    prompt and seeds stay bit-identical, whether they start together or later; a different prompt is not confused
    with it; prompts longer than 256 rows and a ninth distinct prompt are prefilled directly."""
    import dataclasses
    from pega_omni_b200.duplex import PRESETS, Model, Prompt, Step, random_checkpoint
    c = dataclasses.replace(PRESETS["duplex-tiny"], context=400)
    ck = random_checkpoint(c, seed=5, voice_rows=3, head_std=0.3)
    m = Model.load(0, ck, c, max_sessions=12, max_prefill=600)
    rng = np.random.default_rng(9)
    p = make_prompt(c, rng, 21, voice_rows=3)
    q = make_prompt(c, rng, 21, voice_rows=3)
    assert not m.is_cached(p)
    m.warm_prefix(p)
    assert m.is_cached(p) and not m.is_cached(q)
    a, b, x = m.open(), m.open(), m.open()
    m.start([(a, p), (x, q), (b, p)])
    assert m.is_cached(q)
    callers = [[int(v) for v in rng.integers(0, c.card, 8)] for _ in range(4)]
    first = []
    for t in range(4):
        st = Step(caller=callers[t], seed=t + 3)
        out = m.tick([(a, st), (x, st), (b, st)])
        assert np.array_equal(out.emitted[0], out.emitted[2])
        assert np.array_equal(m.text_logits(0), m.text_logits(2)) and np.array_equal(m.audio_logits(0), m.audio_logits(2))
        first.append((out.emitted[0].copy(), m.text_logits(0).copy()))
    late = m.open()  # a later session with the same prompt reads the same cached prefix
    m.start([(late, p)])
    for t in range(4):
        out = m.tick([(late, Step(caller=callers[t], seed=t + 3))])
        assert np.array_equal(out.emitted[0], first[t][0]) and np.array_equal(m.text_logits(0), first[t][1])
    # not eligible: longer than 256 rows
    long_prompt = make_prompt(c, rng, 300)
    s = m.open()
    m.start([(s, long_prompt)])
    assert not m.is_cached(long_prompt) and s.pos == 300
    # the cache holds eight prompts; the ninth distinct one is prefilled directly and stays uncached
    others = [make_prompt(c, rng, 5) for _ in range(7)]
    for o in others:
        m.warm_prefix(o)
    assert all(m.is_cached(o) for o in others[:6]) and not m.is_cached(others[6])
    s2 = m.open()
    m.start([(s2, others[6])])
    out = m.tick([(s2, Step(seed=1))])
    assert out.emitted.shape == (1, 9) and not m.is_cached(others[6])
    m.close()


def test_cached_start_matches_direct_prefill_against_oracle(built_lib):
    """The copied prefix is the prefilled one: teacher-forced ticks after a cached start still match the oracle."""
    from oracle.duplex import DuplexOracle
    from pega_omni_b200.duplex import PRESETS, Model, random_checkpoint
    c = PRESETS["duplex-tiny"]
    ck = random_checkpoint(c, seed=6, head_std=0.15)
    m = Model.load(0, ck, c, max_sessions=4, max_prefill=64)
    orc = DuplexOracle(c, ck)
    rng = np.random.default_rng(10)
    p = make_prompt(c, rng, 9)
    g1, g2 = m.open(), m.open()
    o1, o2 = orc.open(), orc.open()
    m.start([(g1, p), (g2, p)])
    assert m.is_cached(p)
    orc.start([(o1, p), (o2, p)])
    for t in range(4):
        steps = [forced_step(c, rng, seed=t), forced_step(c, rng, seed=t + 50)]
        out = m.tick(list(zip([g1, g2], steps)))
        want = orc.tick(list(zip([o1, o2], steps)))
        assert np.array_equal(out.emitted, want)
        for i in range(2):
            ref = orc.text_logits[i]
            step = np.exp2(np.floor(np.log2(np.maximum(np.abs(ref), 2.0))) - 7)
            assert float((np.abs(m.text_logits(i) - ref) / step).max()) <= 2.0
            assert cosine(m.audio_logits(i), orc.audio_logits[i]) >= 0.9995
    m.close()


def test_graph_replay_equals_per_op_launches(built_lib):
    """A tick replayed as a CUDA graph (the default from the third tick of a bucket on) gives bit-identical draws and
    logits to the same tick issued kernel by kernel; ten and nine sessions share the bucket of 16 (six and seven rows
    on the padding lease), so a change of the session count in between replays the same graph."""
    from pega_omni_b200.duplex import PRESETS, Model, Step, random_checkpoint
    c = PRESETS["duplex-mid"]
    ck = random_checkpoint(c, seed=4, head_std=0.3)
    rng = np.random.default_rng(9)
    prompts = [make_prompt(c, rng, int(rng.integers(3, 9))) for _ in range(10)]
    callers = [[[int(v) for v in rng.integers(0, c.card, 8)] for _ in range(10)] for _ in range(8)]

    def run(use_graphs=True):
        m = Model.load(0, ck, c, max_sessions=16, max_prefill=256, use_graphs=use_graphs)
        ss = [m.open() for _ in prompts]
        m.start(list(zip(ss, prompts)))
        trace = []
        for t in range(8):
            live = ss if t not in (4, 5, 6) else ss[:9]  # three ticks with one session fewer
            out = m.tick([(s, Step(caller=callers[t][i], seed=17 * t + i)) for i, s in enumerate(live)])
            trace.append((out.emitted.copy(), m.text_logits(0).copy(), m.audio_logits(len(live) - 1).copy()))
        m.close()
        return trace

    replayed = run()
    launched = run(use_graphs=False)
    for t, (g, e) in enumerate(zip(replayed, launched)):
        for a, b in zip(g, e):
            assert np.array_equal(a, b), t


def test_warmup_takes_graph_capture_out_of_live_ticks(built_lib):
    """`Model::warmup` (crates/omni-personaplex/src/model.rs:202-240): afterwards the first live tick of a never-seen
    session count replays its bucket's graph: the same kernel count as the steady state and no slower than it by
    more than a quarter (a capture costs several times a tick)."""
    from pega_omni_b200.duplex import PRESETS, Model, Step, random_checkpoint
    c = PRESETS["duplex-mid"]
    ck = random_checkpoint(c, seed=4, head_std=0.3)
    rng = np.random.default_rng(10)
    m = Model.load(0, ck, c, max_sessions=16, max_prefill=256)
    m.warmup()
    prompts = [make_prompt(c, rng, int(rng.integers(3, 9))) for _ in range(5)]  # five sessions: bucket 8
    ss = [m.open() for _ in prompts]
    m.start(list(zip(ss, prompts)))
    steps = lambda t: [(s, Step(caller=[int(v) for v in rng.integers(0, c.card, 8)], seed=31 * t + i)) for i, s in enumerate(ss)]
    m.tick(steps(0))
    first_ms, first_launches = m.stats()
    steady = []
    for t in range(1, 7):
        m.tick(steps(t))
        steady.append(m.stats())
    assert all(n == first_launches for _, n in steady), (first_launches, steady)
    assert first_ms <= 1.25 * float(np.median([ms for ms, _ in steady])), (first_ms, steady)
    m.close()
