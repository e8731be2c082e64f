"""The delay pattern of the Higgs-style model (crates/omni-higgs-audio/src/delay.rs) through the C ABI: the
reference's own known answers and properties (crates/omni-higgs-audio/tests/delay.rs), restated."""
import numpy as np
from hypothesis import given, settings, strategies as st

from pega_omni_b200.higgs import BOC, CODEBOOKS, EOC, Delay, undelay


def delayed(frames):
    """Frames spread over delayed rows: codebook c starts c rows late and ends the run in EOC."""
    frames = np.asarray(frames, dtype=np.int32).reshape(-1, CODEBOOKS)
    rows = []
    for r in range(len(frames) + CODEBOOKS - 1):
        rows.append([BOC if r - c < 0 else (int(frames[r - c][c]) if r - c < len(frames) else EOC)
                     for c in range(CODEBOOKS)])
    return np.array(rows, dtype=np.int32).reshape(-1, CODEBOOKS)


def ends_at(firsts):
    d = Delay()
    for i, f in enumerate(firsts):
        if d.advance(f):
            return i
    return None


def test_the_ramp_unlocks_one_codebook_a_step(built_lib):
    d = Delay()
    forced = []
    for _ in range(CODEBOOKS + 2):
        forced.append(d.forced_from())
        d.advance(EOC)
    assert forced == [1, 2, 3, 4, 5, 6, 7, 8, 8, 8]
    d = Delay()
    assert d.force_row() == [-1] + [BOC] * 7


def test_an_end_inside_the_ramp_is_not_one(built_lib):
    d = Delay()
    assert all(not d.advance(EOC) for _ in range(CODEBOOKS))


@settings(max_examples=200, deadline=None)
@given(st.lists(st.lists(st.integers(0, BOC - 1), min_size=8, max_size=8), min_size=0, max_size=40))
def test_undelay_inverts_the_pattern(built_lib, frames):
    got = undelay(delayed(frames)) if frames else undelay(np.zeros((0, 8), np.int32))
    assert got.tolist() == [list(f) for f in frames]


def test_a_run_shorter_than_a_frame_has_none(built_lib):
    for n in range(CODEBOOKS):
        assert len(undelay(np.zeros((n, CODEBOOKS), np.int32))) == 0


@settings(max_examples=300, deadline=None)
@given(st.lists(st.integers(0, EOC), min_size=0, max_size=80))
def test_the_run_ends_a_countdown_after_the_first_end_past_the_ramp(built_lib, firsts):
    first_end = next((i for i, f in enumerate(firsts) if i >= CODEBOOKS and f == EOC), None)
    expected = None
    if first_end is not None and first_end + CODEBOOKS - 2 < len(firsts):
        expected = first_end + CODEBOOKS - 2
    assert ends_at(firsts) == expected


@settings(max_examples=100, deadline=None)
@given(st.lists(st.integers(0, EOC), min_size=40, max_size=80), st.integers(0, EOC))
def test_an_ended_run_stays_ended(built_lib, firsts, later):
    d = Delay()
    ended = any([d.advance(f) for f in firsts][-1:]) or False
    d2 = Delay()
    ended = False
    for f in firsts:
        ended = d2.advance(f) or ended
    assert (not ended) or d2.advance(later)
