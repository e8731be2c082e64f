"""The streaming codec decoder on the GPU, through the C ABI, against the CPU restatement (oracle/codec.py): frame by
frame against the bf16 streaming oracle, and as a whole against the float64 whole-utterance decoder. The layout follows
the reference's own waveform test (crates/omni-qwen3-tts/tests/golden.rs:106-162): two streams fed the same frames in
one batch must agree bit for bit, and a stream that starts later must decode the same audio."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

from oracle import codec as oc  # noqa: E402
from pega_omni_b200.codec import CODEC_PRESETS, Codec, codec_random_checkpoint  # noqa: E402
from pega_omni_b200.model import Denied, OmniError  # noqa: E402


def _setup(preset, frames, seed=1):
    c = CODEC_PRESETS[preset]
    ck = codec_random_checkpoint(c, 0)
    codes = np.random.default_rng(seed).integers(0, c.codebook_size, size=(frames, 16)).astype(np.int32)
    so = oc.StreamOracle(c, oc.fold(ck, c))
    want = np.stack([so.step(f) for f in codes])
    return c, ck, codes, want


@pytest.mark.parametrize("preset,frames,graphs", [("codec-tiny", 6, False), ("codec-tiny", 80, True),
                                                  ("codec-mid", 5, True)])
def test_streams_match_the_oracle(built_lib, preset, frames, graphs):
    c, ck, codes, want = _setup(preset, frames)
    ref = oc.whole_utterance(ck, c, codes).reshape(frames, -1)
    m = Codec(c, ck, max_batch=4, use_graphs=graphs)
    a, b, late = m.open(), m.open(), m.open()
    lag = 2
    got, lagging = [], []
    for f in range(frames + lag):
        streams, rows = [], []
        if f < frames:
            streams += [a, b]
            rows += [codes[f], codes[f]]
        if f >= lag:
            streams.append(late)
            rows.append(codes[f - lag])
        w = m.decode(streams, np.stack(rows))
        if f < frames:
            assert np.array_equal(w[0], w[1]), "two streams of the same frames in one batch decode differently"
            got.append(w[0])
        if f >= lag:
            lagging.append(w[-1])
    got, lagging = np.stack(got), np.stack(lagging)
    assert a.frames == frames and late.frames == frames
    assert np.isfinite(got).all() and np.abs(got).max() <= 1.0
    # bit-equal bf16 values are not expected: the tensor-core GEMMs sum in another order than the oracle's, and one
    # flipped rounding travels through every later layer. Measured: 29-36 dB against the streaming oracle, and the same
    # distance from the float64 decoder as the oracle's own (26-28 dB)
    assert oc.snr_db(got, want) > 25.0
    assert oc.snr_db(got, ref) > oc.snr_db(want, ref) - 1.5
    assert oc.snr_db(got[0], want[0]) > 33.0  # the first frame has no rounding history behind it
    # the lagging stream ran in other batch rows and buckets: same audio up to the same noise
    assert oc.snr_db(lagging, want) > 25.0
    m.close()


def test_graph_replay_equals_per_op_launches(built_lib):
    c, ck, codes, _ = _setup("codec-tiny", 5)
    out = []
    for graphs in (False, True):
        m = Codec(c, ck, max_batch=2, use_graphs=graphs)
        if graphs:
            m.warmup()
        s = m.open()
        out.append(np.stack([m.decode([s], f[None])[0] for f in codes]))
        ms, launches = m.stats()
        assert launches > 50 and ms > 0
        m.close()
    assert np.array_equal(out[0], out[1])


def test_a_reopened_slot_starts_from_silence(built_lib):
    c, ck, codes, want = _setup("codec-tiny", 3)
    m = Codec(c, ck, max_batch=1, streams=1, use_graphs=False)
    s = m.open()
    first = np.stack([m.decode([s], f[None])[0] for f in codes])
    with pytest.raises(Denied):
        m.open()
    s.close()
    s = m.open()  # the same slot again: its histories, overlap rows and ring must read as zero
    again = np.stack([m.decode([s], f[None])[0] for f in codes])
    assert np.array_equal(first, again)
    m.close()


def test_end_of_speech_and_invalid_codes(built_lib):
    c, ck, codes, _ = _setup("codec-tiny", 1)
    m = Codec(c, ck, max_batch=2, use_graphs=False)
    a, b = m.open(), m.open()
    eos = codes[0].copy()
    eos[0] = c.codebook_size + 102   # the talker's end of speech in codebook 0 reads as code 0
    zero = codes[0].copy()
    zero[0] = 0
    w = m.decode([a, b], np.stack([eos, zero]))
    assert np.array_equal(w[0], w[1])
    bad = codes[0].copy()
    bad[3] = c.codebook_size
    with pytest.raises(OmniError):
        m.decode([a], bad[None])
    with pytest.raises(OmniError):
        m.decode([a, a], np.stack([zero, zero]))
    assert a.frames == 1  # a refused call advances nothing
    m.close()


def test_unsupported_shapes_are_refused(built_lib):
    import dataclasses
    c = dataclasses.replace(CODEC_PRESETS["codec-tiny"], sliding_window=64)
    with pytest.raises(OmniError) as e:
        Codec(c, codec_random_checkpoint(c, 0), max_batch=1)
    assert e.value.status == -5


def test_attached_decoder_fills_wav_of_start_and_step(built_lib):
    """`Out.wav` through the talker's own calls (what the reference's `first` / `decode` programs return): the samples
    are the ones a decoder of its own gives for the same frames, bit for bit, also through step_begin / step_end."""
    import dataclasses
    from pega_omni_b200.config import presets
    from pega_omni_b200.model import Draw, Limits, Model, Prompt
    from pega_omni_b200.synthetic import random_checkpoint
    cfg = presets["tiny128"]()
    model = Model.load(0, random_checkpoint(cfg, seed=0, device="cuda"), cfg, Limits(max_batch=4, max_tokens=128, kv_gib=0.01))
    cc = dataclasses.replace(CODEC_PRESETS["codec-mid"], codebook_size=2048)  # 1,920 samples per frame, 2048-entry books
    ck = codec_random_checkpoint(cc, 0)
    attached, apart = Codec(cc, ck, max_batch=4, streams=4), Codec(cc, ck, max_batch=4, streams=4)
    model.attach_codec(attached)
    rng = np.random.default_rng(3)
    lens = [9, 14, 11]
    prompts = [Prompt(list(rng.integers(0, cfg.text_vocab_size, n)), [-1] * n) for n in lens]
    seqs = [model.open(n, 8) for n in lens]
    streams = [apart.open() for _ in lens]
    draws = lambda: [Draw(list(rng.random(16).astype(np.float32))) for _ in lens]
    out = model.start(list(zip(seqs, prompts, draws())))
    frames = [(out.codes.copy(), out.wav.copy())]
    for _ in range(2):
        out = model.step(list(zip(seqs, draws())))
        frames.append((out.codes.copy(), out.wav.copy()))
    model.step_begin(seqs, draws())
    out = model.step_end(len(seqs))
    frames.append((out.codes.copy(), out.wav.copy()))
    for codes, wav in frames:
        assert np.abs(wav).max() > 0 and np.abs(wav).max() <= 1.0
        want = apart.decode(streams, codes)
        assert np.array_equal(wav, want)
    with pytest.raises(OmniError):
        model.attach_codec(None)  # sequences are open
    for s in seqs:
        model.release(s)
    model.attach_codec(None)
    model.close()
    attached.close()
    apart.close()


def test_full_size_decoder_at_64_streams_matches_the_oracle(built_lib):
    """The headline shape: the 12 Hz decoder's real widths and rates, 64 streams per call, three frames; two of the
    streams are checked frame by frame against the CPU restatement, two fed the same frames must agree bit for bit."""
    c = CODEC_PRESETS["qwen3-tts-12hz"]
    ck = codec_random_checkpoint(c, 0)
    W = oc.fold(ck, c)
    n, frames = 64, 3
    codes = np.random.default_rng(7).integers(0, c.codebook_size, size=(frames, n, 16)).astype(np.int32)
    codes[:, 1] = codes[:, 0]
    m = Codec(c, ck, max_batch=n)
    m.warmup()
    streams = [m.open() for _ in range(n)]
    got = np.stack([m.decode(streams, codes[f]) for f in range(frames)])        # [frames, n, 1920]
    assert np.isfinite(got).all() and np.abs(got).max() <= 1.0
    assert np.array_equal(got[:, 0], got[:, 1])
    for s in (0, 37):
        so = oc.StreamOracle(c, W)
        want = np.stack([so.step(codes[f, s]) for f in range(frames)])
        truth = oc.whole_utterance(ck, c, codes[:, s]).reshape(frames, -1)
        # with random weights the full-depth bf16 pipeline sits 24-25 dB from the float64 decoder whichever way its sums
        # are ordered (measured: this library 25.0 / 24.7 dB, the restatement 24.9 / 24.7 dB for the two streams, and
        # the same frame by frame); the two bf16 realisations are 24-32 dB apart
        assert oc.snr_db(got[:, s], truth) > oc.snr_db(want, truth) - 1.0, s
        assert oc.snr_db(got[:, s], want) > 21.0, s
        assert oc.snr_db(got[0, s], want[0]) > 25.0, s
    ms, launches = m.stats()
    assert launches == 134
    m.close()
