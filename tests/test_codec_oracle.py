"""The codec decoder's CPU restatement pinned against itself: the streaming decoder (one frame per call, state carried in
histories, an overlap row and a 72-frame ring) must reproduce the whole-utterance decoder as published; with the bf16
roundings taken out the two are the same function, with them in the difference is rounding noise. Also the host side
of the C ABI that needs no GPU."""
import ctypes as C

import numpy as np
import pytest

from oracle import codec as oc
from pega_omni_b200.codec import CODEC_PRESETS, CodecConfig, codec_random_checkpoint, codec_tensor_shapes


def _codes(c, frames, seed=1):
    return np.random.default_rng(seed).integers(0, c.codebook_size, size=(frames, 16)).astype(np.int32)


def _stream(c, W, codes):
    so = oc.StreamOracle(c, W)
    return np.concatenate([so.step(f) for f in codes])


@pytest.mark.parametrize("preset,frames", [("codec-tiny", 80), ("codec-mid", 5)])
def test_streaming_is_the_whole_utterance_decoder_when_nothing_is_rounded(preset, frames, monkeypatch):
    # 80 frames of the tiny shape run past the 72-frame attention window and wrap the ring; its short frames also make
    # a history longer than a frame's rows (dilation 9 at 16 rows per frame)
    c = CODEC_PRESETS[preset]
    ck = codec_random_checkpoint(c, 0)
    codes = _codes(c, frames)
    monkeypatch.setattr(oc, "bf", lambda x: np.ascontiguousarray(x, dtype=np.float32))
    wav = _stream(c, oc.fold(ck, c), codes)
    ref = oc.whole_utterance(ck, c, codes)
    assert oc.snr_db(wav, ref) > 90.0  # f32 against f64


@pytest.mark.parametrize("preset,frames", [("codec-tiny", 12), ("codec-mid", 4)])
def test_bf16_streaming_stays_within_rounding_noise_of_the_whole_utterance_decoder(preset, frames):
    c = CODEC_PRESETS[preset]
    ck = codec_random_checkpoint(c, 0)
    codes = _codes(c, frames)
    wav = _stream(c, oc.fold(ck, c), codes)
    ref = oc.whole_utterance(ck, c, codes)
    assert np.abs(ref).max() <= 1.0 and (np.abs(ref) >= 1.0).mean() < 0.05  # the clamp is exercised but rare
    # the reference's own bar on a trained checkpoint is 30 dB (tests/golden.rs:156-162); random weights through
    # 40-odd bf16 layers give 26-28 dB
    assert oc.snr_db(wav, ref) > 22.0


def test_end_of_speech_code_reads_as_code_zero():
    c = CODEC_PRESETS["codec-tiny"]
    ck = codec_random_checkpoint(c, 0)
    W = oc.fold(ck, c)
    codes = _codes(c, 1)
    a = oc.StreamOracle(c, W).step(np.concatenate([[c.codebook_size + 102], codes[0, 1:]]))
    b = oc.StreamOracle(c, W).step(np.concatenate([[0], codes[0, 1:]]))
    assert np.array_equal(a, b)


def test_tap_layouts():
    w = np.arange(2 * 3 * 4, dtype=np.float32).reshape(2, 3, 4)      # [out, in, k]
    t = oc.conv_taps(w)
    assert t.shape == (2, 12) and t[1, 2 * 3 + 1] == w[1, 1, 2]      # tap-major: column j * in + c
    u = oc.transposed_taps(w)                                        # [in, out, k] -> [k * out, in]
    assert u.shape == (12, 2) and u[3 * 3 + 2, 1] == w[1, 2, 3]


def test_full_config_shapes_and_rates():
    c = CodecConfig()
    assert c.samples_per_frame == 1920
    names = dict(codec_tensor_shapes(c))
    assert names["decoder.decoder.1.block.1.conv.weight"] == (1536, 768, 16)
    assert names["decoder.decoder.6.conv.weight"] == (1, 96, 7)
    assert 4.5e9 < c.flops_per_frame() < 5.5e9


def test_config_struct_matches_header(built_lib):
    from pega_omni_b200 import lib as L
    assert C.sizeof(L.CodecCfg) == 120
    assert L.CodecCfg.max_batch.offset == 108 and L.CodecCfg.upsample_rates.offset == 76


def test_no_cpu_fallback_without_a_device(built_lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    from pega_omni_b200.codec import Codec
    from pega_omni_b200.model import OmniError
    c = CODEC_PRESETS["codec-tiny"]
    with pytest.raises(OmniError) as e:
        Codec(c, codec_random_checkpoint(c, 0), max_batch=1)
    assert e.value.status == -2  # OMNI_ERR_CUDA: the decoder exists on the GPU only


def test_codec_entry_points_refuse_null_handles(built_lib):
    """Argument checks run before anything touches a device, so they hold on a machine without one."""
    lib = built_lib
    INVALID = -1
    assert lib.omni_codec_open(None, None) == INVALID
    assert lib.omni_codec_close(None, None) == INVALID
    assert lib.omni_codec_warmup(None) == INVALID
    assert lib.omni_codec_decode(None, 1, None, None, None) == INVALID
    assert lib.omni_codec_stats(None, None, None) == INVALID
    assert lib.omni_codec_stream_frames(None) == -1
    assert lib.omni_codec_samples_per_frame(None) == -1
    assert lib.omni_talker_attach_codec(None, None) == INVALID
    assert lib.omni_codec_last_error(None) == b"null model"
    assert lib.omni_op_codec_rvq(None, None, None, None, 1, 8, 8) == INVALID
    assert lib.omni_op_codec_conv(None, None, 8, 8, 1, 1, None, 1, 1, None, 0, None, None, None) == INVALID
