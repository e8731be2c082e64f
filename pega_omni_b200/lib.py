"""ctypes binding of ``libomni_b200.so`` (declarations of include/omni_b200.h, omni_b200_ops.h, omni_b200_duplex.h,
omni_b200_higgs.h and omni_b200_codec.h).

Loading fails loudly when the library is missing: there is no fallback path.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libomni_b200.so"

OMNI_GROUPS = 16
OMNI_PAGE = 16
OK, DENIED_BUSY, DENIED_EXCEEDS_POOL = 0, 1, 2
ERR_INVALID, ERR_CUDA, ERR_DEVICE, ERR_MISSING_TENSOR, ERR_UNSUPPORTED = -1, -2, -3, -4, -5
BF16, F32 = 0, 1
HOST, DEVICE = 0, 1
BUF_LOGITS, BUF_P_LOGITS, BUF_EMBEDS, BUF_HIDDEN, BUF_PAD_EMBED = 0, 1, 2, 3, 4


class Tensor(C.Structure):
    _fields_ = [("name", C.c_char_p), ("data", C.c_void_p), ("dtype", C.c_int32), ("ndim", C.c_int32),
                ("shape", C.c_int64 * 4), ("location", C.c_int32)]


class StackCfg(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("hidden", "inter", "layers", "q_heads", "kv_heads", "head_dim", "vocab")] + \
               [("rms_eps", C.c_float), ("rope_theta", C.c_float)]


class TalkerCfg(C.Structure):
    _fields_ = [("talker", StackCfg), ("predictor", StackCfg), ("groups", C.c_int32),
                ("tts_pad_token_id", C.c_int32), ("codec_eos_token_id", C.c_int32),
                ("temperature", C.c_float), ("top_k", C.c_int32), ("repetition_penalty", C.c_float),
                ("sub_temperature", C.c_float), ("sub_top_k", C.c_int32), ("top_p", C.c_float),
                ("sampler", C.c_int32), ("min_frames", C.c_int32), ("control_tokens", C.c_int32),
                ("max_batch", C.c_int32), ("max_tokens", C.c_int32), ("kv_gib", C.c_double),
                ("use_graphs", C.c_int32), ("gemm_path", C.c_int32), ("tick_kernel", C.c_int32)]


class Draw(C.Structure):
    _fields_ = [("uniforms", C.c_float * OMNI_GROUPS), ("force", C.c_int32 * OMNI_GROUPS)]


class Stats(C.Structure):
    _fields_ = [("last_call_gpu_ms", C.c_float), ("last_call_launches", C.c_int32), ("bucket", C.c_int32),
                ("pages_total", C.c_int32), ("pages_used", C.c_int32), ("weight_bytes", C.c_int64),
                ("kv_bytes", C.c_int64)]


class DuplexCfg(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("dim", "layers", "heads", "hidden", "context", "dep_dim", "dep_layers",
                                         "dep_heads", "dep_hidden", "text_vocab", "card")] + \
               [("norm_eps", C.c_float), ("rope_period", C.c_float), ("text_temperature", C.c_float),
                ("text_top_k", C.c_int32), ("audio_temperature", C.c_float), ("audio_top_k", C.c_int32),
                ("max_sessions", C.c_int32), ("max_prefill", C.c_int32), ("voice_rows", C.c_int32),
                ("use_graphs", C.c_int32), ("tp_rank", C.c_int32), ("tp_size", C.c_int32)]


class CodecCfg(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("codebook_size", "codebook_dim", "latent_dim", "decoder_dim", "hidden_size",
                                         "intermediate_size", "num_hidden_layers", "num_attention_heads", "head_dim")] + \
               [("rms_norm_eps", C.c_float), ("rope_theta", C.c_float), ("sliding_window", C.c_int32),
                ("num_quantizers", C.c_int32), ("n_upsampling_ratios", C.c_int32), ("upsampling_ratios", C.c_int32 * 4),
                ("n_upsample_rates", C.c_int32), ("upsample_rates", C.c_int32 * 8), ("max_batch", C.c_int32),
                ("max_streams", C.c_int32), ("use_graphs", C.c_int32)]


class DuplexStep(C.Structure):
    _fields_ = [("force", C.c_int32 * 9), ("force_caller", C.c_int32 * 8), ("caller", C.c_int32 * 8),
                ("seed", C.c_uint64)]


class HiggsCfg(C.Structure):
    _fields_ = [("body", StackCfg), ("code_vocab", C.c_int32), ("temperature", C.c_float), ("top_k", C.c_int32),
                ("max_batch", C.c_int32), ("max_tokens", C.c_int32), ("kv_gib", C.c_double), ("use_graphs", C.c_int32),
                ("audio_adapter", C.c_int32)]


class HiggsDraw(C.Structure):
    _fields_ = [("uniforms", C.c_float * 8), ("force", C.c_int32 * 8), ("has_force", C.c_int32)]


class HiggsDelay(C.Structure):
    _fields_ = [("steps", C.c_int32), ("countdown", C.c_int32), ("done", C.c_int32)]


DUPLEX_TEXT_LOGITS, DUPLEX_AUDIO_LOGITS, DUPLEX_ROWS, DUPLEX_DRAWN = 0, 1, 2, 3

P = C.POINTER
VP = C.c_void_p
I32 = C.c_int32

# name -> (restype, argtypes): every symbol the two headers declare
SYMBOLS = {
    "omni_talker_create": (I32, [P(TalkerCfg), P(Tensor), I32, I32, P(VP)]),
    "omni_talker_destroy": (None, [VP]),
    "omni_talker_open": (I32, [VP, I32, I32, P(VP)]),
    "omni_talker_close": (I32, [VP, VP]),
    "omni_talker_seq_seed": (I32, [VP, VP, C.c_uint64]),
    "omni_talker_seq_frames": (I32, [VP]),
    "omni_talker_start": (I32, [VP, I32, P(VP), P(I32), P(I32), P(I32), P(Draw), P(I32), P(C.c_float)]),
    "omni_talker_step": (I32, [VP, I32, P(VP), P(Draw), P(I32), P(C.c_float)]),
    "omni_talker_step_begin": (I32, [VP, I32, P(VP), P(Draw)]),
    "omni_talker_step_end": (I32, [VP, P(I32), P(C.c_float)]),
    "omni_talker_run_ticks": (I32, [VP, I32, P(VP), I32, P(Draw), P(I32), P(C.c_float)]),
    "omni_talker_read": (I32, [VP, I32, I32, VP, C.c_size_t]),
    "omni_talker_is_end": (I32, [VP, P(I32)]),
    "omni_talker_stats": (I32, [VP, P(Stats)]),
    "omni_talker_trace": (I32, [VP, C.c_char_p]),
    "omni_talker_last_error": (C.c_char_p, [VP]),
    "omni_bucket": (I32, [I32]),
    "omni_version": (C.c_char_p, []),
    "omni_ops_create": (I32, [I32, P(VP)]),
    "omni_ops_destroy": (None, [VP]),
    "omni_ops_sync": (I32, [VP, P(C.c_uint32)]),
    "omni_ops_mark": (I32, [VP, I32]),
    "omni_ops_elapsed_ms": (I32, [VP, P(C.c_float)]),
    "omni_ops_last_error": (C.c_char_p, [VP]),
    "omni_op_gemm": (I32, [VP, VP, I32, I32, VP, I32, VP, I32, I32, I32, VP, I32]),
    "omni_op_norm_copy": (I32, [VP, VP, VP, VP, VP, I32, I32, C.c_float]),
    "omni_op_add_norm": (I32, [VP, VP, VP, VP, VP, I32, I32, C.c_float, I32, I32]),
    "omni_op_silu_mul": (I32, [VP, VP, VP, I32, I32]),
    "omni_op_rope_attend": (I32, [VP, VP, VP, VP, VP, I32, VP, VP, VP, VP, VP, I32, I32, I32, I32, C.c_float,
                                  C.c_float, VP]),
    "omni_op_sample": (I32, [VP, VP, I32, C.c_float, I32, C.c_float, C.c_float, I32, I32, I32, I32, VP, VP, VP, VP,
                             VP, C.c_int64, I32, I32, VP, I32, I32]),
    "omni_op_gemm_noalloc": (I32, [VP, I32, I32, VP, I32, VP, I32, I32, VP, I32, VP, C.c_char_p, C.c_size_t]),
    "omni_op_lm_norm": (I32, [VP, VP, VP, VP, VP, I32, I32, C.c_float]),
    "omni_op_lm_tp_add_norm": (I32, [VP, VP, VP, VP, VP, VP, I32, I32, C.c_float, VP]),
    "omni_op_lm_embed": (I32, [VP, VP, VP, I32, VP, I32, VP, I32, I32]),
    "omni_op_lm_rope_attend": (I32, [VP, VP, VP, I32, VP, VP, VP, VP, VP, I32, I32, C.c_float, C.c_float, I32, VP]),
    "omni_op_lm_dep_embed_norm": (I32, [VP, VP, I32, VP, I32, VP, VP, VP, VP, I32, I32, C.c_float]),
    "omni_op_lm_dep_kv_attend": (I32, [VP, VP, VP, I32, VP, I32, I32, C.c_float]),
    "omni_op_lm_sample": (I32, [VP, VP, I32, C.c_int64, C.c_float, I32, VP, VP, I32, VP, I32]),
    "omni_op_lm_advance": (I32, [VP, VP, VP, C.c_int64, VP, VP, VP, VP, VP, I32]),
    "omni_op_higgs_frame_embed": (I32, [VP, VP, VP, C.c_int64, VP, VP, I32, I32, I32]),
    "omni_op_higgs_sample": (I32, [VP, VP, I32, C.c_float, I32, VP, VP, VP, VP, C.c_int64, VP, I32]),
    "omni_op_codec_rvq": (I32, [VP, VP, VP, VP, I32, I32, I32]),
    "omni_op_codec_add_norm": (I32, [VP, VP, C.c_int64, VP, VP, VP, I32, I32, C.c_float]),
    "omni_op_codec_window_attend": (I32, [VP, VP, VP, VP, VP, C.c_int64, C.c_int64, VP, I32, I32, C.c_float]),
    "omni_op_codec_bias_gelu": (I32, [VP, VP, VP, C.c_int64, I32]),
    "omni_op_codec_bias_snake": (I32, [VP, VP, VP, VP, VP, VP, C.c_int64, I32]),
    "omni_op_codec_stage": (I32, [VP, VP, VP, VP, VP, VP, VP, VP, C.c_int64, C.c_int64, VP, I32, I32, I32, I32]),
    "omni_op_codec_gather_taps": (I32, [VP, VP, VP, I32, I32, I32, I32, I32]),
    "omni_op_codec_conv": (I32, [VP, VP, I32, I32, I32, I32, VP, I32, I32, VP, I32, VP, VP, VP]),
    "omni_op_codec_overlap_add": (I32, [VP, VP, VP, VP, VP, VP, C.c_int64, C.c_int64, VP, I32, I32, I32, I32]),
    "omni_op_codec_dwconv_ln": (I32, [VP, VP, VP, VP, VP, VP, VP, VP, VP, VP, C.c_int64, C.c_int64, VP, VP, I32, I32, I32,
                                      I32, C.c_float]),
    "omni_op_codec_out_conv": (I32, [VP, VP, VP, VP, VP, VP, VP, VP, VP, VP, C.c_int64, C.c_int64, VP, I32, I32, I32]),
    "omni_higgs_delay_forced_from": (I32, [P(HiggsDelay)]),
    "omni_higgs_delay_advance": (I32, [P(HiggsDelay), I32]),
    "omni_higgs_undelay": (I32, [P(I32), I32, P(I32)]),
    "omni_higgs_create": (I32, [P(HiggsCfg), P(Tensor), I32, I32, P(VP)]),
    "omni_higgs_destroy": (None, [VP]),
    "omni_higgs_last_error": (C.c_char_p, [VP]),
    "omni_higgs_open": (I32, [VP, I32, I32, P(VP)]),
    "omni_higgs_close": (I32, [VP, VP]),
    "omni_higgs_seq_rows": (I32, [VP]),
    "omni_higgs_start": (I32, [VP, I32, P(VP), P(I32), P(I32), P(HiggsDraw), P(I32), P(I32)]),
    "omni_higgs_step": (I32, [VP, I32, P(VP), P(HiggsDraw), P(I32), P(I32)]),
    "omni_higgs_warmup": (I32, [VP]),
    "omni_higgs_read_logits": (I32, [VP, I32, VP, C.c_size_t]),
    "omni_higgs_stats": (I32, [VP, P(C.c_float), P(I32)]),
    "omni_codec_create": (I32, [P(CodecCfg), P(Tensor), I32, I32, P(VP)]),
    "omni_codec_destroy": (None, [VP]),
    "omni_codec_last_error": (C.c_char_p, [VP]),
    "omni_codec_open": (I32, [VP, P(VP)]),
    "omni_codec_close": (I32, [VP, VP]),
    "omni_codec_stream_frames": (I32, [VP]),
    "omni_codec_samples_per_frame": (I32, [VP]),
    "omni_codec_warmup": (I32, [VP]),
    "omni_codec_decode": (I32, [VP, I32, P(VP), P(I32), P(C.c_float)]),
    "omni_codec_stats": (I32, [VP, P(C.c_float), P(I32)]),
    "omni_talker_attach_codec": (I32, [VP, VP]),
    "omni_duplex_create": (I32, [P(DuplexCfg), P(Tensor), I32, I32, P(VP)]),
    "omni_duplex_destroy": (None, [VP]),
    "omni_duplex_last_error": (C.c_char_p, [VP]),
    "omni_duplex_open": (I32, [VP, P(VP)]),
    "omni_duplex_close": (I32, [VP, VP]),
    "omni_duplex_position": (I32, [VP, P(I32), P(C.c_int64)]),
    "omni_duplex_is_cached": (I32, [VP, I32, P(I32), P(I32)]),
    "omni_duplex_warm_prefix": (I32, [VP, I32, P(I32), P(I32)]),
    "omni_duplex_start": (I32, [VP, I32, P(VP), P(I32), P(I32), P(I32), P(I32), P(I32)]),
    "omni_duplex_tick": (I32, [VP, I32, P(VP), P(DuplexStep), P(I32)]),
    "omni_duplex_warmup": (I32, [VP]),
    "omni_duplex_tp_export": (I32, [VP, VP, C.c_size_t]),
    "omni_duplex_tp_connect": (I32, [VP, VP, C.c_size_t]),
    "omni_duplex_read": (I32, [VP, I32, I32, VP, C.c_size_t]),
    "omni_duplex_stats": (I32, [VP, P(C.c_float), P(I32)]),
}

_lib = None


def load() -> C.CDLL:
    """The shared library with every prototype set. Raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m pega_omni_b200.build` "
                           "(there is no fallback implementation)")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export a declared symbol
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
