"""The streaming codec decoder of the Qwen3-TTS talker over the C ABI (include/omni_b200_codec.h).

Mirrors the decoder the reference builds into the tail of its `first` and `decode` programs
(crates/omni-qwen3-tts/src/codec.rs:112-448): every call turns one new frame of 16 codes of each of up to `max_batch`
streams into `samples_per_frame` samples, nothing recomputed; what a frame needs from the past lives in the stream's
state slot. Field names follow the checkpoint JSON (`config::Codec`, crates/omni-qwen3-tts/src/config.rs:51-67).
"""
from __future__ import annotations

import ctypes as C
import zlib
from dataclasses import dataclass
from typing import Sequence, Tuple

import numpy as np

from . import lib as L
from .model import Denied, OmniError, c_tensors

GROUPS = 16  # quantizers per frame (crates/omni-qwen3-tts/src/talker.rs `GROUPS`)
KERNEL = 7   # taps of every decoder conv (codec.rs:46)


@dataclass(frozen=True)
class CodecConfig:
    codebook_size: int = 2048
    codebook_dim: int = 512
    latent_dim: int = 1024
    decoder_dim: int = 1536
    hidden_size: int = 512
    intermediate_size: int = 1024
    num_hidden_layers: int = 8
    num_attention_heads: int = 16
    head_dim: int = 64
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    sliding_window: int = 72
    num_quantizers: int = GROUPS
    upsample_rates: Tuple[int, ...] = (8, 5, 4, 3)
    upsampling_ratios: Tuple[int, ...] = (2, 2)

    @property
    def samples_per_frame(self) -> int:
        n = 1
        for r in self.upsampling_ratios + self.upsample_rates:
            n *= r
        return n

    def weight_bytes(self) -> int:
        """bf16 bytes of every matrix a frame's decode streams (the books count as the 16 rows a frame gathers)."""
        total = 0
        for name, shape in codec_tensor_shapes(self):
            if "_codebook" in name:
                continue
            n = 1
            for s in shape:
                n *= s
            total += 2 * n
        return total

    def flops_per_frame(self) -> int:
        """Multiply-add flops (2 per MAC) of the dense GEMMs one frame of one stream runs."""
        d, lat, h, inter = self.codebook_dim, self.latent_dim, self.hidden_size, self.intermediate_size
        qd = self.num_attention_heads * self.head_dim
        macs = d * d + 3 * d * lat + lat * h
        macs += self.num_hidden_layers * (3 * qd * h + qd * h + 3 * inter * h)
        macs += h * lat
        t = 1
        for r in self.upsampling_ratios:
            macs += t * r * lat * lat
            t *= r
            macs += t * 8 * lat * lat
        macs += t * KERNEL * lat * self.decoder_dim
        for i, r in enumerate(self.upsample_rates):
            cin, cout = self.decoder_dim >> i, self.decoder_dim >> (i + 1)
            macs += t * 2 * r * cout * cin
            t *= r
            macs += 3 * t * (KERNEL + 1) * cout * cout
        return 2 * macs


CODEC_PRESETS = {
    "qwen3-tts-12hz": CodecConfig(),
    # small shapes for parity tests; short frames, so a history longer than a frame's rows is exercised (dilation 9)
    "codec-tiny": CodecConfig(codebook_size=64, codebook_dim=64, latent_dim=64, decoder_dim=512, hidden_size=256,
                              intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                              upsample_rates=(4, 2, 2, 2), upsampling_ratios=(2, 2)),
    # the full model's rates and group structure at small widths
    "codec-mid": CodecConfig(codebook_size=128, codebook_dim=128, latent_dim=128, decoder_dim=512, hidden_size=256,
                             intermediate_size=512, num_hidden_layers=2, num_attention_heads=4),
}


def codec_tensor_shapes(c: CodecConfig):
    """Checkpoint tensors the decoder reads, by name (codec.rs:134-407)."""
    half, cb, dim, lat, h = c.codebook_dim // 2, c.codebook_size, c.codebook_dim, c.latent_dim, c.hidden_size
    qd, inter = c.num_attention_heads * c.head_dim, c.intermediate_size
    for p in ["decoder.quantizer.rvq_first.vq.layers.0"] + \
            [f"decoder.quantizer.rvq_rest.vq.layers.{i}" for i in range(GROUPS - 1)]:
        yield p + "._codebook.embedding_sum", (cb, half)
        yield p + "._codebook.cluster_usage", (cb,)
    yield "decoder.quantizer.rvq_first.output_proj.weight", (dim, half, 1)
    yield "decoder.quantizer.rvq_rest.output_proj.weight", (dim, half, 1)
    yield "decoder.pre_conv.conv.weight", (lat, dim, 3)
    yield "decoder.pre_conv.conv.bias", (lat,)
    pt = "decoder.pre_transformer"
    yield f"{pt}.input_proj.weight", (h, lat)
    yield f"{pt}.input_proj.bias", (h,)
    for i in range(c.num_hidden_layers):
        q = f"{pt}.layers.{i}."
        yield q + "input_layernorm.weight", (h,)
        yield q + "self_attn.q_proj.weight", (qd, h)
        yield q + "self_attn.k_proj.weight", (qd, h)
        yield q + "self_attn.v_proj.weight", (qd, h)
        yield q + "self_attn.o_proj.weight", (h, qd)
        yield q + "self_attn_layer_scale.scale", (h,)
        yield q + "post_attention_layernorm.weight", (h,)
        yield q + "mlp.gate_proj.weight", (inter, h)
        yield q + "mlp.up_proj.weight", (inter, h)
        yield q + "mlp.down_proj.weight", (h, inter)
        yield q + "mlp_layer_scale.scale", (h,)
    yield f"{pt}.norm.weight", (h,)
    yield f"{pt}.output_proj.weight", (lat, h)
    yield f"{pt}.output_proj.bias", (lat,)
    for i, r in enumerate(c.upsampling_ratios):
        p = f"decoder.upsample.{i}"
        yield f"{p}.0.conv.weight", (lat, lat, r)
        yield f"{p}.0.conv.bias", (lat,)
        yield f"{p}.1.dwconv.conv.weight", (lat, 1, KERNEL)
        yield f"{p}.1.dwconv.conv.bias", (lat,)
        yield f"{p}.1.norm.weight", (lat,)
        yield f"{p}.1.norm.bias", (lat,)
        yield f"{p}.1.pwconv1.weight", (4 * lat, lat)
        yield f"{p}.1.pwconv1.bias", (4 * lat,)
        yield f"{p}.1.gamma", (lat,)
        yield f"{p}.1.pwconv2.weight", (lat, 4 * lat)
        yield f"{p}.1.pwconv2.bias", (lat,)
    yield "decoder.decoder.0.conv.weight", (c.decoder_dim, lat, KERNEL)
    yield "decoder.decoder.0.conv.bias", (c.decoder_dim,)
    for i, rate in enumerate(c.upsample_rates):
        p = f"decoder.decoder.{i + 1}.block"
        cin, cout = c.decoder_dim >> i, c.decoder_dim >> (i + 1)
        yield f"{p}.0.alpha", (cin,)
        yield f"{p}.0.beta", (cin,)
        yield f"{p}.1.conv.weight", (cin, cout, 2 * rate)
        yield f"{p}.1.conv.bias", (cout,)
        for u in range(3):
            q = f"{p}.{u + 2}"
            yield f"{q}.act1.alpha", (cout,)
            yield f"{q}.act1.beta", (cout,)
            yield f"{q}.conv1.conv.weight", (cout, cout, KERNEL)
            yield f"{q}.conv1.conv.bias", (cout,)
            yield f"{q}.act2.alpha", (cout,)
            yield f"{q}.act2.beta", (cout,)
            yield f"{q}.conv2.conv.weight", (cout, cout, 1)
            yield f"{q}.conv2.conv.bias", (cout,)
    n = len(c.upsample_rates) + 1
    out_dim = c.decoder_dim >> len(c.upsample_rates)
    yield f"decoder.decoder.{n}.alpha", (out_dim,)
    yield f"decoder.decoder.{n}.beta", (out_dim,)
    yield f"decoder.decoder.{n + 1}.conv.weight", (1, out_dim, KERNEL)
    yield f"decoder.decoder.{n + 1}.conv.bias", (1,)


def codec_random_checkpoint(c: CodecConfig, seed: int = 0):
    """name -> float32 numpy array. Scales are chosen so activations keep unit order of magnitude through the 40-odd
    layers (fan-in scaled normal weights, small biases, norm gains near 1, layer scales 0.1, usage counts >= 1)."""
    out = {}
    for name, shape in codec_tensor_shapes(c):
        rng = np.random.default_rng((zlib.crc32(name.encode()) + seed) & 0x7fffffff)
        if name.endswith("cluster_usage"):
            t = rng.integers(1, 50, size=shape).astype(np.float32)
        elif name.endswith("embedding_sum"):
            usage = out[name.replace("embedding_sum", "cluster_usage")] if name.replace(
                "embedding_sum", "cluster_usage") in out else np.ones(shape[0], dtype=np.float32)
            t = rng.standard_normal(shape).astype(np.float32) * usage[:, None] * 0.5   # divided by the usage at load
        elif name.endswith("layernorm.weight") or name.endswith(".norm.weight"):
            t = 1.0 + 0.1 * rng.standard_normal(shape).astype(np.float32)
        elif name.endswith("layer_scale.scale") or name.endswith(".gamma"):
            t = np.full(shape, 0.1, dtype=np.float32) + 0.01 * rng.standard_normal(shape).astype(np.float32)
        elif name.endswith(".alpha") or name.endswith(".beta"):
            t = 0.3 * rng.standard_normal(shape).astype(np.float32)    # log-scale SnakeBeta parameters
        elif name.endswith(".bias"):
            t = 0.02 * rng.standard_normal(shape).astype(np.float32)
        else:
            fan_in = 1
            for s in shape[1:]:
                fan_in *= s
            gain = 1.0
            if "dwconv" in name:
                fan_in = KERNEL
            elif ".block.1.conv.weight" in name:
                fan_in = 2 * shape[0]                                  # transposed conv [in, out, 2 * rate]
            elif "upsample" in name and ".0.conv.weight" in name:
                fan_in = shape[0]                                      # transposed conv [in, out, r], stride = kernel
            elif ".conv2.conv.weight" in name:
                gain = 0.3                                             # residual branches stay below their stream
            elif name == f"decoder.decoder.{len(c.upsample_rates) + 2}.conv.weight":
                gain = 0.1                                             # keeps most of the waveform inside the clamp
            t = rng.standard_normal(shape).astype(np.float32) * (gain / np.sqrt(fan_in))
        out[name] = np.ascontiguousarray(t, dtype=np.float32)
    return out


class Stream:
    """One stream's lease of a state slot (the codec's share of `Seq`, crates/omni-qwen3-tts/src/model.rs)."""

    def __init__(self, model: "Codec", handle):
        self._model, self._h = model, handle

    @property
    def frames(self) -> int:
        return self._model._lib.omni_codec_stream_frames(self._h)

    def close(self):
        if self._h is not None:
            self._model._check(self._model._lib.omni_codec_close(self._model._m, self._h))
            self._h = None


class Codec:
    """`codec::build`'s decoder as a model of its own: `open` a stream, `decode` one frame of every given stream."""

    def __init__(self, cfg: CodecConfig, checkpoint: dict, max_batch: int = 64, streams: int = 0, device: int = 0,
                 use_graphs: bool = True):
        self.cfg = cfg
        self._lib = L.load()
        rates = list(cfg.upsampling_ratios) + [0] * (4 - len(cfg.upsampling_ratios))
        ups = list(cfg.upsample_rates) + [0] * (8 - len(cfg.upsample_rates))
        c = L.CodecCfg(cfg.codebook_size, cfg.codebook_dim, cfg.latent_dim, cfg.decoder_dim, cfg.hidden_size,
                       cfg.intermediate_size, cfg.num_hidden_layers, cfg.num_attention_heads, cfg.head_dim,
                       cfg.rms_norm_eps, cfg.rope_theta, cfg.sliding_window, cfg.num_quantizers,
                       len(cfg.upsampling_ratios), (C.c_int32 * 4)(*rates), len(cfg.upsample_rates),
                       (C.c_int32 * 8)(*ups), max_batch, streams or max_batch, 1 if use_graphs else 0)
        import torch
        checkpoint = {k: (torch.from_numpy(np.ascontiguousarray(v)) if isinstance(v, np.ndarray) else v)
                      for k, v in checkpoint.items()}
        arr, self._keep = c_tensors(checkpoint)
        m = C.c_void_p()
        rc = self._lib.omni_codec_create(C.byref(c), arr, len(checkpoint), device, C.byref(m))
        if rc != 0:
            msg = self._lib.omni_codec_last_error(m).decode() if m else "create failed"
            if m:
                self._lib.omni_codec_destroy(m)
            raise OmniError(rc, msg)
        self._m = m
        self.max_batch = max_batch

    def _check(self, rc):
        if rc in (L.DENIED_BUSY, L.DENIED_EXCEEDS_POOL):
            raise Denied("busy" if rc == L.DENIED_BUSY else "exceeds_pool")
        if rc != 0:
            raise OmniError(rc, self._lib.omni_codec_last_error(self._m).decode())

    def open(self) -> Stream:
        h = C.c_void_p()
        self._check(self._lib.omni_codec_open(self._m, C.byref(h)))
        return Stream(self, h)

    def warmup(self):
        self._check(self._lib.omni_codec_warmup(self._m))

    def decode(self, streams: Sequence[Stream], codes) -> np.ndarray:
        """codes [n, 16] int32 -> wav [n, samples_per_frame] float32; every stream advances by one frame."""
        n = len(streams)
        codes = np.ascontiguousarray(np.asarray(codes, dtype=np.int32).reshape(n, GROUPS))
        wav = np.empty((n, self.cfg.samples_per_frame), dtype=np.float32)
        hs = (C.c_void_p * n)(*[s._h for s in streams])
        self._check(self._lib.omni_codec_decode(self._m, n, hs, codes.ctypes.data_as(C.POINTER(C.c_int32)),
                                                wav.ctypes.data_as(C.POINTER(C.c_float))))
        return wav

    def stats(self):
        ms, launches = C.c_float(), C.c_int32()
        self._check(self._lib.omni_codec_stats(self._m, C.byref(ms), C.byref(launches)))
        return ms.value, launches.value

    def close(self):
        if self._m is not None:
            self._lib.omni_codec_destroy(self._m)
            self._m = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
