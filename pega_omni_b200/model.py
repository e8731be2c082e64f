"""Python mirror of the reference's talker model shell over the C ABI.

Names and argument meaning follow crates/omni-qwen3-tts/src/model.rs: ``Limits``, ``Seq``, ``Draw``,
``Out``, ``Model.{load, open, is_end, start, step, embeds, talker_logits, predictor_logits}``.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np

from . import lib as L
from .config import TalkerConfig

GROUPS = L.OMNI_GROUPS
NO_CODEC = -1  # prompt.rs:25
SAMPLES_PER_FRAME = 1920


class OmniError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"omni_b200 status {status}: {message}")
        self.status = status


class Denied(Exception):
    """`kern_pool::Denied`: ``busy`` passes when sequences close, ``exceeds_pool`` never will."""

    def __init__(self, kind: str):
        super().__init__(kind)
        self.kind = kind


@dataclass
class Limits:  # model.rs:56-64
    max_batch: int = 64
    max_tokens: int = 8192
    kv_gib: float = 16.0


@dataclass
class Prompt:  # prompt.rs:27-31
    text: list
    codec: list

    def __len__(self) -> int:
        return len(self.text)


@dataclass
class Draw:  # model.rs:75-79
    uniforms: Sequence[float] = field(default_factory=lambda: [0.5] * GROUPS)
    force: Optional[Sequence[int]] = None


@dataclass
class Out:  # model.rs:92-96
    codes: np.ndarray  # [n, 16] int32
    wav: np.ndarray    # [n, samples_per_frame] float32


class Seq:
    """One sequence's KV pages and state slot (model.rs:67-71)."""

    def __init__(self, model: "Model", handle: int, prompt: int):
        self._model, self._h, self.prompt = model, handle, prompt

    @property
    def frames(self) -> int:
        return L.load().omni_talker_seq_frames(self._h)


def _stack_cfg(c) -> L.StackCfg:
    return L.StackCfg(c.hidden_size, c.intermediate_size, c.num_hidden_layers, c.num_attention_heads,
                      c.num_key_value_heads, c.head_dim, c.vocab_size, c.rms_norm_eps, c.rope_theta)


def c_config(cfg: TalkerConfig, limits: Limits, use_graphs: bool = True, gemm_path: int = 0,
             tick_kernel: bool = True) -> L.TalkerCfg:
    g = cfg.generation
    return L.TalkerCfg(_stack_cfg(cfg.talker), _stack_cfg(cfg.predictor), cfg.num_code_groups,
                       cfg.tts_pad_token_id, cfg.codec_eos_token_id, g.temperature, g.top_k,
                       g.repetition_penalty, g.subtalker_temperature, g.subtalker_top_k, g.top_p,
                       1 if g.sampler == "philox" else 0, cfg.min_frames, cfg.control_tokens,
                       limits.max_batch, limits.max_tokens, limits.kv_gib, int(use_graphs), gemm_path,
                       int(tick_kernel))


def c_tensors(checkpoint: dict):
    """(array of omni_tensor, keep-alive list) from name -> torch tensor (bf16 or f32, host or device)."""
    import torch
    arr = (L.Tensor * len(checkpoint))()
    keep = []
    for i, (name, t) in enumerate(checkpoint.items()):
        if t.dtype == torch.bfloat16:
            dt = L.BF16
        elif t.dtype == torch.float32:
            dt = L.F32
        else:
            raise TypeError(f"{name}: dtype {t.dtype}")
        t = t.contiguous()
        bname = name.encode()
        keep += [t, bname]
        shape = (C.c_int64 * 4)(*(list(t.shape) + [0] * (4 - t.dim())))
        arr[i] = L.Tensor(bname, t.data_ptr(), dt, t.dim(), shape, L.DEVICE if t.is_cuda else L.HOST)
    return arr, keep


DRAW_DTYPE = np.dtype([("uniforms", np.float32, (GROUPS,)), ("force", np.int32, (GROUPS,))])


class DrawBatch:
    """The draws of one call as two arrays, laid out as the C ABI's `omni_draw[n]`: for callers that prepare a step's
    inputs ahead of time (an engine's staging buffer) instead of building `Draw` objects per row."""

    def __init__(self, uniforms, force=None):
        uniforms = np.asarray(uniforms, dtype=np.float32).reshape(-1, GROUPS)
        self.raw = np.zeros(len(uniforms), dtype=DRAW_DTYPE)
        self.raw["uniforms"] = uniforms
        self.raw["force"] = -1 if force is None else np.asarray(force, dtype=np.int32).reshape(-1, GROUPS)

    def __len__(self) -> int:
        return len(self.raw)

    def pointer(self):
        return self.raw.ctypes.data_as(C.POINTER(L.Draw))


def _draws(draws):
    if isinstance(draws, DrawBatch):
        return draws.pointer()
    arr = (L.Draw * len(draws))()
    for i, d in enumerate(draws):
        u = list(d.uniforms) + [0.5] * (GROUPS - len(d.uniforms))
        f = list(d.force) + [-1] * (GROUPS - len(d.force)) if d.force is not None else [-1] * GROUPS
        arr[i] = L.Draw((C.c_float * GROUPS)(*u), (C.c_int32 * GROUPS)(*f))
    return arr


class Model:
    def __init__(self, handle: int, config: TalkerConfig, limits: Limits):
        self._h, self.config, self.limits = handle, config, limits
        self._lib = L.load()

    # -- Model::load (model.rs:111-131) --
    @classmethod
    def load(cls, device: int, checkpoint: dict, config: TalkerConfig, limits: Limits = Limits(),
             use_graphs: bool = True, gemm_path: int = 0, tick_kernel: bool = True) -> "Model":
        lib = L.load()
        cfg = c_config(config, limits, use_graphs, gemm_path, tick_kernel)
        tensors, keep = c_tensors(checkpoint)
        h = C.c_void_p()
        rc = lib.omni_talker_create(C.byref(cfg), tensors, len(checkpoint), device, C.byref(h))
        del keep
        if rc != L.OK:
            msg = lib.omni_talker_last_error(h).decode() if h else "create failed"
            if h:
                lib.omni_talker_destroy(h)
            raise OmniError(rc, msg)
        return cls(h, config, limits)

    def close(self) -> None:
        if self._h:
            self._lib.omni_talker_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc: int) -> None:
        if rc != L.OK:
            raise OmniError(rc, self._lib.omni_talker_last_error(self._h).decode())

    # -- Model::open (model.rs:135-146) --
    def open(self, prompt: int, frames: int) -> Seq:
        h = C.c_void_p()
        rc = self._lib.omni_talker_open(self._h, prompt, frames, C.byref(h))
        if rc == L.DENIED_BUSY:
            raise Denied("busy")
        if rc == L.DENIED_EXCEEDS_POOL:
            raise Denied("exceeds_pool")
        self._check(rc)
        return Seq(self, h, prompt)

    def attach_codec(self, codec) -> None:
        """Puts a `pega_omni_b200.codec.Codec` behind this model (`omni_talker_attach_codec`): `start` / `step` then
        return the frames' samples in `Out.wav` as the reference's `first` / `decode` programs do. None detaches."""
        self._check(self._lib.omni_talker_attach_codec(self._h, codec._m if codec is not None else None))
        self._codec = codec  # kept alive as long as it is attached

    def release(self, seq: Seq) -> None:
        """Dropping a `Seq`: its lease returns to the pool."""
        self._check(self._lib.omni_talker_close(self._h, seq._h))
        seq._h = None

    def seed(self, seq: Seq, seed: int) -> None:
        self._check(self._lib.omni_talker_seq_seed(self._h, seq._h, seed))

    def is_end(self, frame) -> bool:  # model.rs:148-150
        return int(frame[0]) == self.config.codec_eos_token_id

    def _seq_array(self, seqs: Sequence[Seq]):
        key = tuple(id(s) for s in seqs)
        if getattr(self, "_seq_key", None) != key:  # the same batch call after call: keep its handle array
            self._seq_key, self._seq_arr = key, (C.c_void_p * len(seqs))(*[s._h for s in seqs])
        return self._seq_arr

    # -- Model::start (model.rs:153-177) --
    def start(self, rows: Sequence[tuple]) -> Out:
        n = len(rows)
        seqs = [r[0] for r in rows]
        text = np.asarray([t for r in rows for t in r[1].text], dtype=np.int32)
        codec = np.asarray([t for r in rows for t in r[1].codec], dtype=np.int32)
        lens = np.asarray([len(r[1]) for r in rows], dtype=np.int32)
        codes = np.zeros((n, GROUPS), dtype=np.int32)
        wav = np.zeros((n, SAMPLES_PER_FRAME), dtype=np.float32)
        i32p = C.POINTER(C.c_int32)
        self._check(self._lib.omni_talker_start(
            self._h, n, self._seq_array(seqs), text.ctypes.data_as(i32p), codec.ctypes.data_as(i32p),
            lens.ctypes.data_as(i32p), _draws([r[2] for r in rows]), codes.ctypes.data_as(i32p),
            wav.ctypes.data_as(C.POINTER(C.c_float))))
        return Out(codes, wav)

    # -- Model::step (model.rs:180-192) --
    def step(self, rows: Sequence[tuple]) -> Out:
        return self.step_batch([r[0] for r in rows], [r[1] for r in rows])

    def step_batch(self, seqs: Sequence[Seq], draws, out: Optional[Out] = None) -> Out:
        """`step` with the sequences and their draws as two parallel sequences; `draws` may be a `DrawBatch` and `out`
        a previous call's `Out` to write into (both spare per-row Python work in a tight serving loop)."""
        n = len(seqs)
        if out is None:
            out = Out(np.zeros((n, GROUPS), dtype=np.int32), np.zeros((n, SAMPLES_PER_FRAME), dtype=np.float32))
        self._check(self._lib.omni_talker_step(
            self._h, n, self._seq_array(seqs), _draws(draws),
            out.codes.ctypes.data_as(C.POINTER(C.c_int32)), out.wav.ctypes.data_as(C.POINTER(C.c_float))))
        return out

    def step_begin(self, seqs: Sequence[Seq], draws) -> None:
        """Enqueues one decode step and returns at once (`omni_talker_step_begin`); up to two may be under way."""
        self._check(self._lib.omni_talker_step_begin(self._h, len(seqs), self._seq_array(seqs), _draws(draws)))

    def step_end(self, n: int, out: Optional[Out] = None) -> Out:
        """Waits for the oldest step begun (of `n` sequences) and returns its frames."""
        if out is None:
            out = Out(np.zeros((n, GROUPS), dtype=np.int32), np.zeros((n, SAMPLES_PER_FRAME), dtype=np.float32))
        self._check(self._lib.omni_talker_step_end(
            self._h, out.codes.ctypes.data_as(C.POINTER(C.c_int32)), out.wav.ctypes.data_as(C.POINTER(C.c_float))))
        return out

    def run_ticks(self, seqs: Sequence[Seq], draws: Sequence[Sequence[Draw]]):
        """`len(draws)` decode ticks with all inputs staged on the device first; returns (codes, tick_ms)."""
        ticks, n = len(draws), len(seqs)
        flat = _draws([d for tick in draws for d in tick])
        codes = np.zeros((ticks, n, GROUPS), dtype=np.int32)
        ms = np.zeros(ticks, dtype=np.float32)
        self._check(self._lib.omni_talker_run_ticks(
            self._h, n, self._seq_array(seqs), ticks, flat, codes.ctypes.data_as(C.POINTER(C.c_int32)),
            ms.ctypes.data_as(C.POINTER(C.c_float))))
        return codes, ms

    # -- debug getters (model.rs:241-262); bf16 widened to f32 --
    def _read(self, what: int, s: int, count: int) -> np.ndarray:
        raw = np.zeros(count, dtype=np.uint16)
        self._check(self._lib.omni_talker_read(self._h, what, s, raw.ctypes.data, raw.nbytes))
        return (raw.astype(np.uint32) << 16).view(np.float32)

    def embeds(self, tokens: int) -> np.ndarray:
        h = self.config.talker.hidden_size
        return self._read(L.BUF_EMBEDS, 0, tokens * h).reshape(tokens, h)

    def talker_logits(self, s: int) -> np.ndarray:
        return self._read(L.BUF_LOGITS, s, self.config.talker.vocab_size)

    def predictor_logits(self, s: int) -> np.ndarray:
        g, v = self.config.num_code_groups - 1, self.config.predictor.vocab_size
        return self._read(L.BUF_P_LOGITS, s, g * v).reshape(g, v)

    def hidden(self, s: int) -> np.ndarray:
        return self._read(L.BUF_HIDDEN, s, self.config.talker.hidden_size)

    def pad_embed(self) -> np.ndarray:
        return self._read(L.BUF_PAD_EMBED, 0, self.config.talker.hidden_size)

    def trace(self, path) -> None:
        """Per-phase device timestamps of the last tick of every later `run_ticks` call go to `path` (None: off)."""
        self._check(self._lib.omni_talker_trace(self._h, str(path).encode() if path else None))

    def stats(self) -> L.Stats:
        st = L.Stats()
        self._check(self._lib.omni_talker_stats(self._h, C.byref(st)))
        return st
