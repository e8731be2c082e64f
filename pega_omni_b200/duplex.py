"""Python mirror of the reference's duplex (PersonaPlex) model shell over the C ABI (include/omni_b200_duplex.h).

Names and argument meaning follow crates/omni-personaplex/src/model.rs: ``Session``, ``Step``, ``Out``,
``Model.{load, open, start, tick, input_row, text_logits, audio_logits}``; ``advance`` is the host specification
of the token bookkeeping (crates/omni-personaplex/src/prompt.rs:167-183).
"""
from __future__ import annotations

import ctypes as C
import zlib
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np

from . import lib as L
from .model import Denied, OmniError, c_tensors

STREAMS, CODEBOOKS, DRAWN, STATE = 17, 8, 9, 24
DEP_STEPS = 8


@dataclass
class DuplexConfig:
    """Shapes of crates/omni-personaplex/src/config.rs:5-37 (defaults: PersonaPlex-7B) and its sampling (:55-69)."""
    dim: int = 4096
    layers: int = 32
    heads: int = 32
    hidden: int = 11264
    context: int = 3000
    dep_dim: int = 1024
    dep_layers: int = 6
    dep_heads: int = 16
    dep_hidden: int = 2816
    text_vocab: int = 32000
    card: int = 2048
    norm_eps: float = 1e-8
    rope_period: float = 10000.0
    text_temperature: float = 0.7
    text_top_k: int = 25
    audio_temperature: float = 0.8
    audio_top_k: int = 250

    def tick_weight_bytes(self) -> int:
        """bf16 weight bytes one tick streams: Helium layers + text head + depformer input, 8 steps x layers, heads."""
        d, h, dd, dh = self.dim, self.hidden, self.dep_dim, self.dep_hidden
        helium = self.layers * (3 * d * d + d * d + 2 * h * d + d * h) + self.text_vocab * d
        dep = DEP_STEPS * dd * d + DEP_STEPS * (self.dep_layers * (3 * dd * dd + dd * dd + 2 * dh * dd + dd * dh) +
                                                 self.card * dd)
        return 2 * (helium + dep)


PRESETS = {
    "personaplex-7b": DuplexConfig(),
    # small shapes for parity tests: every kernel path (tensor-core and vector GEMM, ring wrap) at CPU-oracle cost
    "duplex-tiny": DuplexConfig(dim=256, layers=2, heads=2, hidden=512, context=40, dep_dim=256, dep_layers=2,
                                dep_heads=4, dep_hidden=384, text_vocab=320, card=96, text_top_k=25, audio_top_k=40),
    "duplex-mid": DuplexConfig(dim=512, layers=3, heads=4, hidden=1408, context=96, dep_dim=256, dep_layers=2,
                               dep_heads=4, dep_hidden=704, text_vocab=1000, card=256),
}


def tensor_shapes(c: DuplexConfig, voice_rows: int = 0):
    d, h, dd, dh, card1 = c.dim, c.hidden, c.dep_dim, c.dep_hidden, c.card + 1
    yield "h.text_emb", (c.text_vocab + 1, d)
    yield "h.audio_emb", (16 * card1, d)
    yield "h.out_norm", (d,)
    yield "h.text_linear", (c.text_vocab, d)
    for i in range(c.layers):
        p = f"h.l{i}."
        yield p + "norm1", (d,)
        yield p + "qkv", (3 * d, d)
        yield p + "o", (d, d)
        yield p + "norm2", (d,)
        yield p + "gate_up", (2 * h, d)
        yield p + "down", (d, h)
    yield "d.input", (DEP_STEPS * dd, d)
    yield "d.text_emb", (c.text_vocab + 1, dd)
    yield "d.emb", ((DEP_STEPS - 1) * card1, dd)
    yield "d.heads", (DEP_STEPS * c.card, dd)
    for i in range(c.dep_layers):
        p = f"d.l{i}."
        yield p + "norm1", (dd,)
        yield p + "qkv", (DEP_STEPS * 3 * dd, dd)
        yield p + "out", (DEP_STEPS * dd, dd)
        yield p + "norm2", (dd,)
        yield p + "gate_in", (DEP_STEPS * 2 * dh, dd)
        yield p + "gate_out", (DEP_STEPS * dd, dh)
    if voice_rows:
        yield "voices", (voice_rows, d)


def random_checkpoint(c: DuplexConfig, seed: int = 0, std: float = 0.02, device="cpu", voice_rows: int = 0,
                      head_std: Optional[float] = None):
    """name -> bf16 tensor: norm gains 1.0, embeddings N(0, 1) (so the first norm sees unit-scale rows), everything
    else N(0, std) from a per-tensor seed derived from its name; `head_std` widens the two output heads."""
    import torch
    out = {}
    on_device = torch.device(device).type == "cuda"  # full-size models are drawn on the GPU (a different stream of
    for name, shape in tensor_shapes(c, voice_rows):  # numbers than the CPU generator's: fine for timing)
        if "norm" in name:
            t = torch.ones(shape, dtype=torch.float32, device=device if on_device else "cpu")
        else:
            g = torch.Generator(device=device if on_device else "cpu")
            g.manual_seed((zlib.crc32(name.encode()) + seed) & 0x7fffffff)
            s = std
            if name.endswith("_emb") or name in ("d.emb", "voices"):
                s = 1.0
            elif head_std is not None and name in ("h.text_linear", "d.heads"):
                s = head_std
            t = torch.randn(shape, generator=g, dtype=torch.float32, device=device if on_device else "cpu") * s
        out[name] = t.to(torch.bfloat16).to(device)
    return out


@dataclass
class Step:  # model.rs:98-107, with the caller's codes in place of its PCM
    force: Sequence[int] = field(default_factory=lambda: [-1] * DRAWN)
    force_caller: Sequence[int] = field(default_factory=lambda: [-1] * CODEBOOKS)
    caller: Sequence[int] = field(default_factory=lambda: [0] * CODEBOOKS)
    seed: int = 0


@dataclass
class Prompt:
    """What `prompt::build` hands to prefill (prompt.rs:120-157): the rows, the first input row, the pending caller
    codes and what the first tick must take."""
    rows: np.ndarray                     # [steps, 17] int32, -1 = no token
    first: Sequence[int]                 # [17]
    pending: Sequence[int]               # [7]
    first_force: Sequence[int] = field(default_factory=lambda: [-1] * DRAWN)
    voice: Optional[Sequence[int]] = None  # per row: row of "voices" taken instead of the ids

    def __len__(self) -> int:
        return len(self.rows)


@dataclass
class Out:  # model.rs:111-116
    emitted: np.ndarray  # [n, 9] int32: the text token spoken now and the agent's frame


def advance(row, pending, drawn, caller):
    """`prompt::advance` (prompt.rs:167-183): (next row, next pending, text, frame)."""
    nxt = [drawn[k] if k <= CODEBOOKS else caller[0] if k == 1 + CODEBOOKS else pending[k - 2 - CODEBOOKS]
           for k in range(STREAMS)]
    return nxt, [caller[i + 1] for i in range(CODEBOOKS - 1)], row[0], [row[1]] + [drawn[1 + i] for i in range(1, CODEBOOKS)]


class Session:
    """A lease of `context` KV positions and a token-state slot (model.rs:82-95)."""

    def __init__(self, model: "Model", handle: int):
        self._model, self._h = model, handle

    def _where(self):
        pos, frame = C.c_int32(), C.c_int64()
        L.load().omni_duplex_position(self._h, C.byref(pos), C.byref(frame))
        return pos.value, frame.value

    @property
    def pos(self) -> int:
        return self._where()[0]

    @property
    def frame(self) -> int:
        return self._where()[1]


def shard_checkpoint(checkpoint: dict, c: "DuplexConfig", rank: int, size: int) -> dict:
    """Rank `rank`'s tensors of a tensor-parallel group of `size`: of every Helium layer the q, k and v rows of its
    heads, the matching columns of o, its gate and up rows and the matching columns of down; everything else whole."""
    d, h = c.dim, c.hidden
    dl, hl = d // size, h // size
    out = {}
    for name, t in checkpoint.items():
        if name.startswith("h.l") and name.endswith(".qkv"):
            parts = [t[k * d + rank * dl: k * d + (rank + 1) * dl] for k in range(3)]
            out[name] = _cat(parts)
        elif name.startswith("h.l") and name.endswith(".o"):
            out[name] = _contig(t[:, rank * dl:(rank + 1) * dl])
        elif name.startswith("h.l") and name.endswith(".gate_up"):
            out[name] = _cat([t[k * h + rank * hl: k * h + (rank + 1) * hl] for k in range(2)])
        elif name.startswith("h.l") and name.endswith(".down"):
            out[name] = _contig(t[:, rank * hl:(rank + 1) * hl])
        else:
            out[name] = t
    return out


def _cat(parts):
    if isinstance(parts[0], np.ndarray):
        return np.ascontiguousarray(np.concatenate(parts))
    import torch
    return torch.cat(parts).contiguous()


def _contig(t):
    return np.ascontiguousarray(t) if isinstance(t, np.ndarray) else t.contiguous()


class Model:
    def __init__(self, handle, config: DuplexConfig, max_sessions: int):
        self._h, self.config, self.max_sessions = handle, config, max_sessions
        self._lib = L.load()

    @classmethod
    def load(cls, device: int, checkpoint: dict, config: DuplexConfig, max_sessions: int = 128,
             max_prefill: int = 2048, use_graphs: bool = True, tp_rank: int = 0, tp_size: int = 1) -> "Model":
        """`tp_size = 2`: this process is rank `tp_rank` of a tensor-parallel pair; `checkpoint` is the whole model and
        the rank's rows / columns of Helium's projections are cut out here (`shard_checkpoint`). The pair must then be
        connected: each rank's `tp_export()` bytes go to the other rank's `tp_connect()`."""
        lib = L.load()
        c = config
        if tp_size > 1:
            checkpoint = shard_checkpoint(checkpoint, c, tp_rank, tp_size)
        voice_rows = checkpoint["voices"].shape[0] if "voices" in checkpoint else 0
        cfg = L.DuplexCfg(c.dim, c.layers, c.heads, c.hidden, c.context, c.dep_dim, c.dep_layers, c.dep_heads,
                          c.dep_hidden, c.text_vocab, c.card, c.norm_eps, c.rope_period, c.text_temperature,
                          c.text_top_k, c.audio_temperature, c.audio_top_k, max_sessions, max_prefill, voice_rows,
                          int(use_graphs), tp_rank, tp_size)
        tensors, keep = c_tensors(checkpoint)
        h = C.c_void_p()
        rc = lib.omni_duplex_create(C.byref(cfg), tensors, len(checkpoint), device, C.byref(h))
        del keep
        if rc != L.OK:
            msg = lib.omni_duplex_last_error(h).decode() if h else "create failed"
            if h:
                lib.omni_duplex_destroy(h)
            raise OmniError(rc, msg)
        return cls(h, config, max_sessions)

    def close(self):
        if self._h:
            self._lib.omni_duplex_destroy(self._h)
            self._h = None

    def tp_export(self) -> bytes:
        """The handle under which the other rank's process maps this rank's exchange region."""
        buf = C.create_string_buffer(64)
        self._check(self._lib.omni_duplex_tp_export(self._h, buf, 64))
        return buf.raw

    def tp_connect(self, peer_handle: bytes) -> None:
        buf = C.create_string_buffer(bytes(peer_handle), 64)
        self._check(self._lib.omni_duplex_tp_connect(self._h, buf, 64))

    def _check(self, rc: int):
        if rc in (L.DENIED_BUSY, L.DENIED_EXCEEDS_POOL):
            raise Denied("busy" if rc == L.DENIED_BUSY else "exceeds_pool")
        if rc != L.OK:
            raise OmniError(rc, self._lib.omni_duplex_last_error(self._h).decode())

    # -- Model::open (model.rs:287-296) --
    def open(self) -> Session:
        h = C.c_void_p()
        self._check(self._lib.omni_duplex_open(self._h, C.byref(h)))
        return Session(self, h)

    def release(self, session: Session):
        self._check(self._lib.omni_duplex_close(self._h, session._h))
        session._h = None

    def _prompt_arrays(self, prompt: "Prompt"):
        ids = np.ascontiguousarray(np.asarray(prompt.rows, dtype=np.int32).reshape(-1, STREAMS))
        voice = None if prompt.voice is None else np.ascontiguousarray(np.asarray(prompt.voice, dtype=np.int32))
        return ids, voice

    # -- Model::is_cached / warm_prefix (model.rs:243-259) --
    def is_cached(self, prompt: "Prompt") -> bool:
        ids, voice = self._prompt_arrays(prompt)
        i32p = C.POINTER(C.c_int32)
        return bool(self._lib.omni_duplex_is_cached(self._h, len(ids), ids.ctypes.data_as(i32p),
                                                    voice.ctypes.data_as(i32p) if voice is not None else None))

    def warm_prefix(self, prompt: "Prompt"):
        ids, voice = self._prompt_arrays(prompt)
        i32p = C.POINTER(C.c_int32)
        self._check(self._lib.omni_duplex_warm_prefix(self._h, len(ids), ids.ctypes.data_as(i32p),
                                                      voice.ctypes.data_as(i32p) if voice is not None else None))

    # -- Model::start (model.rs:325-370) --
    def start(self, rows: Sequence[tuple]):
        """rows: [(session, prompt)]."""
        n = len(rows)
        handles = (C.c_void_p * n)(*[s._h for s, _ in rows])
        counts = np.array([len(p) for _, p in rows], dtype=np.int32)
        ids = np.ascontiguousarray(np.concatenate([np.asarray(p.rows, dtype=np.int32).reshape(-1, STREAMS)
                                                   for _, p in rows]))
        any_voice = any(p.voice is not None for _, p in rows)
        voice = np.ascontiguousarray(np.concatenate(
            [np.asarray(p.voice if p.voice is not None else [-1] * len(p), dtype=np.int32) for _, p in rows]))
        init = np.ascontiguousarray(np.array([list(p.first) + list(p.pending) for _, p in rows], dtype=np.int32))
        ff = np.ascontiguousarray(np.array([list(p.first_force) for _, p in rows], dtype=np.int32))
        i32p = C.POINTER(C.c_int32)
        self._check(self._lib.omni_duplex_start(self._h, n, handles, counts.ctypes.data_as(i32p),
                                                ids.ctypes.data_as(i32p),
                                                voice.ctypes.data_as(i32p) if any_voice else None,
                                                init.ctypes.data_as(i32p), ff.ctypes.data_as(i32p)))

    # -- Model::tick (model.rs:373-433) --
    def warmup(self) -> None:
        """`Model::warmup` (model.rs:202-240): every bucket's tick on the padding lease, so live ticks replay graphs."""
        self._check(self._lib.omni_duplex_warmup(self._h))

    def tick(self, rows: Sequence[tuple]) -> Out:
        """rows: [(session, step)]."""
        n = len(rows)
        handles = (C.c_void_p * n)(*[s._h for s, _ in rows])
        steps = (L.DuplexStep * n)()
        for i, (_, x) in enumerate(rows):
            steps[i] = L.DuplexStep((C.c_int32 * DRAWN)(*x.force), (C.c_int32 * CODEBOOKS)(*x.force_caller),
                                    (C.c_int32 * CODEBOOKS)(*x.caller), x.seed & 0xFFFFFFFFFFFFFFFF)
        emitted = np.zeros((n, DRAWN), dtype=np.int32)
        self._check(self._lib.omni_duplex_tick(self._h, n, handles, steps,
                                               emitted.ctypes.data_as(C.POINTER(C.c_int32))))
        return Out(emitted)

    def _read(self, which: int, s: int, count: int, dtype) -> np.ndarray:
        buf = np.zeros(count, dtype=dtype)
        self._check(self._lib.omni_duplex_read(self._h, which, s, buf.ctypes.data_as(C.c_void_p), buf.nbytes))
        return buf

    def _bf16(self, which: int, s: int, count: int) -> np.ndarray:
        raw = self._read(which, s, count, np.uint16)
        return (raw.astype(np.uint32) << 16).view(np.float32)

    def text_logits(self, s: int) -> np.ndarray:  # model.rs:446-448
        return self._bf16(L.DUPLEX_TEXT_LOGITS, s, self.config.text_vocab)

    def audio_logits(self, s: int) -> np.ndarray:  # model.rs:456-466
        return self._bf16(L.DUPLEX_AUDIO_LOGITS, s, DEP_STEPS * self.config.card).reshape(DEP_STEPS, self.config.card)

    def input_row(self, s: int) -> np.ndarray:  # model.rs:436-438
        return self._read(L.DUPLEX_ROWS, s, STREAMS, np.int32)

    def drawn(self, s: int) -> np.ndarray:
        return self._read(L.DUPLEX_DRAWN, s, DRAWN, np.int32)

    def stats(self):
        ms, launches = C.c_float(), C.c_int32()
        self._lib.omni_duplex_stats(self._h, C.byref(ms), C.byref(launches))
        return ms.value, launches.value
