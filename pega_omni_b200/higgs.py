"""Host side of the Higgs-style speech model's delay pattern over the C ABI (include/omni_b200_ops.h).

Names follow crates/omni-higgs-audio/src/delay.rs: ``Delay.forced_from``, ``Delay.advance``, ``undelay``; ``BOC`` and
``EOC`` are the last two codes of every codebook.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import lib as L

CODEBOOKS, BOC, EOC = 8, 1024, 1025


class Delay:
    """Which codebooks of the next step are not drawn, and when generation ends (delay.rs:19-46)."""

    def __init__(self):
        self._d = L.HiggsDelay(0, 0, 0)
        self._lib = L.load()

    def forced_from(self) -> int:
        return self._lib.omni_higgs_delay_forced_from(C.byref(self._d))

    def advance(self, first: int) -> bool:
        return bool(self._lib.omni_higgs_delay_advance(C.byref(self._d), int(first)))

    def force_row(self, draw_all: bool = False):
        """The `force` row of the next step: -1 for the codebooks that draw, BOC from `forced_from` on."""
        f = self.forced_from()
        return [-1 if b < f else BOC for b in range(CODEBOOKS)]


def undelay(rows) -> np.ndarray:
    """Frames inside delayed rows: frame t takes codebook c from row t + c (delay.rs:50-54)."""
    rows = np.ascontiguousarray(np.asarray(rows, dtype=np.int32).reshape(-1, CODEBOOKS))
    frames = np.zeros((max(len(rows) - CODEBOOKS + 1, 0), CODEBOOKS), dtype=np.int32)
    i32p = C.POINTER(C.c_int32)
    n = L.load().omni_higgs_undelay(rows.ctypes.data_as(i32p), len(rows), frames.ctypes.data_as(i32p))
    assert n == len(frames)
    return frames


# ---- the model shell (crates/omni-higgs-audio/src/model.rs) --------------------------------------------------------

from dataclasses import dataclass, field  # noqa: E402
from typing import Optional, Sequence  # noqa: E402

from .config import StackConfig  # noqa: E402
from .model import Denied, OmniError, c_tensors  # noqa: E402

VOCAB = 1026  # codes per codebook, BOC and EOC last (config.rs:13)


@dataclass
class HiggsConfig:
    """The body's shape (`config::Stack`) and `Sampling` (model.rs:84-87); defaults: the Higgs-style 4B body."""
    body: StackConfig = field(default_factory=lambda: StackConfig(
        hidden_size=2560, intermediate_size=9728, num_hidden_layers=36, num_attention_heads=20, num_key_value_heads=4,
        head_dim=128, vocab_size=128256, rms_norm_eps=1e-6, rope_theta=500000.0))
    code_vocab: int = VOCAB
    temperature: float = 1.0
    top_k: int = 50
    # a second, audio-only MLP of the same width beside every layer's MLP, run on audio positions (every decode row);
    # the reference's Higgs body has none
    audio_adapter: bool = False

    def step_weight_bytes(self) -> int:
        b = self.body
        q, kv = b.num_attention_heads * b.head_dim, b.num_key_value_heads * b.head_dim
        mlps = 2 if self.audio_adapter else 1
        layer = (q + 2 * kv) * b.hidden_size + b.hidden_size * q + mlps * 3 * b.intermediate_size * b.hidden_size
        return 2 * (b.num_hidden_layers * layer + CODEBOOKS * self.code_vocab * b.hidden_size)


HIGGS_PRESETS = {
    "higgs-4b": HiggsConfig(),
    # small shapes for parity tests: 5 query heads per kv head as in the full model
    "higgs-tiny": HiggsConfig(body=StackConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                                               num_attention_heads=5, num_key_value_heads=1, head_dim=64,
                                               vocab_size=300, rms_norm_eps=1e-6, rope_theta=500000.0)),
    "higgs-mid": HiggsConfig(body=StackConfig(hidden_size=512, intermediate_size=1408, num_hidden_layers=3,
                                              num_attention_heads=10, num_key_value_heads=2, head_dim=128,
                                              vocab_size=1000, rms_norm_eps=1e-6, rope_theta=500000.0)),
}


def higgs_tensor_shapes(c: HiggsConfig):
    b = c.body
    h, d = b.hidden_size, b.head_dim
    q, kv, i = b.num_attention_heads * d, b.num_key_value_heads * d, b.intermediate_size
    for l in range(b.num_hidden_layers):
        p = f"body.layers.{l}."
        yield p + "input_layernorm.weight", (h,)
        yield p + "self_attn.q_proj.weight", (q, h)
        yield p + "self_attn.k_proj.weight", (kv, h)
        yield p + "self_attn.v_proj.weight", (kv, h)
        yield p + "self_attn.q_norm.weight", (d,)
        yield p + "self_attn.k_norm.weight", (d,)
        yield p + "self_attn.o_proj.weight", (h, q)
        yield p + "post_attention_layernorm.weight", (h,)
        yield p + "mlp.gate_proj.weight", (i, h)
        yield p + "mlp.up_proj.weight", (i, h)
        yield p + "mlp.down_proj.weight", (h, i)
        if c.audio_adapter:
            yield p + "audio_mlp.gate_proj.weight", (i, h)
            yield p + "audio_mlp.up_proj.weight", (i, h)
            yield p + "audio_mlp.down_proj.weight", (h, i)
    yield "body.norm.weight", (h,)
    yield "tied.embedding.text_embedding.weight", (b.vocab_size, h)
    yield "tied.embedding.modality_embeddings.0.embedding.weight", (CODEBOOKS * c.code_vocab, h)


def higgs_random_checkpoint(c: HiggsConfig, seed: int = 0, std: float = 0.02, device="cpu", embed_std: float = 0.3):
    """name -> bf16 tensor: norm gains 1.0, the two embedding tables N(0, embed_std) (the fused one is also the output
    head), everything else N(0, std); per-tensor seeds derived from the names."""
    import zlib

    import torch
    on_device = torch.device(device).type == "cuda"
    out = {}
    for name, shape in higgs_tensor_shapes(c):
        if "norm" in name:
            t = torch.ones(shape, dtype=torch.float32, device=device if on_device else "cpu")
        else:
            g = torch.Generator(device=device if on_device else "cpu")
            g.manual_seed((zlib.crc32(name.encode()) + seed) & 0x7fffffff)
            s = embed_std if "embedding" in name else std
            t = torch.randn(shape, generator=g, dtype=torch.float32, device=device if on_device else "cpu") * s
        out[name] = t.to(torch.bfloat16).to(device)
    return out


@dataclass
class HiggsDraw:  # model.rs:99-104
    uniforms: Sequence[float] = field(default_factory=lambda: [0.5] * CODEBOOKS)
    force: Optional[Sequence[int]] = None


@dataclass
class HiggsOut:  # model.rs:114-117
    rows: np.ndarray   # [n, 8] int32: one delayed row of codes per sequence
    ended: np.ndarray  # [n] bool


class HiggsSeq:
    def __init__(self, handle, prompt: int):
        self._h, self.prompt = handle, prompt

    @property
    def rows(self) -> int:
        return L.load().omni_higgs_seq_rows(self._h)


class HiggsModel:
    def __init__(self, handle, config: HiggsConfig):
        self._h, self.config = handle, config
        self._lib = L.load()

    @classmethod
    def load(cls, device: int, checkpoint: dict, config: HiggsConfig, max_batch: int = 32, max_tokens: int = 8192,
             kv_gib: float = 4.0, use_graphs: bool = True) -> "HiggsModel":
        lib = L.load()
        b = config.body
        body = L.StackCfg(b.hidden_size, b.intermediate_size, b.num_hidden_layers, b.num_attention_heads,
                          b.num_key_value_heads, b.head_dim, b.vocab_size, b.rms_norm_eps, b.rope_theta)
        cfg = L.HiggsCfg(body, config.code_vocab, config.temperature, config.top_k, max_batch, max_tokens, kv_gib,
                         int(use_graphs), int(config.audio_adapter))
        tensors, keep = c_tensors(checkpoint)
        h = C.c_void_p()
        rc = lib.omni_higgs_create(C.byref(cfg), tensors, len(checkpoint), device, C.byref(h))
        del keep
        if rc != L.OK:
            msg = lib.omni_higgs_last_error(h).decode() if h else "create failed"
            if h:
                lib.omni_higgs_destroy(h)
            raise OmniError(rc, msg)
        return cls(h, config)

    def close(self):
        if self._h:
            self._lib.omni_higgs_destroy(self._h)
            self._h = None

    def _check(self, rc: int):
        if rc in (L.DENIED_BUSY, L.DENIED_EXCEEDS_POOL):
            raise Denied("busy" if rc == L.DENIED_BUSY else "exceeds_pool")
        if rc != L.OK:
            raise OmniError(rc, self._lib.omni_higgs_last_error(self._h).decode())

    def open(self, prompt: int, rows: int) -> HiggsSeq:  # model.rs:152-163
        h = C.c_void_p()
        self._check(self._lib.omni_higgs_open(self._h, prompt, rows, C.byref(h)))
        return HiggsSeq(h, prompt)

    def release(self, seq: HiggsSeq):
        self._check(self._lib.omni_higgs_close(self._h, seq._h))
        seq._h = None

    @staticmethod
    def _draws(draws):
        arr = (L.HiggsDraw * len(draws))()
        for i, d in enumerate(draws):
            f = list(d.force) if d.force is not None else [-1] * CODEBOOKS
            arr[i] = L.HiggsDraw((C.c_float * 8)(*d.uniforms), (C.c_int32 * 8)(*f), int(d.force is not None))
        return arr

    def _out(self, n):
        return np.zeros((n, CODEBOOKS), dtype=np.int32), np.zeros(n, dtype=np.int32)

    def start(self, rows: Sequence[tuple]) -> HiggsOut:  # model.rs:166-187; rows: [(seq, prompt ids, draw)]
        n = len(rows)
        handles = (C.c_void_p * n)(*[r[0]._h for r in rows])
        ids = np.ascontiguousarray(np.concatenate([np.asarray(r[1], dtype=np.int32) for r in rows]))
        lens = np.array([len(r[1]) for r in rows], dtype=np.int32)
        codes, ended = self._out(n)
        i32p = C.POINTER(C.c_int32)
        self._check(self._lib.omni_higgs_start(self._h, n, handles, ids.ctypes.data_as(i32p), lens.ctypes.data_as(i32p),
                                               self._draws([r[2] for r in rows]), codes.ctypes.data_as(i32p),
                                               ended.ctypes.data_as(i32p)))
        return HiggsOut(codes, ended.astype(bool))

    def warmup(self) -> None:
        """Every bucket's decode step on the padding lease, so live steps replay captured graphs."""
        rc = self._lib.omni_higgs_warmup(self._h)
        if rc != L.OK:
            raise OmniError(rc, self._lib.omni_higgs_last_error(self._h).decode())

    def step(self, rows: Sequence[tuple]) -> HiggsOut:  # model.rs:190-199; rows: [(seq, draw)]
        n = len(rows)
        handles = (C.c_void_p * n)(*[r[0]._h for r in rows])
        codes, ended = self._out(n)
        i32p = C.POINTER(C.c_int32)
        self._check(self._lib.omni_higgs_step(self._h, n, handles, self._draws([r[1] for r in rows]),
                                              codes.ctypes.data_as(i32p), ended.ctypes.data_as(i32p)))
        return HiggsOut(codes, ended.astype(bool))

    def logits(self, s: int) -> np.ndarray:  # model.rs:258-260
        raw = np.zeros(CODEBOOKS * self.config.code_vocab, dtype=np.uint16)
        self._check(self._lib.omni_higgs_read_logits(self._h, s, raw.ctypes.data_as(C.c_void_p), raw.nbytes))
        return (raw.astype(np.uint32) << 16).view(np.float32).reshape(CODEBOOKS, self.config.code_vocab)

    def stats(self):
        ms, launches = C.c_float(), C.c_int32()
        self._lib.omni_higgs_stats(self._h, C.byref(ms), C.byref(launches))
        return ms.value, launches.value
