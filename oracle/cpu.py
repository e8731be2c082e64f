"""ctypes wrapper of the CPU oracle (``talker_oracle.cpp``).

TEST INFRASTRUCTURE: imported only by tests, the smoke check and the benchmark's CPU-baseline leg.
Takes the same checkpoint-named tensors and the same config objects as the product (duck-typed:
anything with the attribute names of ``pega_omni_b200.config.TalkerConfig``).
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

LIB_PATH = Path(__file__).resolve().parent / "liboracle.so"
GROUPS = 16


class _Tensor(C.Structure):
    _fields_ = [("name", C.c_char_p), ("data", C.c_void_p), ("dtype", C.c_int32), ("ndim", C.c_int32),
                ("shape", C.c_int64 * 4), ("location", C.c_int32)]


class _Stack(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("hidden", "inter", "layers", "q_heads", "kv_heads", "head_dim", "vocab")] + \
               [("rms_eps", C.c_float), ("rope_theta", C.c_float)]


class _Config(C.Structure):
    _fields_ = [("talker", _Stack), ("predictor", _Stack), ("groups", C.c_int32), ("tts_pad_token_id", C.c_int32),
                ("codec_eos_token_id", C.c_int32), ("temperature", C.c_float), ("top_k", C.c_int32),
                ("repetition_penalty", C.c_float), ("sub_temperature", C.c_float), ("sub_top_k", C.c_int32),
                ("top_p", C.c_float), ("sampler", C.c_int32), ("min_frames", C.c_int32),
                ("control_tokens", C.c_int32)]


_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            from . import build
            build.build()
        lib = C.CDLL(str(LIB_PATH))
        lib.orc_create.restype = C.c_void_p
        lib.orc_create.argtypes = [C.POINTER(_Config), C.POINTER(_Tensor), C.c_int]
        lib.orc_destroy.argtypes = [C.c_void_p]
        lib.orc_open.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_uint64]
        lib.orc_close.argtypes = [C.c_void_p, C.c_int]
        vp = C.c_void_p
        lib.orc_start.argtypes = [vp, C.c_int, vp, vp, vp, vp, vp, vp, vp]
        lib.orc_step.argtypes = [vp, C.c_int, vp, vp, vp, vp]
        lib.orc_read.argtypes = [vp, C.c_int, C.c_int, vp, C.c_int64]
        lib.orc_gemm.argtypes = [vp, C.c_int, vp, C.c_int, C.c_int, vp]
        lib.orc_add_norm.argtypes = [vp, vp, vp, vp, C.c_int, C.c_int, C.c_float, C.c_int, C.c_int]
        lib.orc_norm_copy.argtypes = [vp, vp, vp, vp, C.c_int, C.c_int, C.c_float]
        lib.orc_silu_mul.argtypes = [vp, vp, C.c_int, C.c_int]
        lib.orc_rope_head.argtypes = [vp, vp, C.c_int, C.c_int, C.c_float, C.c_float]
        lib.orc_attend.argtypes = [vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, vp]
        lib.orc_sample.argtypes = [vp, C.c_int, C.c_float, C.c_int, C.c_float, C.c_float, C.c_int, C.c_int, C.c_int,
                                   C.c_int, C.c_int, C.c_float, C.c_int, vp, vp, C.c_int, C.c_int]
        lib.orc_philox_uniform.restype = C.c_float
        lib.orc_philox_uniform.argtypes = [C.c_uint64, C.c_uint32, C.c_uint32]
        lib.orc_f2bf.restype = C.c_uint16
        lib.orc_f2bf.argtypes = [C.c_float]
        lib.orc_set_threads.argtypes = [C.c_int]
        lib.orc_round_logits.argtypes = [C.c_int]
        _lib = lib
    return _lib


def bf16_bits(x: np.ndarray) -> np.ndarray:
    """f32 array -> bf16 bit patterns (uint16), round-to-nearest-even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return r.astype(np.uint16)


def bf16_round(x: np.ndarray) -> np.ndarray:
    return (bf16_bits(x).astype(np.uint32) << 16).view(np.float32)


def bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def _stack(c) -> _Stack:
    return _Stack(c.hidden_size, c.intermediate_size, c.num_hidden_layers, c.num_attention_heads,
                  c.num_key_value_heads, c.head_dim, c.vocab_size, c.rms_norm_eps, c.rope_theta)


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


class CpuOracle:
    """The whole talker frame loop on the CPU, same call shapes as the product's model shell."""

    def __init__(self, config, checkpoint: dict):
        import torch
        self.lib = load()
        g = config.generation
        self.config = config
        cfg = _Config(_stack(config.talker), _stack(config.predictor), config.num_code_groups,
                      config.tts_pad_token_id, config.codec_eos_token_id, g.temperature, g.top_k,
                      g.repetition_penalty, g.subtalker_temperature, g.subtalker_top_k, g.top_p,
                      1 if g.sampler == "philox" else 0, config.min_frames, config.control_tokens)
        arr = (_Tensor * len(checkpoint))()
        keep = []
        for i, (name, t) in enumerate(checkpoint.items()):
            t = t.detach().cpu().contiguous()
            dt = 0 if t.dtype == torch.bfloat16 else 1
            if dt == 1:
                t = t.float()
            b = name.encode()
            keep += [t, b]
            arr[i] = _Tensor(b, t.data_ptr(), dt, t.dim(), (C.c_int64 * 4)(*(list(t.shape) + [0] * (4 - t.dim()))), 0)
        self.h = self.lib.orc_create(C.byref(cfg), arr, len(checkpoint))
        if not self.h:
            raise RuntimeError("oracle: create failed (missing tensor?)")

    def close(self):
        if self.h:
            self.lib.orc_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def open(self, prompt: int, frames: int, seed: int = 0) -> int:
        return self.lib.orc_open(self.h, prompt, frames, seed)

    def release(self, sid: int) -> None:
        self.lib.orc_close(self.h, sid)

    @staticmethod
    def _draws(draws):
        n = len(draws)
        u = np.full((n, GROUPS), 0.5, dtype=np.float32)
        f = np.full((n, GROUPS), -1, dtype=np.int32)
        for i, d in enumerate(draws):
            uu = list(d.uniforms)
            u[i, :len(uu)] = uu
            if d.force is not None:
                ff = list(d.force)
                f[i, :len(ff)] = ff
        return u, f

    def start(self, sids, prompts, draws) -> np.ndarray:
        n = len(sids)
        text = np.asarray([t for p in prompts for t in p.text], dtype=np.int32)
        codec = np.asarray([t for p in prompts for t in p.codec], dtype=np.int32)
        lens = np.asarray([len(p.text) for p in prompts], dtype=np.int32)
        u, f = self._draws(draws)
        codes = np.zeros((n, GROUPS), dtype=np.int32)
        ids = np.asarray(sids, dtype=np.int32)
        rc = self.lib.orc_start(self.h, n, _ptr(ids), _ptr(text), _ptr(codec), _ptr(lens), _ptr(u), _ptr(f), _ptr(codes))
        if rc:
            raise RuntimeError(f"oracle start: {rc}")
        return codes

    def step(self, sids, draws) -> np.ndarray:
        n = len(sids)
        u, f = self._draws(draws)
        codes = np.zeros((n, GROUPS), dtype=np.int32)
        ids = np.asarray(sids, dtype=np.int32)
        rc = self.lib.orc_step(self.h, n, _ptr(ids), _ptr(u), _ptr(f), _ptr(codes))
        if rc:
            raise RuntimeError(f"oracle step: {rc}")
        return codes

    def _read(self, what, s, count):
        out = np.zeros(count, dtype=np.float32)
        rc = self.lib.orc_read(self.h, what, s, _ptr(out), count)
        if rc:
            raise RuntimeError("oracle read")
        return out

    def talker_logits(self, s):
        return self._read(0, s, self.config.talker.vocab_size)

    def predictor_logits(self, s):
        g, v = self.config.num_code_groups - 1, self.config.predictor.vocab_size
        return self._read(1, s, g * v).reshape(g, v)

    def embeds(self, tokens):
        h = self.config.talker.hidden_size
        return self._read(2, 0, tokens * h).reshape(tokens, h)

    def hidden(self, s):
        return self._read(3, s, self.config.talker.hidden_size)

    def pad_embed(self):
        return self._read(4, 0, self.config.talker.hidden_size)


# ---- operator-level oracles (inputs are f32 arrays holding bf16-representable values) ----

def gemm(x: np.ndarray, w_bits: np.ndarray) -> np.ndarray:
    rows, k = x.shape
    n = w_bits.shape[0]
    x = np.ascontiguousarray(x, dtype=np.float32)
    w_bits = np.ascontiguousarray(w_bits, dtype=np.uint16)
    y = np.zeros((rows, n), dtype=np.float32)
    load().orc_gemm(_ptr(x), rows, _ptr(w_bits), n, k, _ptr(y))
    return y


def add_norm(x, res, w_bits, eps, every=1, which=0):
    rows, dim = x.shape
    x = np.ascontiguousarray(x, dtype=np.float32)
    res = np.array(res, dtype=np.float32, copy=True)
    out = np.zeros(((rows + every - 1) // every, dim), dtype=np.float32)
    load().orc_add_norm(_ptr(x), _ptr(res), _ptr(np.ascontiguousarray(w_bits)), _ptr(out), rows, dim, eps, every, which)
    return out, res


def norm_copy(x, w_bits, eps):
    rows, dim = x.shape
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.zeros_like(x)
    res = np.zeros_like(x)
    load().orc_norm_copy(_ptr(x), _ptr(np.ascontiguousarray(w_bits)), _ptr(out), _ptr(res), rows, dim, eps)
    return out, res


def silu_mul(gate_up):
    rows, two_i = gate_up.shape
    gate_up = np.ascontiguousarray(gate_up, dtype=np.float32)
    act = np.zeros((rows, two_i // 2), dtype=np.float32)
    load().orc_silu_mul(_ptr(gate_up), _ptr(act), rows, two_i // 2)
    return act


def rope_head(head, w_bits, pos, eps, theta):
    h = np.array(head, dtype=np.float32, copy=True)
    load().orc_rope_head(_ptr(h), _ptr(np.ascontiguousarray(w_bits)), h.shape[0], pos, eps, theta)
    return h


def attend(q, kv_bits, hq, hk, d):
    """q: [hq*d] f32; kv_bits: [len, 2*hk*d] uint16 -> [hq*d]."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    kv_bits = np.ascontiguousarray(kv_bits, dtype=np.uint16)
    out = np.zeros(hq * d, dtype=np.float32)
    load().orc_attend(_ptr(q), _ptr(kv_bits), kv_bits.shape[0], hq, hk, d, _ptr(out))
    return out


def sample(logits, temperature, top_k, top_p, penalty, suppress_lo, suppress_hi, exempt, min_frames, frame, u, forced,
           last_frame, seen, penalize, group):
    """One sampler row; `last_frame` (int32[16]) and `seen` (uint32 bitmap) are updated in place."""
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    return load().orc_sample(_ptr(logits), logits.shape[0], temperature, top_k, top_p, penalty, suppress_lo,
                             suppress_hi, exempt, min_frames, frame, u, forced, _ptr(last_frame), _ptr(seen),
                             int(penalize), group)


def philox_uniform(seed: int, frame: int, group: int) -> float:
    return load().orc_philox_uniform(seed, frame, group)
