"""Operator-level calls (include/omni_b200_ops.h) over torch CUDA tensors, for parity tests and micro-benchmarks."""
from __future__ import annotations

import ctypes as C

from . import lib as L


class OpsError(RuntimeError):
    pass


def _p(t):
    return None if t is None else C.c_void_p(t.data_ptr())


class Ops:
    def __init__(self, device: int = 0):
        self._lib = L.load()
        h = C.c_void_p()
        rc = self._lib.omni_ops_create(device, C.byref(h))
        self._h = h
        if rc != L.OK:
            msg = self._lib.omni_ops_last_error(h).decode() if h else "create failed"
            raise OpsError(f"status {rc}: {msg}")

    def close(self):
        if self._h:
            self._lib.omni_ops_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc):
        if rc != L.OK:
            raise OpsError(f"status {rc}: {self._lib.omni_ops_last_error(self._h).decode()}")

    def sync(self):
        word = C.c_uint32(0)
        self._check(self._lib.omni_ops_sync(self._h, C.byref(word)))

    def mark(self, which: int):
        self._check(self._lib.omni_ops_mark(self._h, which))

    def elapsed_ms(self) -> float:
        ms = C.c_float(0)
        self._check(self._lib.omni_ops_elapsed_ms(self._h, C.byref(ms)))
        return ms.value

    def gemm(self, w, x, y, path=0, splits=0, bias=None, epilogue=0):
        n, k = w.shape
        rows = x.shape[0]
        assert x.shape[1] == k and y.shape[0] >= rows
        self._check(self._lib.omni_op_gemm(self._h, _p(w), n, k, _p(x), rows, _p(y), y.stride(0), path, splits,
                                           _p(bias), epilogue))

    def norm_copy(self, x, w, out, res, eps):
        self._check(self._lib.omni_op_norm_copy(self._h, _p(x), _p(w), _p(out), _p(res), x.shape[0], x.shape[1], eps))

    def add_norm(self, x, res, w, out, eps, every=1, which=0):
        self._check(self._lib.omni_op_add_norm(self._h, _p(x), _p(res), _p(w), _p(out), x.shape[0], x.shape[1], eps,
                                               every, which))

    def silu_mul(self, gate_up, act):
        self._check(self._lib.omni_op_silu_mul(self._h, _p(gate_up), _p(act), gate_up.shape[0], act.shape[1]))

    def rope_attend(self, qkv, q_norm, k_norm, kv, kv_pages, pos, slot, seq, indptr, pages, hq, hk, d, eps, theta,
                    out):
        self._check(self._lib.omni_op_rope_attend(self._h, _p(qkv), _p(q_norm), _p(k_norm), _p(kv), kv_pages, _p(pos),
                                                  _p(slot), _p(seq), _p(indptr), _p(pages), qkv.shape[0], hq, hk, d,
                                                  eps, theta, _p(out)))

    def sample(self, logits, temperature, top_k, top_p, penalty, suppress_lo, suppress_hi, exempt, min_frames, frames,
               uniforms, force, state, lines, stride, penalize, philox, codes, group):
        rows, vocab = logits.shape
        self._check(self._lib.omni_op_sample(self._h, _p(logits), vocab, temperature, top_k, top_p, penalty,
                                             suppress_lo, suppress_hi, exempt, min_frames, _p(frames), _p(uniforms),
                                             _p(force), _p(state), _p(lines), stride, penalize, philox, _p(codes),
                                             group, rows))


    # ---- duplex (PersonaPlex) kernels ----
    def lm_norm(self, x, alpha, out, eps, y=None):
        rows, dim = x.shape
        self._check(self._lib.omni_op_lm_norm(self._h, _p(y), _p(x), _p(alpha), _p(out), rows, dim, eps))

    def lm_tp_add_norm(self, mine, peer, x, alpha, out, eps, words):
        rows, dim = x.shape
        self._check(self._lib.omni_op_lm_tp_add_norm(self._h, _p(mine), _p(peer), _p(x), _p(alpha), _p(out), rows, dim,
                                                     eps, _p(words)))

    def lm_embed(self, ids, text_emb, audio_emb, out):
        rows, dim = out.shape
        self._check(self._lib.omni_op_lm_embed(self._h, _p(ids), _p(text_emb), text_emb.shape[0], _p(audio_emb),
                                               audio_emb.shape[0] // 16, _p(out), rows, dim))

    def lm_rope_attend(self, qkv, kv, kv_pages, pos, slot, seq, indptr, pages, heads, coef, scale, context, out):
        self._check(self._lib.omni_op_lm_rope_attend(self._h, _p(qkv), _p(kv), kv_pages, _p(pos), _p(slot), _p(seq),
                                                     _p(indptr), _p(pages), qkv.shape[0], heads, coef, scale, context,
                                                     _p(out)))

    def lm_dep_embed_norm(self, projected, k, table, drawn, alpha, x, xn, eps):
        rows, dim = x.shape
        self._check(self._lib.omni_op_lm_dep_embed_norm(self._h, _p(projected), k, _p(table), table.shape[0],
                                                        _p(drawn), _p(alpha), _p(x), _p(xn), rows, dim, eps))

    def lm_dep_kv_attend(self, qkv, ws, step, out, heads, scale):
        self._check(self._lib.omni_op_lm_dep_kv_attend(self._h, _p(qkv), _p(ws), step, _p(out), qkv.shape[0], heads,
                                                       scale))

    def lm_sample(self, logits, temperature, top_k, force, seeds, col, drawn):
        rows, vocab = logits.shape
        self._check(self._lib.omni_op_lm_sample(self._h, _p(logits), vocab, logits.stride(0), temperature, top_k,
                                                _p(force), _p(seeds), col, _p(drawn), rows))

    def lm_advance(self, state, lines, stride, rows, init=None, drawn=None, caller=None, force_caller=None,
                   emitted=None):
        self._check(self._lib.omni_op_lm_advance(self._h, _p(state), _p(lines), stride, _p(init), _p(drawn),
                                                 _p(caller), _p(force_caller), _p(emitted), rows))


    # ---- Higgs glue ----
    def higgs_frame_embed(self, state, lines, stride, table, out, vocab):
        rows, dim = out.shape
        self._check(self._lib.omni_op_higgs_frame_embed(self._h, _p(state), _p(lines), stride, _p(table), _p(out), rows,
                                                        dim, vocab))

    def higgs_sample(self, logits, temperature, top_k, uniforms, force, state, lines, stride, codes):
        rows, books, vocab = logits.shape
        assert books == 8
        self._check(self._lib.omni_op_higgs_sample(self._h, _p(logits), vocab, temperature, top_k, _p(uniforms),
                                                   _p(force), _p(state), _p(lines), stride, _p(codes), rows))

    # ---- streaming codec decoder (state: a byte tensor; lines / pos: int32 tensors, one entry per stream) ----
    def codec_rvq(self, codes, books, out, book_rows):
        n, dim = out.shape
        self._check(self._lib.omni_op_codec_rvq(self._h, _p(codes), _p(books), _p(out), n, dim // 2, book_rows))

    def codec_add_norm(self, add, res, w, out, eps):
        rows, dim = res.shape
        stride = 0 if add.dim() == 1 else dim
        self._check(self._lib.omni_op_codec_add_norm(self._h, _p(add), stride, _p(res), _p(w), _p(out), rows, dim, eps))

    def codec_window_attend(self, qkv, state, lines, pos, stride, ring_offset, out, heads, theta):
        self._check(self._lib.omni_op_codec_window_attend(self._h, _p(qkv), _p(state), _p(lines), _p(pos), stride,
                                                          ring_offset, _p(out), qkv.shape[0], heads, theta))

    def codec_bias_gelu(self, x, bias):
        rows, cols = x.shape
        self._check(self._lib.omni_op_codec_bias_gelu(self._h, _p(x), _p(bias), rows, cols))

    def codec_bias_snake(self, x, bias, alpha, inv_b, out):
        rows, cols = x.shape
        self._check(self._lib.omni_op_codec_bias_snake(self._h, _p(x), _p(bias), _p(alpha), _p(inv_b), _p(out), rows, cols))

    def codec_stage(self, x, bias, alpha, inv_b, state, lines, pos, stride, hist_offset, padded, n, T, H):
        C = x.shape[-1]
        self._check(self._lib.omni_op_codec_stage(self._h, _p(x), _p(bias), _p(alpha) if alpha is not None else None,
                                                  _p(inv_b) if inv_b is not None else None, _p(state), _p(lines), _p(pos),
                                                  stride, hist_offset, _p(padded), n, T, C, H))

    def codec_gather_taps(self, padded, col, n, T, C, taps, dil):
        self._check(self._lib.omni_op_codec_gather_taps(self._h, _p(padded), _p(col), n, T, C, taps, dil))

    def codec_conv(self, w, C, taps, dil, padded, T, n, y, epilogue=0, bias=None, alpha=None, inv_b=None):
        opt = lambda t: _p(t) if t is not None else None
        self._check(self._lib.omni_op_codec_conv(self._h, _p(w), w.shape[0], C, taps, dil, _p(padded), T, n, _p(y), epilogue,
                                                 opt(bias), opt(alpha), opt(inv_b)))

    def codec_overlap_add(self, z, bias, state, lines, pos, stride, prev_offset, out, n, L, r, C):
        self._check(self._lib.omni_op_codec_overlap_add(self._h, _p(z), _p(bias), _p(state), _p(lines), _p(pos), stride,
                                                        prev_offset, _p(out), n, L, r, C))

    def codec_dwconv_ln(self, z, zb, w, b, ln_w, ln_b, state, lines, pos, stride, hist_offset, xin, out, n, T, r, eps):
        C = xin.shape[-1]
        self._check(self._lib.omni_op_codec_dwconv_ln(self._h, _p(z), _p(zb), _p(w), _p(b), _p(ln_w), _p(ln_b), _p(state),
                                                      _p(lines), _p(pos), stride, hist_offset, _p(xin), _p(out), n, T, r, C,
                                                      eps))

    def codec_out_conv(self, x, bias, alpha, inv_b, w, wb, state, lines, pos, stride, hist_offset, wav, n, T):
        C = x.shape[-1]
        self._check(self._lib.omni_op_codec_out_conv(self._h, _p(x), _p(bias), _p(alpha), _p(inv_b), _p(w), _p(wb),
                                                     _p(state), _p(lines), _p(pos), stride, hist_offset, _p(wav), n, T, C))


def gemm_noalloc(w, x, y, splits=0, bias=None, epilogue=0, stream=None):
    """`omni_op_gemm_noalloc`: the tensor-core GEMM with its split-K scratch inside the library image, for callers
    that cannot allocate device memory (no context object, no cudaMalloc). Waits for the result; raises OpsError
    with the library's message on refusal."""
    lib = L.load()
    n, k = w.shape
    msg = C.create_string_buffer(512)
    rc = lib.omni_op_gemm_noalloc(_p(w), n, k, _p(x), x.shape[0], _p(y), y.stride(0), splits, _p(bias), epilogue,
                                  C.c_void_p(stream) if stream else None, msg, len(msg))
    if rc != L.OK:
        raise OpsError(f"status {rc}: {msg.value.decode()}")
