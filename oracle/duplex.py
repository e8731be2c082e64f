"""CPU restatement (numpy) of the reference's duplex (PersonaPlex) token loop. TEST INFRASTRUCTURE ONLY: nothing
outside tests/, the smoke check and bench.py's CPU legs may import this file.

What it follows, by reference file:line (paths inside the reference project):
  op order of a tick .......... crates/omni-personaplex/src/helium.rs:189-284, depformer.rs:137-259
  embedding sums .............. crates/omni-personaplex/kernels/lm.cu:25-43
  RMSNorm / add+norm / add .... lm.cu:74-120
  rotary + FP8 KV write ....... lm.cu:129-184 (pair rotation: kernels/attend.cuh:112-129)
  FP8 ring attention .......... lm.cu:197-290
  depformer embed / attention . lm.cu:301-366
  Gumbel-max top-k draw ....... lm.cu:368-537
  token bookkeeping ........... lm.cu:546-573, crates/omni-personaplex/src/prompt.rs:167-183
  ring positions, first force . crates/omni-personaplex/src/model.rs:373-433, :496

Rounding points are the reference's: every buffer it keeps in bf16 is rounded to bf16 here (f32 accumulation in
between), K and V are quantised to E4M3 per (token, head) with scale max(amax / 448, 1e-12).

Parity status: UNPINNED against a real checkpoint (the reference's golden files are not available offline). It is
pinned against the reference's own kernels replayed on a GPU (tests/test_duplex_replay_gpu.py): draws and token
bookkeeping bit-exact, the float kernels to a bf16 step.
"""
from __future__ import annotations

import numpy as np

STREAMS, BOOKS, DRAWN, STATE, DEP_STEPS = 17, 8, 9, 24, 8
HEAD, DEP_HEAD = 128, 64


def bf16r(x):
    """f32 -> nearest bf16 (ties to even), returned as f32."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return r.astype(np.uint32).view(np.float32).reshape(np.shape(x))


def e4m3(x):
    """f32 -> nearest E4M3 value (ties to even, saturating at 448), returned as f32."""
    x = np.asarray(x, dtype=np.float32)
    a = np.abs(x)
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(a > 0, a, 1.0)))
    e = np.maximum(e, -6.0)                      # below 2^-6 the grid is the subnormal one
    step = np.exp2(e - 3.0).astype(np.float32)   # 3 mantissa bits
    q = np.rint(a / step) * step
    q = np.minimum(q, 448.0)
    return (np.sign(x) * q).astype(np.float32)


def mix(x):
    x = np.asarray(x, dtype=np.uint64) & 0xFFFFFFFF
    x ^= x >> 16
    x = (x * 0x7FEB352D) & 0xFFFFFFFF
    x ^= x >> 15
    x = (x * 0x846CA68B) & 0xFFFFFFFF
    x ^= x >> 16
    return x


def order_key16(logits_bf16_as_f32):
    u = (np.ascontiguousarray(logits_bf16_as_f32, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint32)
    return np.where(u & 0x8000, (~u) & 0xFFFF, u | 0x8000)


def gumbel_scores(logits, temperature, top_k, seed_lo, seed_hi, col):
    """(scores f32 with -inf outside the top-k, kept mask) of `lm_sample` for one row (lm.cu:423-537)."""
    logits = np.asarray(logits, dtype=np.float32)
    vocab = logits.shape[0]
    keep = top_k if 0 < top_k < vocab else vocab
    key = order_key16(logits)
    kept = np.ones(vocab, dtype=bool)
    if temperature > 0 and keep < vocab:
        kept = key >= np.sort(key)[::-1][keep - 1]  # the k-th largest key; ties are kept
    inv_t = np.float32(1.0) / np.float32(temperature) if temperature > 0 else np.float32(1.0)
    score = logits * inv_t
    if temperature > 0:
        seed = mix((np.uint64(seed_lo) & 0xFFFFFFFF) ^
                   mix(((np.uint64(seed_hi) & 0xFFFFFFFF) + np.uint64(0x9E3779B9) * np.uint64(col + 1)) & 0xFFFFFFFF))
        u = ((mix(seed ^ mix(np.arange(vocab, dtype=np.uint64))) >> 8).astype(np.float32) + np.float32(0.5)) * \
            np.float32(1.0 / 16777216.0)
        with np.errstate(divide="ignore"):  # u rounds to 1.0 for the largest hash, as on the device
            score = (score - np.log(-np.log(u))).astype(np.float32)
    return np.where(kept, score, -np.inf).astype(np.float32), kept


def sample(logits, temperature, top_k, seed_lo, seed_hi, col):
    score, _ = gumbel_scores(logits, temperature, top_k, seed_lo, seed_hi, col)
    return int(np.argmax(score))  # first maximum = lowest index on ties


def advance(row, pending, drawn, caller):
    """`prompt::advance` (prompt.rs:167-183): (next row, next pending, text, frame)."""
    nxt = [drawn[k] if k <= BOOKS else caller[0] if k == 1 + BOOKS else pending[k - 2 - BOOKS] for k in range(STREAMS)]
    return nxt, [caller[i + 1] for i in range(BOOKS - 1)], row[0], [row[1]] + [drawn[1 + i] for i in range(1, BOOKS)]


def gemm(x, w):
    return bf16r(x.astype(np.float32) @ w.astype(np.float32).T)


def rms_norm(v, alpha, eps):
    r = np.float32(1.0) / np.sqrt((v.astype(np.float32) ** 2).mean(axis=-1, keepdims=True, dtype=np.float32) + np.float32(eps))
    return bf16r(v * (alpha * r))


def silu_mul(gu, inter):
    g, u = gu[..., :inter], gu[..., inter:]
    return bf16r(bf16r(g / (np.float32(1.0) + np.exp(-g))) * u)


def rope_pairs(x, pos, coef):
    """x: [..., 128] interleaved (real, imag) pairs; unrounded f32 result (attend.cuh:112-129)."""
    i = np.arange(HEAD // 2, dtype=np.float32)
    freq = np.exp(i * np.float32(coef)).astype(np.float32)
    ang = (freq * np.float32(pos)).astype(np.float32)
    c, s = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    r, im = x[..., 0::2], x[..., 1::2]
    out = np.empty_like(x, dtype=np.float32)
    out[..., 0::2] = r * c - im * s
    out[..., 1::2] = r * s + im * c
    return out


def quantize_heads(x):
    """x: [heads, 128] -> (E4M3 values as f32, scales [heads])."""
    amax = np.abs(x).max(axis=-1)
    sc = np.maximum(amax * np.float32(1.0 / 448.0), np.float32(1e-12)).astype(np.float32)
    inv = (np.float32(1.0) / sc).astype(np.float32)
    return e4m3(x * inv[:, None]), sc


class DuplexOracle:
    def __init__(self, cfg, checkpoint: dict):
        """checkpoint: name -> array-like of bf16-representable values (torch bf16 tensors or f32 arrays)."""
        self.c = cfg
        self.w = {}
        for k, v in checkpoint.items():
            self.w[k] = np.asarray(v.float().cpu().numpy() if hasattr(v, "float") else v, dtype=np.float32)
        self.coef = np.float32(-np.log(np.float64(cfg.rope_period)) * 2.0 / HEAD)
        self.sessions = {}
        self.next_id = 0
        self.text_logits = self.audio_logits = self.rows = self.drawn = None

    # -- leases --
    def open(self) -> int:
        c = self.c
        sid = self.next_id
        self.next_id += 1
        self.sessions[sid] = dict(pos=0, frame=0, state=[0] * STATE, first_force=[-1] * DRAWN,
                                  kq=np.zeros((c.layers, c.context, c.heads, HEAD), np.float32),
                                  ks=np.zeros((c.layers, c.context, c.heads), np.float32),
                                  vq=np.zeros((c.layers, c.context, c.heads, HEAD), np.float32),
                                  vs=np.zeros((c.layers, c.context, c.heads), np.float32))
        return sid

    # -- embeddings (lm.cu:25-43) --
    def embed(self, ids):
        c, w = self.c, self.w
        acc = np.zeros(c.dim, np.float32)
        for k in range(STREAMS):
            stream = k + 1 if k < STREAMS - 1 else 0
            i = int(ids[stream])
            if i < 0:
                continue
            row = w["h.text_emb"][i] if stream == 0 else w["h.audio_emb"][k * (c.card + 1) + i]
            acc = bf16r(acc + row)
        return acc

    # -- one Helium row through every layer (helium.rs:225-284) --
    def helium_row(self, s, x, pos):
        c, w = self.c, self.w
        D, nh = c.dim, c.heads
        scale = np.float32(1.0 / np.sqrt(np.float32(HEAD)))
        ring = pos % c.context
        xn = rms_norm(x, w["h.l0.norm1"], c.norm_eps)
        for i in range(c.layers):
            p = f"h.l{i}."
            qkv = gemm(xn, w[p + "qkv"]).reshape(3, nh, HEAD)
            q = bf16r(rope_pairs(qkv[0], pos, self.coef))
            kq, ks = quantize_heads(rope_pairs(qkv[1], pos, self.coef))
            vq, vs = quantize_heads(qkv[2])
            s["kq"][i, ring], s["ks"][i, ring], s["vq"][i, ring], s["vs"][i, ring] = kq, ks, vq, vs
            n = min(pos + 1, c.context)
            K, KS, V, VS = s["kq"][i, :n], s["ks"][i, :n], s["vq"][i, :n], s["vs"][i, :n]
            sc = np.einsum("hd,thd->ht", q, K).astype(np.float32) * (KS.T * scale)
            pr = np.exp(sc - sc.max(axis=1, keepdims=True)).astype(np.float32)
            attn = bf16r(np.einsum("ht,thd->hd", pr * VS.T, V) / pr.sum(axis=1, keepdims=True)).reshape(D)
            x = bf16r(x + gemm(attn, w[p + "o"]))
            xn = rms_norm(x, w[p + "norm2"], c.norm_eps)
            act = silu_mul(gemm(xn, w[p + "gate_up"]), c.hidden)
            x = bf16r(x + gemm(act, w[p + "down"]))
            xn = rms_norm(x, w[f"h.l{i + 1}.norm1"] if i + 1 < c.layers else w["h.out_norm"], c.norm_eps)
        return xn

    # -- Model::start (model.rs:325-370) --
    def start(self, rows):
        for sid, prompt in rows:
            s = self.sessions[sid]
            assert s["pos"] == 0
            for p, ids in enumerate(np.asarray(prompt.rows).reshape(-1, STREAMS)):
                v = -1 if prompt.voice is None else int(prompt.voice[p])
                x = self.w["voices"][v] if v >= 0 else self.embed(ids)
                self.helium_row(s, x, p)
            s["pos"], s["frame"] = len(prompt), 0
            s["state"] = list(prompt.first) + list(prompt.pending)
            s["first_force"] = list(prompt.first_force)

    # -- the eight depformer passes of one session (depformer.rs:137-259) --
    def depformer(self, xn, drawn, force, seed_lo, seed_hi):
        c, w = self.c, self.w
        D, H, nh = c.dep_dim, c.dep_hidden, c.dep_heads
        scale = np.float32(1.0 / np.sqrt(np.float32(DEP_HEAD)))
        proj = gemm(xn, w["d.input"]).reshape(DEP_STEPS, D)
        ws = np.zeros((c.dep_layers, DEP_STEPS, 2, nh, DEP_HEAD), np.float32)
        logits_all = np.zeros((DEP_STEPS, c.card), np.float32)
        for k in range(DEP_STEPS):
            table = w["d.text_emb"] if k == 0 else w["d.emb"][(k - 1) * (c.card + 1):k * (c.card + 1)]
            x = bf16r(proj[k] + table[drawn[k]])
            xn_d = rms_norm(x, w["d.l0.norm1"], c.norm_eps)
            for i in range(c.dep_layers):
                p = f"d.l{i}."
                qkv = gemm(xn_d, w[p + "qkv"][k * 3 * D:(k + 1) * 3 * D]).reshape(3, nh, DEP_HEAD)
                ws[i, k, 0], ws[i, k, 1] = qkv[1], qkv[2]
                sc = np.einsum("hd,thd->ht", qkv[0], ws[i, :k + 1, 0]).astype(np.float32) * scale
                pr = np.exp(sc - sc.max(axis=1, keepdims=True)).astype(np.float32)
                attn = bf16r(np.einsum("ht,thd->hd", pr, ws[i, :k + 1, 1]) / pr.sum(axis=1, keepdims=True)).reshape(D)
                x = bf16r(x + gemm(attn, w[p + "out"][k * D:(k + 1) * D]))
                xn_d = rms_norm(x, w[p + "norm2"], c.norm_eps)
                act = silu_mul(gemm(xn_d, w[p + "gate_in"][k * 2 * H:(k + 1) * 2 * H]), H)
                x = bf16r(x + gemm(act, w[p + "gate_out"][k * D:(k + 1) * D]))
                if i + 1 < c.dep_layers:
                    xn_d = rms_norm(x, w[f"d.l{i + 1}.norm1"], c.norm_eps)
            logits = gemm(x, w["d.heads"][k * c.card:(k + 1) * c.card])
            logits_all[k] = logits
            f = force[1 + k]
            drawn[1 + k] = f if f >= 0 else sample(logits, c.audio_temperature, c.audio_top_k, seed_lo, seed_hi, 1 + k)
        return logits_all

    # -- Model::tick (model.rs:373-433) --
    def tick(self, rows):
        c = self.c
        n = len(rows)
        emitted = np.zeros((n, DRAWN), np.int32)
        self.text_logits = np.zeros((n, c.text_vocab), np.float32)
        self.audio_logits = np.zeros((n, DEP_STEPS, c.card), np.float32)
        self.rows = np.zeros((n, STREAMS), np.int32)
        self.drawn = np.zeros((n, DRAWN), np.int32)
        for r, (sid, step) in enumerate(rows):
            s = self.sessions[sid]
            assert s["pos"] > 0
            force = [s["first_force"][k] if s["frame"] == 0 and step.force[k] < 0 else step.force[k] for k in range(DRAWN)]
            seed_lo, seed_hi = step.seed & 0xFFFFFFFF, (step.seed >> 32) & 0xFFFFFFFF
            row = s["state"][:STREAMS]
            self.rows[r] = row
            xn = self.helium_row(s, self.embed(row), s["pos"])
            tl = gemm(xn, self.w["h.text_linear"])
            self.text_logits[r] = tl
            drawn = [0] * DRAWN
            drawn[0] = force[0] if force[0] >= 0 else sample(tl, c.text_temperature, c.text_top_k, seed_lo, seed_hi, 0)
            self.audio_logits[r] = self.depformer(xn, drawn, force, seed_lo, seed_hi)
            self.drawn[r] = drawn
            heard = [step.force_caller[k] if step.force_caller[k] >= 0 else step.caller[k] for k in range(BOOKS)]
            nxt, pending, text, frame = advance(row, s["state"][STREAMS:], drawn, heard)
            emitted[r] = [text] + frame
            s["state"] = nxt + pending
            s["pos"] += 1
            s["frame"] += 1
        return emitted
