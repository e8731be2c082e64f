"""CPU restatement of the Higgs-style speech model's token loop. TEST INFRASTRUCTURE ONLY: nothing outside tests/, the
smoke check and bench.py's CPU legs may import this file.

Every arithmetic step goes through the operator-level C++ oracle (oracle/talker_oracle.cpp via oracle/cpu.py: GEMM,
norms, SwiGLU, q/k norm + rotary embedding, attention, the draw), sequenced here as the reference's manifest does:
  prefill / decode / first programs ... crates/omni-higgs-audio/src/model.rs:339-405
  body pass ............................ crates/omni-qwen3/src/stack.rs:152-203
  frame embedding, draws ............... crates/omni-higgs-audio/kernels/higgs.cu:24-37, :186-208
  delay pattern ........................ crates/omni-higgs-audio/src/delay.rs:19-54
  positions, ramp, finish .............. crates/omni-higgs-audio/src/model.rs:166-199, :262-272

Parity status: UNPINNED against a real checkpoint (none is available offline); the glue kernels are pinned against the
reference's own higgs.cu cubin on the GPU (tests/test_higgs_gpu.py), the delay pattern against the reference's tests.
"""
from __future__ import annotations

import numpy as np

from . import cpu

BOOKS, BOC, EOC = 8, 1024, 1025


class Delay:
    """delay.rs:19-46."""

    def __init__(self):
        self.steps, self.countdown, self.done = 0, None, False

    def forced_from(self):
        return min(self.steps + 1, BOOKS)

    def advance(self, first):
        if self.done:
            return True
        if self.steps < BOOKS:
            self.steps += 1
        elif self.countdown is not None:
            left = self.countdown
            self.countdown = left - 1
            self.done = left <= 1
        elif first == EOC:
            self.countdown = BOOKS - 2
        return self.done


def undelay(rows):
    rows = np.asarray(rows).reshape(-1, BOOKS)
    n = max(len(rows) - (BOOKS - 1), 0)
    return np.array([[rows[t + c][c] for c in range(BOOKS)] for t in range(n)], dtype=np.int32).reshape(n, BOOKS)


def _bits(t):
    a = t.float().cpu().numpy() if hasattr(t, "float") else np.asarray(t, dtype=np.float32)
    return cpu.bf16_bits(a)


class HiggsOracle:
    def __init__(self, cfg, checkpoint: dict):
        self.c = cfg
        b = cfg.body
        w = {k: _bits(v) for k, v in checkpoint.items()}
        self.layers = []
        for i in range(b.num_hidden_layers):
            p = f"body.layers.{i}."
            self.layers.append(dict(
                ln1=w[p + "input_layernorm.weight"], ln2=w[p + "post_attention_layernorm.weight"],
                qkv=np.concatenate([w[p + "self_attn.q_proj.weight"], w[p + "self_attn.k_proj.weight"],
                                    w[p + "self_attn.v_proj.weight"]]),
                q_norm=w[p + "self_attn.q_norm.weight"], k_norm=w[p + "self_attn.k_norm.weight"],
                o=w[p + "self_attn.o_proj.weight"],
                gate_up=np.concatenate([w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"]]),
                down=w[p + "mlp.down_proj.weight"]))
            if getattr(cfg, "audio_adapter", False):
                # an audio position's MLP: the text and the audio branch side by side along the channel axis, so the
                # down projection sums both branches in f32 before its one bf16 rounding (this library's definition:
                # the reference's Higgs body has no such adapter)
                self.layers[-1]["gate_up_audio"] = np.concatenate(
                    [w[p + "mlp.gate_proj.weight"], w[p + "audio_mlp.gate_proj.weight"],
                     w[p + "mlp.up_proj.weight"], w[p + "audio_mlp.up_proj.weight"]])
                self.layers[-1]["down_audio"] = np.concatenate(
                    [w[p + "mlp.down_proj.weight"], w[p + "audio_mlp.down_proj.weight"]], axis=1)
        self.norm = w["body.norm.weight"]
        self.text = cpu.bits_to_f32(w["tied.embedding.text_embedding.weight"])
        self.fused_bits = w["tied.embedding.modality_embeddings.0.embedding.weight"]
        self.fused = cpu.bits_to_f32(self.fused_bits)
        self.seqs = {}
        self.next_id = 0
        self.logits = None

    def open(self, prompt: int, rows: int) -> int:
        sid = self.next_id
        self.next_id += 1
        self.seqs[sid] = dict(prompt=prompt, rows=0, delay=Delay(), codes=[0] * BOOKS,
                              kv=[[] for _ in self.layers])
        return sid

    def _body_row(self, s, x_in, pos, audio=False):
        """One row through every layer (stack.rs:152-203); returns the final norm's row. `audio`: the row is an audio
        position (a frame row), whose MLP includes the audio branch when the model has the adapter."""
        b = self.c.body
        hq, hk, d = b.num_attention_heads, b.num_key_value_heads, b.head_dim
        x, res = cpu.norm_copy(x_in[None, :], self.layers[0]["ln1"], b.rms_norm_eps)
        for i, L in enumerate(self.layers):
            qkv = cpu.gemm(x, L["qkv"])[0]
            q = qkv[:hq * d].reshape(hq, d).copy()
            k = qkv[hq * d:(hq + hk) * d].reshape(hk, d).copy()
            v = qkv[(hq + hk) * d:]
            for j in range(hq):
                q[j] = cpu.rope_head(q[j], L["q_norm"], pos, b.rms_norm_eps, b.rope_theta)
            for j in range(hk):
                k[j] = cpu.rope_head(k[j], L["k_norm"], pos, b.rms_norm_eps, b.rope_theta)
            s["kv"][i].append(cpu.bf16_bits(np.concatenate([k.ravel(), v])))
            attn = cpu.attend(q.ravel(), np.stack(s["kv"][i]), hq, hk, d)
            o = cpu.gemm(attn[None, :], L["o"])
            x, res = cpu.add_norm(o, res, L["ln2"], b.rms_norm_eps)
            both = audio and "gate_up_audio" in L
            act = cpu.silu_mul(cpu.gemm(x, L["gate_up_audio" if both else "gate_up"]))
            down = cpu.gemm(act, np.ascontiguousarray(L["down_audio"]) if both else L["down"])
            nxt = self.layers[i + 1]["ln1"] if i + 1 < len(self.layers) else self.norm
            x, res = cpu.add_norm(down, res, nxt, b.rms_norm_eps)
        return x[0]

    def _tail(self, rows, hidden):
        """head GEMM + the eight draws + `finish` (model.rs:381-404, :267-272)."""
        c = self.c
        n = len(rows)
        out, ended = np.zeros((n, BOOKS), np.int32), np.zeros(n, bool)
        self.logits = np.zeros((n, BOOKS, c.code_vocab), np.float32)
        for r, (sid, draw) in enumerate(rows):
            s = self.seqs[sid]
            logits = cpu.gemm(hidden[r][None, :], self.fused_bits)[0].reshape(BOOKS, c.code_vocab)
            self.logits[r] = logits
            from_ = s["delay"].forced_from()
            force = list(draw.force) if draw.force is not None else [BOC if b >= from_ else -1 for b in range(BOOKS)]
            last, seen = np.zeros(16, np.int32), np.zeros(c.code_vocab // 32 + 1, np.uint32)
            for b in range(BOOKS):
                out[r, b] = cpu.sample(logits[b], c.temperature, c.top_k, 1.0, 1.0, 0, 0, -1, 0, 0,
                                       float(np.float32(draw.uniforms[b])), int(force[b]), last, seen, False, b)
            s["codes"] = [int(v) for v in out[r]]
            s["rows"] += 1
            ended[r] = s["delay"].advance(int(out[r, 0]))
        return out, ended

    def start(self, rows):
        """rows: [(sid, prompt ids, draw)] (model.rs:166-187)."""
        hidden = []
        for sid, ids, _ in rows:
            s = self.seqs[sid]
            assert s["rows"] == 0 and len(ids) == s["prompt"]
            h = None
            for p, t in enumerate(ids):
                h = self._body_row(s, self.text[int(t)], p)
            hidden.append(h)
        return self._tail([(sid, d) for sid, _, d in rows], hidden)

    def step(self, rows):
        """rows: [(sid, draw)] (model.rs:190-199): frame embedding of the last row's codes at position prompt+rows-1."""
        c = self.c
        hidden = []
        for sid, _ in rows:
            s = self.seqs[sid]
            assert s["rows"] > 0
            acc = np.zeros(c.body.hidden_size, np.float32)
            for b in range(BOOKS):  # f32 sum in codebook order, one rounding (higgs.cu:24-37)
                acc = acc + self.fused[b * c.code_vocab + s["codes"][b]]
            hidden.append(self._body_row(s, cpu.bf16_round(acc), s["prompt"] + s["rows"] - 1, audio=True))
        return self._tail(rows, hidden)
