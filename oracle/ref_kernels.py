"""The reference's own CUDA kernels, compiled for sm_100a and replayed on the GPU (TEST INFRASTRUCTURE).

build(): when the reference checkout is present, compiles `crates/omni-qwen3/kernels/qwen3.cu`,
`crates/omni-qwen3-tts/kernels/talker.cu`, `crates/omni-qwen3-tts/kernels/codec.cu`,
`crates/omni-personaplex/kernels/lm.cu` and `crates/omni-higgs-audio/kernels/higgs.cu` where they lie (include path
`crates/omni-kern/kernels`) into
`oracle/_ref/*.cubin` with the reference's own flags except the architecture
(crates/omni-qwen3/build.rs:17-27: `nvcc -cubin -O3 -std=c++17`). Sources are never copied.

`RefTalker` then replays a talker decode tick exactly as the reference's manifest sequences it
(crates/omni-qwen3/src/stack.rs:152-241, crates/omni-qwen3-tts/src/talker.rs:224-356): the reference's kernels
launched through the driver API, GEMMs as bf16 `x @ w.T` through cuBLAS (the reference uses cuBLASLt bf16 TN inside
its un-vendored runtime; algorithm choices there are unknown), optionally captured as one CUDA graph per bucket like
the reference's `decode` program. It serves two purposes: a second oracle (the reference's real arithmetic, including
its sampler, on the same GPU) and the "reference build on the same box" timing baseline.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
# the reference checkout: named by OMNI_REFERENCE, else looked for beside this repository's checkout
REFERENCE = Path(os.environ.get("OMNI_REFERENCE") or HERE.parent.parent / "reference")
SOURCES = {
    "qwen3": "crates/omni-qwen3/kernels/qwen3.cu",
    "talker": "crates/omni-qwen3-tts/kernels/talker.cu",
    "lm": "crates/omni-personaplex/kernels/lm.cu",
    "higgs": "crates/omni-higgs-audio/kernels/higgs.cu",
    "codec": "crates/omni-qwen3-tts/kernels/codec.cu",
}


def available() -> bool:
    return all((OUT / f"{n}.cubin").exists() for n in SOURCES)


def build(force: bool = False) -> bool:
    """Compiles the cubins if the reference is here; returns whether they exist afterwards."""
    if not REFERENCE.exists():
        return available()
    OUT.mkdir(exist_ok=True)
    for name, rel in SOURCES.items():
        src, dst = REFERENCE / rel, OUT / f"{name}.cubin"
        if not force and dst.exists() and dst.stat().st_mtime >= src.stat().st_mtime:
            continue
        cmd = ["nvcc", "-cubin", "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a",
               "-I", str(REFERENCE / "crates/omni-kern/kernels"), "-I", str(src.parent), "-o", str(dst), str(src)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {rel}:\n{res.stderr}")
    return available()


class _Module:
    """One cubin loaded with the driver API; kernels are launched on torch's current stream."""

    def __init__(self, path: Path):
        from cuda.bindings import driver
        self.drv = driver
        err, self.mod = driver.cuModuleLoadData(path.read_bytes())
        if int(err) != 0:
            raise RuntimeError(f"cuModuleLoadData({path.name}): {err}")
        self.fns = {}

    def launch(self, name: str, grid, block: int, args):
        """args: list of (ctype, value); pointers are passed as (c_void_p, int)."""
        import torch
        drv = self.drv
        if name not in self.fns:
            err, fn = drv.cuModuleGetFunction(self.mod, name.encode())
            if int(err) != 0:
                raise RuntimeError(f"cuModuleGetFunction({name}): {err}")
            self.fns[name] = fn
        vals = tuple(v for _, v in args)
        types = tuple(t for t, _ in args)
        stream = torch.cuda.current_stream().cuda_stream
        gx, gy, gz = (list(grid) + [1, 1])[:3]
        (err,) = drv.cuLaunchKernel(self.fns[name], gx, gy, gz, block, 1, 1, 0, stream, (vals, types), 0)
        if int(err) != 0:
            raise RuntimeError(f"cuLaunchKernel({name}): {err}")


def _p(t):
    return (ctypes.c_void_p, t.data_ptr())


def _i(v):
    return (ctypes.c_int, int(v))


def _f(v):
    return (ctypes.c_float, float(v))


def _l(v):
    return (ctypes.c_int64, int(v))


class RefTalker:
    """Decode ticks of the talker through the reference's kernels (see the module docstring).

    Sessions are dense here (session s owns pages [s * pages_per_seq, (s+1) * pages_per_seq)); the KV layout is the
    reference's `[slot][K heads | V heads][128]`. Prompts are prefilled with the reference's ragged path
    (`Talker::prefill`, talker.rs:186-221).
    """

    def __init__(self, cfg, ck: dict, sessions: int, max_positions: int, device: str = "cuda"):
        import torch
        self.torch = torch
        self.cfg, self.b = cfg, sessions
        self.q = _Module(OUT / "qwen3.cubin")
        self.t = _Module(OUT / "talker.cubin")
        t, p = cfg.talker, cfg.predictor
        assert t.head_dim == 128 and p.head_dim == 128 and cfg.num_code_groups == 16, "the reference's own limits"
        dev = torch.device(device)

        def fuse(prefix, c):
            layers = []
            for i in range(c.num_hidden_layers):
                g = lambda n: ck[f"{prefix}.layers.{i}.{n}"]
                layers.append(dict(
                    ln1=g("input_layernorm.weight"),
                    qkv=torch.cat([g("self_attn.q_proj.weight"), g("self_attn.k_proj.weight"),
                                   g("self_attn.v_proj.weight")]).contiguous(),
                    q_norm=g("self_attn.q_norm.weight"), k_norm=g("self_attn.k_norm.weight"),
                    o=g("self_attn.o_proj.weight"), ln2=g("post_attention_layernorm.weight"),
                    gate_up=torch.cat([g("mlp.gate_proj.weight"), g("mlp.up_proj.weight")]).contiguous(),
                    down=g("mlp.down_proj.weight")))
            return layers, ck[f"{prefix}.norm.weight"]

        self.tl, self.tnorm = fuse("talker.model", t)
        self.pl, self.pnorm = fuse("talker.code_predictor.model", p)
        self.text_emb = ck["talker.model.text_embedding.weight"]
        self.codec_emb = ck["talker.model.codec_embedding.weight"]
        self.codec_head = ck["talker.codec_head.weight"]
        self.fc1 = (ck["talker.text_projection.linear_fc1.weight"], ck["talker.text_projection.linear_fc1.bias"])
        self.fc2 = (ck["talker.text_projection.linear_fc2.weight"], ck["talker.text_projection.linear_fc2.bias"])
        self.mtp = (ck["talker.code_predictor.small_to_mtp_projection.weight"],
                    ck["talker.code_predictor.small_to_mtp_projection.bias"])
        self.p_emb = torch.cat([ck[f"talker.code_predictor.model.codec_embedding.{g}.weight"] for g in range(15)])
        self.lm_heads = torch.cat([ck[f"talker.code_predictor.lm_head.{g}.weight"] for g in range(15)])

        b, h, ph = sessions, t.hidden_size, p.hidden_size
        bf = dict(dtype=torch.bfloat16, device=dev)
        i32 = dict(dtype=torch.int32, device=dev)
        self.pages_per_seq = (max_positions + 15) // 16
        slots = b * self.pages_per_seq * 16
        self.kv = [torch.zeros((slots, 2 * t.num_key_value_heads, 128), **bf) for _ in range(t.num_hidden_layers)]
        self.pkv = [torch.zeros((b * 16, 2 * p.num_key_value_heads, 128), **bf) for _ in range(p.num_hidden_layers)]
        self.stride = ((4 * (16 + (t.vocab_size + 31) // 32) + 255) // 256) * 256
        self.state = torch.zeros((b, self.stride), dtype=torch.uint8, device=dev)
        self.lines = torch.arange(b, **i32)
        self.frames = torch.zeros(b, **i32)
        self.uniforms = torch.full((b, 16), 0.5, dtype=torch.float32, device=dev)
        self.force = torch.full((b, 16), -1, **i32)
        self.t_pos = torch.zeros(b, **i32)
        self.t_slot = torch.zeros(b, **i32)
        self.t_seq = torch.arange(b, **i32)
        self.indptr = torch.arange(b + 1, **i32) * self.pages_per_seq
        self.pages = torch.arange(b * self.pages_per_seq, **i32)
        self.codes = torch.zeros((b, 16), **i32)
        self.logits = torch.zeros((b, t.vocab_size), **bf)
        self.p_logits = torch.zeros((15 * b, p.vocab_size), **bf)
        self.hidden = torch.zeros((b, h), **bf)
        self.t_e = torch.zeros((b, h), **bf)
        self.p_in = torch.zeros((2 * b, h), **bf)
        self.p_last = torch.zeros((b, ph), **bf)
        self.prompt_len = torch.zeros(b, dtype=torch.int64)
        self.n_frames = 0
        self.graph = None
        self.launches = 0
        # `Talker::init`: the <tts_pad> embedding through the text projection
        e = self.text_emb[cfg.tts_pad_token_id][None]
        pp = self._gemm(e, self.fc1[0])
        self._bias(pp, self.fc1[1], silu=True)
        self.pad_embed = self._gemm(pp, self.fc2[0])
        self._bias(self.pad_embed, self.fc2[1], silu=False)

    # ---- pieces ----
    def _gemm(self, x, w):
        self.launches += 1
        return x @ w.t()

    def _bias(self, x, bias, silu):
        rows, cols = x.shape
        total = rows * cols // 8
        self.t.launch("talker_bias_silu" if silu else "talker_bias", [(total + 255) // 256], 256,
                      [_p(x), _p(bias), _i(cols), _i(total)])
        self.launches += 1

    def _stack(self, layers, final_norm, c, x_in, rows, paged, per=1, base=0, pos=None, slot=None, seq=None,
               ragged=0, indptr=None, pages=None, kv=None, every=1, which=0):
        torch = self.torch
        h, hq, hk, inter = c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.intermediate_size
        eps, theta = c.rms_norm_eps, c.rope_theta
        x = torch.empty((rows, h), dtype=torch.bfloat16, device=x_in.device)
        res = torch.empty_like(x)
        attn = torch.empty((rows, hq * 128), dtype=torch.bfloat16, device=x_in.device)
        act = torch.empty((rows, inter), dtype=torch.bfloat16, device=x_in.device)
        out = torch.empty((rows // every, h), dtype=torch.bfloat16, device=x_in.device)
        self.q.launch("qwen3_norm_copy", [rows], h // 8, [_p(x_in), _p(layers[0]["ln1"]), _p(x), _p(res), _i(h), _f(eps)])
        self.launches += 1
        heads = (hq + 2 * hk + 7) // 8
        scale = 1.0 / (128 ** 0.5)
        for i, L in enumerate(layers):
            qkv = self._gemm(x, L["qkv"])
            if paged:
                self.q.launch("qwen3_rope", [rows, heads], 256, [_p(qkv), _p(L["q_norm"]), _p(L["k_norm"]), _p(pos), _p(slot),
                                                                  _p(kv[i]), _i(hq), _i(hk), _f(eps), _f(theta)])
                self.q.launch("qwen3_attend", [rows, hk], 128, [_p(qkv), _p(kv[i]), _p(pos), _p(seq), _i(ragged), _p(indptr),
                                                                _p(pages), _i(16), _p(attn), _i(hq), _i(hk), _f(scale)])
            else:
                self.q.launch("qwen3_rope_dense", [rows, heads], 256, [_p(qkv), _p(L["q_norm"]), _p(L["k_norm"]), _p(kv[i]),
                                                                        _i(per), _i(base), _i(16), _i(hq), _i(hk), _f(eps),
                                                                        _f(theta)])
                self.q.launch("qwen3_attend_dense", [rows, hk], 128, [_p(qkv), _p(kv[i]), _i(per), _i(base), _i(16), _p(attn),
                                                                      _i(hq), _i(hk), _f(scale)])
            o = self._gemm(attn, L["o"])
            self.q.launch("qwen3_add_norm", [rows], h // 8, [_p(o), _p(res), _p(L["ln2"]), _p(x), _i(h), _f(eps), _i(1), _i(0)])
            gu = self._gemm(x, L["gate_up"])
            total = rows * inter // 8
            self.q.launch("qwen3_silu_mul", [(total + 255) // 256], 256, [_p(gu), _p(act), _i(inter), _i(total)])
            d = self._gemm(act, L["down"])
            last = i + 1 == len(layers)
            self.q.launch("qwen3_add_norm", [rows], h // 8,
                          [_p(d), _p(res), _p(final_norm if last else layers[i + 1]["ln1"]), _p(out if last else x), _i(h),
                           _f(eps), _i(every if last else 1), _i(which if last else 0)])
            self.launches += 5
        return out

    def _sample(self, group, logits):
        cfg, g = self.cfg, self.cfg.generation
        if group == 0:
            v = cfg.talker.vocab_size
            consts = (v, g.temperature, g.top_k, g.repetition_penalty, v - cfg.control_tokens, v, cfg.codec_eos_token_id,
                      cfg.min_frames, 1)
        else:
            consts = (cfg.predictor.vocab_size, g.subtalker_temperature, g.subtalker_top_k, 1.0, 0, 0, -1, 0, 0)
        vocab, temp, top_k, pen, lo, hi, exempt, min_frames, penalize = consts
        self.t.launch("talker_sample", [self.b], 1024,
                      [_p(logits), _i(vocab), _f(temp), _i(top_k), _f(pen), _i(lo), _i(hi), _i(exempt), _i(min_frames),
                       _p(self.frames), _p(self.uniforms), _p(self.force), _p(self.state), _p(self.lines), _l(self.stride),
                       _i(penalize), _p(self.codes), _i(group)])
        self.launches += 1

    def _tail(self):
        cfg, b = self.cfg, self.b
        t, p = cfg.talker, cfg.predictor
        h, pv = t.hidden_size, p.vocab_size
        self.logits.copy_(self._gemm(self.hidden, self.codec_head))
        self._sample(0, self.logits)
        self.t.launch("talker_pred_input", [b, 2], h // 8, [_p(self.hidden), _p(self.codec_emb), _p(self.codes), _p(self.p_in),
                                                            _i(h)])
        self.launches += 1
        for g in range(1, 16):
            per, rows = (2, 2 * b) if g == 1 else (1, b)
            if g > 1:
                table = self.p_emb[(g - 2) * pv:(g - 1) * pv]
                self.t.launch("talker_gather", [b], h // 8, [(ctypes.c_void_p, self.codes.data_ptr() + 4 * (g - 1)), _i(16),
                                                             _p(table), _p(self.p_in), _i(h)])
                self.launches += 1
            ph = self._gemm(self.p_in[:rows], self.mtp[0])
            self._bias(ph, self.mtp[1], silu=False)
            last = self._stack(self.pl, self.pnorm, p, ph, rows, paged=False, per=per, base=0 if g == 1 else g, kv=self.pkv,
                               every=per, which=per - 1)
            lg = self.p_logits[(g - 1) * b:g * b]
            lg.copy_(self._gemm(last, self.lm_heads[(g - 1) * pv:g * pv]))
            self._sample(g, lg)

    def _decode(self):
        cfg, b = self.cfg, self.b
        t = cfg.talker
        h = t.hidden_size
        self.t.launch("talker_frame_embed", [b], h // 8, [_p(self.state), _p(self.lines), _l(self.stride), _p(self.pad_embed),
                                                          _p(self.codec_emb), _p(self.p_emb), _p(self.t_e), _i(h),
                                                          _i(cfg.predictor.vocab_size)])
        self.launches += 1
        out = self._stack(self.tl, self.tnorm, t, self.t_e, b, paged=True, pos=self.t_pos, slot=self.t_slot, seq=self.t_seq,
                          ragged=0, indptr=self.indptr, pages=self.pages, kv=self.kv)
        self.hidden.copy_(out)
        self._tail()

    # ---- the model-shell calls ----
    def start(self, prompts, uniforms, force):
        """Prefill (ragged) + the first frame. prompts: objects with .text / .codec; uniforms, force: [b, 16]."""
        torch, cfg, b = self.torch, self.cfg, self.b
        dev = self.hidden.device
        lens = [len(p.text) for p in prompts]
        tokens = sum(lens)
        ids = torch.tensor([x for p in prompts for x in p.text], dtype=torch.int32, device=dev)
        codec = torch.tensor([x for p in prompts for x in p.codec], dtype=torch.int32, device=dev)
        pos = torch.tensor([i for n in lens for i in range(n)], dtype=torch.int32, device=dev)
        seq = torch.tensor([s for s, n in enumerate(lens) for _ in range(n)], dtype=torch.int32, device=dev)
        slot = (seq * self.pages_per_seq * 16 + pos).to(torch.int32)
        h = cfg.talker.hidden_size
        e = self.text_emb[ids.long()]
        pp = self._gemm(e, self.fc1[0])
        self._bias(pp, self.fc1[1], silu=True)
        emb = self._gemm(pp, self.fc2[0]).contiguous()
        self.t.launch("talker_prompt_codec", [tokens], h // 8, [_p(emb), _p(self.fc2[1]), _p(self.codec_emb), _p(codec), _i(h)])
        self.embeds = emb
        out = self._stack(self.tl, self.tnorm, cfg.talker, emb, tokens, paged=True, pos=pos, slot=slot, seq=seq, ragged=1,
                          indptr=self.indptr, pages=self.pages, kv=self.kv)
        last_rows = torch.tensor(lens, device=dev).cumsum(0) - 1
        self.hidden.copy_(out[last_rows])
        self.prompt_len = torch.tensor(lens, dtype=torch.int64)
        self.frames.zero_()
        self.uniforms.copy_(torch.as_tensor(uniforms, dtype=torch.float32))
        self.force.copy_(torch.as_tensor(force, dtype=torch.int32))
        self._tail()
        torch.cuda.synchronize()
        self.n_frames = 1
        return self.codes.cpu().numpy().copy()

    def _stage(self, uniforms, force):
        torch = self.torch
        position = (self.prompt_len + self.n_frames - 1).to(torch.int32)
        self.t_pos.copy_(position)
        self.t_slot.copy_((torch.arange(self.b) * self.pages_per_seq * 16 + position).to(torch.int32))
        self.frames.fill_(self.n_frames)
        self.uniforms.copy_(torch.as_tensor(uniforms, dtype=torch.float32))
        self.force.copy_(torch.as_tensor(force, dtype=torch.int32))

    def step(self, uniforms, force, graph: bool = False):
        """One decode tick (`Model::step`, model.rs:180-192); with `graph`, replayed from a captured CUDA graph."""
        torch = self.torch
        self._stage(uniforms, force)
        if graph:
            if self.graph is None:
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    self.launches = 0
                    self._decode()  # warm-up: cuBLAS workspaces and heuristics before capture
                torch.cuda.current_stream().wait_stream(side)
                torch.cuda.synchronize()
                raise_if = self.codes.clone()  # the warm-up drew a frame: callers capture on a throw-away tick
                del raise_if
                self.graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(self.graph):
                    self.launches = 0
                    self._decode()
                self.graph_nodes = self.launches
            self.graph.replay()
        else:
            self.launches = 0
            self._decode()
        torch.cuda.synchronize()
        self.n_frames += 1
        return self.codes.cpu().numpy().copy()

    def talker_logits(self, s):
        return self.logits[s].float().cpu().numpy()

    def predictor_logits(self, s):
        pv = self.cfg.predictor.vocab_size
        return self.p_logits.view(15, self.b, pv)[:, s].float().cpu().numpy()
