"""CPU restatement of the Qwen3-TTS streaming codec decoder. TEST INFRASTRUCTURE ONLY: nothing outside tests/, the
smoke check and bench.py's CPU legs may import this file.

Two decoders over the same checkpoint tensors:

  whole_utterance(): the decoder as published (RVQ -> causal conv -> sliding-window transformer -> two x2 upsamplers
      (transposed conv + ConvNeXt) -> four SnakeBeta / transposed-conv blocks with dilated residual units -> SnakeBeta,
      conv, clamp), float64, unfolded weights, all frames at once. It is the centre the streaming decoders are
      measured against (the reference's own bar: snr > 30 dB, crates/omni-qwen3-tts/tests/golden.rs:156-162).
  StreamOracle: the reference's streaming restatement, one frame per call, bf16 buffers and f32 arithmetic with a
      rounding at every point the reference's kernels round:
        weight folding at load ............ crates/omni-qwen3-tts/src/codec.rs:112-448 (`fold`)
        tap layouts ....................... crates/omni-kern/src/weights.rs:98-121
        RVQ gather, gelu, snake, norms .... crates/omni-qwen3-tts/kernels/codec.cu:66-170
        window attention .................. codec.cu:177-283
        im2col + history, overlap-add ..... codec.cu:291-372
        depthwise conv + LayerNorm ........ codec.cu:381-446
        output conv ....................... codec.cu:455-513

Parity status: UNPINNED against a real checkpoint (none is available offline, and the reference's golden file is not in
its tree); the two decoders here pin each other (tests/test_codec_oracle.py), and the CUDA path is compared with both.
The CUDA kernels themselves are also compared one by one with the reference's codec.cu compiled for sm_100a
(tests/test_codec_ops_gpu.py), which this file takes no part in.
"""
from __future__ import annotations

import math

import numpy as np

GROUPS, KERNEL, WINDOW, HEAD = 16, 7, 72, 64


def bf(x):
    """float32 -> nearest-even bf16, returned as float32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    r = ((u >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF)
    return ((u + r) & np.uint32(0xFFFF0000)).view(np.float32)


def f32(x):
    return np.asarray(x, dtype=np.float32)


def conv_taps(w):
    """[out, in, k] -> [out, k * in], tap-major (weights.rs:98-105)."""
    o, i, k = w.shape
    return np.ascontiguousarray(w.transpose(0, 2, 1).reshape(o, k * i))


def transposed_taps(w):
    """[in, out, k] -> [k * out, in] (weights.rs:107-115)."""
    i, o, k = w.shape
    return np.ascontiguousarray(w.transpose(2, 1, 0).reshape(k * o, i))


def snake_params(ck, prefix):
    """codec.rs:48-56: a = exp(alpha), inv_b = 1 / (exp(beta) + 1e-9), both f32."""
    a = np.exp(f32(ck[prefix + ".alpha"])).astype(np.float32)
    inv_b = (np.float32(1.0) / (np.exp(f32(ck[prefix + ".beta"])).astype(np.float32) + np.float32(1e-9)))
    return a, inv_b.astype(np.float32)


def fold(ck, c):
    """The named tensors `codec::build` hands the runtime: layouts transformed, scales and biases folded on the host in
    f32, matrices and bias vectors rounded to bf16, SnakeBeta parameters kept in f32."""
    W = {}
    half, cb, dim, lat, h = c.codebook_dim // 2, c.codebook_size, c.codebook_dim, c.latent_dim, c.hidden_size
    names = ["decoder.quantizer.rvq_first.vq.layers.0"] + \
        [f"decoder.quantizer.rvq_rest.vq.layers.{i}" for i in range(GROUPS - 1)]
    books = [f32(ck[p + "._codebook.embedding_sum"]) / np.maximum(f32(ck[p + "._codebook.cluster_usage"]),
                                                                  np.float32(1e-5))[:, None] for p in names]
    W["rvq.books"] = bf(np.concatenate(books, 0))
    first = f32(ck["decoder.quantizer.rvq_first.output_proj.weight"]).reshape(dim, half)
    rest = f32(ck["decoder.quantizer.rvq_rest.output_proj.weight"]).reshape(dim, half)
    W["rvq.out"] = bf(np.concatenate([first, rest], 1))
    W["pre_conv.w"] = bf(conv_taps(f32(ck["decoder.pre_conv.conv.weight"])))
    pre_b = f32(ck["decoder.pre_conv.conv.bias"])
    pt = "decoder.pre_transformer"
    in_w = f32(ck[f"{pt}.input_proj.weight"])
    W["input_proj.b"] = bf(f32(ck[f"{pt}.input_proj.bias"]) + in_w @ pre_b)
    W["input_proj.w"] = bf(in_w)
    for i in range(c.num_hidden_layers):
        q = f"{pt}.layers.{i}."
        W[f"l{i}.ln1"] = bf(ck[q + "input_layernorm.weight"])
        W[f"l{i}.qkv"] = bf(np.concatenate([f32(ck[q + f"self_attn.{n}_proj.weight"]) for n in "qkv"], 0))
        W[f"l{i}.o"] = bf(f32(ck[q + "self_attn.o_proj.weight"]) * f32(ck[q + "self_attn_layer_scale.scale"])[:, None])
        W[f"l{i}.ln2"] = bf(ck[q + "post_attention_layernorm.weight"])
        W[f"l{i}.gate_up"] = bf(np.concatenate([f32(ck[q + "mlp.gate_proj.weight"]), f32(ck[q + "mlp.up_proj.weight"])], 0))
        W[f"l{i}.down"] = bf(f32(ck[q + "mlp.down_proj.weight"]) * f32(ck[q + "mlp_layer_scale.scale"])[:, None])
    W["norm"] = bf(ck[f"{pt}.norm.weight"])
    W["output_proj.w"] = bf(ck[f"{pt}.output_proj.weight"])
    pending = f32(ck[f"{pt}.output_proj.bias"])
    for i, r in enumerate(c.upsampling_ratios):
        p = f"decoder.upsample.{i}"
        up = transposed_taps(f32(ck[f"{p}.0.conv.weight"]))                       # [r * lat, lat]
        zb = (up @ pending).reshape(r, lat) + f32(ck[f"{p}.0.conv.bias"])[None, :]
        W[f"up{i}.w"], W[f"up{i}.b"] = bf(up), bf(zb)
        W[f"up{i}.dw.w"] = bf(f32(ck[f"{p}.1.dwconv.conv.weight"]).reshape(lat, KERNEL).T)   # [7, lat]
        W[f"up{i}.dw.b"] = bf(ck[f"{p}.1.dwconv.conv.bias"])
        W[f"up{i}.ln.w"], W[f"up{i}.ln.b"] = bf(ck[f"{p}.1.norm.weight"]), bf(ck[f"{p}.1.norm.bias"])
        W[f"up{i}.pw1.w"], W[f"up{i}.pw1.b"] = bf(ck[f"{p}.1.pwconv1.weight"]), bf(ck[f"{p}.1.pwconv1.bias"])
        gamma = f32(ck[f"{p}.1.gamma"])
        W[f"up{i}.pw2.w"] = bf(f32(ck[f"{p}.1.pwconv2.weight"]) * gamma[:, None])
        pending = f32(ck[f"{p}.1.pwconv2.bias"]) * gamma
    W["conv_in.in_b"] = bf(pending)
    W["conv_in.w"] = bf(conv_taps(f32(ck["decoder.decoder.0.conv.weight"])))
    pending = f32(ck["decoder.decoder.0.conv.bias"])
    for i, rate in enumerate(c.upsample_rates):
        p = f"decoder.decoder.{i + 1}.block"
        W[f"b{i}.snake"] = snake_params(ck, f"{p}.0")
        W[f"b{i}.in_b"] = bf(pending)
        W[f"b{i}.up.w"] = bf(transposed_taps(f32(ck[f"{p}.1.conv.weight"])))     # [2 * rate * cout, cin]
        W[f"b{i}.up.b"] = bf(ck[f"{p}.1.conv.bias"])
        pending = np.zeros(c.decoder_dim >> (i + 1), dtype=np.float32)
        for u in range(3):
            q = f"{p}.{u + 2}"
            W[f"b{i}.u{u}.s1"] = snake_params(ck, f"{q}.act1")
            W[f"b{i}.u{u}.conv1.w"] = bf(conv_taps(f32(ck[f"{q}.conv1.conv.weight"])))
            W[f"b{i}.u{u}.conv1.b"] = bf(ck[f"{q}.conv1.conv.bias"])
            W[f"b{i}.u{u}.s2"] = snake_params(ck, f"{q}.act2")
            W[f"b{i}.u{u}.conv2.w"] = bf(conv_taps(f32(ck[f"{q}.conv2.conv.weight"])))
            W[f"b{i}.u{u}.in_b"] = bf(pending)
            pending = pending + f32(ck[f"{q}.conv2.conv.bias"])
    n = len(c.upsample_rates) + 1
    W["conv_out.snake"] = snake_params(ck, f"decoder.decoder.{n}")
    W["conv_out.in_b"] = bf(pending)
    W["conv_out.w"] = bf(conv_taps(f32(ck[f"decoder.decoder.{n + 1}.conv.weight"])).reshape(KERNEL, -1))
    W["conv_out.b"] = bf(ck[f"decoder.decoder.{n + 1}.conv.bias"])
    return W


# ---- the reference's streaming arithmetic ---------------------------------------------------------------------------

def gemm(x, w):
    """bf16 rows times bf16 [n, k] weights, f32 accumulation, bf16 result."""
    return bf(f32(x) @ f32(w).T)


def gemm_acc(y, x, w):
    """y = bf16(y + x . w^T): one rounding of the f32 sum (the runtime's accumulating GEMM)."""
    return bf(f32(y) + f32(x) @ f32(w).T)


def fast_sin(y):
    """codec.cu:34-37: two-step reduction to [-pi, pi], then the sine (hardware approximation there, error ~4e-7)."""
    y = f32(y)
    k = np.rint(y * np.float32(0.159154943091895336)).astype(np.float32)
    r = (-k).astype(np.float64) * np.float64(np.float32(6.28318548202514648)) + y.astype(np.float64)
    r = r.astype(np.float32).astype(np.float64) + (-k).astype(np.float64) * np.float64(np.float32(-1.74845553e-7))
    return np.sin(r.astype(np.float32).astype(np.float64)).astype(np.float32)


def snake(x, a, inv_b):
    s = fast_sin(a * f32(x))
    return f32(x) + inv_b * s * s


def rms_norm_add(add, res, w, eps):
    """codec.cu:117-152: v = res + add (f32); res = bf16(v); out = bf16(v * (rs * w)), rs over the unrounded v."""
    v = f32(res) + f32(add)
    rs = np.float32(1.0) / np.sqrt((v * v).sum(-1, keepdims=True, dtype=np.float32) / np.float32(v.shape[-1]) + np.float32(eps))
    return bf(v), bf(v * (rs.astype(np.float32) * f32(w)))


def silu_mul(gu, inter):
    g, u = f32(gu[..., :inter]), f32(gu[..., inter:])
    return bf(bf(g / (np.float32(1.0) + np.exp(-g))) * u)


def gelu_bias(x, b):
    y = bf(f32(x) + f32(b))
    erf = np.vectorize(math.erf, otypes=[np.float64])
    return bf((np.float32(0.5) * y * (np.float32(1.0) + erf(y.astype(np.float64) * 0.70710678118654752).astype(np.float32))))


class ConvState:
    """History of one causal conv: the last (k - 1) * d rows of its transformed input, zero before the stream starts."""

    def __init__(self, k, d, cin):
        self.h = (k - 1) * d
        self.rows = np.zeros((self.h, cin), dtype=np.float32)


def conv(state, x, bias, act, w, k, d):
    """codec.rs:60-93 + codec.cu:291-318: out = (im2col of act(x + bias) and its history) . w^T, bias of the conv left
    to the consumer."""
    u = f32(x) + f32(bias)
    if act is not None:
        u = snake(u, *act)
    u = bf(u)
    ext = np.concatenate([state.rows, u], 0)
    T = len(u)
    col = np.concatenate([ext[j * d: j * d + T] for j in range(k)], 1)
    state.rows = ext[T:] if state.h else state.rows
    return gemm(col, w)


class StreamOracle:
    """One stream: `step(codes[16]) -> wav[samples_per_frame]` (bf16 values as float32)."""

    def __init__(self, cfg, W):
        self.c, self.W, self.pos = cfg, W, 0
        c = cfg
        qd = c.num_attention_heads * c.head_dim
        self.pre = ConvState(3, 1, c.codebook_dim)
        self.kring = np.zeros((c.num_hidden_layers, WINDOW, qd), dtype=np.float32)
        self.vring = np.zeros_like(self.kring)
        self.dw = [np.zeros((KERNEL - 1, c.latent_dim), dtype=np.float32) for _ in c.upsampling_ratios]
        self.conv_in = ConvState(KERNEL, 1, c.latent_dim)
        self.prev, self.units = [], []
        for i, rate in enumerate(c.upsample_rates):
            cout = c.decoder_dim >> (i + 1)
            self.prev.append(np.zeros((rate, cout), dtype=np.float32))
            self.units.append([ConvState(KERNEL, d, cout) for d in (1, 3, 9)])
        self.out_hist = np.zeros((KERNEL - 1, c.decoder_dim >> len(c.upsample_rates)), dtype=np.float32)

    def attention(self, layer, qkv):
        c, p = self.c, self.pos
        heads, qd = c.num_attention_heads, c.num_attention_heads * HEAD
        q, k, v = (qkv[i * qd:(i + 1) * qd].reshape(heads, HEAD) for i in range(3))
        lane = np.arange(32, dtype=np.float32)
        inv_freq = np.float32(1.0) / np.power(np.float32(c.rope_theta), np.float32(2.0) * lane / np.float32(HEAD)).astype(np.float32)
        ang = (np.float32(p) * inv_freq).astype(np.float32)
        s, co = np.sin(ang.astype(np.float64)).astype(np.float32), np.cos(ang.astype(np.float64)).astype(np.float32)

        def rot(x):
            lo, hi = f32(x[:, :32]), f32(x[:, 32:])
            return bf(np.concatenate([lo * co - hi * s, hi * co + lo * s], 1))
        q, k = rot(q), rot(k)
        self.kring[layer, p % WINDOW] = k.reshape(-1)
        self.vring[layer, p % WINDOW] = f32(v).reshape(-1)
        n = min(p + 1, WINDOW)
        idx = [(p - n + 1 + j) % WINDOW for j in range(n)]
        K = self.kring[layer, idx].reshape(n, heads, HEAD)
        V = self.vring[layer, idx].reshape(n, heads, HEAD)
        sc = np.einsum("hd,nhd->hn", q, K).astype(np.float32) * np.float32(1.0 / math.sqrt(HEAD))
        m = sc.max(-1, keepdims=True)
        e = np.exp(sc - m).astype(np.float32)
        o = np.einsum("hn,nhd->hd", e, V).astype(np.float32) / e.sum(-1, keepdims=True, dtype=np.float32)
        return bf(o.reshape(-1))

    def step(self, codes):
        c, W = self.c, self.W
        half, cb, lat, inter = c.codebook_dim // 2, c.codebook_size, c.latent_dim, c.intermediate_size
        books = W["rvq.books"]
        c0 = int(codes[0]) if int(codes[0]) < cb else 0
        rest = np.zeros(half, dtype=np.float32)
        for g in range(1, GROUPS):
            rest = rest + books[g * cb + int(codes[g])]
        col = np.concatenate([books[c0], bf(rest)])[None, :]
        a = gemm(col, W["rvq.out"])
        b = conv(self.pre, a, np.zeros(c.codebook_dim, dtype=np.float32), None, W["pre_conv.w"], 3, 1)
        res = gemm(b, W["input_proj.w"])
        res, x = rms_norm_add(W["input_proj.b"], res, W["l0.ln1"], c.rms_norm_eps)
        for i in range(c.num_hidden_layers):
            qkv = gemm(x, W[f"l{i}.qkv"])
            att = self.attention(i, qkv[0])[None, :]
            x = gemm(att, W[f"l{i}.o"])
            res, x = rms_norm_add(x, res, W[f"l{i}.ln2"], c.rms_norm_eps)
            gu = gemm(x, W[f"l{i}.gate_up"])
            x = gemm(silu_mul(gu, inter), W[f"l{i}.down"])
            nxt = W[f"l{i + 1}.ln1"] if i + 1 < c.num_hidden_layers else W["norm"]
            res, x = rms_norm_add(x, res, nxt, c.rms_norm_eps)
        cur = gemm(x, W["output_proj.w"])
        t = 1
        for i, r in enumerate(c.upsampling_ratios):
            z = gemm(cur, W[f"up{i}.w"]).reshape(t * r, lat)
            t *= r
            xin = bf(z + np.tile(W[f"up{i}.b"], (t // r, 1)))
            ext = np.concatenate([self.dw[i], xin], 0)
            acc = np.tile(W[f"up{i}.dw.b"][None, :], (t, 1)).astype(np.float32)
            for j in range(KERNEL):
                acc = acc + W[f"up{i}.dw.w"][j][None, :] * ext[j:j + t]
            self.dw[i] = ext[t:]
            acc = bf(acc)
            mean = acc.sum(-1, keepdims=True, dtype=np.float32) / np.float32(lat)
            var = ((acc - mean) ** 2).sum(-1, keepdims=True, dtype=np.float32) / np.float32(lat)
            rstd = (np.float32(1.0) / np.sqrt(var + np.float32(1e-6))).astype(np.float32)
            xn = bf((acc - mean) * rstd * W[f"up{i}.ln.w"] + W[f"up{i}.ln.b"])
            hcol = gelu_bias(gemm(xn, W[f"up{i}.pw1.w"]), W[f"up{i}.pw1.b"])
            cur = gemm_acc(xin, hcol, W[f"up{i}.pw2.w"])
        cur = conv(self.conv_in, cur, W["conv_in.in_b"], None, W["conv_in.w"], KERNEL, 1)
        for i, rate in enumerate(c.upsample_rates):
            cout = c.decoder_dim >> (i + 1)
            tmp = bf(snake(f32(cur) + W[f"b{i}.in_b"], *W[f"b{i}.snake"]))
            z = gemm(tmp, W[f"b{i}.up.w"]).reshape(t, 2 * rate, cout)
            before = np.concatenate([self.prev[i][None], z[:-1, rate:]], 0)      # taps rate.. of the row before
            self.prev[i] = z[-1, rate:].copy()
            cur = bf((W[f"b{i}.up.b"][None, None, :] + z[:, :rate]) + before).reshape(t * rate, cout)
            t *= rate
            for u, d in enumerate((1, 3, 9)):
                y = conv(self.units[i][u], cur, W[f"b{i}.u{u}.in_b"], W[f"b{i}.u{u}.s1"], W[f"b{i}.u{u}.conv1.w"], KERNEL, d)
                xs = bf(snake(f32(y) + W[f"b{i}.u{u}.conv1.b"], *W[f"b{i}.u{u}.s2"]))
                cur = gemm_acc(cur, xs, W[f"b{i}.u{u}.conv2.w"])
        v = bf(snake(f32(cur) + W["conv_out.in_b"], *W["conv_out.snake"]))
        ext = np.concatenate([self.out_hist, v], 0)
        self.out_hist = ext[t:]
        acc = np.zeros(t, dtype=np.float32)
        for j in range(KERNEL):
            acc = acc + (ext[j:j + t] * W["conv_out.w"][j][None, :]).sum(-1, dtype=np.float32)
        self.pos += 1
        return bf(np.clip(bf(acc + W["conv_out.b"][0]), -1.0, 1.0))


# ---- the decoder as published: float64, unfolded, all frames at once -----------------------------------------------

def _causal_conv(x, w, b, d=1):
    """x [T, cin], w [cout, cin, k]: left-padded by (k - 1) * d."""
    k = w.shape[2]
    T = len(x)
    ext = np.concatenate([np.zeros(((k - 1) * d, x.shape[1])), x], 0)
    out = np.zeros((T, w.shape[0]))
    for j in range(k):
        out += ext[j * d: j * d + T] @ w[:, :, j].T
    return out + b


def _snake64(x, alpha, beta):
    return x + (1.0 / (np.exp(beta) + 1e-9)) * np.sin(np.exp(alpha) * x) ** 2


def whole_utterance(ck, c, codes):
    """codes [F, 16] -> wav [F * samples_per_frame] in float64."""
    g = {k: np.asarray(v, dtype=np.float64) for k, v in ck.items()}
    codes = np.asarray(codes).reshape(-1, GROUPS)
    F = len(codes)
    half, cb, dim, lat, h = c.codebook_dim // 2, c.codebook_size, c.codebook_dim, c.latent_dim, c.hidden_size

    def book(p):
        return g[p + "._codebook.embedding_sum"] / np.maximum(g[p + "._codebook.cluster_usage"], 1e-5)[:, None]
    c0 = np.where(codes[:, 0] < cb, codes[:, 0], 0)
    e0 = book("decoder.quantizer.rvq_first.vq.layers.0")[c0]
    er = sum(book(f"decoder.quantizer.rvq_rest.vq.layers.{i}")[codes[:, i + 1]] for i in range(GROUPS - 1))
    x = e0 @ g["decoder.quantizer.rvq_first.output_proj.weight"].reshape(dim, half).T + \
        er @ g["decoder.quantizer.rvq_rest.output_proj.weight"].reshape(dim, half).T
    x = _causal_conv(x, g["decoder.pre_conv.conv.weight"], g["decoder.pre_conv.conv.bias"])
    pt = "decoder.pre_transformer"
    x = x @ g[f"{pt}.input_proj.weight"].T + g[f"{pt}.input_proj.bias"]
    heads = c.num_attention_heads
    pos = np.arange(F)[:, None]
    inv_freq = 1.0 / c.rope_theta ** (2.0 * np.arange(32) / HEAD)
    cs, sn = np.cos(pos * inv_freq)[:, None, :], np.sin(pos * inv_freq)[:, None, :]
    mask = (pos >= pos.T) & (pos - pos.T < c.sliding_window)

    def norm(v, w):
        return v / np.sqrt((v * v).mean(-1, keepdims=True) + c.rms_norm_eps) * w

    def rot(v):
        lo, hi = v[..., :32], v[..., 32:]
        return np.concatenate([lo * cs - hi * sn, hi * cs + lo * sn], -1)
    for i in range(c.num_hidden_layers):
        q_ = f"{pt}.layers.{i}."
        y = norm(x, g[q_ + "input_layernorm.weight"])
        q = rot((y @ g[q_ + "self_attn.q_proj.weight"].T).reshape(F, heads, HEAD))
        k = rot((y @ g[q_ + "self_attn.k_proj.weight"].T).reshape(F, heads, HEAD))
        v = (y @ g[q_ + "self_attn.v_proj.weight"].T).reshape(F, heads, HEAD)
        sc = np.einsum("ihd,jhd->hij", q, k) / math.sqrt(HEAD)
        sc = np.where(mask[None], sc, -np.inf)
        pr = np.exp(sc - sc.max(-1, keepdims=True))
        pr /= pr.sum(-1, keepdims=True)
        att = np.einsum("hij,jhd->ihd", pr, v).reshape(F, heads * HEAD)
        x = x + (att @ g[q_ + "self_attn.o_proj.weight"].T) * g[q_ + "self_attn_layer_scale.scale"]
        y = norm(x, g[q_ + "post_attention_layernorm.weight"])
        gate, up = y @ g[q_ + "mlp.gate_proj.weight"].T, y @ g[q_ + "mlp.up_proj.weight"].T
        x = x + ((gate / (1.0 + np.exp(-gate)) * up) @ g[q_ + "mlp.down_proj.weight"].T) * g[q_ + "mlp_layer_scale.scale"]
    x = norm(x, g[f"{pt}.norm.weight"])
    x = x @ g[f"{pt}.output_proj.weight"].T + g[f"{pt}.output_proj.bias"]
    erf = np.vectorize(math.erf, otypes=[np.float64])
    for i, r in enumerate(c.upsampling_ratios):
        p = f"decoder.upsample.{i}"
        w = g[f"{p}.0.conv.weight"]                                   # [in, out, r], stride = kernel
        x = np.einsum("tc,cor->tro", x, w).reshape(len(x) * r, lat) + g[f"{p}.0.conv.bias"]
        w7 = g[f"{p}.1.dwconv.conv.weight"][:, 0, :]                   # depthwise: one 7-tap filter per channel
        ext = np.concatenate([np.zeros((KERNEL - 1, lat)), x], 0)
        y = sum(ext[j:j + len(x)] * w7[:, j] for j in range(KERNEL)) + g[f"{p}.1.dwconv.conv.bias"]
        mu = y.mean(-1, keepdims=True)
        y = (y - mu) / np.sqrt(((y - mu) ** 2).mean(-1, keepdims=True) + 1e-6) * g[f"{p}.1.norm.weight"] + g[f"{p}.1.norm.bias"]
        y = y @ g[f"{p}.1.pwconv1.weight"].T + g[f"{p}.1.pwconv1.bias"]
        y = 0.5 * y * (1.0 + erf(y * 0.70710678118654752))
        y = y @ g[f"{p}.1.pwconv2.weight"].T + g[f"{p}.1.pwconv2.bias"]
        x = x + y * g[f"{p}.1.gamma"]
    x = _causal_conv(x, g["decoder.decoder.0.conv.weight"], g["decoder.decoder.0.conv.bias"])
    for i, rate in enumerate(c.upsample_rates):
        p = f"decoder.decoder.{i + 1}.block"
        x = _snake64(x, g[f"{p}.0.alpha"], g[f"{p}.0.beta"])
        w = g[f"{p}.1.conv.weight"]                                   # [cin, cout, 2 * rate], stride rate, right-trimmed
        z = np.einsum("tc,cok->tko", x, w)                            # [L, 2 rate, cout]
        L = len(x)
        out = np.zeros((L + 1, rate, w.shape[1]))
        out[:L] += z[:, :rate]
        out[1:] += z[:, rate:]
        x = out[:L].reshape(L * rate, -1) + g[f"{p}.1.conv.bias"]
        for u, d in enumerate((1, 3, 9)):
            q_ = f"{p}.{u + 2}"
            y = _causal_conv(_snake64(x, g[f"{q_}.act1.alpha"], g[f"{q_}.act1.beta"]), g[f"{q_}.conv1.conv.weight"],
                             g[f"{q_}.conv1.conv.bias"], d)
            y = _causal_conv(_snake64(y, g[f"{q_}.act2.alpha"], g[f"{q_}.act2.beta"]), g[f"{q_}.conv2.conv.weight"],
                             g[f"{q_}.conv2.conv.bias"])
            x = x + y
    n = len(c.upsample_rates) + 1
    x = _snake64(x, g[f"decoder.decoder.{n}.alpha"], g[f"decoder.decoder.{n}.beta"])
    x = _causal_conv(x, g[f"decoder.decoder.{n + 1}.conv.weight"], g[f"decoder.decoder.{n + 1}.conv.bias"])
    return np.clip(x[:, 0], -1.0, 1.0)


def snr_db(ours, theirs):
    ours, theirs = np.asarray(ours, dtype=np.float64).ravel(), np.asarray(theirs, dtype=np.float64).ravel()
    noise = ((ours - theirs) ** 2).sum()
    return 10.0 * math.log10((theirs ** 2).sum() / max(noise, 1e-300))
