"""The codec decoder's kernels, one call each through the C ABI, against the reference's own `codec.cu` compiled for
sm_100a (oracle/ref_kernels.py -> oracle/_ref/codec.cubin). Elementwise kernels, histories, overlap rows and the K/V ring
must agree bit for bit; where a sum is taken in another order (attention, LayerNorm, the output conv, the tensor-core
conv against im2col + an f32 matmul) the bf16 results may differ by one rounding step."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    from oracle import ref_kernels as R
    if not (R.OUT / "codec.cubin").exists():
        pytest.skip("reference cubins not built (the reference checkout was absent at build time)")
    import torch
    torch.zeros(1, device="cuda")
    return R, R._Module(R.OUT / "codec.cubin")


@pytest.fixture(scope="module")
def ops(built_lib):
    from pega_omni_b200.ops import Ops
    o = Ops(0)
    yield o
    o.close()


def _gen(seed):
    import torch
    return torch.Generator().manual_seed(seed)


def _bf(shape, g, scale=1.0):
    import torch
    return (torch.randn(shape, generator=g) * scale).to(torch.bfloat16).cuda()


def _i32(values):
    import torch
    return torch.tensor(values, dtype=torch.int32).cuda()


def _steps(got, want):
    """Largest difference in bf16 steps of the reference value (a step is 2^-7 of its binade)."""
    got, want = got.float().cpu().numpy(), want.float().cpu().numpy()
    step = np.exp2(np.floor(np.log2(np.maximum(np.abs(want), 1e-3))) - 7)
    return float((np.abs(got - want) / step).max())


def _snake_params(c, g):
    import torch
    alpha = torch.exp(0.3 * torch.randn(c, generator=g)).cuda()
    inv_b = (1.0 / (torch.exp(0.3 * torch.randn(c, generator=g)) + 1e-9)).cuda()
    return alpha, inv_b


def _state(slots, stride, g):
    """A per-stream state of `slots` slots with random bf16 contents (histories in flight), twice."""
    import torch
    s = (torch.randn(slots * stride // 2, generator=g) * 0.5).to(torch.bfloat16).cuda()
    return s, s.clone()


def _at(state, offset):
    """The state as the reference's kernels take it: the base pointer plus the layer's byte offset."""
    import torch
    return state.view(torch.uint8)[offset:]


def test_rvq_is_bit_exact(ref, ops):
    import torch
    R, cu = ref
    g = _gen(1)
    n, half, cb = 5, 256, 128
    books = _bf((16 * cb, half), g)
    codes = torch.randint(0, cb, (n, 16), generator=g, dtype=torch.int32)
    codes[2, 0] = cb + 102  # end of speech in codebook 0
    codes = codes.cuda()
    a = torch.zeros(n, 2 * half, dtype=torch.bfloat16, device="cuda")
    b = torch.zeros_like(a)
    ops.codec_rvq(codes, books, a, cb)
    ops.sync()
    cu.launch("codec_rvq", [n], half // 8, [R._p(codes), R._p(books), R._p(b), R._i(half), R._i(cb)])
    torch.cuda.synchronize()
    assert torch.equal(a, b)


def test_bias_gelu_and_bias_snake_are_bit_exact(ref, ops):
    import torch
    R, cu = ref
    g = _gen(2)
    rows, cols = 37, 256
    x = _bf((rows, cols), g, 2.0)
    bias = _bf((cols,), g, 0.3)
    total = rows * cols // 8
    a, b = x.clone(), x.clone()
    ops.codec_bias_gelu(a, bias)
    ops.sync()
    cu.launch("codec_bias_gelu", [(total + 255) // 256], 256, [R._p(b), R._p(bias), R._i(cols), R._i(total)])
    torch.cuda.synchronize()
    assert torch.equal(a, b)
    alpha, inv_b = _snake_params(cols, g)
    a, b = torch.zeros_like(x), torch.zeros_like(x)
    ops.codec_bias_snake(x, bias, alpha, inv_b, a)
    ops.sync()
    cu.launch("codec_bias_snake", [(total + 255) // 256], 256,
              [R._p(x), R._p(bias), R._p(alpha), R._p(inv_b), R._p(b), R._i(cols), R._i(total)])
    torch.cuda.synchronize()
    assert torch.equal(a, b)


@pytest.mark.parametrize("dim", [256, 512, 1024])
def test_add_norm_is_bit_exact(ref, ops, dim):
    import torch
    R, cu = ref
    g = _gen(3)
    rows, eps = 9, 1e-5
    x, res, w, bias = _bf((rows, dim), g), _bf((rows, dim), g), _bf((dim,), g, 0.2) + 1, _bf((dim,), g, 0.1)
    xa, ra, xb, rb = x.clone(), res.clone(), x.clone(), res.clone()
    ops.codec_add_norm(xa, ra, w, xa, eps)  # in place, as the reference's add_rms_norm
    ops.sync()
    cu.launch("codec_add_rms_norm", [(rows + 3) // 4], 128, [R._p(xb), R._p(rb), R._p(w), R._i(dim), R._f(eps), R._i(rows)])
    torch.cuda.synchronize()
    assert torch.equal(xa, xb) and torch.equal(ra, rb)
    oa, ob, ra, rb = torch.zeros_like(x), torch.zeros_like(x), res.clone(), res.clone()
    ops.codec_add_norm(bias, ra, w, oa, eps)  # one bias row for all
    ops.sync()
    cu.launch("codec_bias_rms_norm", [(rows + 3) // 4], 128,
              [R._p(rb), R._p(bias), R._p(w), R._p(ob), R._i(dim), R._f(eps), R._i(rows)])
    torch.cuda.synchronize()
    assert torch.equal(oa, ob) and torch.equal(ra, rb)


def test_window_attention_ring_is_bit_exact_and_rows_within_a_step(ref, ops):
    import torch
    R, cu = ref
    g = _gen(4)
    heads, n, offset = 4, 4, 256
    width = heads * 64
    stride = offset + 2 * 72 * width * 2 + 256
    sa, sb = _state(6, stride, g)
    qkv = _bf((n, 3 * width), g)
    lines, pos = _i32([3, 0, 5, 1]), _i32([0, 7, 71, 200])  # a first frame, a short history, a full window, a wrapped ring
    a = torch.zeros(n, width, dtype=torch.bfloat16, device="cuda")
    b = torch.zeros_like(a)
    ops.codec_window_attend(qkv, sa, lines, pos, stride, offset, a, heads, 10000.0)
    ops.sync()
    cu.launch("codec_attention", [n, heads], 128, [R._p(qkv), R._p(pos), R._p(lines), R._p(_at(sb, offset)), R._p(b),
                                                    R._l(stride), R._i(heads), R._f(10000.0)])
    torch.cuda.synchronize()
    assert torch.equal(sa, sb)        # rotated k and v landed in the same ring rows, bit for bit
    assert _steps(a, b) <= 1.0        # the weighted sums run in another order


@pytest.mark.parametrize("T,C,d,snake", [(5, 64, 3, True), (40, 96, 1, True), (4, 128, 1, False), (32, 64, 9, True)])
def test_stage_and_gather_reproduce_the_reference_im2col(ref, ops, T, C, d, snake):
    import torch
    R, cu = ref
    g = _gen(5)
    n, K, offset = 3, 7, 512
    H = (K - 1) * d
    stride = offset + 2 * H * C * 2 + 256
    sa, sb = _state(5, stride, g)
    x, bias = _bf((n * T, C), g, 1.5), _bf((C,), g, 0.3)
    alpha, inv_b = _snake_params(C, g) if snake else (None, None)
    lines, pos = _i32([4, 1, 2]), _i32([0, 3, 8])
    padded = torch.zeros(n, H + T, C, dtype=torch.bfloat16, device="cuda")
    a = torch.zeros(n * T, K * C, dtype=torch.bfloat16, device="cuda")
    b = torch.zeros_like(a)
    ops.codec_stage(x, bias, alpha, inv_b, sa, lines, pos, stride, offset, padded, n, T, H)
    ops.codec_gather_taps(padded, a, n, T, C, K, d)
    ops.sync()
    total = n * (H + T) * C // 8
    tail = [R._p(_at(sb, offset)), R._p(pos), R._p(lines), R._p(b), R._i(T), R._i(C), R._i(K), R._i(d), R._l(stride),
            R._i(total)]
    if snake:
        cu.launch("codec_im2col_snake", [(total + 255) // 256], 256, [R._p(x), R._p(bias), R._p(alpha), R._p(inv_b)] + tail)
    else:
        cu.launch("codec_im2col", [(total + 255) // 256], 256, [R._p(x), R._p(bias)] + tail)
    torch.cuda.synchronize()
    assert torch.equal(a, b)          # the matrix the reference multiplies
    assert torch.equal(sa, sb)        # and the history it leaves for the next frame


@pytest.mark.parametrize("T,C,N,d,n", [(256, 96, 96, 9, 3), (160, 192, 192, 3, 3), (32, 128, 256, 1, 6), (4, 64, 48, 1, 40)])
def test_implicit_conv_matches_im2col_and_a_matmul(ref, ops, T, C, N, d, n):
    """The tensor-core conv (no im2col matrix; 96 channels take the zero-filled boxes; 160 and 32 rows per stream put
    several streams into one tile, the last tile partly past the last stream) against the reference's path: its
    im2col kernel, an f32-accumulating matmul, its SnakeBeta kernel."""
    import torch
    R, cu = ref
    g = _gen(6)
    K, offset = 7, 0
    H = (K - 1) * d
    stride = 2 * H * C * 2 + 256
    sa, sb = _state(n, stride, g)
    x, bias = _bf((n * T, C), g, 1.5), _bf((C,), g, 0.3)
    s1 = _snake_params(C, g)
    w = _bf((N, K * C), g, 1.0 / np.sqrt(K * C))
    c1_b, s2 = _bf((N,), g, 0.2), _snake_params(N, g)
    lines, pos = _i32(list(range(n))), _i32([i % 3 for i in range(n)])
    padded = torch.zeros(n, H + T, C, dtype=torch.bfloat16, device="cuda")
    ops.codec_stage(x, bias, s1[0], s1[1], sa, lines, pos, stride, offset, padded, n, T, H)
    y = torch.zeros(n * T, N, dtype=torch.bfloat16, device="cuda")
    ops.codec_conv(w, C, K, d, padded, T, n, y, epilogue=2, bias=c1_b, alpha=s2[0], inv_b=s2[1])
    plain = torch.zeros_like(y)
    ops.codec_conv(w, C, K, d, padded, T, n, plain, epilogue=0)
    ops.sync()
    col = torch.zeros(n * T, K * C, dtype=torch.bfloat16, device="cuda")
    total = n * (H + T) * C // 8
    cu.launch("codec_im2col_snake", [(total + 255) // 256], 256,
              [R._p(x), R._p(bias), R._p(s1[0]), R._p(s1[1]), R._p(sb), R._p(pos), R._p(lines), R._p(col), R._i(T), R._i(C),
               R._i(K), R._i(d), R._l(stride), R._i(total)])
    z = (col.float() @ w.float().T).to(torch.bfloat16)
    want = torch.zeros_like(z)
    tot2 = n * T * N // 8
    cu.launch("codec_bias_snake", [(tot2 + 255) // 256], 256,
              [R._p(z), R._p(c1_b), R._p(s2[0]), R._p(s2[1]), R._p(want), R._i(N), R._i(tot2)])
    torch.cuda.synchronize()
    assert _steps(plain, z) <= 1.0                       # one rounding of sums taken in two orders
    flips = (plain != z).float().mean().item()
    assert flips < 0.02
    same = plain == z
    assert torch.equal(y[same], want[same])              # where the GEMMs agree the fused SnakeBeta epilogue is exact
    # accumulate: y = bf16(y + a) with one rounding, against the f32 sum
    base = _bf((n * T, N), g)
    acc = base.clone()
    ops.codec_conv(w[:, :C].contiguous(), C, 1, 1, x, T, n, acc, epilogue=1)
    ops.sync()
    want_acc = (base.float() + x.float() @ w[:, :C].float().T).to(torch.bfloat16)
    assert _steps(acc, want_acc) <= 1.0 and (acc != want_acc).float().mean().item() < 0.02


def test_overlap_add_is_bit_exact(ref, ops):
    import torch
    R, cu = ref
    g = _gen(7)
    n, L, r, C, offset = 3, 4, 5, 64, 128
    stride = offset + r * C * 2 + 256
    sa, sb = _state(4, stride, g)
    z, bias = _bf((n, L, 2 * r * C), g), _bf((C,), g, 0.2)
    lines, pos = _i32([2, 0, 3]), _i32([1, 1, 1])
    a = torch.zeros(n * L * r, C, dtype=torch.bfloat16, device="cuda")
    b = torch.zeros_like(a)
    ops.codec_overlap_add(z, bias, sa, lines, pos, stride, offset, a, n, L, r, C)
    ops.sync()
    total = n * L * r * C // 8
    cu.launch("codec_col2im", [(total + 255) // 256], 256, [R._p(z), R._p(bias), R._p(_at(sb, offset)), R._p(lines),
                                                            R._p(b), R._i(L), R._i(r), R._i(C), R._l(stride), R._i(total)])
    torch.cuda.synchronize()
    assert torch.equal(a, b) and torch.equal(sa, sb)


@pytest.mark.parametrize("T,C", [(2, 256), (8, 1024), (4, 512)])
def test_dwconv_ln_history_is_bit_exact_and_rows_within_a_step(ref, ops, T, C):
    import torch
    R, cu = ref
    g = _gen(8)
    n, r, offset, eps = 3, 2, 64, 1e-6
    stride = offset + 2 * 6 * C * 2 + 256
    sa, sb = _state(4, stride, g)
    z, zb = _bf((n * T, C), g), _bf((r, C), g, 0.2)
    w, b_, lw, lb = _bf((7, C), g, 0.4), _bf((C,), g, 0.1), _bf((C,), g, 0.2) + 1, _bf((C,), g, 0.1)
    lines, pos = _i32([1, 3, 0]), _i32([0, 1, 6])
    xa, oa = torch.zeros(n * T, C, dtype=torch.bfloat16, device="cuda"), torch.zeros(n * T, C, dtype=torch.bfloat16, device="cuda")
    xb, ob = torch.zeros_like(xa), torch.zeros_like(oa)
    ops.codec_dwconv_ln(z, zb, w, b_, lw, lb, sa, lines, pos, stride, offset, xa, oa, n, T, r, eps)
    ops.sync()
    cu.launch("codec_dwconv_ln", [n * T], C // 8,
              [R._p(z), R._p(zb), R._p(w), R._p(b_), R._p(lw), R._p(lb), R._p(_at(sb, offset)), R._p(pos), R._p(lines),
               R._p(xb), R._p(ob), R._i(T), R._i(r), R._i(C), R._l(stride), R._f(eps)])
    torch.cuda.synchronize()
    assert torch.equal(xa, xb) and torch.equal(sa, sb)
    assert _steps(oa, ob) <= 1.0      # the two block-wide sums run in another order


@pytest.mark.parametrize("C", [96, 128, 32])
def test_output_conv_history_is_bit_exact_and_samples_within_a_step(ref, ops, C):
    import torch
    R, cu = ref
    g = _gen(9)
    n, T, offset = 3, 192, 0
    stride = 2 * 6 * C * 2 + 256
    sa, sb = _state(3, stride, g)
    x, bias = _bf((n * T, C), g), _bf((C,), g, 0.2)
    alpha, inv_b = _snake_params(C, g)
    w, wb = _bf((7, C), g, 0.3 / np.sqrt(7 * C)), _bf((1,), g, 0.05)
    lines, pos = _i32([2, 0, 1]), _i32([0, 1, 4])
    a = torch.zeros(n, T, dtype=torch.float32, device="cuda")
    b = torch.zeros(n, T, dtype=torch.bfloat16, device="cuda")
    ops.codec_out_conv(x, bias, alpha, inv_b, w, wb, sa, lines, pos, stride, offset, a, n, T)
    ops.sync()
    cu.launch("codec_conv_out", [T // 64, n], 256,
              [R._p(x), R._p(bias), R._p(alpha), R._p(inv_b), R._p(w), R._p(wb), R._p(sb), R._p(pos), R._p(lines), R._p(b),
               R._i(T), R._i(C), R._l(stride)])
    torch.cuda.synchronize()
    assert torch.equal(sa, sb)
    assert torch.equal(a.to(torch.bfloat16).float(), a)   # the f32 samples are bf16 values
    assert _steps(a, b) <= 1.0 and a.abs().max() <= 1.0
