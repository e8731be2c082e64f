"""The duplex kernels against the reference's own `lm.cu`, compiled to an sm_100a cubin and launched on the same GPU
(oracle/ref_kernels.py): draws and token bookkeeping bit for bit, the float kernels to rounding."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    from oracle import ref_kernels as R
    if not (R.OUT / "lm.cubin").exists():
        pytest.skip("reference cubins not built (the reference checkout was absent at build time)")
    import torch
    torch.zeros(1, device="cuda")  # the driver context the cubin is loaded into
    return R, R._Module(R.OUT / "lm.cubin")


@pytest.fixture(scope="module")
def ops(built_lib):
    from pega_omni_b200.ops import Ops
    o = Ops(0)
    yield o
    o.close()


def bf16(t):
    import torch
    return t.to(torch.bfloat16).cuda()


@pytest.mark.parametrize("vocab,top_k,temperature", [(2048, 250, 0.8), (2048, 0, 0.8), (32000, 25, 0.7),
                                                      (1000, 25, 0.0), (2048, 2048, 1.0)])
def test_draw_is_bit_exact(ref, ops, vocab, top_k, temperature):
    """`lm_sample`: both vocabulary paths of the reference (registers up to 2048, strided above), ties in the top-k,
    forced columns, greedy."""
    import torch
    R, lm = ref
    rows, col = 96, 3
    g = torch.Generator().manual_seed(vocab + top_k)
    logits = bf16(torch.randn(rows, vocab, generator=g) * 2.5)
    logits[:, 5] = logits[:, 700]  # ties
    force = torch.full((rows, 9), -1, dtype=torch.int32)
    force[::7, col] = 11
    force = force.cuda()
    seeds = torch.randint(-2 ** 31, 2 ** 31 - 1, (rows, 2), generator=g, dtype=torch.int64).to(torch.int32).cuda()
    ours = torch.zeros(rows, 9, dtype=torch.int32, device="cuda")
    theirs = torch.zeros_like(ours)
    ops.lm_sample(logits, temperature, top_k, force, seeds, col, ours)
    ops.sync()
    lm.launch("lm_sample", [rows], 1024, [R._p(logits), R._i(vocab), R._l(vocab), R._f(temperature), R._i(top_k),
                                           R._p(force), R._p(seeds), R._i(col), R._p(theirs)])
    torch.cuda.synchronize()
    assert torch.equal(ours, theirs)
    assert (ours[::7, col] == 11).all() and len(set(ours[:, col].tolist())) > (1 if temperature == 0 else 20)


def test_token_bookkeeping_is_bit_exact(ref, ops):
    """`lm_init` + `lm_advance` over several ticks with shuffled state lines."""
    import torch
    R, lm = ref
    n, stride = 40, 256
    g = torch.Generator().manual_seed(9)
    lines = torch.randperm(64, generator=g)[:n].to(torch.int32).cuda()
    init = torch.randint(0, 2048, (n, 24), generator=g, dtype=torch.int32).cuda()
    a = torch.zeros(64 * stride, dtype=torch.uint8, device="cuda")
    b = torch.zeros_like(a)
    ops.lm_advance(a, lines, stride, n, init=init)
    lm.launch("lm_init", [n], 32, [R._p(b), R._p(lines), R._l(stride), R._p(init)])
    for t in range(5):
        drawn = torch.randint(0, 2048, (n, 9), generator=g, dtype=torch.int32).cuda()
        caller = torch.randint(0, 2048, (n, 8), generator=g, dtype=torch.int32).cuda()
        fc = torch.randint(-1, 3, (n, 8), generator=g, dtype=torch.int32).cuda()
        ea = torch.zeros(n, 9, dtype=torch.int32, device="cuda")
        eb = torch.zeros_like(ea)
        ops.lm_advance(a, lines, stride, n, drawn=drawn, caller=caller, force_caller=fc, emitted=ea)
        ops.sync()
        lm.launch("lm_advance", [(n + 127) // 128], 128, [R._p(b), R._p(lines), R._l(stride), R._p(drawn), R._p(caller),
                                                         R._p(fc), R._p(eb), R._i(n)])
        torch.cuda.synchronize()
        assert torch.equal(ea, eb) and torch.equal(a, b)


def test_norms_and_embedding_match(ref, ops):
    import torch
    R, lm = ref
    g = torch.Generator().manual_seed(3)
    rows, dim, card_rows, text_rows = 24, 1024, 65, 301
    x = bf16(torch.randn(rows, dim, generator=g) * 3)
    y = bf16(torch.randn(rows, dim, generator=g))
    alpha = bf16(1 + 0.1 * torch.randn(dim, generator=g))
    eps = 1e-8
    o1, o2 = torch.zeros_like(x), torch.zeros_like(x)
    ops.lm_norm(x, alpha, o1, eps)
    ops.sync()
    lm.launch("lm_norm", [rows], dim // 8, [R._p(x), R._p(alpha), R._p(o2), R._i(dim), R._f(eps)])
    torch.cuda.synchronize()
    # the row sum is taken in a different association order: at most one bf16 step on a handful of elements
    d = (o1.float() - o2.float()).abs()
    assert (d > 0).float().mean() < 0.01 and d.max() <= 2.0 ** -5
    xa, xb = x.clone(), x.clone()
    ops.lm_norm(xa, alpha, o1, eps, y=y)
    ops.sync()
    lm.launch("lm_add_norm", [rows], dim // 8, [R._p(y), R._p(xb), R._p(alpha), R._p(o2), R._i(dim), R._f(eps)])
    torch.cuda.synchronize()
    assert torch.equal(xa, xb)
    d = (o1.float() - o2.float()).abs()
    assert (d > 0).float().mean() < 0.01 and d.max() <= 2.0 ** -5
    text_emb = bf16(torch.randn(text_rows, dim, generator=g))
    audio_emb = bf16(torch.randn(16 * card_rows, dim, generator=g))
    ids = torch.randint(0, card_rows, (rows, 17), generator=g, dtype=torch.int32)
    ids[:, 0] = torch.randint(0, text_rows, (rows,), generator=g)
    ids[torch.rand(rows, 17, generator=g) < 0.15] = -1
    ids = ids.cuda()
    voice = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
    if card_rows == 2049:  # the reference's table stride is fixed at 2049 rows per stream
        pass
    e1 = torch.zeros(rows, dim, dtype=torch.bfloat16, device="cuda")
    ops.lm_embed(ids, text_emb, audio_emb, e1)
    ops.sync()
    # reference layout: 2049 rows per audio stream
    wide = torch.zeros(16 * 2049, dim, dtype=torch.bfloat16, device="cuda")
    for k in range(16):
        wide[k * 2049:k * 2049 + card_rows] = audio_emb[k * card_rows:(k + 1) * card_rows]
    e2 = torch.zeros_like(e1)
    lm.launch("lm_embed_prompt", [rows], dim // 8, [R._p(ids), R._p(voice), R._p(text_emb), R._p(text_emb), R._p(wide),
                                                   R._p(e2), R._i(dim)])
    torch.cuda.synchronize()
    assert torch.equal(e1, e2)


def test_rope_fp8_kv_and_attention_match(ref, ops):
    """`lm_rope` + `lm_attend`: q rotated in place bit for bit, the FP8 keys, values and scales byte for byte (after
    mapping the reference's slot-major layout to this library's page blocks), attention output to a bf16 step — over
    several positions so later rows read earlier rows' slots, with a ring that wraps."""
    import torch
    R, lm = ref
    heads, sessions, context, steps = 4, 5, 24, 30
    ppseq = (context + 15) // 16
    kv_pages = sessions * ppseq
    coef = float(np.float32(-np.log(10000.0) * 2.0 / 128))
    scale = 1.0 / np.sqrt(128.0)
    slot_bytes = 2 * heads * 128 + 2 * heads * 4
    ours_kv = torch.zeros(kv_pages * heads * (2 * 16 * 128 + 2 * 16 * 4), dtype=torch.uint8, device="cuda")
    ref_kv = torch.zeros(kv_pages * 16 * slot_bytes, dtype=torch.uint8, device="cuda")
    g = torch.Generator().manual_seed(5)
    perm = torch.randperm(kv_pages, generator=g).to(torch.int32)
    pages = perm.cuda()
    indptr = torch.arange(0, kv_pages + 1, ppseq, dtype=torch.int32).cuda()
    for p in range(steps):
        qkv = bf16(torch.randn(sessions, 3 * heads * 128, generator=g) * 2)
        ring = p % context
        pos = torch.full((sessions,), p, dtype=torch.int32).cuda()
        slot = torch.tensor([int(perm[s * ppseq + ring // 16]) * 16 + ring % 16 for s in range(sessions)],
                            dtype=torch.int32).cuda()
        qa, qb = qkv.clone(), qkv.clone()
        oa = torch.zeros(sessions, heads * 128, dtype=torch.bfloat16, device="cuda")
        ob = torch.zeros_like(oa)
        ops.lm_rope_attend(qa, ours_kv, kv_pages, pos, slot, None, indptr, pages, heads, coef, scale, context, oa)
        ops.sync()
        lm.launch("lm_rope", [sessions, (3 * heads + 7) // 8], 256,
                  [R._p(qb), R._p(pos), R._p(slot), R._p(ref_kv), R._i(heads), R._f(coef)])
        lm.launch("lm_attend", [sessions, heads], 128,
                  [R._p(qb), R._p(ref_kv), R._p(pos), R._p(pos), R._i(0), R._p(indptr), R._p(pages), R._i(16), R._p(ob),
                   R._i(heads), R._f(scale), R._i(context)])
        torch.cuda.synchronize()
        assert torch.equal(qa[:, :heads * 128], qb[:, :heads * 128]), p
        d = (oa.float() - ob.float()).abs()
        assert d.max() <= 2.0 ** -6 * max(1.0, float(ob.float().abs().max())), (p, float(d.max()))
    # KV bytes: reference slot = [K heads | V heads | K scales | V scales]; ours = per (page, head) blocks
    a = ours_kv.cpu().numpy().reshape(kv_pages, heads, 2 * 16 * 128 + 128)
    b = ref_kv.cpu().numpy().reshape(kv_pages, 16, slot_bytes)
    for h in range(heads):
        assert np.array_equal(a[:, h, :2048].reshape(kv_pages, 16, 128), b[:, :, h * 128:(h + 1) * 128])
        assert np.array_equal(a[:, h, 2048:4096].reshape(kv_pages, 16, 128), b[:, :, (heads + h) * 128:(heads + h + 1) * 128])
        ks = 2 * heads * 128
        assert np.array_equal(a[:, h, 4096:4160].reshape(kv_pages, 16, 4), b[:, :, ks + h * 4:ks + h * 4 + 4])
        assert np.array_equal(a[:, h, 4160:4224].reshape(kv_pages, 16, 4), b[:, :, ks + (heads + h) * 4:ks + (heads + h) * 4 + 4])


def test_depformer_kernels_match(ref, ops):
    import torch
    R, lm = ref
    g = torch.Generator().manual_seed(7)
    rows, dim, heads, table_rows = 20, 1024, 16, 300
    eps, scale = 1e-8, 0.125
    projected = bf16(torch.randn(rows, 8 * dim, generator=g))
    table = bf16(torch.randn(table_rows, dim, generator=g))
    alpha = bf16(1 + 0.1 * torch.randn(dim, generator=g))
    drawn = torch.randint(0, table_rows, (rows, 9), generator=g, dtype=torch.int32).cuda()
    wa = torch.zeros(rows * 8 * 2 * dim, dtype=torch.bfloat16, device="cuda")
    wb = torch.zeros_like(wa)
    for k in range(8):
        xa, xna = (torch.zeros(rows, dim, dtype=torch.bfloat16, device="cuda") for _ in range(2))
        xb, xnb = torch.zeros_like(xa), torch.zeros_like(xa)
        ops.lm_dep_embed_norm(projected, k, table, drawn, alpha, xa, xna, eps)
        ops.sync()
        lm.launch("lm_dep_embed_norm", [rows], dim // 8, [R._p(projected), R._i(k), R._p(table), R._p(drawn), R._p(alpha),
                                                         R._p(xb), R._p(xnb), R._i(dim), R._f(eps)])
        torch.cuda.synchronize()
        assert torch.equal(xa, xb)
        d = (xna.float() - xnb.float()).abs()
        assert (d > 0).float().mean() < 0.01 and d.max() <= 2.0 ** -5
        qkv = bf16(torch.randn(rows, 3 * dim, generator=g))
        oa = torch.zeros(rows, dim, dtype=torch.bfloat16, device="cuda")
        ob = torch.zeros_like(oa)
        ops.lm_dep_kv_attend(qkv, wa, k, oa, heads, scale)
        ops.sync()
        lm.launch("lm_dep_kv_attend", [rows, heads], 32, [R._p(qkv), R._p(wb), R._i(k), R._p(ob), R._i(heads), R._f(scale)])
        torch.cuda.synchronize()
        assert torch.equal(wa, wb) and torch.equal(oa, ob), k
