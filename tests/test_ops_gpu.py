"""Kernel-level parity on the GPU: every operator of include/omni_b200_ops.h against the CPU oracle on the
same seeded inputs. Elementwise ops must agree to one bf16 rounding step; GEMMs (different f32 summation
order) to the same; the sampler must pick identical token ids for identical logits and uniforms."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

BF16_ULP = 2.0 ** -8


def to_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().view(torch.int16).numpy().view(np.uint16)


def to_f32(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy()


def close_bf16(got: np.ndarray, want: np.ndarray, ulps: float = 1.0, floor: float = 1e-3):
    tol = ulps * BF16_ULP * np.maximum(np.abs(want), floor) * 2
    bad = np.abs(got - want) > tol
    assert not bad.any(), f"{bad.sum()} of {bad.size} beyond {ulps} bf16 steps; worst {np.abs(got - want).max()}"


@pytest.fixture(scope="module")
def ops(built_lib):
    from pega_omni_b200.ops import Ops
    o = Ops(0)
    yield o
    o.close()


def rand_bf16(shape, seed, scale=1.0):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


@pytest.mark.parametrize("rows,n,k", [(1, 512, 256), (3, 200, 1024), (8, 1024, 2048), (20, 256, 512)])
def test_gemv_matches_oracle(ops, oracle_lib, rows, n, k):
    w, x = rand_bf16((n, k), 1, 0.05), rand_bf16((rows, k), 2)
    y = torch.zeros((rows, n), dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    ops.gemm(w, x, y, path=1)
    ops.sync()
    close_bf16(to_f32(y), oracle_lib.gemm(to_f32(x), to_bits(w)))


@pytest.mark.parametrize("rows,n,k,splits", [
    (16, 128, 64, 1), (16, 256, 512, 0), (24, 384, 1024, 2), (64, 4096, 2048, 0), (64, 2048, 6144, 8),
    (64, 200, 256, 1), (128, 1024, 1024, 0), (130, 256, 512, 0), (256, 512, 512, 3), (300, 256, 256, 1),
    (48, 3072, 2048, 0), (12, 1024, 512, 0),
])
def test_tensor_core_gemm_matches_oracle(ops, oracle_lib, rows, n, k, splits):
    w, x = rand_bf16((n, k), 3, 0.05), rand_bf16((rows, k), 4)
    y = torch.full((rows, n), 7.0, dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    ops.gemm(w, x, y, path=2, splits=splits)
    ops.sync()
    want = oracle_lib.gemm(to_f32(x), to_bits(w))
    close_bf16(to_f32(y), want)
    # and the two device paths agree with each other
    y2 = torch.zeros_like(y)
    ops.gemm(w, x, y2, path=1)
    ops.sync()
    close_bf16(to_f32(y), to_f32(y2))
    # a second launch reuses the split-K counters: they must have been reset
    y3 = torch.zeros_like(y)
    ops.gemm(w, x, y3, path=2, splits=splits)
    ops.sync()
    assert torch.equal(y, y3)


@pytest.mark.parametrize("path", [1, 2])
@pytest.mark.parametrize("epi", [1, 2])
def test_gemm_bias_epilogues(ops, oracle_lib, path, epi):
    rows, n, k = 32, 512, 256
    w, x, b = rand_bf16((n, k), 5, 0.05), rand_bf16((rows, k), 6), rand_bf16((n,), 7, 0.5)
    y = torch.zeros((rows, n), dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    ops.gemm(w, x, y, path=path, bias=b, epilogue=epi)
    ops.sync()
    t = oracle_lib.bf16_round(oracle_lib.gemm(to_f32(x), to_bits(w)) + to_f32(b)[None])
    if epi == 2:
        t = oracle_lib.bf16_round(t / (1.0 + np.exp(-t)))
    # the accumulator (|a| ~ 1) may round one step apart on the two sides; after the bias and the SiLU that step is
    # an absolute error, so the floor is the accumulator's scale, not the output's
    close_bf16(to_f32(y), t, ulps=2.0, floor=0.5)


@pytest.mark.parametrize("rows,n,k", [(128, 1024, 1024), (128, 3072, 1024), (100, 1000, 2816), (32, 3584, 2560),
                                      (9, 320, 256), (128, 22528, 4096), (64, 72, 64), (128, 12288, 4096), (77, 4096, 4096)])
def test_gemm_rows_on_m(ops, oracle_lib, rows, n, k):
    """The no-split tensor-core path (input rows on the MMA M dimension): ragged row counts, N not a multiple of the
    tile, all three tile widths, a strided output."""
    w, x = rand_bf16((n, k), 21, 0.05), rand_bf16((rows, k), 22)
    big = torch.zeros((rows, n + 16), dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    ops.gemm(w, x, big[:, 8:8 + n], path=3)
    ops.sync()
    # outputs near zero are sums of thousands of O(0.05) products: the floor is the accumulator's scale
    close_bf16(to_f32(big[:, 8:8 + n]), oracle_lib.gemm(to_f32(x), to_bits(w)), floor=0.05)
    assert not big[:, :8].any() and not big[:, 8 + n:].any()


def test_gemm_strided_output(ops, oracle_lib):
    # logits of group g land in a wider buffer (ldy > N), the way p_logits is addressed
    rows, n, k = 16, 256, 128
    w, x = rand_bf16((n, k), 8, 0.05), rand_bf16((rows, k), 9)
    big = torch.zeros((rows, 3 * n), dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    ops.gemm(w, x, big[:, n:2 * n], path=2)
    ops.sync()
    close_bf16(to_f32(big[:, n:2 * n]), oracle_lib.gemm(to_f32(x), to_bits(w)))
    assert not big[:, :n].any() and not big[:, 2 * n:].any()


@pytest.mark.parametrize("rows,dim", [(1, 128), (5, 1024), (64, 2048)])
def test_norms_match_oracle(ops, oracle_lib, rows, dim):
    x, res, w = rand_bf16((rows, dim), 10), rand_bf16((rows, dim), 11), rand_bf16((dim,), 12, 0.3) + 1
    out, r2 = torch.zeros_like(x), torch.zeros_like(x)
    torch.cuda.synchronize()
    ops.norm_copy(x, w, out, r2, 1e-6)
    ops.sync()
    want, want_res = oracle_lib.norm_copy(to_f32(x), to_bits(w), 1e-6)
    close_bf16(to_f32(out), want)
    assert np.array_equal(to_f32(r2), want_res)
    for every, which in ((1, 0), (2, 1)):
        if rows % every:
            continue
        res_d = res.clone()
        out = torch.zeros((rows // every, dim), dtype=torch.bfloat16, device="cuda")
        torch.cuda.synchronize()
        ops.add_norm(x, res_d, w, out, 1e-6, every, which)
        ops.sync()
        want, want_res = oracle_lib.add_norm(to_f32(x), to_f32(res), to_bits(w), 1e-6, every, which)
        close_bf16(to_f32(out), want)
        assert np.array_equal(to_f32(res_d), want_res)


def test_silu_mul_matches_oracle(ops, oracle_lib):
    gu = rand_bf16((9, 2 * 768), 13, 2.0)
    act = torch.zeros((9, 768), dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    ops.silu_mul(gu, act)
    ops.sync()
    close_bf16(to_f32(act), oracle_lib.silu_mul(to_f32(gu)), ulps=2.0)


@pytest.mark.parametrize("hq,hk,d", [(4, 2, 128), (4, 2, 64), (16, 8, 128), (8, 8, 128), (8, 2, 128), (5, 1, 128)])
def test_rope_attend_ragged_paged(ops, oracle_lib, hq, hk, d):
    """A ragged prefill over shuffled pages: every row's attention equals the oracle's over positions 0..pos."""
    rng = np.random.default_rng(hq * 100 + d)
    lens = [5, 19, 40, 16]
    rows = sum(lens)
    n_pages = 32
    width = (hq + 2 * hk) * d
    qkv = rand_bf16((rows, width), 14)
    qn, kn = rand_bf16((d,), 15, 0.2) + 1, rand_bf16((d,), 16, 0.2) + 1
    kv = torch.zeros((n_pages, hk, 2, 16, d), dtype=torch.bfloat16, device="cuda")
    perm = rng.permutation(n_pages)
    pos, slot, seq, indptr, pages = [], [], [], [0], []
    at = 0
    for s, n in enumerate(lens):
        mine = [int(p) for p in perm[at:at + (n + 15) // 16]]
        at += len(mine)
        pages += mine
        indptr.append(len(pages))
        for t in range(n):
            pos.append(t)
            slot.append(mine[t // 16] * 16 + t % 16)
            seq.append(s)
    dev = lambda a: torch.tensor(a, dtype=torch.int32, device="cuda")
    out = torch.zeros((rows, hq * d), dtype=torch.bfloat16, device="cuda")
    qkv_in = to_f32(qkv)
    torch.cuda.synchronize()
    ops.rope_attend(qkv, qn, kn, kv, n_pages, dev(pos), dev(slot), dev(seq), dev(indptr), dev(pages), hq, hk, d, 1e-6,
                    1e6, out)
    ops.sync()
    # oracle: rotate every q/k head, then attend row by row
    eps, theta = 1e-6, 1e6
    want = np.zeros((rows, hq * d), dtype=np.float32)
    r = 0
    got_q = to_f32(qkv)
    for s, n in enumerate(lens):
        kvrows = np.zeros((n, 2 * hk * d), dtype=np.float32)
        qrows = np.zeros((n, hq * d), dtype=np.float32)
        for t in range(n):
            row = qkv_in[r + t]
            for h in range(hq):
                qrows[t, h * d:(h + 1) * d] = oracle_lib.rope_head(row[h * d:(h + 1) * d], to_bits(qn), t, eps, theta)
            for h in range(hk):
                a = (hq + h) * d
                kvrows[t, h * d:(h + 1) * d] = oracle_lib.rope_head(row[a:a + d], to_bits(kn), t, eps, theta)
            kvrows[t, hk * d:] = row[(hq + hk) * d:]
        close_bf16(got_q[r:r + n, :hq * d], qrows, ulps=2.0, floor=0.5)  # a*cos - b*sin cancels: absolute scale of a, b
        bits = oracle_lib.bf16_bits(kvrows)
        for t in range(n):
            want[r + t] = oracle_lib.attend(qrows[t], bits[:t + 1], hq, hk, d)
        r += n
    close_bf16(to_f32(out), want, ulps=3.0, floor=0.25)  # averages of O(1) values: absolute scale


def test_rope_attend_decode_rows_over_long_paged_contexts(ops, oracle_lib):
    """Decode rows (one per sequence) at positions from 0 to several hundred over shuffled pages: a warp of the
    attention team then goes through its staging slots many times, and the last block holds the token written by the
    same call. Every row equals the oracle's attention over the pool's rows 0..pos."""
    hq, hk, d = 16, 8, 128
    rng = np.random.default_rng(77)
    lens = [1, 17, 129, 200, 333, 512, 64, 33]  # keys per sequence, the new token included
    rows = len(lens)
    n_pages = sum((n + 15) // 16 for n in lens) + 3
    width = (hq + 2 * hk) * d
    qkv = rand_bf16((rows, width), 21)
    qn, kn = rand_bf16((d,), 22, 0.2) + 1, rand_bf16((d,), 23, 0.2) + 1
    kv = rand_bf16((n_pages, hk, 2, 16, d), 24)
    perm = rng.permutation(n_pages)
    pos, slot, seq, indptr, pages = [], [], [], [0], []
    at = 0
    for s, n in enumerate(lens):
        mine = [int(p) for p in perm[at:at + (n + 15) // 16]]
        at += len(mine)
        pages += mine
        indptr.append(len(pages))
        pos.append(n - 1)
        slot.append(mine[(n - 1) // 16] * 16 + (n - 1) % 16)
        seq.append(s)
    dev = lambda a: torch.tensor(a, dtype=torch.int32, device="cuda")
    out = torch.zeros((rows, hq * d), dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    ops.rope_attend(qkv, qn, kn, kv, n_pages, dev(pos), dev(slot), dev(seq), dev(indptr), dev(pages), hq, hk, d, 1e-6,
                    1e6, out)
    ops.sync()
    pool = to_f32(kv)      # after the call: the new tokens' rotated keys and values are in their slots
    q_rot = to_f32(qkv)    # and the query heads were rotated in place
    for s, n in enumerate(lens):
        mine = pages[indptr[s]:indptr[s + 1]]
        rows_kv = np.zeros((n, 2 * hk * d), dtype=np.float32)
        for t in range(n):
            blk = pool[mine[t // 16]]  # [hk, 2, 16, d]
            rows_kv[t, :hk * d] = blk[:, 0, t % 16, :].reshape(-1)
            rows_kv[t, hk * d:] = blk[:, 1, t % 16, :].reshape(-1)
        want = oracle_lib.attend(q_rot[s, :hq * d], oracle_lib.bf16_bits(rows_kv), hq, hk, d)
        close_bf16(to_f32(out)[s:s + 1], want[None, :], ulps=3.0, floor=0.25)


def _slots(rows, vocab):
    words = (vocab + 31) // 32
    stride = ((4 * (16 + words + (words & 1)) + 8 + 255) // 256) * 256
    return words, stride


@pytest.mark.parametrize("vocab,group,temperature,top_k", [(3072, 0, 0.9, 50), (2048, 3, 0.9, 50), (2048, 1, 0.0, 50),
                                                            (3072, 0, 1.0, 0), (1000, 2, 0.7, 5)])
def test_sampler_picks_the_oracle_token(ops, oracle_lib, vocab, group, temperature, top_k):
    rows = 48
    rng = np.random.default_rng(vocab + group)
    logits = rand_bf16((rows, vocab), 17, 2.0)
    words, stride = _slots(rows, vocab)
    state = np.zeros((rows + 3, stride // 4), dtype=np.uint32)
    lines = rng.permutation(rows + 3)[:rows].astype(np.int32)
    penalize = group == 0
    for s in range(rows):
        for t in rng.integers(0, min(vocab, 2048), 30):
            state[lines[s], 16 + t // 32] |= np.uint32(1 << (t % 32))
    frames = rng.integers(0, 5, rows).astype(np.int32)
    uniforms = rng.random((rows, 16)).astype(np.float32)
    force = np.full((rows, 16), -1, dtype=np.int32)
    force[5, group] = 77
    lo, hi, exempt, min_frames = (vocab - 1024, vocab, vocab - 900, 2) if penalize else (0, 0, -1, 0)
    d_state = torch.tensor(state.view(np.int32), device="cuda")
    d_codes = torch.full((rows, 16), -9, dtype=torch.int32, device="cuda")
    dev = lambda a: torch.tensor(a, device="cuda")
    torch.cuda.synchronize()
    ops.sample(logits, temperature, top_k, 1.0, 1.05, lo, hi, exempt, min_frames, dev(frames), dev(uniforms), dev(force),
               d_state, dev(lines), stride, int(penalize), 0, d_codes, group)
    ops.sync()
    got_codes = d_codes.cpu().numpy()
    got_state = d_state.cpu().numpy().view(np.uint32)
    lg = to_f32(logits)
    mismatches = 0
    for s in range(rows):
        last = state[lines[s], :16].view(np.int32).copy()
        seen = state[lines[s], 16:16 + words].copy()
        tok = oracle_lib.sample(lg[s], temperature, top_k, 1.0, 1.05, lo, hi, exempt, min_frames, int(frames[s]),
                                float(uniforms[s, group]), int(force[s, group]), last, seen, penalize, group)
        if tok != got_codes[s, group]:
            mismatches += 1  # only a uniform landing within rounding of a CDF step may differ (__expf vs expf)
            continue
        assert got_state[lines[s], group] == tok
        assert np.array_equal(got_state[lines[s], 16:16 + words], seen)
    assert mismatches <= 1, mismatches
    assert got_codes[5, group] == 77


def test_sampler_philox_and_top_p(ops, oracle_lib):
    rows, vocab, group = 32, 2048, 4
    logits = rand_bf16((rows, vocab), 18, 2.5)
    words, stride = _slots(rows, vocab)
    state = np.zeros((rows, stride // 4), dtype=np.uint32)
    seeds = np.arange(rows, dtype=np.uint64) * np.uint64(0x9E3779B97F4A7C15) + np.uint64(11)
    state.view(np.uint8).reshape(rows, stride)[:, 4 * (16 + words):4 * (16 + words) + 8] = \
        seeds.view(np.uint8).reshape(rows, 8)
    frames = np.arange(rows, dtype=np.int32)
    d_state = torch.tensor(state.view(np.int32), device="cuda")
    d_codes = torch.zeros((rows, 16), dtype=torch.int32, device="cuda")
    dev = lambda a: torch.tensor(a, device="cuda")
    lines = np.arange(rows, dtype=np.int32)
    force = np.full((rows, 16), -1, dtype=np.int32)
    torch.cuda.synchronize()
    ops.sample(logits, 0.9, 50, 0.8, 1.0, 0, 0, -1, 0, dev(frames), dev(np.zeros((rows, 16), np.float32)), dev(force),
               d_state, dev(lines), stride, 0, 1, d_codes, group)
    ops.sync()
    got = d_codes.cpu().numpy()[:, group]
    lg = to_f32(logits)
    mismatches = 0
    for s in range(rows):
        u = oracle_lib.philox_uniform(int(seeds[s]), int(frames[s]), group)
        last, seen = np.zeros(16, np.int32), np.zeros(words, np.uint32)
        tok = oracle_lib.sample(lg[s], 0.9, 50, 0.8, 1.0, 0, 0, -1, 0, int(frames[s]), u, -1, last, seen, False, group)
        mismatches += tok != got[s]
    assert mismatches <= 1, mismatches
