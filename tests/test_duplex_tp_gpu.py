"""The tensor-parallel pair of the duplex path on two GPUs: one process per rank, each with half of Helium's heads and
MLP channels, partial rows exchanged over peer memory inside the add + norm kernel. Both ranks must agree bit for bit,
and agree with the whole model on one GPU up to the extra bf16 rounding of the two partial sums. Needs two GPUs; on a
single-GPU box it is skipped."""
import multiprocessing as mp

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

PRESET, SESSIONS, TICKS = "duplex-mid", 12, 5


def _script(c, rng_seed=5):
    """The prompts and forced steps every run plays (seeded, so every process builds the same ones)."""
    from tests.test_duplex_gpu import forced_step, make_prompt
    rng = np.random.default_rng(rng_seed)
    lens = [int(rng.integers(3, 14)) for _ in range(SESSIONS)]
    prompts = [make_prompt(c, rng, n, voice_rows=4 if i % 2 == 0 else 0) for i, n in enumerate(lens)]
    steps = [[forced_step(c, rng, seed=t * 100 + i) for i in range(SESSIONS)] for t in range(TICKS)]
    return prompts, steps


def _play(m, c):
    prompts, steps = _script(c)
    sessions = [m.open() for _ in prompts]
    m.start(list(zip(sessions, prompts)))
    emitted, text, audio = [], [], []
    for t in range(TICKS):
        out = m.tick(list(zip(sessions, steps[t])))
        emitted.append(np.array(out.emitted))
        text.append(np.stack([m.text_logits(i) for i in range(SESSIONS)]))
        audio.append(np.stack([m.audio_logits(i) for i in range(SESSIONS)]))
    return np.stack(emitted), np.stack(text), np.stack(audio)


def _rank(rank, to_peer, from_peer, results, use_graphs):
    import torch
    torch.cuda.set_device(rank)
    from pega_omni_b200.duplex import PRESETS, Model, random_checkpoint
    c = PRESETS[PRESET]
    ck = random_checkpoint(c, seed=1, voice_rows=4, head_std=0.15)
    m = Model.load(rank, ck, c, max_sessions=16, max_prefill=256, use_graphs=use_graphs, tp_rank=rank, tp_size=2)
    to_peer.put(m.tp_export())
    m.tp_connect(from_peer.get(timeout=300))
    if use_graphs:
        m.warmup()
    out = _play(m, c)
    results.put((rank,) + out)
    to_peer.put("done")  # neither rank unmaps its exchange region while the other may still read it
    assert from_peer.get(timeout=300) == "done"
    m.close()


def _rows(shape, seed, scale=1.0):
    import torch
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


def test_exchange_kernel_sums_both_ranks_rows_then_adds_and_norms(built_lib):
    """One GPU standing in for a rank whose peer has already raised its flag: y = bf16(mine + peer), x = bf16(x + y),
    out = x * (alpha * rsqrt(eps + mean x^2)); twice in a row, so the second launch runs on the counter the first left."""
    import torch
    from pega_omni_b200.ops import Ops
    ops = Ops(0)
    rows, dim, eps = 37, 1024, 1e-5
    words = torch.zeros(64, dtype=torch.int32, device="cuda")
    words[0] = 2  # the peer is two exchanges ahead at most: both launches find their number reached
    alpha = _rows((dim,), 3, 0.2) + 1
    for call in range(2):
        mine, peer, x = _rows((rows, dim), 10 + call), _rows((rows, dim), 20 + call), _rows((rows, dim), 30 + call)
        out = torch.zeros((rows, dim), dtype=torch.bfloat16, device="cuda")
        y = (mine.float() + peer.float()).to(torch.bfloat16)
        want_x = (x.float() + y.float()).to(torch.bfloat16)
        v = want_x.float()
        want = (v * (alpha.float() * torch.rsqrt(eps + (v * v).mean(dim=1, keepdim=True)))).to(torch.bfloat16)
        torch.cuda.synchronize()
        ops.lm_tp_add_norm(mine, peer, x, alpha, out, eps, words)
        ops.sync()
        assert torch.equal(x, want_x)
        step = torch.exp2(torch.floor(torch.log2(want.float().abs().clamp_min(2.0 ** -6))) - 7)
        assert ((out.float() - want.float()).abs() <= step).all()  # the row's mean is summed in another order
        w = words.cpu().numpy()
        assert w[32] == call + 1 and w[16] == call + 1 and w[48] == 0
    ops.close()


def test_a_flag_that_nothing_raises_runs_the_wait_out(built_lib):
    """The peer never arrives: after the bounded wait the kernel sets the device error word, takes the peer's rows as
    zero and finishes; the host reads status OMNI_ERR_DEVICE, and the context stays usable."""
    import time
    import torch
    from pega_omni_b200.ops import Ops, OpsError
    ops = Ops(0)
    rows, dim, eps = 5, 512, 1e-5
    words = torch.zeros(64, dtype=torch.int32, device="cuda")
    mine, peer, x = _rows((rows, dim), 1), _rows((rows, dim), 2), _rows((rows, dim), 3)
    x0 = x.clone()
    alpha = torch.ones(dim, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros((rows, dim), dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    t0 = time.monotonic()
    ops.lm_tp_add_norm(mine, peer, x, alpha, out, eps, words)
    with pytest.raises(OpsError) as e:
        ops.sync()
    assert "status -3" in str(e.value)
    assert 1.0 < time.monotonic() - t0 < 10.0
    assert torch.equal(x, (x0.float() + mine.float()).to(torch.bfloat16))  # the peer counted as zero
    # the error word was read and cleared: the next launch, with the flag raised, runs normally
    words.zero_()
    words[0] = 1
    ops.lm_tp_add_norm(mine, peer, x, alpha, out, eps, words)
    ops.sync()
    ops.close()


@pytest.mark.parametrize("use_graphs", [False, True])
def test_pair_agrees_with_itself_and_with_one_gpu(built_lib, use_graphs):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from pega_omni_b200.duplex import PRESETS, Model, random_checkpoint
    c = PRESETS[PRESET]
    ck = random_checkpoint(c, seed=1, voice_rows=4, head_std=0.15)
    whole = Model.load(0, ck, c, max_sessions=16, max_prefill=256, use_graphs=use_graphs)
    want = _play(whole, c)
    whole.close()
    ctx = mp.get_context("spawn")
    a_to_b, b_to_a, results = ctx.Queue(), ctx.Queue(), ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(0, a_to_b, b_to_a, results, use_graphs)),
             ctx.Process(target=_rank, args=(1, b_to_a, a_to_b, results, use_graphs))]
    for p in procs:
        p.start()
    got = {}
    for _ in procs:
        r = results.get(timeout=600)
        got[r[0]] = r[1:]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for a, b in zip(got[0], got[1]):  # the ranks round the same sums: bit-identical logits, the same tokens
        assert np.array_equal(a, b)
    emitted, text, audio = got[0]
    assert np.array_equal(emitted, want[0])
    worst = 0.0
    for g, w in ((text, want[1]), (audio, want[2])):
        step = np.exp2(np.floor(np.log2(np.maximum(np.abs(w), 2.0))) - 7)
        worst = max(worst, float((np.abs(g - w) / step).max()))
        num = (g.astype(np.float64) * w).sum(axis=-1)
        den = np.linalg.norm(g.astype(np.float64), axis=-1) * np.linalg.norm(w.astype(np.float64), axis=-1) + 1e-30
        assert (num / den).min() >= 0.9995
    # each rank's partial rows are rounded to bf16 before they are summed: one rounding more per projection than the
    # whole model's, through three layers
    assert worst <= 3.0, worst
