"""`omni_op_gemm_noalloc`: the split-K tensor-core GEMM whose scratch is a fixed array inside the library, for
callers that cannot allocate device memory (a process whose KV pool already owns all free HBM, or an engine thread
in mid-tick where a cudaMalloc would stall every other stream). Its output must equal the allocating entry point's
bit for bit, on two calls in a row (the second call finds the first call's partials and counters in the shared
array). Collected last so that a run stopping at the first failure has already run every other test."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def rand_bf16(shape, seed, scale=1.0):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


def test_noalloc_gemm_equals_the_allocating_entry_point(built_lib):
    from pega_omni_b200.ops import Ops, OpsError, gemm_noalloc
    ops = Ops(0)
    for call, (rows, n, k, splits) in enumerate([(64, 2048, 2048, 8), (48, 1024, 6144, 4)]):
        w, x = rand_bf16((n, k), 40 + call, 0.05), rand_bf16((rows, k), 50 + call)
        want = torch.zeros((rows, n), dtype=torch.bfloat16, device="cuda")
        got = torch.full((rows, n), 3.0, dtype=torch.bfloat16, device="cuda")
        torch.cuda.synchronize()
        ops.gemm(w, x, want, path=2, splits=splits)
        ops.sync()
        before = torch.cuda.memory_allocated()
        gemm_noalloc(w, x, got, splits=splits)
        assert torch.cuda.memory_allocated() == before
        assert torch.equal(got, want), f"call {call}: {(got.float() - want.float()).abs().max().item()}"
        assert np.isfinite(got.float().cpu().numpy()).all() and got.float().abs().max().item() > 0
    # beyond the built-in scratch: refused with the sizes in the message, nothing launched
    rows, n, k = 256, 8192, 1024
    w, x = rand_bf16((n, k), 60, 0.05), rand_bf16((rows, k), 61)
    y = torch.zeros((rows, n), dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    with pytest.raises(OpsError) as e:
        gemm_noalloc(w, x, y, splits=8)
    assert "status -5" in str(e.value) and "limit" in str(e.value)
    assert not y.any()
    ops.close()
