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
    side = torch.cuda.Stream()
    # (rows, N, K, splits, epilogue, stream): the plain product twice in a row, then a bias epilogue on a stream of the
    # caller's with 300 rows (two row tiles through the shared scratch)
    cases = [(64, 2048, 2048, 8, 0, None), (48, 1024, 6144, 4, 0, None), (300, 1024, 2048, 4, 1, side)]
    for call, (rows, n, k, splits, epilogue, stream) in enumerate(cases):
        w, x = rand_bf16((n, k), 40 + call, 0.05), rand_bf16((rows, k), 50 + call)
        bias = rand_bf16((n,), 70 + call) if epilogue else None
        want = torch.zeros((rows, n), dtype=torch.bfloat16, device="cuda")
        got = torch.full((rows, n), 3.0, dtype=torch.bfloat16, device="cuda")
        torch.cuda.synchronize()
        ops.gemm(w, x, want, path=2, splits=splits, bias=bias, epilogue=epilogue)
        ops.sync()
        if call == 0:  # module load and the entry point's first-call set-up happen here, outside the memory check
            gemm_noalloc(w, x, got, splits=splits, bias=bias, epilogue=epilogue)
            got.fill_(3.0)
            torch.cuda.synchronize()
        # the driver's own count of free device memory: a cudaMalloc anywhere in the library would show here
        # (torch's allocator counters only see torch's allocations)
        free_before, _ = torch.cuda.mem_get_info()
        gemm_noalloc(w, x, got, splits=splits, bias=bias, epilogue=epilogue, stream=stream.cuda_stream if stream else None)
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after == free_before, (free_before, free_after)
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
