"""The allocation-free entry point of the fused GEMM, called straight through the C ABI.

``swiglu_b200_gemm_fwd_noalloc`` serves callers that may not allocate device memory (a process whose
memory planner already owns the whole device, a loop where cudaMalloc is banned because it
synchronises, a plug-in handed only its tensors): the kernel's status word sits in a small array
inside the library instead of being passed in.  This file is collected last on purpose, so that a
run that stops at the first failure has already executed every other test.

Two calls in a row must each reproduce the output of the ordinary entry point (same kernel, same
operands: the comparison is exact, and also held to the bf16 tolerance of the other GEMM tests
against the fp32 reference), the second call must not be disturbed by what the first left in the
shared array, and the PyTorch allocator must see no allocation during the calls.
"""
import pytest
import torch

from kernel_pocs_b200 import _lib

pytestmark = pytest.mark.gpu
DEVICE = "cuda"


def _operands(m, n, k, seed):
    g = torch.Generator(device=DEVICE).manual_seed(seed)
    x = torch.randn(m, k, generator=g, device=DEVICE).bfloat16()
    wg = (0.05 * torch.randn(n, k, generator=g, device=DEVICE)).bfloat16()
    wu = (0.05 * torch.randn(n, k, generator=g, device=DEVICE)).bfloat16()
    return x, wg, wu


def test_no_alloc_entry_matches_the_regular_entry_twice_in_a_row():
    lib = _lib.lib
    stream = torch.cuda.current_stream().cuda_stream
    status_dev = torch.zeros(1, dtype=torch.int32, device=DEVICE)
    status_host = torch.full((1,), -1, dtype=torch.int32).pin_memory()
    cases = [(300, 272, 200, 0.7, 1.3), (1024, 1408, 512, 1.0, 1.0)]
    prepared = []
    for i, (m, n, k, gm, dm) in enumerate(cases):
        x, wg, wu = _operands(m, n, k, 30 + i)
        want = torch.empty(m, n, dtype=torch.bfloat16, device=DEVICE)
        _lib.check("regular entry", lib.swiglu_b200_gemm_fwd(
            want.data_ptr(), None, None, x.data_ptr(), wg.data_ptr(), wu.data_ptr(), m, n, k, gm, dm,
            status_dev.data_ptr(), 0, stream))
        torch.cuda.synchronize()
        assert int(status_dev.item()) == 0
        got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEVICE)
        prepared.append((x, wg, wu, m, n, k, gm, dm, want, got))

    # every buffer exists now; from here on the allocator must stay untouched
    torch.cuda.synchronize()
    allocs_before = torch.cuda.memory_stats()["allocation.all.allocated"]
    bytes_before = torch.cuda.memory_allocated()
    launches_before = lib.swiglu_b200_gemm_launch_count()
    for x, wg, wu, m, n, k, gm, dm, want, got in prepared:  # two calls in a row, no sync between them
        _lib.check("no-alloc entry", lib.swiglu_b200_gemm_fwd_noalloc(
            got.data_ptr(), x.data_ptr(), wg.data_ptr(), wu.data_ptr(), m, n, k, gm, dm,
            status_host.data_ptr(), 0, stream))
    torch.cuda.synchronize()
    assert lib.swiglu_b200_gemm_launch_count() == launches_before + 2
    assert torch.cuda.memory_stats()["allocation.all.allocated"] == allocs_before
    assert torch.cuda.memory_allocated() == bytes_before
    assert int(status_host.item()) == 0

    for x, wg, wu, m, n, k, gm, dm, want, got in prepared:
        assert torch.equal(got, want)
        ref = torch.nn.functional.silu((x.float() @ wg.float().t()) * gm) * (x.float() @ wu.float().t()) * dm
        tol = 2.0 ** -7 * ref.abs() + 2.0 ** -9 * ref.pow(2).mean().sqrt()
        assert bool(((got.float() - ref).abs() <= tol).all())

    # argument errors are reported like those of the regular entry point, and an empty problem is a no-op
    x, wg, wu, m, n, k, gm, dm, want, got = prepared[0]
    assert lib.swiglu_b200_gemm_fwd_noalloc(got.data_ptr(), x.data_ptr(), wg.data_ptr(), wu.data_ptr(), m, n, 20, gm, dm,
                                            None, 0, stream) == 3
    assert lib.swiglu_b200_gemm_fwd_noalloc(None, x.data_ptr(), wg.data_ptr(), wu.data_ptr(), m, n, k, gm, dm,
                                            None, 0, stream) == 2
    assert lib.swiglu_b200_gemm_fwd_noalloc(got.data_ptr(), x.data_ptr(), wg.data_ptr(), wu.data_ptr(), 0, n, k, gm, dm,
                                            None, 0, stream) == 0
    # with a status word given, an empty problem reports success there (nothing ran, nothing failed)
    status_host.fill_(-1)
    assert lib.swiglu_b200_gemm_fwd_noalloc(got.data_ptr(), x.data_ptr(), wg.data_ptr(), wu.data_ptr(), 0, n, k, gm, dm,
                                            status_host.data_ptr(), 0, stream) == 0
    torch.cuda.synchronize()
    assert int(status_host.item()) == 0
