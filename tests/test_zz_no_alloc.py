"""dcg_colsum_noalloc: the column sum (bias gradient) for callers that cannot allocate.

Who needs it: code that is handed operand pointers and nothing else - a runtime handler with the
reference's void(rt::Node*) shape, a process whose device-memory budget was fixed at start-up, a
loop that must not enter the driver's allocator - cannot provide the scratch the two-stage column
sum wants and cannot cudaMalloc it.  This entry point keeps its scratch in a 256 KiB array that is
part of the library image, allocates nothing, and refuses shapes that do not fit.

The test calls it through the C ABI, twice in a row on different shapes (the calls share the one
scratch array, which keeps the previous call's contents), and expects exactly what dcg_colsum
produces with caller-provided scratch: both run the same kernels in the same order.

This file sorts last on purpose, so that a run stopping at the first failure has already been
through every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _stream():
    return torch.cuda.current_stream().cuda_stream


def test_no_alloc_colsum_matches_colsum(pkg, dev):
    L = pkg.lib
    g = torch.Generator().manual_seed(11)
    assert L.dcg_colsum_noalloc_max_bytes() == 256 << 10
    # conv bias gradients of the DCGAN layers (batch 64), a dense bias gradient, an odd shape
    for rows, cols in ((64 * 32 * 32, 64), (64 * 4 * 4, 512), (64, 8192), (1001, 7)):
        a = (torch.rand((rows, cols), generator=g) * 2 - 1).to(dev)
        want = pkg.functional.colsum(a)                      # caller-provided scratch
        torch.cuda.synchronize()
        got = torch.full((cols,), float("nan"), device=dev)
        mem_before = torch.cuda.memory_allocated(dev)
        for _ in range(2):                                   # two calls in a row on the shared scratch
            pkg._lib.check(L.dcg_colsum_noalloc(a.data_ptr(), got.data_ptr(), rows, cols, _stream()))
        torch.cuda.synchronize()
        assert torch.equal(got, want), (rows, cols)
        assert torch.cuda.memory_allocated(dev) == mem_before
        ref = a.double().sum(0)
        assert (got.double() - ref).abs().max().item() <= 1e-5 * rows ** 0.5 + 1e-5 * ref.abs().max().item()


def test_no_alloc_colsum_interleaved_shapes_and_limit(pkg, dev):
    L = pkg.lib
    g = torch.Generator().manual_seed(12)
    a1 = (torch.rand((4096, 128), generator=g)).to(dev)
    a2 = (torch.rand((300, 36), generator=g)).to(dev)
    o1, o2 = torch.empty(128, device=dev), torch.empty(36, device=dev)
    # back to back on one stream: the second call reuses scratch the first one has finished with
    pkg._lib.check(L.dcg_colsum_noalloc(a1.data_ptr(), o1.data_ptr(), 4096, 128, _stream()))
    pkg._lib.check(L.dcg_colsum_noalloc(a2.data_ptr(), o2.data_ptr(), 300, 36, _stream()))
    pkg._lib.check(L.dcg_colsum_noalloc(a1.data_ptr(), o1.data_ptr(), 4096, 128, _stream()))
    torch.cuda.synchronize()
    assert torch.equal(o1, pkg.functional.colsum(a1)) and torch.equal(o2, pkg.functional.colsum(a2))
    # a shape whose partial sums exceed the built-in scratch is refused, nothing is launched
    rows, cols = 4096, 1 << 16
    assert L.dcg_colsum_workspace_bytes(rows, cols) > L.dcg_colsum_noalloc_max_bytes()
    before = pkg.launches_total()
    status = L.dcg_colsum_noalloc(a1.data_ptr(), o1.data_ptr(), rows, cols, _stream())
    assert status == pkg._lib.ERR_WORKSPACE
    assert b"built-in" in L.dcg_last_error()
    assert pkg.launches_total() == before
    assert L.dcg_colsum_noalloc(None, None, 4, 4, _stream()) == pkg._lib.ERR_INVALID
