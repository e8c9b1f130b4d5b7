"""The allocation-free split-K product (pamk_matmul_static_scratch) against the ordinary entry
point (pamk_matmul with a caller-allocated workspace), through the C ABI.

Some callers of this library cannot allocate device memory: code inside a stream capture or a
real-time loop, a host that hands a plugin fixed buffers and no allocator, a process whose device
memory belongs to another pool.  For them the split-K partial sums live in a fixed array inside
the library.  Both entry points run the same kernels in the same order, so the results must be
identical bit for bit — also on a second call with other shapes, which reuses the array while it
still holds the first call's partial sums.

This file is collected last on purpose: if it fails, a run that stops at the first failure has
already run every other test.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(lib, A, B, split, offset=1.0):
    from pam_b200 import _lib
    dev = A.device
    M, K = A.shape
    N = B.shape[1]
    stream = torch.cuda.current_stream(dev).cuda_stream
    strides = (0, A.stride(0), A.stride(1), 0, B.stride(0), B.stride(1))
    ref = torch.empty(M, N, device=dev)
    ws = torch.empty(lib.pamk_matmul_workspace_bytes(1, M, N, split), dtype=torch.uint8, device=dev)
    _lib.check(lib.pamk_matmul(0, A.data_ptr(), B.data_ptr(), ref.data_ptr(), 1, M, N, K, *strides, offset, split,
                               ws.data_ptr(), ws.numel(), stream), "pamk_matmul")
    out = torch.full((M, N), float("nan"), device=dev)
    _lib.check(lib.pamk_matmul_static_scratch(A.data_ptr(), B.data_ptr(), out.data_ptr(), 1, M, N, K, *strides,
                                              offset, split, stream), "pamk_matmul_static_scratch")
    torch.cuda.synchronize(dev)
    return out, ref


def test_static_scratch_matches_workspace_entry_point_twice():
    from pam_b200 import _lib
    lib = _lib.lib()
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(2026)
    assert lib.pamk_matmul_static_scratch_bytes() == 32 << 20

    # first call: a weight-gradient shape (small output, long K), 24 ranges, transposed A
    X, G = torch.randn(12608, 192, generator=g).to(dev), torch.randn(12608, 576, generator=g).to(dev)
    out1, ref1 = _both(lib, X.T, G, 24)
    assert torch.equal(out1.view(torch.int32), ref1.view(torch.int32))

    # second call straight after, other shape / split / offset, operands with zeros and huge values:
    # the array still holds the first call's partial sums and none of them may leak through
    A = torch.randn(100, 1000, generator=g)
    B = torch.randn(1000, 70, generator=g)
    A[::7, ::5] = 0.0
    B[3, :] = 1e30
    A, B = A.to(dev), B.to(dev)
    out2, ref2 = _both(lib, A, B, 5, offset=1.0552)
    same = (out2.view(torch.int32) == ref2.view(torch.int32)) | (out2.isnan() & ref2.isnan())
    assert bool(same.all())
    assert bool(ref2.isfinite().any())

    # the first problem again gives the first answer again
    out3, _ = _both(lib, X.T, G, 24)
    assert torch.equal(out3.view(torch.int32), ref1.view(torch.int32))


def test_static_scratch_refuses_what_does_not_fit():
    from pam_b200 import _lib
    lib = _lib.lib()
    dev = torch.device("cuda", 0)
    x = torch.ones(16, device=dev)
    s = torch.cuda.current_stream(dev).cuda_stream
    limit = lib.pamk_matmul_static_scratch_bytes() // 4
    # 4 x 2048 x 2048 partial sums are twice the array: refused before anything is launched
    assert 4 * 2048 * 2048 > limit
    assert lib.pamk_matmul_static_scratch(x.data_ptr(), x.data_ptr(), x.data_ptr(), 1, 2048, 2048, 64,
                                          0, 64, 1, 0, 2048, 1, 1.0, 4, s) == -2
    assert lib.pamk_matmul_static_scratch(x.data_ptr(), x.data_ptr(), x.data_ptr(), 1, 4, 4, 4,
                                          0, 4, 1, 0, 4, 1, 1.0, 0, s) == -1          # split_k must be >= 1
    torch.cuda.synchronize(dev)
