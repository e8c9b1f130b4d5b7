"""`pamk_matmul_strided` through the C ABI against `pamk_matmul` on contiguous copies.

Same products, same order of summation and the same split-K ranges, so the results must be equal bit for
bit; the output lands in a padded, strided buffer whose other elements (canaries) must stay untouched.
"""
import pytest
import torch

from conftest import assert_bits_equal

pytestmark = pytest.mark.gpu


def _strided(shape, strides_order, pad, gen, dev):
    """A tensor of `shape` whose memory order is `strides_order` (outermost first) with `pad` unused
    elements after every innermost run."""
    sizes = [shape[d] for d in strides_order]
    sizes[-1] += pad
    base = torch.randn(*sizes, generator=gen).to(dev)
    view = base[..., :shape[strides_order[-1]]]
    inverse = [strides_order.index(d) for d in range(len(shape))]
    return view.permute(*inverse)


@pytest.mark.parametrize("outer,inner,M,N,K", [(3, 2, 70, 33, 40), (1, 1, 64, 64, 64), (2, 5, 9, 200, 77), (4, 3, 197, 64, 197), (1, 7, 130, 5, 1000)])
@pytest.mark.parametrize("a_order,b_order", [((0, 2, 1, 3), (0, 2, 1, 3)), ((1, 0, 3, 2), (0, 1, 2, 3)), ((0, 1, 2, 3), (2, 0, 1, 3)), ((0, 1, 3, 2), (1, 0, 3, 2))])
@pytest.mark.parametrize("split,scale", [(1, None), (3, None), (1, 0.125), (2, 0.37)])
def test_strided_product_equals_the_plain_product_on_copies(outer, inner, M, N, K, a_order, b_order, split, scale):
    import pam_b200 as pam
    from pam_b200 import _lib, cuda_bindings
    dev = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(outer * 100 + inner * 10 + M + split)
    # A[o, i, m, k] and B[o, i, k, n] as views whose matrix part has one unit stride
    if a_order[-1] not in (2, 3) or b_order[-1] not in (2, 3):
        pytest.skip("the matrix part needs a unit stride")
    A = _strided((outer, inner, M, K), list(a_order), 3, gen, dev)
    B = _strided((outer, inner, K, N), list(b_order), 5, gen, dev)
    assert 1 in A.stride()[2:] and 1 in B.stride()[2:]
    # output [o, m, i, n] in memory (token-major, like an attention context) with 4 unused columns per row
    Cbuf = torch.full((outer, M, inner, N + 4), 777.0, device=dev)
    handle = _lib.lib()
    ws_bytes = handle.pamk_matmul_workspace_bytes(outer * inner, M, N, split)
    ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=dev)
    sc = Cbuf.stride()
    with _lib.device_guard(dev):
        rc = handle.pamk_matmul_strided(A.data_ptr(), B.data_ptr(), Cbuf.data_ptr(), outer, inner, M, N, K,
                                        A.stride(0), A.stride(1), A.stride(2), A.stride(3),
                                        B.stride(0), B.stride(1), B.stride(2), B.stride(3),
                                        sc[0], sc[2], sc[1], 1.0, int(scale is not None), float(scale or 0.0),
                                        split, ws.data_ptr() if ws_bytes else None, ws_bytes, _lib.stream_ptr(dev))
    _lib.check(rc, "pamk_matmul_strided")
    want = cuda_bindings._matmul(_lib.MUL_PAM, A.reshape(outer * inner, M, K).contiguous(),
                                 B.reshape(outer * inner, K, N).contiguous(), 1.0, 3, split_k=split)
    if scale is not None:
        want = pam.mul(want, scale)
    got = Cbuf[..., :N].permute(0, 2, 1, 3).reshape(outer * inner, M, N)
    assert_bits_equal(got, want, "strided product")
    assert bool((Cbuf[..., N:] == 777.0).all()), "columns beyond N were written"


def test_strided_product_rejects_bad_arguments():
    from pam_b200 import _lib
    dev = torch.device("cuda", 0)
    handle = _lib.lib()
    a = torch.randn(2, 3, 4, 64, device=dev)
    b = torch.randn(2, 3, 64, 6, device=dev)
    c = torch.empty(2, 3, 4, 6, device=dev)
    def call(**over):
        args = dict(outer=2, inner=3, M=4, N=6, K=64, sa=a.stride(), sb=b.stride(), sc=(c.stride(0), c.stride(1), c.stride(2)), split=1)
        args.update(over)
        with _lib.device_guard(dev):
            return handle.pamk_matmul_strided(a.data_ptr(), b.data_ptr(), c.data_ptr(), args["outer"], args["inner"],
                                              args["M"], args["N"], args["K"], *args["sa"], *args["sb"], *args["sc"],
                                              1.0, 0, 0.0, args["split"], None, 0, _lib.stream_ptr(dev))
    assert call() == 0
    assert call(outer=-1) == -1
    assert call(sc=(c.stride(0), c.stride(1), 5)) == -1          # rows of the output would overlap
    assert call(sa=(768, 256, 2, 3)) == -3                        # no unit stride in the matrix part
    assert call(split=2) == -4                               # an explicit split needs its scratch
    assert call(outer=0) == 0


def test_nvtx_ranges_do_not_change_results():
    import pam_b200 as pam
    dev = torch.device("cuda", 0)
    a, b = torch.randn(70, 50, device=dev), torch.randn(50, 30, device=dev)
    plain = pam.matmul(a, b)
    pam.set_nvtx(True)
    try:
        traced = pam.matmul(a, b)
        probs = pam.softmax(traced, dim=-1)
    finally:
        pam.set_nvtx(False)
    assert_bits_equal(traced, plain, "matmul under NVTX ranges")
    assert_bits_equal(probs, pam.softmax(plain, dim=-1), "softmax under NVTX ranges")
