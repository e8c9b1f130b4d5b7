"""The CPU-baseline port of the reference's float-log path against values produced by the real
pam/native.py (fixtures), and its distance from the integer arithmetic of the kernels."""
import torch

from conftest import assert_close_nan


def test_port_matches_reference_native(golden):
    from oracle import native_port as N
    a, b = golden["native/a"], golden["native/b"]
    assert torch.equal(N.pam(a, b), golden["native/pam"])
    assert torch.equal(N.pam(a, b, 1.0552), golden["native/pam_off"])
    assert torch.equal(N.pad(a, b), golden["native/pad"])
    A, B, G = golden["native/A"], golden["native/B"], golden["native/G"]
    assert torch.equal(N.matmul(A, B), golden["native/mm/y"])
    assert torch.equal(N.matmul(A, B, row_chunk=3), golden["native/mm/y"])       # chunking changes nothing
    dA, dB = N.matmul_approx_bwd(A, B, G)
    assert_close_nan(dA, golden["native/mm/dA"], 1e-6, 1e-7)
    assert_close_nan(dB, golden["native/mm/dB"], 1e-6, 1e-7)
    y = N.layer_norm(golden["ln/x"].reshape(-1, 48), golden["ln/w"], golden["ln/b"], 1e-5)
    assert_close_nan(y.reshape(7, 3, 48), golden["native/ln/y"], 1e-6, 1e-6)


def test_native_and_integer_semantics_agree_to_allclose(oracle, golden):
    # the reference's own tests compare its two implementations with torch.allclose defaults
    from oracle import native_port as N
    a, b = golden["native/a"], golden["native/b"]
    integer = oracle.kernels().pam_fwd(a, b, 1.0)
    assert torch.allclose(N.pam(a, b), integer)
    assert not torch.equal(N.pam(a, b), integer)     # ... but not bit for bit
