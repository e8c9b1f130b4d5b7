"""The shipped scalar header, compiled for the host, against the CPU oracle (no GPU needed)."""
import subprocess

import pytest
import torch

from conftest import ROOT, assert_bits_equal


@pytest.fixture(scope="module")
def host_header(oracle, tmp_path_factory):
    out = tmp_path_factory.mktemp("hostscalar") / "libhostscalar.so"
    subprocess.check_call(["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off",
                           "-o", str(out), str(ROOT / "tests" / "host_scalar_shim.cpp")])
    k = oracle.CpuKernels.__new__(oracle.CpuKernels)
    k.kind, k.lib = "host-header", oracle._load(out)
    return k


def _patterns(n, seed):
    g = torch.Generator().manual_seed(seed)
    raw = torch.randint(-2**31, 2**31 - 1, (n,), generator=g, dtype=torch.int64).to(torch.int32).view(torch.float32)
    wide = torch.randn(n, generator=g) * torch.exp2(torch.randint(-70, 70, (n,), generator=g).float())
    # values hugging the flush / pass thresholds and powers of two
    edge = torch.tensor([0x02081CEA, 0x02081CEB, 0x7CF0BDC2, 0x7CF0BDC3, 0x00800000, 0x007FFFFF, 1, 0,
                         0x3F800000, 0x3F7FFFFF, 0x40FFFFFF, 0x41000000, 0x7F7FFFFF, 0x7F800000],
                        dtype=torch.int32).view(torch.float32)
    edge = torch.cat([edge, -edge]).repeat(n // 28 + 1)[:n]
    return raw, wide, edge


@pytest.mark.parametrize("offset", [1.0, 1.0552, 0.97])
def test_binary_ops(oracle, host_header, offset):
    K = oracle.kernels()
    raw, wide, edge = _patterns(400_000, 3)
    dc = torch.randn(raw.numel())
    for a, b in ((raw, raw.flip(0)), (wide, wide.flip(0)), (wide, raw), (edge, wide), (edge, edge.roll(5))):
        assert_bits_equal(host_header.pam_fwd(a, b, offset), K.pam_fwd(a, b, offset), "pam")
        assert_bits_equal(host_header.pad_fwd(a, b, offset), K.pad_fwd(a, b, offset), "pad")
        assert_bits_equal(host_header.pam_bwd(a, b, dc, offset), K.pam_bwd(a, b, dc, offset), "pam_bwd")
        assert_bits_equal(host_header.pad_bwd(a, b, dc, offset), K.pad_bwd(a, b, dc, offset), "pad_bwd")


@pytest.mark.parametrize("base", [2.0, 2.718281828459045, 10.0, 0.5])
def test_exp_log(oracle, host_header, base):
    K = oracle.kernels()
    raw, wide, edge = _patterns(400_000, 4)
    g = torch.Generator().manual_seed(5)
    x = torch.cat([raw, wide, edge, torch.randn(400_000, generator=g) * 60,
                   torch.arange(-200, 200).float(), torch.arange(-200, 200).float() - 2.0 ** -20])
    dy = torch.randn(x.numel(), generator=g) * torch.exp2(torch.randint(-60, 60, (x.numel(),), generator=g).float())
    for off in (1.0, 1.0552):
        assert_bits_equal(host_header.pa_exp_fwd(x, base, off), K.pa_exp_fwd(x, base, off), "exp")
        assert_bits_equal(host_header.pa_exp_bwd(x, dy, base, off), K.pa_exp_bwd(x, dy, base, off), "exp_bwd")
        assert_bits_equal(host_header.pa_log_fwd(x, base, off), K.pa_log_fwd(x, base, off), "log")
        assert_bits_equal(host_header.pa_log_bwd(x, dy, base, off), K.pa_log_bwd(x, dy, base, off), "log_bwd")


def test_exp2_log2_exhaustive_exponents(oracle, host_header):
    # every binade of fp32, both ends and the middle, through exp2(log2(x)) building blocks
    K = oracle.kernels()
    e = torch.arange(0, 255, dtype=torch.int32)
    m = torch.tensor([0, 1, 0x400000, 0x7FFFFF], dtype=torch.int32)
    x = ((e[:, None] << 23) | m[None, :]).reshape(-1).view(torch.float32)
    assert_bits_equal(host_header.pa_log_fwd(x, 2.0, 1.0), K.pa_log_fwd(x, 2.0, 1.0))
    assert_bits_equal(host_header.pa_log_bwd(x, x.flip(0), 2.0, 1.0), K.pa_log_bwd(x, x.flip(0), 2.0, 1.0))
    t = torch.linspace(-160, 135, 50_000)
    assert_bits_equal(host_header.pa_exp_fwd(t, 2.0, 1.0), K.pa_exp_fwd(t, 2.0, 1.0))
    assert_bits_equal(host_header.pa_exp_bwd(t, t.flip(0), 2.0, 1.0), K.pa_exp_bwd(t, t.flip(0), 2.0, 1.0))


def test_shared_divisor_division_is_exact(oracle, host_header):
    """div_by(a, make_divisor(d)) == pad(a, d) bit for bit: for divisors of every magnitude (and the
    special ones) against dividends that hug both thresholds of each divisor from either side."""
    import ctypes
    K = oracle.kernels()
    lib = host_header.lib
    lib.host_div_by.argtypes = [ctypes.c_void_p, ctypes.c_float, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int]
    lib.host_div_by.restype = None
    g = torch.Generator().manual_seed(99)
    raw = torch.randint(-2**31, 2**31 - 1, (20000,), generator=g, dtype=torch.int64).to(torch.int32).view(torch.float32)
    divisors = [0.0, -0.0, float("inf"), float("-inf"), float("nan"), 1.0, -1.0, 1.4e-45, 1e-40, 1.1754944e-38,
                3.4028235e38, 1e37, 9.9e36, 1e-37, 1.0000001e-37, 0.33333334, 3.0, 192.0, 1e-19, 1e19]
    divisors += (torch.randn(60, generator=g) * torch.exp2(torch.randint(-126, 127, (60,), generator=g).float())).tolist()
    steps = torch.arange(-6, 7, dtype=torch.int32)
    for d in divisors:
        dt = torch.tensor(d, dtype=torch.float32)
        for offset in (1.0, 1.0552):
            cands = [raw, torch.tensor([0.0, -0.0, float("inf"), float("-inf"), float("nan")])]
            if bool(dt.isfinite()) and float(dt) != 0.0:
                for bound_bits in (0x02081CEA, 0x7CF0BDC2):
                    centre = (torch.tensor(bound_bits, dtype=torch.int32).view(torch.float32) * dt.abs()).reshape(1)
                    if bool(centre.isfinite()):
                        around = (centre.view(torch.int32) + steps).clamp(0, 0x7F7FFFFF).view(torch.float32)
                        cands += [around, -around]
            a = torch.cat(cands).contiguous()
            got = torch.empty_like(a)
            lib.host_div_by(a.data_ptr(), float(dt), got.data_ptr(), a.numel(), oracle.offset_to_int(offset))
            want = K.pad_fwd(a, dt.expand_as(a).contiguous(), offset)
            assert_bits_equal(got, want, f"divisor {d!r} offset {offset}")
