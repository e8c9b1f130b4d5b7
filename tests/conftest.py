import pathlib
import sys

import numpy as np
import pytest
import torch

ROOT = pathlib.Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    """Fixtures generated from the reference by tests/golden/make_golden.py."""
    data = np.load(ROOT / "tests" / "golden" / "pam_golden.npz")
    return {k: torch.from_numpy(data[k]) for k in data.files}


@pytest.fixture(scope="session")
def oracle():
    from oracle import build, pam_oracle
    build.build_oracle()
    return pam_oracle


def bits_equal(x, y):
    """Elementwise fp32 bit equality; any NaN matches any NaN (payloads are not part of parity)."""
    x = torch.as_tensor(x, dtype=torch.float32).cpu()
    y = torch.as_tensor(y, dtype=torch.float32).cpu()
    assert x.shape == y.shape, (x.shape, y.shape)
    return (x.contiguous().view(torch.int32) == y.contiguous().view(torch.int32)) | (x.isnan() & y.isnan())


def assert_bits_equal(x, y, what=""):
    ok = bits_equal(x, y)
    if not bool(ok.all()):
        bad = (~ok).nonzero()
        first = tuple(bad[0].tolist())
        x = torch.as_tensor(x).cpu()
        y = torch.as_tensor(y).cpu()
        raise AssertionError(f"{what}: {bad.shape[0]} of {ok.numel()} elements differ; first at {first}: "
                             f"{x[first].item()!r} vs {y[first].item()!r}")


def assert_close_nan(x, y, rtol, atol, what=""):
    """allclose on the finite lanes; NaN lanes and infinities must coincide."""
    x = torch.as_tensor(x, dtype=torch.float32).cpu()
    y = torch.as_tensor(y, dtype=torch.float32).cpu()
    assert x.shape == y.shape, (what, x.shape, y.shape)
    assert bool((x.isnan() == y.isnan()).all()), f"{what}: NaN lanes differ"
    fin = ~(x.isnan())
    xf, yf = x[fin], y[fin]
    ok = torch.isclose(xf, yf, rtol=rtol, atol=atol)
    if not bool(ok.all()):
        err = (xf - yf).abs()
        i = int(torch.where(ok, torch.zeros_like(err), err).argmax())
        raise AssertionError(f"{what}: {(~ok).sum().item()} of {ok.numel()} lanes off; worst {xf[i].item()!r} vs {yf[i].item()!r}")
