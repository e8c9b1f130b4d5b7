"""Host-side multi-process logic on CPU (gloo, world size 2): row sharding with no collective and
the data-parallel gradient sum followed by the PAM Adam step.  The PAM arithmetic runs through the
oracle-backed fake library (tests/cpu_backend.py), so no GPU is involved."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    import sys
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from _pytest.monkeypatch import MonkeyPatch
        import cpu_backend
        mpatch = MonkeyPatch()
        cpu_backend.install(mpatch)
        import pam_b200 as pam
        from pam_b200 import optim, parallel

        g = torch.Generator().manual_seed(3)
        X, G = torch.randn(37, 24, generator=g), torch.randn(37, 10, generator=g)
        W0 = torch.randn(10, 24, generator=g) * 0.1

        # (1) row-sharded product: each rank computes its rows, nothing is exchanged
        lo, hi = parallel.shard_rows(37, rank, world)
        Y_rows = pam.linear(X[lo:hi], W0)

        # (2) data-parallel step: local gradients, one all-reduce, PAM Adam
        lin = pam.Linear(24, 10, approx_bwd=True)
        ln = pam.LayerNorm(10, approx_bwd=True)
        with torch.no_grad():
            lin.weight.copy_(W0)
            lin.bias.zero_()
        params = list(lin.parameters()) + list(ln.parameters())
        opt = optim.Adam(params, lr=1e-2, betas=(0.9, 0.98), weight_decay=1e-4, opt_functional_cfg="pam")
        out = ln(lin(X[lo:hi]))
        out.backward(G[lo:hi])
        local_w_grad = lin.weight.grad.clone()
        parallel.all_reduce_gradients(params)
        reduced_w_grad = lin.weight.grad.clone()
        # the same sum, started bucket by bucket from gradient hooks during the backward pass
        for prm in params:
            prm.grad = None
        buckets = parallel.GradientBuckets(params, bucket_bytes=256)      # tiny buckets: several per step
        ln(lin(X[lo:hi])).backward(G[lo:hi])
        buckets.finish()
        bucketed_w_grad = lin.weight.grad.clone()
        ln(lin(X[lo:hi])).backward(G[lo:hi])                              # a second step re-arms the buckets
        buckets.finish()
        buckets.remove()
        second_w_grad = lin.weight.grad.clone()
        lin.weight.grad = reduced_w_grad.clone()
        opt.step()
        slowest = parallel.max_over_ranks(1.0 + rank, torch.device("cpu"))
        torch.save({"rows": (lo, hi), "Y": Y_rows.detach(), "local": local_w_grad, "reduced": reduced_w_grad,
                    "bucketed": bucketed_w_grad, "second": second_w_grad,
                    "weight": lin.weight.detach().clone(), "gamma": ln.weight.detach().clone(), "slowest": slowest},
                   os.path.join(out_dir, f"rank{rank}.pt"))
        mpatch.undo()
    finally:
        dist.destroy_process_group()


def test_row_sharding_and_gradient_all_reduce(tmp_path, oracle, monkeypatch):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    r = [torch.load(tmp_path / f"rank{k}.pt") for k in range(world)]

    import cpu_backend
    cpu_backend.install(monkeypatch)
    import pam_b200 as pam
    g = torch.Generator().manual_seed(3)
    X, G = torch.randn(37, 24, generator=g), torch.randn(37, 10, generator=g)
    W0 = torch.randn(10, 24, generator=g) * 0.1

    # shards tile the row range and reproduce the unsharded product bit for bit
    assert r[0]["rows"] == (0, 19) and r[1]["rows"] == (19, 37)
    full = pam.linear(X, W0)
    assert torch.equal(torch.cat([r[0]["Y"], r[1]["Y"]]), full)

    # the all-reduce is the sum of the two local gradients, identical on both ranks
    assert torch.equal(r[0]["reduced"], r[1]["reduced"])
    assert torch.equal(r[0]["reduced"], r[0]["local"] + r[1]["local"])
    # the overlapped, bucketed reduction gives the same sums; a second backward accumulates onto them
    assert torch.equal(r[0]["bucketed"], r[0]["reduced"]) and torch.equal(r[1]["bucketed"], r[0]["reduced"])
    assert torch.equal(r[0]["second"], r[1]["second"])
    # after the optimizer step the replicas hold the same parameters
    assert torch.equal(r[0]["weight"], r[1]["weight"]) and torch.equal(r[0]["gamma"], r[1]["gamma"])
    assert not torch.equal(r[0]["weight"], W0)
    assert r[0]["slowest"] == r[1]["slowest"] == 2.0


def test_shard_rows_edges():
    from pam_b200.parallel import shard_rows
    assert [shard_rows(10, k, 4) for k in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert [shard_rows(2, k, 4) for k in range(4)] == [(0, 1), (1, 2), (2, 2), (2, 2)]
    assert shard_rows(0, 0, 1) == (0, 0)
    with pytest.raises(ValueError):
        shard_rows(5, 2, 2)


def test_gradient_buckets_default_size_overlaps_small_models():
    """The default bucket size is 25 MB or an eighth of all gradients, whichever is less: a model whose
    gradients would fit one 25 MB bucket still gets about eight reductions to overlap with its backward
    pass (no process group is needed to look at the grouping)."""
    import torch
    from pam_b200 import parallel
    small = [torch.nn.Parameter(torch.zeros(250_000)) for _ in range(23)]           # 23 MB of gradients
    buckets = parallel.GradientBuckets(small)
    assert 7 <= len(buckets.buckets) <= 12
    assert sum(len(b) for b in buckets.buckets) == len(small)
    large = [torch.nn.Parameter(torch.zeros(4_000_000)) for _ in range(40)]         # 640 MB: 25 MB buckets
    assert len(parallel.GradientBuckets(large).buckets) >= 20
    assert len(parallel.GradientBuckets(small, bucket_bytes=25 << 20).buckets) == 1
