"""Benchmark of the PAM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (one "step"): the DeiT-tiny PAM linear-layer set — activations X[12608 x 192] (batch 64 x
197 tokens) N(0,1), trunc-normal(0.02) weights, the four GEMMs 192->576, 192->192, 192->768,
768->192 forward and backward with approx_bwd (12 PAM GEMMs, 16.73 G PAM multiply-accumulates),
plus pam_ln (LayerNorm) over the 192-wide rows forward and backward.  Synthetic seeded data.

Prints ONE JSON line: PAM-GEMM MAC/s (GEMM multiply-accumulates of the step / step time, the
LayerNorm included in the time), with the issue-rate roofline of the dominant kernel, the
end-to-end figure with host buffers, clocks sampled during the timed region and the CPU baseline.
With N > 1 (torchrun) every rank runs the same per-GPU workload on its own rows (weak scaling,
no collective on the data path); the time is the max over ranks.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

LAYERS = ((192, 576), (192, 192), (192, 768), (768, 192))
TOKENS = 12608
LN_WIDTH = 192
MACS_PER_STEP = 3 * TOKENS * sum(k * n for k, n in LAYERS)
METRIC = "PAM-GEMM MAC/s (fp32), DeiT-tiny linear-layer set fwd+bwd(approx) + pam_ln"


# mean DRAM traffic of one PAM GEMM launch of the 192->576 layer, from the ncu capture summarised in
# profiles/gemm_pam_tile64_deit_shapes_ncu.md (operands mostly stay in the 126 MB L2)
GEMM_DRAM_BYTES_PER_LAUNCH = (10.2e6 + 36.0e6 + 333.5e6) / 3


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-rows", type=int, default=0, help="rows of X in the CPU sample (0 = auto)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--case", default=None,
                    help="run one kernel in isolation (for profiling) instead of the benchmark: "
                         "gemm | gemm_specials | deit_gemms | deit_gemms_exact | mul | layer_norm_fwd | layer_norm_bwd | "
                         "softmax_fwd | softmax_bwd | adam | column_sum; or a full training step, also under torchrun "
                         "with --gpus N: deit_step | transformer_step")
    ap.add_argument("--size", type=int, default=4096, help="--case size: GEMM edge, or log2 of the element count")
    ap.add_argument("--reps", type=int, default=2)
    ap.add_argument("--exact-bwd", action="store_true",
                    help="training-step cases: exact piecewise-affine gradients (approx_bwd=False) instead of approx_bwd=True")
    return ap.parse_args()


def make_inputs(seed, device=None, pin=False):
    g = torch.Generator().manual_seed(seed)
    data = {"X": [], "W": [], "G": []}
    for k, n in LAYERS:
        data["X"].append(torch.randn(TOKENS, k, generator=g))
        data["W"].append(torch.nn.init.trunc_normal_(torch.empty(n, k), std=0.02, generator=g))
        data["G"].append(torch.randn(TOKENS, n, generator=g))
    data["LNX"] = torch.randn(TOKENS, LN_WIDTH, generator=g)
    data["LNG"] = torch.randn(TOKENS, LN_WIDTH, generator=g)

    def place(t):
        if device is not None:
            return t.to(device)
        return t.pin_memory() if pin else t
    return {k: [place(t) for t in v] if isinstance(v, list) else place(v) for k, v in data.items()}


# ---- clocks ---------------------------------------------------------------------------------------

class ClockSampler:
    """Samples nvidia-smi for one GPU every 20 ms while the device-timed regions run."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.25)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, r[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# ---- our arm ------------------------------------------------------------------------------------------

def run_ours(args):
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    if args.warmup < 3:
        raise SystemExit("timing rules need --warmup >= 3")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    import pam_b200 as pam
    from pam_b200 import _lib
    torch.backends.cuda.matmul.allow_tf32 = False
    lib = _lib.lib()                       # fails loudly if the CUDA library is missing

    d = make_inputs(1234 + rank, device=dev)
    ln = pam.LayerNorm(LN_WIDTH, eps=1e-6, approx_bwd=True).to(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)     # > 126 MB L2

    def step(data, keep=False):
        outs = []
        for X, W, G in zip(data["X"], data["W"], data["G"]):
            X = X.detach().requires_grad_()
            W = W.detach().requires_grad_()
            Y = pam.linear(X, W, approx_bwd=True)
            Y.backward(G)
            if keep:
                outs += [Y.detach(), X.grad, W.grad]
        x = data["LNX"].detach().requires_grad_()
        y = ln(x)
        y.backward(data["LNG"])
        ln.weight.grad = ln.bias.grad = None
        if keep:
            outs += [y.detach(), x.grad]
        return outs

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(args.warmup):
        step(d)
    barrier()

    # ---- value: inputs resident in HBM, per-step CUDA events, L2 flushed between steps ----------
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    launches0 = lib.pamk_launch_count()
    clocks = ClockSampler(local)
    clocks.__enter__()
    barrier()
    for e0, e1 in ev:
        flush.zero_()
        e0.record()
        step(d)
        e1.record()
    barrier()
    launches = lib.pamk_launch_count() - launches0
    total_ms = sum(e0.elapsed_time(e1) for e0, e1 in ev)

    # ---- roofline of the dominant kernel: the 12 GEMM launches alone -------------------------------
    def gemms_only():
        ck = pam.cuda_bindings
        for X, W, G in zip(d["X"], d["W"], d["G"]):
            ck._matmul(0, X, W.T, 1.0, 2)
            ck._matmul(0, G, W, 1.0, 2)
            ck._matmul(0, X.T, G, 1.0, 2)
    for _ in range(3):
        gemms_only()
    torch.cuda.synchronize()
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = max(3, args.steps // 2)
    gemm_ms = 0.0
    for _ in range(reps):
        flush.zero_()
        g0.record()
        gemms_only()
        g1.record()
        torch.cuda.synchronize()
        gemm_ms += g0.elapsed_time(g1)
    gemm_rate = MACS_PER_STEP * reps / (gemm_ms * 1e-3)

    import ctypes
    peak = {}
    scratch = torch.zeros(4, dtype=torch.int32, device=dev)
    for name, variant in (("fadd", 0), ("iadd", 1), ("iadd_fadd", 2), ("imad_fadd", 3), ("mixed_fadd", 4)):
        ms, steps_done = ctypes.c_float(), ctypes.c_double()
        _lib.check(lib.pamk_issue_rate(variant, 8000, 4, scratch.data_ptr(), ctypes.byref(ms), ctypes.byref(steps_done),
                                       torch.cuda.current_stream().cuda_stream), "issue_rate")
        peak[name] = steps_done.value / (ms.value * 1e-3)
    mac_peak = max(peak["iadd_fadd"], peak["imad_fadd"], peak["mixed_fadd"])
    clocks.__exit__(None, None, None)

    # ---- e2e: host buffers in, results out, through the public API ------------------------------------
    # Copies are pipelined against the compute on two extra streams (PCIe is full duplex): inputs
    # upload and results download while other layers compute.
    host = make_inputs(1234 + rank, pin=True)
    h2d = sum(t.numel() * 4 for v in host.values() for t in (v if isinstance(v, list) else [v]))
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    main = torch.cuda.current_stream(dev)
    out_host = {}

    def download(key, tensors):
        ready = torch.cuda.Event()
        ready.record(main)
        s_out.wait_event(ready)
        with torch.cuda.stream(s_out):
            for j, t in enumerate(tensors):
                slot = out_host.get((key, j))
                if slot is None:
                    slot = out_host[(key, j)] = torch.empty(t.shape, dtype=t.dtype).pin_memory()
                slot.copy_(t, non_blocking=True)
                t.record_stream(s_out)

    def e2e_step():
        uploads = []
        with torch.cuda.stream(s_in):
            for i in range(len(LAYERS)):
                trio = [host[k][i].to(dev, non_blocking=True) for k in ("X", "W", "G")]
                ev = torch.cuda.Event()
                ev.record(s_in)
                uploads.append((trio, ev))
            ln_in = [host["LNX"].to(dev, non_blocking=True), host["LNG"].to(dev, non_blocking=True)]
            ln_ev = torch.cuda.Event()
            ln_ev.record(s_in)
        for i, ((X, W, G), ev) in enumerate(uploads):
            main.wait_event(ev)
            for t in (X, W, G):
                t.record_stream(main)
            X.requires_grad_()
            W.requires_grad_()
            Y = pam.linear(X, W, approx_bwd=True)
            Y.backward(G)
            download(i, [Y.detach(), X.grad, W.grad])
        main.wait_event(ln_ev)
        x = ln_in[0].requires_grad_()
        for t in ln_in:
            t.record_stream(main)
        y = ln(x)
        y.backward(ln_in[1])
        ln.weight.grad = ln.bias.grad = None
        download("ln", [y.detach(), x.grad])

    # The K steps are timed as one region: step i+1's uploads are queued while step i computes and
    # downloads (the way a prefetching input pipeline feeds a training loop), so the steady state is
    # whichever of upload, compute and download is slowest; every byte of every step crosses PCIe
    # inside the region.
    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(2):
        e2e_step()
    main.wait_stream(s_out)
    torch.cuda.synchronize()
    barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(e2e_steps):
        e2e_step()
    main.wait_stream(s_out)
    t1.record()
    torch.cuda.synchronize()
    e2e_ms = t0.elapsed_time(t1)
    d2h = sum(t.numel() * 4 for t in out_host.values())

    from pam_b200 import parallel
    total_ms, e2e_ms = (parallel.max_over_ranks(v, dev) for v in (total_ms, e2e_ms))

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_sample(args, target_seconds=12.0)

    if rank == 0:
        value = world * MACS_PER_STEP * args.steps / (total_ms * 1e-3)
        line = {
            "metric": METRIC, "value": value, "unit": "MAC/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int32 add + fp32 accumulate", "data": "synthetic",
            "config": {"workload": "configs[1]: DeiT-tiny PAM linear-layer set, X[12608x192], GEMMs 192->576, "
                                   "192->192, 192->768, 768->192 fwd+bwd approx_bwd, pam_ln over 192-wide rows fwd+bwd",
                       "macs_per_step_per_gpu": MACS_PER_STEP, "l2": "flushed between timed steps (256 MB write)",
                       "sharding": "per-GPU replica of the workload on its own rows; no collective"},
            "e2e": {"value": world * MACS_PER_STEP * e2e_steps / (e2e_ms * 1e-3), "unit": "MAC/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "note": "pinned host inputs -> device -> pam.linear/LayerNorm fwd+bwd -> all outputs and gradients "
                            "back to pinned host; uploads and downloads overlap the compute on their own streams"},
            "gpu_launches": int(launches),
            "clocks": clocks.summary(),
            "roofline": {"bound": "issue (INT32 add + FP32 add per MAC)", "achieved": gemm_rate / 1e12, "peak": mac_peak / 1e12,
                         "unit": "T PAM-MAC/s", "frac": gemm_rate / mac_peak, "traffic": GEMM_DRAM_BYTES_PER_LAUNCH,
                         "traffic_note": "DRAM bytes per GEMM launch, mean of the three captured launches of the 192->576 layer "
                                         "(ncu dram__bytes_read.sum + dram__bytes_write.sum: 10 MB forward, 36 MB input gradient, "
                                         "333 MB weight gradient incl. its 43 split-K partials); algorithmic 40 MB; irrelevant to an "
                                         "issue-bound kernel (about 1 % of HBM bandwidth)",
                         "kernel": "gemm_kernel<pam> (12 launches of the step, timed alone)",
                         "peak_source": "measured live: 1:1 INT32-add/FP32-add register chains (pamk_issue_rate)",
                         "issue_rates_T_per_s": {k: v / 1e12 for k, v in peak.items()}},
            "cpu_baseline": cpu,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# ---- single kernels, for profilers -------------------------------------------------------------------

def run_case(args):
    """Launches one kernel `--reps` times after one warm-up and prints its CUDA-event time.  Meant
    to be wrapped by ncu (`-k regex:<kernel> -s 1 -c 1`); sizes default to a few hundred MB."""
    import pam_b200 as pam
    from pam_b200 import cuda_bindings as cb
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(7)
    n = args.size
    if args.case in ("gemm", "gemm_specials"):
        A, B = torch.randn(n, n, generator=g), torch.randn(n, n, generator=g)
        if args.case == "gemm_specials":       # 1% zeros / denormals / +-1e30 / +-1e-30
            vals = torch.tensor([0.0, -0.0, 1e-40, -1e-40, 1.4e-45, -1.4e-45, 1e30, -1e30, 1e-30, -1e-30])
            for t in (A, B):
                idx = torch.randperm(t.numel(), generator=g)[: t.numel() // 100]
                t.view(-1)[idx] = vals[torch.arange(idx.numel()) % 10]
        A, W = A.to(dev), B.to(dev)
        fn, work, unit = (lambda: cb._matmul(0, A, W.T, 1.0, 2)), float(n) ** 3, "MAC"
    elif args.case == "deit_gemms":
        d = make_inputs(1234, device=dev)

        def fn():
            for X, W, G in zip(d["X"], d["W"], d["G"]):
                cb._matmul(0, X, W.T, 1.0, 2)
                cb._matmul(0, G, W, 1.0, 2)
                cb._matmul(0, X.T, G, 1.0, 2)
        work, unit = float(MACS_PER_STEP), "MAC"
    elif args.case == "deit_gemms_exact":      # the eight exact-gradient products of the linear-layer set
        d = make_inputs(1234, device=dev)

        def fn():
            for X, W, G in zip(d["X"], d["W"], d["G"]):
                cb._matmul_bwd(G, W, X, True, 1.0, 2)            # dX[i,k] = sum_n G[i,n] * slope(X[i,k], W[n,k])
                cb._matmul_bwd(X.T, G, W.T, False, 1.0, 2)       # dW^T[k,n] = sum_i G[i,n] * slope(W[n,k], X[i,k])
        work, unit = float(MACS_PER_STEP) * 2 / 3, "MAC"
    elif args.case == "mul":
        count = 1 << n if n < 40 else n
        a, b = torch.randn(count, device=dev), torch.randn(count, device=dev)
        fn, work, unit = (lambda: cb.cuda_kernels.pam_fwd(a, b, 1.0)), 12.0 * count, "B"
    elif args.case in ("layer_norm_fwd", "layer_norm_bwd"):
        rows = (1 << n if n < 40 else n) // LN_WIDTH
        x = torch.randn(rows, LN_WIDTH, device=dev, requires_grad=True)
        gy = torch.randn(rows, LN_WIDTH, device=dev)
        ln = pam.LayerNorm(LN_WIDTH, eps=1e-6, approx_bwd=True).to(dev)
        if args.case == "layer_norm_fwd":
            def fn():
                with torch.no_grad():
                    ln(x)
            work = 8.0 * rows * LN_WIDTH
        else:
            y = ln(x)
            fn = lambda: torch.autograd.grad(y, (x, ln.weight, ln.bias), gy, retain_graph=True)
            work = 12.0 * rows * LN_WIDTH
        unit = "B"
    elif args.case in ("softmax_fwd", "softmax_bwd"):
        length = 1024
        rows = (1 << n if n < 40 else n) // length
        x = torch.randn(rows, length, device=dev, requires_grad=True)
        gy = torch.randn(rows, length, device=dev)
        if args.case == "softmax_fwd":
            def fn():
                with torch.no_grad():
                    pam.softmax(x, dim=-1, approx_bwd=True)
            work = 12.0 * rows * length           # maximum pass 4 B + row pass 8 B per element
        else:
            y = pam.softmax(x, dim=-1, approx_bwd=True)
            fn = lambda: torch.autograd.grad(y, (x,), gy, retain_graph=True)
            work = 16.0 * rows * length           # maximum pass 4 B + row pass 12 B per element
        unit = "B"
    elif args.case == "column_sum":            # bias gradient of a linear layer: 768-wide rows
        count = 1 << n if n < 40 else n
        x = torch.randn(count // 768, 768, device=dev)
        fn, work, unit = (lambda: cb._column_sum(x)), 4.0 * x.numel(), "B"
    elif args.case == "adam":
        from pam_b200 import optim
        count = 1 << n if n < 40 else n
        p = torch.nn.Parameter(torch.randn(count, device=dev))
        p.grad = torch.randn(count, device=dev) * 0.01
        opt = optim.Adam([p], lr=5e-4, betas=(0.9, 0.98), weight_decay=1e-4, opt_functional_cfg="pam")
        fn, work, unit = opt.step, 28.0 * count, "B"
    else:
        raise SystemExit(f"unknown --case {args.case}")
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.reps
    print(json.dumps({"case": args.case, "size": n, "ms": ms, f"G{unit}_per_s": work / ms / 1e6}))


# ---- full training steps (BASELINE configs 3 and 4) -----------------------------------------------------

def run_step_case(args):
    """One data-parallel training step per iteration: batch upload, forward, backward, gradient
    all-reduce over the ranks (NCCL; summed, as the reference's fairseq path leaves them), fused PAM
    Adam.  Every rank holds the same parameters and its own batch (seed + rank).  Prints the step
    time (slowest rank, CUDA events) and the PAM multiply-accumulate rate of the whole job."""
    import torch.distributed as dist
    import pam_b200 as pam
    from pam_b200 import _lib, optim, parallel, steps
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    kw = dict(approx_bwd=not args.exact_bwd)
    g = torch.Generator().manual_seed(1000 + rank)
    if args.case == "deit_step":
        cfg, batch = steps.DeitConfig(), 64
        params = steps.to_device(steps.deit_params(cfg, torch.Generator().manual_seed(5)), dev)
        host = (torch.randn(batch, cfg.channels, cfg.image, cfg.image, generator=g).pin_memory(),
                torch.randint(0, cfg.classes, (batch,), generator=g).pin_memory())
        loss_fn = lambda images, labels: steps.deit_loss(pam, params, images, labels, cfg, kw)
        macs, hyper = 3 * steps.deit_macs(cfg, batch), dict(lr=5e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.05)
        what = f"DeiT-tiny step, batch {batch} per GPU"
    else:
        cfg = steps.TransformerConfig()
        params = steps.to_device(steps.transformer_params(cfg, torch.Generator().manual_seed(5)), dev)
        host = tuple(t.pin_memory() for t in steps.transformer_batch(cfg, g))
        loss_fn = lambda src, prev, tgt: steps.transformer_loss(pam, params, src, prev, tgt, cfg, kw)
        macs, hyper = 3 * steps.transformer_macs(cfg), dict(lr=5e-4, betas=(0.9, 0.98), eps=1e-8, weight_decay=1e-4)
        what = "6+6 transformer step, 4096 tokens per GPU"
    leaves = list(params.values())
    opt = optim.Adam(leaves, opt_functional_cfg="pam", **hyper)
    launches0 = None
    times, losses = [], []
    for it in range(args.warmup + args.steps):
        if it == args.warmup:
            launches0 = _lib.lib().pamk_launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        batch_dev = [t.to(dev, non_blocking=True) for t in host]
        opt.zero_grad(set_to_none=True)
        loss = loss_fn(*batch_dev)
        loss.backward()
        parallel.all_reduce_gradients(leaves)
        opt.step()
        e1.record()
        torch.cuda.synchronize()
        if it >= args.warmup:
            times.append(e0.elapsed_time(e1))
        losses.append(float(loss.detach()))
    ms = parallel.max_over_ranks(sum(times) / len(times), dev)
    launches = (_lib.lib().pamk_launch_count() - launches0) / max(1, args.steps)
    if rank == 0:
        print(json.dumps({"case": args.case, "workload": what, "approx_bwd": not args.exact_bwd, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                          "ms_per_step": ms, "PAM_MAC_per_s": macs * world / (ms * 1e-3), "MAC_per_step_per_gpu": macs,
                          "library_launches_per_step": launches, "loss_first": losses[0], "loss_last": losses[-1],
                          "params": sum(t.numel() for t in leaves)}))
    if world > 1:
        dist.destroy_process_group()


# ---- CPU baseline / reference arm ---------------------------------------------------------------------

def cpu_sample(args, target_seconds):
    """Times the port of the reference's native PyTorch CPU path (oracle/native_port.py) on a bounded
    sample of the workload: the first `rows` rows of X through every layer, forward and both
    approx_bwd gradients.  Returns the cpu_baseline object."""
    from oracle import native_port as N
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    d = make_inputs(1234)
    rows = args.cpu_rows
    if rows <= 0:
        t0 = time.perf_counter()
        N.matmul(d["X"][0][:8], d["W"][0].T)
        probe = (time.perf_counter() - t0) / (8 * 192 * 576)          # seconds per MAC
        per_row = 3 * sum(k * n for k, n in LAYERS) * probe
        rows = int(max(4, min(TOKENS, target_seconds / max(per_row, 1e-12))))
    macs = 3 * rows * sum(k * n for k, n in LAYERS)
    t0 = time.perf_counter()
    for X, W, G in zip(d["X"], d["W"], d["G"]):
        N.matmul(X[:rows], W.T)
        N.matmul(G[:rows], W)
        N.matmul(X[:rows].T, G[:rows])
    dt = time.perf_counter() - t0
    return {"value": macs / dt, "unit": "MAC/s", "cores": threads, "kind": "port",
            "sample": f"first {rows} of {TOKENS} rows through all four layers, fwd + dX + dW "
                      f"({macs / 1e6:.0f} M MAC, {dt:.1f} s); port of pam/native.py (float log2/exp2 PAM) in PyTorch CPU",
            "seconds": dt, "rows": rows}


def run_reference(args):
    if int(os.environ.get("RANK", 0)) != 0:
        return
    per_step = []
    base = None
    for _ in range(args.warmup + args.steps):
        base = cpu_sample(args, target_seconds=60.0 / max(1, args.steps + args.warmup))
        per_step.append(base)
        if not args.cpu_rows:
            args.cpu_rows = base["rows"]                         # keep the sample fixed across steps
    timed = per_step[args.warmup:]
    seconds = sum(b["seconds"] for b in timed)
    rows = args.cpu_rows
    macs = 3 * rows * sum(k * n for k, n in LAYERS)
    value = macs * len(timed) / seconds
    base = dict(timed[-1], value=value)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "MAC/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * seconds / len(timed),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32 (float log2/exp2 PAM)",
        "data": "synthetic",
        "config": {"workload": "configs[1]: DeiT-tiny PAM linear-layer set (bounded row sample per step)",
                   "rows_per_step": rows},
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": "MAC/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


if __name__ == "__main__":
    a = parse()
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    if a.case in ("deit_step", "transformer_step"):
        run_step_case(a)
    elif a.case:
        run_case(a)
    elif a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
