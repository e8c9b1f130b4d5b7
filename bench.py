"""Benchmark of the PAM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--size n]

Headline workload (one "step"): the largest square product of the scaling sweep — one PAM matrix
product C = A (x) B with M = N = K = 16384 in fp32, entries N(0,1) with 1 % injected special values
(zeros of both signs, denormals, magnitudes 1e30 and 1e-30) generated on the device from a seed.
With N > 1 ranks (torchrun) the rows of A are sharded: every rank holds its own 16384-row block of
a [N*16384 x 16384] A and the whole B (weak scaling, no collective on the data path); the time is the
max over ranks.

Prints ONE JSON line: PAM-GEMM MAC/s, the issue-rate roofline of the product kernel on this input,
the end-to-end figure with host buffers, clocks sampled during the timed region, per-rank times, and
secondary objects measured in the same run: the same product without special values, the DeiT-tiny
linear-layer set, the HBM-bound kernels (mul / div / pam_ln) against the measured copy bandwidth,
the reference's own CUDA kernel on the same inputs (when its build is present), the two training
steps, and the reference's CPU implementation on a bounded sample.
"""
import argparse
import ctypes
import json
import os
import pathlib
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = pathlib.Path(__file__).resolve().parent

# the DeiT-tiny linear-layer set (secondary workload)
LAYERS = ((192, 576), (192, 192), (192, 768), (768, 192))
TOKENS = 12608
LN_WIDTH = 192
LAYER_SET_MACS = 3 * TOKENS * sum(k * n for k, n in LAYERS)

SPECIALS = [0.0, -0.0, 1e-40, -1e-40, 1.4e-45, -1.4e-45, 1e30, -1e30, 1e-30, -1e-30]
METRIC = "PAM-GEMM MAC/s (fp32)"
SM_LANES = 128          # fp32 / int32 lanes per SM: one INT32 add + one FP32 add per MAC -> lanes * clock / 2

# DRAM bytes (ncu dram__bytes_read.sum + dram__bytes_write.sum) of one product launch of the
# headline kernel on an 8192^3 input with 1 % specials; a 16384^3 launch streams each operand from
# DRAM once per wave of output tiles, so its traffic is scaled by the number of multiply-accumulates.
GEMM_DRAM_BYTES_8192 = 7.933e9 + 0.269e9


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--size", type=int, default=None,
                    help="edge of the headline product (default 16384); with --case: GEMM edge or log2 of the element count")
    ap.add_argument("--cpu-rows", type=int, default=0, help="rows of A in the CPU sample (0 = auto)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="headline only (for profilers)")
    ap.add_argument("--case", default=None,
                    help="run one kernel in isolation (for profiling) instead of the benchmark: "
                         "gemm | gemm_specials | gemm_relu | deit_gemms | deit_gemms_exact | attention_gemms | mul | div | "
                         "layer_norm_fwd | layer_norm_bwd | softmax_fwd | softmax_bwd | adam | column_sum; or a full training "
                         "step, also under torchrun with --gpus N: deit_step | transformer_step")
    ap.add_argument("--reps", type=int, default=2)
    ap.add_argument("--exact-bwd", action="store_true",
                    help="training-step cases: exact piecewise-affine gradients (approx_bwd=False) instead of approx_bwd=True")
    return ap.parse_args()


def randn_with_specials(shape, seed, dev, frac=0.01, values=SPECIALS):
    """N(0,1) entries with a fraction overwritten by a cycle of special values (seeded, on `dev`)."""
    g = torch.Generator(device=dev).manual_seed(seed)
    t = torch.randn(shape, generator=g, device=dev)
    if frac > 0:
        flat = t.view(-1)
        count = max(1, int(flat.numel() * frac))
        idx = torch.randint(0, flat.numel(), (count,), generator=g, device=dev)
        vals = torch.tensor(values, dtype=torch.float32, device=dev)
        flat[idx] = vals[torch.arange(count, device=dev) % vals.numel()]
    return t


def layer_set_inputs(seed, device=None):
    g = torch.Generator().manual_seed(seed)
    data = {"X": [], "W": [], "G": []}
    for k, n in LAYERS:
        data["X"].append(torch.randn(TOKENS, k, generator=g))
        data["W"].append(torch.nn.init.trunc_normal_(torch.empty(n, k), std=0.02, generator=g))
        data["G"].append(torch.randn(TOKENS, n, generator=g))
    data["LNX"] = torch.randn(TOKENS, LN_WIDTH, generator=g)
    data["LNG"] = torch.randn(TOKENS, LN_WIDTH, generator=g)
    place = (lambda t: t.to(device)) if device is not None else (lambda t: t)
    return {k: [place(t) for t in v] if isinstance(v, list) else place(v) for k, v in data.items()}


def hbm_peak():
    """Measured copy bandwidth of this pool's B200s (GB/s) and where the figure comes from."""
    path = ROOT / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    except (OSError, ValueError, KeyError):
        return 6650.0, "fallback (earlier measurement on this pool)"


# ---- clocks ---------------------------------------------------------------------------------------

class ClockSampler:
    """Samples nvidia-smi for one GPU every 50 ms while the device-timed regions run."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
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
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, power, reasons = [], [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
                power.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, r[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_min_mhz": min(sm), "sm_max_mhz": max(mx), "power_w_max": max(power),
                "reasons": sorted(reasons), "samples": len(sm)}


def timed(fn, reps, flush=None, back_to_back=False):
    """Mean CUDA-event milliseconds of `fn` over `reps` calls (one warm-up call first).  With
    `back_to_back` the calls are queued without a host synchronisation in between, so that short
    kernels are not charged the host's launch latency."""
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if back_to_back:
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps
    total = 0.0
    for _ in range(reps):
        if flush is not None:
            flush.zero_()
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / reps


def issue_rates(lib, dev):
    """Live INT32/FP32 issue rates from register-only chains (instructions-pairs per second)."""
    from pam_b200 import _lib
    peak = {}
    scratch = torch.zeros(4, dtype=torch.int32, device=dev)
    for name, variant in (("fadd", 0), ("iadd", 1), ("iadd_fadd", 2), ("imad_fadd", 3), ("mixed_fadd", 4)):
        ms, steps_done = ctypes.c_float(), ctypes.c_double()
        _lib.check(lib.pamk_issue_rate(variant, 8000, 4, scratch.data_ptr(), ctypes.byref(ms), ctypes.byref(steps_done),
                                       torch.cuda.current_stream().cuda_stream), "issue_rate")
        peak[name] = steps_done.value / (ms.value * 1e-3)
    return peak


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
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    import pam_b200 as pam
    from pam_b200 import _lib, parallel
    torch.backends.cuda.matmul.allow_tf32 = False
    lib = _lib.lib()                       # fails loudly if the CUDA library is missing
    n = args.size or 16384
    macs = float(n) ** 3
    sms = torch.cuda.get_device_properties(dev).multi_processor_count

    # rank r's block of rows of A (seed + rank) and the shared B
    A = randn_with_specials((n, n), 4000 + rank, dev)
    B = randn_with_specials((n, n), 3999, dev)

    def step():
        with torch.no_grad():
            return pam.matmul(A, B)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()

    # ---- value: inputs resident in HBM; operands (1 GiB each at the default size) exceed the L2 ----
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    launches0 = lib.pamk_launch_count()
    clocks = ClockSampler(local)
    clocks.__enter__()
    barrier()
    region0, region1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    region0.record()
    enqueue_s = 0.0
    for e0, e1 in ev:
        t0 = time.perf_counter()
        e0.record()
        step()
        e1.record()
        enqueue_s += time.perf_counter() - t0
    region1.record()
    barrier()
    clocks.__exit__(None, None, None)
    launches = lib.pamk_launch_count() - launches0
    kernel_ms = sum(e0.elapsed_time(e1) for e0, e1 in ev)
    region_ms = region0.elapsed_time(region1)
    clk = clocks.summary()

    peak_chains = issue_rates(lib, dev)
    live_peak = max(peak_chains["iadd_fadd"], peak_chains["imad_fadd"], peak_chains["mixed_fadd"])
    clock_peak = 0.98 * sms * SM_LANES * (clk["sm_mhz"] or 0.0) * 1e6 / 2
    mac_peak = max(live_peak, clock_peak)

    secondary = {}
    if not args.no_secondary:
        secondary = run_secondary(args, pam, lib, dev, A, B, n, mac_peak, rank)

    # ---- e2e: host buffers in, result out, through the public API ---------------------------------------
    e2e_steps = max(3, min(args.steps, 5))
    hA, hB = A.cpu().pin_memory(), B.cpu().pin_memory()
    hC = torch.empty(n, n, dtype=torch.float32).pin_memory()

    # B goes up first; A follows in row blocks on a copy stream, each block's product starts when its rows
    # have arrived, and each block of C returns on a third stream while the next product runs
    blocks = 8 if n % 8 == 0 and n >= 2048 else 1
    rows = n // blocks
    up, down = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def e2e_step():
        cur = torch.cuda.current_stream(dev)
        up.wait_stream(cur)
        arrived = []
        with torch.cuda.stream(up):
            dB = hB.to(dev, non_blocking=True)
            for b in range(blocks):
                dA = hA[b * rows:(b + 1) * rows].to(dev, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(up)
                arrived.append((dA, ev))
        dB.record_stream(cur)
        for b, (dA, ev) in enumerate(arrived):
            cur.wait_event(ev)
            dA.record_stream(cur)
            with torch.no_grad():
                out = pam.matmul(dA, dB)
            done = torch.cuda.Event()
            done.record(cur)
            down.wait_event(done)
            with torch.cuda.stream(down):
                hC[b * rows:(b + 1) * rows].copy_(out, non_blocking=True)
            out.record_stream(down)
        cur.wait_stream(down)

    e2e_step()
    barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(e2e_steps):
        e2e_step()
    t1.record()
    torch.cuda.synchronize()
    e2e_ms = t0.elapsed_time(t1)
    del hA, hB, hC

    per_rank = [[round(region_ms / args.steps, 4), round(kernel_ms / args.steps, 4), round(1e3 * enqueue_s / args.steps, 4)]]
    if world > 1:
        gathered = [torch.zeros(3, dtype=torch.float64, device=dev) for _ in range(world)]
        dist.all_gather(gathered, torch.tensor([region_ms / args.steps, kernel_ms / args.steps, 1e3 * enqueue_s / args.steps],
                                               dtype=torch.float64, device=dev))
        per_rank = [[round(float(v), 4) for v in g.tolist()] for g in gathered]
    region_ms, e2e_ms = (parallel.max_over_ranks(v, dev) for v in (region_ms, e2e_ms))

    train = None
    if not args.no_secondary:
        train = {name: training_step(args, name, rank, world, dev, steps=5, warmup=3) for name in ("deit_step", "transformer_step")}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_sample(args, n, target_seconds=12.0)

    if rank == 0:
        value = world * macs * args.steps / (region_ms * 1e-3)
        kernel_rate = macs * args.steps / (kernel_ms * 1e-3)
        line = {
            "metric": METRIC, "value": value, "unit": "MAC/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": region_ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int32 add + fp32 accumulate", "data": "synthetic",
            "config": {"workload": f"configs[4]: scaling sweep, square PAM GEMM M=N=K={n}, fp32, N(0,1) inputs with 1% injected "
                                   "specials (+-0, denormals, +-1e30, +-1e-30), forward product through pam.matmul",
                       "macs_per_step_per_gpu": macs, "l2": "operands larger than L2 (1 GiB each at 16384)",
                       "sharding": "rows of A sharded over the ranks (each rank its own n-row block, B replicated); no collective"},
            "e2e": {"value": world * macs * e2e_steps / (e2e_ms * 1e-3), "unit": "MAC/s",
                    "h2d_bytes_per_step": 2 * n * n * 4, "d2h_bytes_per_step": n * n * 4,
                    "note": "every step: pinned host B, then A in 8 row blocks -> device on a copy stream; pam.matmul per block as its "
                            "rows arrive; each block of C back to pinned host on a third stream"},
            "gpu_launches": int(launches),
            "clocks": clk,
            "timed_region_s": region_ms * 1e-3,
            "macs_per_sm_clock": (kernel_rate / ((clk["sm_mhz"] or float("nan")) * 1e6)),
            "per_rank": {"columns": ["ms_per_step", "kernel_ms_per_step", "host_enqueue_ms_per_step"], "rows": per_rank},
            "roofline": {"bound": "issue (INT32 add + FP32 add per MAC)", "achieved": kernel_rate / 1e12, "peak": mac_peak / 1e12,
                         "unit": "T PAM-MAC/s", "frac": kernel_rate / mac_peak,
                         "traffic": None if GEMM_DRAM_BYTES_8192 is None else GEMM_DRAM_BYTES_8192 * (n / 8192.0) ** 3,
                         "kernel": "gemm_kernel<pam, 128x128x16> (one launch per step, rank 0)",
                         "peak_source": "max(live 1:1 INT32-add/FP32-add register chains, 0.98 * SMs * 128 lanes * median sampled "
                                        "SM clock / 2)",
                         "peak_live_chains": live_peak / 1e12, "peak_from_sampled_clock": clock_peak / 1e12,
                         "peak_nominal_at_max_clock": sms * SM_LANES * (clk["sm_max_mhz"] or 0.0) * 1e6 / 2 / 1e12,
                         "issue_rates_T_per_s": {k: v / 1e12 for k, v in peak_chains.items()}},
            "cpu_baseline": cpu,
        }
        line.update(secondary)
        if train is not None:
            line["train_steps"] = train
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_secondary(args, pam, lib, dev, A, B, n, mac_peak, rank):
    """Figures measured beside the headline in the same run (rank-local; rank 0's are printed)."""
    from pam_b200 import cuda_bindings as cb
    out = {}
    macs = float(n) ** 3
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)     # > 126 MB L2

    # the same product without special values (every slab takes the two-instruction loop)
    A0, B0 = torch.randn(n, n, device=dev), torch.randn(n, n, device=dev)
    ms = timed(lambda: cb._matmul(0, A0, B0, 1.0, 2), 3)
    out["gemm_no_specials"] = {"T_mac_per_s": macs / ms / 1e9, "ms": ms, "frac_of_peak": macs / (ms * 1e-3) / mac_peak}
    del A0, B0

    # the reference's own CUDA kernel (compiled for sm_100a by baseline/build_ref.py) on the same inputs
    ref = None
    try:
        from baseline import build_ref
        ref = build_ref.load()
    except Exception as exc:                                        # noqa: BLE001 (absence is reported, not fatal)
        out["ref_gpu_kernel"] = {"unavailable": f"{type(exc).__name__}: {exc}"}
    if ref is not None:
        ours_ms = timed(lambda: cb._matmul(0, A, B, 1.0, 2), 2)
        ref_ms = timed(lambda: ref.pam_matmul_fwd(A, B, True, True, 1.0), 1)
        out["ref_gpu_kernel"] = {
            "what": "pam_matmul_fwd of the reference's pam/cuda_kernels.cu built for sm_100a, same inputs, same run, CUDA events",
            "headline_gemm": {"ref_ms": ref_ms, "ours_ms": ours_ms, "ref_T_mac_per_s": macs / ref_ms / 1e9,
                              "speedup_vs_ref_kernel": ref_ms / ours_ms}}
    elif "ref_gpu_kernel" not in out:
        out["ref_gpu_kernel"] = {"unavailable": "baseline/_ref/pam_ref_cuda_kernels.so was not built"}

    # the DeiT-tiny linear-layer set: 12 products forward + approx_bwd, pam_ln over the 192-wide rows
    d = layer_set_inputs(1234 + rank, device=dev)
    ln = pam.LayerNorm(LN_WIDTH, eps=1e-6, approx_bwd=True).to(dev)

    def layer_set_step():
        for X, W, G in zip(d["X"], d["W"], d["G"]):
            X = X.detach().requires_grad_()
            W = W.detach().requires_grad_()
            pam.linear(X, W, approx_bwd=True).backward(G)
        x = d["LNX"].detach().requires_grad_()
        ln(x).backward(d["LNG"])
        ln.weight.grad = ln.bias.grad = None

    def layer_set_gemms():
        for X, W, G in zip(d["X"], d["W"], d["G"]):
            cb._matmul(0, X, W.T, 1.0, 2)
            cb._matmul(0, G, W, 1.0, 2)
            cb._matmul(0, X.T, G, 1.0, 2)

    for _ in range(3):
        layer_set_step()
    step_ms = timed(layer_set_step, 10, flush)
    gemm_ms = timed(layer_set_gemms, 10, flush)
    out["config2_linear_set"] = {
        "workload": "configs[1]: DeiT-tiny PAM linear-layer set, X[12608x192], GEMMs 192->576, 192->192, 192->768, 768->192 "
                    "fwd+bwd approx_bwd, pam_ln over 192-wide rows fwd+bwd; L2 flushed between steps",
        "T_mac_per_s": LAYER_SET_MACS / step_ms / 1e9, "ms_per_step": step_ms,
        "gemms_only_T_mac_per_s": LAYER_SET_MACS / gemm_ms / 1e9, "gemms_only_frac_of_peak": LAYER_SET_MACS / (gemm_ms * 1e-3) / mac_peak}
    if ref is not None:
        def ref_gemms():
            for X, W, G in zip(d["X"], d["W"], d["G"]):
                ref.pam_matmul_fwd(X, W.T, True, False, 1.0)
                ref.pam_matmul_fwd(G, W, True, True, 1.0)
                ref.pam_matmul_fwd(X.T, G, False, True, 1.0)
        ref_ms = timed(ref_gemms, 3, flush)
        out["ref_gpu_kernel"]["config2_gemms"] = {"ref_ms": ref_ms, "ours_ms": gemm_ms, "speedup_vs_ref_kernel": ref_ms / gemm_ms}

    # HBM-bound kernels: algorithmic bytes / CUDA-event time, against the measured copy bandwidth
    peak_gbs, peak_src = hbm_peak()
    hbm = {"peak_GBps": peak_gbs, "peak_source": peak_src, "kernels": {}}
    for log2n in (26, 28):
        count = 1 << log2n
        a = randn_with_specials((count,), 50 + log2n, dev)
        b = randn_with_specials((count,), 60 + log2n, dev)
        for name, fn in (("mul", pam.mul), ("div", pam.div)):
            ms = timed(lambda: fn(a, b), 5, back_to_back=True)
            gbs = 12.0 * count / ms / 1e6
            hbm["kernels"][f"{name}_2^{log2n}"] = {"GBps": gbs, "frac": gbs / peak_gbs, "bytes_per_element": 12}
        del a, b
        # pam_ln through the C ABI on preallocated buffers (through the module a call at 2^26 elements is as
        # long on the host as on the GPU): the forward kernel; the backward kernel plus its parameter-gradient pass
        rows = count // LN_WIDTH
        x = randn_with_specials((rows, LN_WIDTH), 70 + log2n, dev)
        gy = torch.randn(rows, LN_WIDTH, device=dev)
        y, dx = torch.empty_like(x), torch.empty_like(x)
        dw, db = torch.empty(LN_WIDTH, device=dev), torch.empty(LN_WIDTH, device=dev)
        w, bias = ln.weight.detach(), ln.bias.detach()
        ws_bytes = lib.pamk_layer_norm_bwd_workspace_bytes(rows, LN_WIDTH)
        ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)
        st = torch.cuda.current_stream(dev).cuda_stream

        def ln_fwd():
            rc = lib.pamk_layer_norm_fwd(x.data_ptr(), w.data_ptr(), bias.data_ptr(), y.data_ptr(), rows, LN_WIDTH, 1e-6, 1.0, st)
            assert rc == 0, rc

        # (the backward pass as the modules run it with approx_bwd: from the row scalars the forward pass saved)
        stats = torch.empty(rows, lib.pamk_layer_norm_stats_per_row(), device=dev)
        rc = lib.pamk_layer_norm_fwd_save(x.data_ptr(), w.data_ptr(), bias.data_ptr(), y.data_ptr(), stats.data_ptr(),
                                          rows, LN_WIDTH, 1e-6, 1.0, st)
        assert rc == 0, rc

        def ln_bwd():
            rc = lib.pamk_layer_norm_bwd_saved(x.data_ptr(), w.data_ptr(), gy.data_ptr(), stats.data_ptr(), dx.data_ptr(),
                                               dw.data_ptr(), db.data_ptr(), rows, LN_WIDTH, 1.0, ws.data_ptr(), ws_bytes, st)
            assert rc == 0, rc

        for name, fn, per in (("pam_ln_fwd", ln_fwd, 8), ("pam_ln_bwd", ln_bwd, 12)):
            ms = timed(fn, 10, back_to_back=True)
            gbs = float(per) * rows * LN_WIDTH / ms / 1e6
            hbm["kernels"][f"{name}_2^{log2n}"] = {"GBps": gbs, "frac": gbs / peak_gbs, "bytes_per_element": per}
        del x, gy, y, dx, stats
    out["hbm_kernels"] = hbm
    return out


# ---- single kernels, for profilers -------------------------------------------------------------------

def run_case(args):
    """Launches one kernel `--reps` times after one warm-up and prints its CUDA-event time.  Meant
    to be wrapped by ncu (`-k regex:<kernel> -s 1 -c 1`); sizes default to a few hundred MB."""
    import pam_b200 as pam
    from pam_b200 import cuda_bindings as cb
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(7)
    n = args.size or 4096
    if args.case in ("gemm", "gemm_specials", "gemm_relu"):
        if args.case == "gemm_specials":       # 1% zeros / denormals / +-1e30 / +-1e-30
            A, W = randn_with_specials((n, n), 1, dev), randn_with_specials((n, n), 2, dev)
        elif args.case == "gemm_relu":          # an activation after ReLU times a dense weight
            A, W = torch.relu(torch.randn(n, n, device=dev)), torch.randn(n, n, device=dev)
        else:
            A, W = torch.randn(n, n, device=dev), torch.randn(n, n, device=dev)
        fn, work, unit = (lambda: cb._matmul(0, A, W.T, 1.0, 2)), float(n) ** 3, "MAC"
    elif args.case == "deit_gemms":
        d = layer_set_inputs(1234, device=dev)

        def fn():
            for X, W, G in zip(d["X"], d["W"], d["G"]):
                cb._matmul(0, X, W.T, 1.0, 2)
                cb._matmul(0, G, W, 1.0, 2)
                cb._matmul(0, X.T, G, 1.0, 2)
        work, unit = float(LAYER_SET_MACS), "MAC"
    elif args.case == "deit_gemms_exact":      # the eight exact-gradient products of the linear-layer set
        d = layer_set_inputs(1234, device=dev)

        def fn():
            for X, W, G in zip(d["X"], d["W"], d["G"]):
                cb._matmul_bwd(G, W, X, True, 1.0, 2)            # dX[i,k] = sum_n G[i,n] * slope(X[i,k], W[n,k])
                cb._matmul_bwd(X.T, G, W.T, False, 1.0, 2)       # dW^T[k,n] = sum_i G[i,n] * slope(W[n,k], X[i,k])
        work, unit = float(LAYER_SET_MACS) * 2 / 3, "MAC"
    elif args.case == "attention_gemms":       # DeiT-tiny attention: 192 x (197x64 . 64x197) and (197x197 . 197x64)
        q = torch.randn(192, 197, 64, device=dev)
        k = torch.randn(192, 197, 64, device=dev)
        p = torch.softmax(torch.randn(192, 197, 197, device=dev), -1)

        def fn():
            cb._matmul(0, q, k.transpose(1, 2), 1.0, 3)
            cb._matmul(0, p, q, 1.0, 3)
        work, unit = 2.0 * 192 * 197 * 197 * 64, "MAC"
    elif args.case in ("mul", "div"):
        count = 1 << n if n < 40 else n
        a, b = torch.randn(count, device=dev), torch.randn(count, device=dev)
        kernel = cb.cuda_kernels.pam_fwd if args.case == "mul" else cb.cuda_kernels.pad_fwd
        fn, work, unit = (lambda: kernel(a, b, 1.0)), 12.0 * count, "B"
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
            work = 12.0 * rows * length           # from the saved exponentials: e, dy in, dx out
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

def training_step(args, case, rank, world, dev, steps, warmup):
    """One data-parallel training step per iteration: batch upload, forward, backward with the
    gradient all-reduce over the ranks started bucket by bucket as gradients become ready (NCCL;
    summed, as the reference's fairseq path leaves them), fused PAM Adam.  Every rank holds the same parameters and its own batch (seed + rank).  Returns the step
    time (slowest rank, CUDA events), the share of the all-reduce and the PAM multiply-accumulate
    rate of the whole job."""
    import torch.distributed as dist
    import pam_b200 as pam
    from pam_b200 import _lib, optim, parallel, steps as workloads
    # the models are built as the reference's forks build them: every swappable layer from a configuration
    # string through the factories (pam_b200/models.py), then filled with the seeded parameters
    from pam_b200 import models
    cfgs = models.pam_cfgs(approx_bwd=not args.exact_bwd)
    g = torch.Generator().manual_seed(1000 + rank)
    if case == "deit_step":
        cfg, batch = workloads.DeitConfig(), 64
        model = models.VisionTransformer(cfg, linear_cfg=cfgs["linear"], conv_cfg=cfgs["linear"], norm_cfg=cfgs["norm"],
                                         functional_cfg=cfgs["function"])
        model.load_parameters(workloads.deit_params(cfg, torch.Generator().manual_seed(5))).to(dev)
        host = (torch.randn(batch, cfg.channels, cfg.image, cfg.image, generator=g).pin_memory(),
                torch.randint(0, cfg.classes, (batch,), generator=g).pin_memory())
        loss_fn = lambda images, labels: torch.nn.functional.cross_entropy(model(images), labels)
        macs, hyper = 3 * workloads.deit_macs(cfg, batch), dict(lr=5e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.05)
        what = f"configs[3]: DeiT-tiny step, batch {batch} per GPU"
    else:
        cfg = workloads.TransformerConfig()
        model = models.Transformer(cfg, linear_cfg=cfgs["linear"], norm_cfg=cfgs["norm"], functional_cfg=cfgs["function"],
                                   loss_functional_cfg=cfgs["function"])
        model.load_parameters(workloads.transformer_params(cfg, torch.Generator().manual_seed(5))).to(dev)
        host = tuple(t.pin_memory() for t in workloads.transformer_batch(cfg, g))
        loss_fn = lambda src, prev, tgt: model.loss(src, prev, tgt, fused=True)
        macs, hyper = 3 * workloads.transformer_macs(cfg), dict(lr=5e-4, betas=(0.9, 0.98), eps=1e-8, weight_decay=1e-4)
        what = "configs[2]: 6+6 transformer step, 4096 tokens per GPU"
    params = model
    leaves = list(model.parameters())
    opt = optim.Adam(leaves, opt_functional_cfg="pam", **hyper)
    buckets = parallel.GradientBuckets(leaves)       # bucketed all-reduce, overlapped with the backward pass
    launches0 = None
    times, reduce_times, losses = [], [], []
    for it in range(warmup + steps):
        if it == warmup:
            launches0 = _lib.lib().pamk_launch_count()
        e0, e1, r0, r1 = (torch.cuda.Event(enable_timing=True) for _ in range(4))
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        batch_dev = [t.to(dev, non_blocking=True) for t in host]
        opt.zero_grad(set_to_none=True)
        loss = loss_fn(*batch_dev)
        loss.backward()
        r0.record()
        buckets.finish()                              # what is left of the reductions after the backward pass
        r1.record()
        opt.step()
        e1.record()
        torch.cuda.synchronize()
        if it >= warmup:
            times.append(e0.elapsed_time(e1))
            reduce_times.append(r0.elapsed_time(r1))
        losses.append(float(loss.detach()))
    ms = parallel.max_over_ranks(sum(times) / len(times), dev)
    reduce_ms = parallel.max_over_ranks(sum(reduce_times) / len(reduce_times), dev)
    launches = (_lib.lib().pamk_launch_count() - launches0) / max(1, steps)
    buckets.remove()
    del opt, params, model, leaves, buckets
    torch.cuda.empty_cache()
    return {"workload": what, "approx_bwd": not args.exact_bwd, "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": ms, "all_reduce_exposed_ms": reduce_ms, "all_reduce_exposed_share": reduce_ms / ms,
            "PAM_MAC_per_s": macs * world / (ms * 1e-3), "MAC_per_step_per_gpu": macs,
            "library_launches_per_step": launches, "loss_first": losses[0], "loss_last": losses[-1]}


def run_step_case(args):
    import torch.distributed as dist
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    res = training_step(args, args.case, rank, world, dev, args.steps, args.warmup)
    if rank == 0:
        print(json.dumps(dict(res, case=args.case)))
    if world > 1:
        dist.destroy_process_group()


# ---- CPU baseline / reference arm ---------------------------------------------------------------------

def cpu_matmul():
    """The reference's CPU implementation of the product, row-chunked: pam/native.py `pam_matmul`
    (staged by oracle/build.py into oracle/_ref/pam_native) when present, else its port
    (oracle/native_port.py).  Returns (function(A, B) -> C, kind, description)."""
    from oracle import build as oracle_build
    native = None
    try:
        oracle_build.build_native()
        native = oracle_build.load_native()
    except Exception:                                               # noqa: BLE001
        native = None
    if native is not None:
        def run(A, B):
            # native.pam_matmul materialises [rows, K, cols]; output rows and columns are independent, so
            # it is fed blocks of about 256 MB of temporaries (identical results, bounded memory)
            K, N = B.shape
            cols = max(1, min(N, (64 << 20) // max(1, K)))
            rows = max(1, (64 << 20) // max(1, K * cols))
            with torch.no_grad():
                return torch.cat([torch.cat([native.pam_matmul(A[r:r + rows], B[:, c:c + cols]) for c in range(0, N, cols)], dim=1)
                                  for r in range(0, A.shape[0], rows)])
        return run, "reference", "the reference's pam/native.py pam_matmul (float log2/exp2 PAM, PyTorch CPU), evaluated in blocks"
    from oracle import native_port
    return (lambda A, B: native_port.matmul(A, B)), "port", "port of pam/native.py (float log2/exp2 PAM) in PyTorch CPU"


class CpuSample:
    """The reference's CPU path on a bounded sample of the headline workload: the first `rows` rows
    of A against the whole B (same recipe and seeds as rank 0's device inputs)."""

    def __init__(self, n):
        self.n = n
        self.run, self.kind, self.what = cpu_matmul()
        self.threads = os.cpu_count() or 1
        torch.set_num_threads(self.threads)
        self.B = randn_with_specials((n, n), 3999, torch.device("cpu"))

    def rows_for(self, seconds):
        A1 = randn_with_specials((1, self.n), 4000, torch.device("cpu"))
        self.run(A1, self.B)
        t0 = time.perf_counter()
        self.run(A1, self.B)
        per_row = time.perf_counter() - t0
        return int(max(1, min(self.n, seconds / max(per_row, 1e-9))))

    def measure(self, rows):
        A = randn_with_specials((rows, self.n), 4000, torch.device("cpu"))
        t0 = time.perf_counter()
        self.run(A, self.B)
        dt = time.perf_counter() - t0
        macs = float(rows) * self.n * self.n
        return {"value": macs / dt, "unit": "MAC/s", "cores": self.threads, "kind": self.kind,
                "sample": f"first {rows} of {self.n} rows of A against the whole B ({macs / 1e9:.2f} G MAC, {dt:.1f} s); {self.what}",
                "seconds": dt, "rows": rows}


def cpu_sample(args, n, target_seconds):
    sample = CpuSample(n)
    return sample.measure(args.cpu_rows or sample.rows_for(target_seconds))


def run_reference(args):
    if int(os.environ.get("RANK", 0)) != 0:
        return
    n = args.size or 16384
    sample = CpuSample(n)
    budget = 150.0 / max(1, args.steps + args.warmup)          # the whole run ends within a few minutes
    rows = args.cpu_rows or sample.rows_for(min(budget, 15.0))  # fixed across steps, independent of --gpus
    per_step = [sample.measure(rows) for _ in range(args.warmup + args.steps)]
    timed_steps = per_step[args.warmup:]
    seconds = sum(b["seconds"] for b in timed_steps)
    macs = float(rows) * n * n
    value = macs * len(timed_steps) / seconds
    base = dict(timed_steps[-1], value=value)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "MAC/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * seconds / len(timed_steps),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32 (float log2/exp2 PAM)",
        "data": "synthetic",
        "config": {"workload": f"configs[4]: scaling sweep, square PAM GEMM M=N=K={n}, fp32, N(0,1) inputs with 1% injected "
                               "specials; each step a bounded row sample of the same product on the host cores",
                   "rows_per_step": rows},
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": "MAC/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


if __name__ == "__main__":
    a = parse()
    sys.path.insert(0, str(ROOT))
    if a.case in ("deit_step", "transformer_step"):
        run_step_case(a)
    elif a.case:
        run_case(a)
    elif a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
