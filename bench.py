#!/usr/bin/env python
"""Benchmark of the hot path: one shampoo2-AdamW 4-bit optimizer step on ViT-Base/32
parameter shapes (every interval firing: statistics refresh, inverse 4th root, apply,
AdamW tail), plus the blockwise quantize / dequantize rate of the same state.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line (rank 0).  `--impl reference` times the CPU side on this machine's host
cores and never imports the CUDA package: the whole ViT-B/32 step on the CPU port of the
reference's step (oracle/shampoo_oracle.py + oracle/qoracle.c; the reference's own Python
quantizer needs minutes per step), and the 1024 x 1024 quantize -> dequantize round trip on the
reference's own pure-PyTorch quantizer when a copy of it is present under oracle/_ref/py.
Multi-GPU runs are launched with torch.distributed.run.
"""
import argparse
import ctypes as ct
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "low-bit-shampoo_b200")
sys.path.insert(0, ROOT)


def use_package():
    """Puts the CUDA package on the import path (GPU arm only; the CPU arm must not see it)."""
    if PKG not in sys.path:
        sys.path.insert(0, PKG)


def load_workloads():
    """The model definitions (plain torch) loaded from their file, without exposing the package."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench_workloads", os.path.join(PKG, "workloads.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod

METRIC = "shampoo2 4-bit optimizer step ms (ViT-B/32); quant/dequant HBM GB/s"
HYPER = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.05, start_prec_step=1,
             stat_compute_steps=1, prec_compute_steps=1, stat_decay=0.95, matrix_eps=1e-6,
             prec_maxorder=1200, prec_bits=4, min_lowbit_size=4096, quan_blocksize=64,
             rect_t1=1, rect_t2=4, inv_root_mode=0)
WORKLOAD = ("vit_base_patch32_224 parameter set (88.2M params, 226 preconditioner matrices of order "
            "50..1200), shampoo2-adamw 4-bit block 64, T1=T2=1 so statistics refresh, inverse root and "
            "apply all run every step")


def measured_peaks():
    """(HBM GB/s, bf16 TFLOP/s burst, bf16 TFLOP/s sustained, "measured" | "fallback").  The burst
    figure is the denominator for a kernel timed alone, the sustained one for work timed inside a
    long step."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d.get("hbm_gbs", 6650.0), d.get("bf16_tflops", 1590.0), d.get("bf16_tflops_sustained", 1400.0), "measured"
    return 6650.0, 1590.0, 1400.0, "fallback"


def ncu_traffic(kernel):
    """DRAM bytes per launch of `kernel` from the committed capture table (dram__bytes_read.sum +
    dram__bytes_write.sum of one launch under ncu; a profiler cannot run inside the timed bench)."""
    try:
        with open(os.path.join(ROOT, "profiles", "roofline_traffic.json")) as f:
            return float(json.load(f)[kernel]["bytes"])
    except (OSError, KeyError, ValueError, TypeError):
        return None


def step_algorithmic_flops(shapes, maxorder=1200):
    """Algorithmic flops of one firing shampoo2 step (mode 0) over `shapes`, counted the way the
    reference spends them: per preconditioner matrix of order n  4 n^3 (Bjorck step) + 1.5 n^3
    (V^T diag(S) V) + 2 n^3 (L V^T) + 4 n^3 (V^T L V) + 5.5 n^3 (four Bjorck steps on n/2 rows and the
    root) = 17 n^3 of products plus 8/3 n^3 for the Householder QR; per gradient block m x k
    2 (m^2 k + m k^2) for the two Gram matrices and the same for P_L G P_R."""
    import itertools
    total = 0.0
    for s in shapes:
        dims = [d for d in s if d != 1]
        if len(dims) < 2:
            continue
        rows, cols = dims[0], 1
        for d in dims[1:]:
            cols *= d
        cut = lambda d: [maxorder] * (d // maxorder) + ([d % maxorder] if d % maxorder else []) if d > maxorder else [d]
        for m, k in itertools.product(cut(rows), cut(cols)):
            total += (17.0 + 8.0 / 3.0) * (m ** 3 + k ** 3) + 4.0 * (m * m * k + m * k * k)
    return total


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs (read-only NVML queries
    from a thread of this process every 10 ms, so that even a timed region of a few dozen
    milliseconds is covered; nvidia-smi in a loop as the fallback)."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index):
        self.index, self.rows, self.proc, self.stop = index, [], None, threading.Event()
        self.nvml = self.handle = None
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = index
            if visible:
                ids = [v.strip() for v in visible.split(",") if v.strip()]
                if index < len(ids) and ids[index].isdigit():
                    phys = int(ids[index])
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.nvml = pynvml
        except Exception:
            self.nvml = None

    def __enter__(self):
        if self.nvml is not None:
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return self
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _poll(self):
        n = self.nvml
        bits = {"hw_slowdown": getattr(n, "nvmlClocksEventReasonHwSlowdown", 0x8),
                "hw_thermal_slowdown": getattr(n, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                "sw_thermal_slowdown": getattr(n, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                "sw_power_cap": getattr(n, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        reasons_fn = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or getattr(n, "nvmlDeviceGetCurrentClocksThrottleReasons")
        while not self.stop.is_set():
            try:
                sm = n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)
                mx = n.nvmlDeviceGetMaxClockInfo(self.handle, n.NVML_CLOCK_SM)
                mask = reasons_fn(self.handle)
                self.rows.append([str(sm), str(mx)] + ["Active" if mask & bits[k] else "Not Active" for k in self.NAMES])
            except Exception:
                pass
            self.stop.wait(0.01)

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        self.stop.set()
        if self.nvml is not None:
            self.thread.join(timeout=2)
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], 0, set()
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx = max(mx, float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(self.NAMES, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------
# CPU arm.  Runs in a process of its own that never imports the CUDA package (only the model
# definitions of workloads.py, which are plain torch), so no GPU library is mapped into it.
# ---------------------------------------------------------------------------------------

CPU_STEP_BUDGET_S = 200.0       # stop taking timed steps once this much time has been spent stepping


def host_threads():
    """Threads the CPU arm uses: every core this process may run on (torch.distributed.run
    exports OMP_NUM_THREADS=1, which would otherwise leave one)."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    return max(1, min(n, 64))


def config1_matrix(torch, n=1024):
    """Q diag(lambda) Q^T, Q from the QR of a seeded N(0,1) matrix, lambda log-uniform in [1e-6, 1]."""
    g = torch.Generator().manual_seed(0)
    q, _ = torch.linalg.qr(torch.randn(n, n, dtype=torch.float64, generator=g))
    lam = torch.exp(torch.empty(n, dtype=torch.float64).uniform_(-13.815510557964274, 0.0, generator=g))
    a = (q * lam) @ q.T
    return (0.5 * (a + a.T)).float().contiguous()


def cpu_config1(torch):
    """The 1024 x 1024 round trip (4-bit, block 64) on the host: the reference's own pure-PyTorch
    quantizer (qtensor/functional.py:526-688) when oracle/_ref/py holds a copy of it, else the C port."""
    n, bs = 1024, 64
    A = config1_matrix(torch, n)
    nbytes = 4 * n * n + n * n // 2 + 4 * n * (n // bs)
    refpy = os.path.join(ROOT, "oracle", "_ref", "py")
    if os.path.isfile(os.path.join(refpy, "qtensor", "functional.py")):
        sys.path.insert(0, refpy)
        import qtensor.functional as RF                    # the reference's module (this process has no other qtensor)
        assert os.path.realpath(RF.__file__).startswith(os.path.realpath(refpy))
        code = RF.create_linear_map(True, 4, 2)
        tq, td = [], []
        for _ in range(2):
            t0 = time.perf_counter()
            q, am = RF.quantize_blockwise(A, code, n, blocksize=bs, bits=4)
            t1 = time.perf_counter()
            RF.dequantize_blockwise(q, code, n, am, blocksize=bs, bits=4)
            t2 = time.perf_counter()
            tq.append(t1 - t0)
            td.append(t2 - t1)
        kind = "reference"
    else:
        from oracle import qoracle
        code = qoracle.linear_map(True, 4, 2)
        a = A.numpy()
        tq, td = [], []
        for _ in range(3):
            t0 = time.perf_counter()
            q, am = qoracle.quantize(a, code, n, bs, 4)[:2]
            t1 = time.perf_counter()
            qoracle.dequantize(q, code, n, am, bs, 4)
            t2 = time.perf_counter()
            tq.append(t1 - t0)
            td.append(t2 - t1)
        kind = "port"
    return {"case": "1 x 1024^2 SPD fp32, 4-bit linear-2 code, block 64", "kind": kind, "cores": 1 if kind == "port" else torch.get_num_threads(),
            "quantize_s": min(tq), "dequantize_s": min(td), "bytes_per_direction": nbytes,
            "quantize_gbs": nbytes / min(tq) / 1e9, "dequantize_gbs": nbytes / min(td) / 1e9}


def cpu_reference_step(steps, warmup):
    """The full ViT-B/32 step (all 226 preconditioner matrices, every interval firing) on the CPU
    port, gradients from the same bf16-autocast backward as the GPU arm (seed 0, batch 256)."""
    import torch
    torch.set_num_threads(host_threads())
    from oracle.shampoo_oracle import OracleShampoo
    workloads = load_workloads()
    torch.manual_seed(0)
    model = workloads.vit_base_patch32_224()
    workloads.synthetic_gradients(model, 256, 224, 1000, "cpu", autocast_bf16=True, seed=0)
    params = [p.detach().clone() for p in model.parameters()]
    grads = [p.grad.detach().clone() for p in model.parameters()]
    del model
    opt = OracleShampoo(params, kind="adamw", flavour="s2", **{
        "lr": HYPER["lr"], "betas": HYPER["betas"], "eps": HYPER["eps"], "weight_decay": HYPER["weight_decay"],
        "stat_compute_steps": 1, "prec_compute_steps": 1, "stat_decay": HYPER["stat_decay"],
        "matrix_eps": HYPER["matrix_eps"], "prec_maxorder": 1200, "prec_bits": 4, "quan_blocksize": 64,
        "rect_t1": 1, "rect_t2": 4, "inv_root_mode": 0})
    times, spent = [], 0.0
    warm = max(1, min(warmup, 2))
    for it in range(warm + steps):
        t0 = time.perf_counter()
        opt.step([g.clone() for g in grads])
        dt = time.perf_counter() - t0
        if it >= warm:
            times.append(dt)
            spent += dt
            if spent > CPU_STEP_BUDGET_S:
                break
    ms = 1e3 * sum(times) / len(times)
    sample = (f"whole workload (all {len(params)} tensors, 226 preconditioner matrices), {len(times)} timed step(s) of {steps} requested "
              f"after {warm} warm-up, {torch.get_num_threads()} threads; CPU port of the reference's step (torch CPU products and QR, C quantizer)")
    return ms, torch.get_num_threads(), sample, len(times), warm, torch


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    ms, cores, sample, steps_run, warm_run, torch = cpu_reference_step(args.steps, args.warmup)
    c1 = cpu_config1(torch)
    line = {"impl": "reference", "metric": METRIC, "value": ms, "unit": "ms/step", "n_gpus": args.gpus,
            "steps": steps_run, "warmup": warm_run, "requested": {"steps": args.steps, "warmup": args.warmup},
            "ms_per_step": ms, "higher_is_better": False, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32 arithmetic on 4-bit state", "data": "synthetic",
            "config": {"workload": WORKLOAD, "gradients": "one bf16-autocast cross-entropy backward on the host, batch 256 of N(0,1) "
                       "224x224 images, uniform labels, seed 0 (computed once, reused every step)",
                       "hyper": {k: (list(v) if isinstance(v, tuple) else v) for k, v in HYPER.items()}},
            "cpu_baseline": {"value": ms, "unit": "ms/step", "cores": cores, "kind": "port", "sample": sample},
            "config1": c1,
            "e2e": {"value": ms, "unit": "ms/step", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def cpu_baseline_subprocess(steps=2, warmup=1, timeout=600):
    """Runs the CPU arm as a separate process (so that the reference's `qtensor` package and this
    package's never meet) and returns its parsed JSON line, or None."""
    env = dict(os.environ)
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "OMP_NUM_THREADS"):
        env.pop(k, None)
    env["CUDA_VISIBLE_DEVICES"] = ""
    try:
        out = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference", "--steps", str(steps),
                              "--warmup", str(warmup)], capture_output=True, text=True, timeout=timeout, env=env)
        for ln in reversed(out.stdout.strip().splitlines()):
            if ln.startswith("{"):
                return json.loads(ln)
    except (subprocess.SubprocessError, ValueError, OSError):
        pass
    return None


# ---------------------------------------------------------------------------------------
# GPU arm.
# ---------------------------------------------------------------------------------------

def quantizer_roofline(torch, lib, device, iters=20):
    """Quantize / dequantize rate on the workload's largest order class (125 matrices of
    order 768, 4-bit diagreal, block 64; 320 MB of fp32 per pass, larger than L2)."""
    import qtensor.functional as F
    n, count, bs = 768, 125, 64
    nb = (n + bs - 1) // bs
    A = torch.randn(count, n, n, device=device)
    packed = torch.empty(count, n * n // 2, dtype=torch.uint8, device=device)
    absmax = torch.empty(count, n * nb, device=device)
    diag = torch.empty(count, n, device=device)
    out = torch.empty_like(A)
    code = F.create_linear_map(True, 4, 2).to(device)
    p = lambda t: ct.c_void_p(t.data_ptr())
    st = ct.c_void_p(torch.cuda.current_stream().cuda_stream)

    def q():
        rc = lib.qt_quantize_blockwise(p(A), 0, n * n, p(code), n, count, p(absmax), n * nb, p(diag), n,
                                       p(packed), n * n // 2, bs, 4, st)
        assert rc == 0

    def d():
        rc = lib.qt_dequantize_blockwise(p(packed), n * n // 2, p(code), n, count, p(absmax), n * nb, p(diag), n,
                                         p(out), 0, n * n, bs, 4, st)
        assert rc == 0

    bytes_per_launch = count * (4 * n * n + n * n // 2 + 4 * n * nb + 4 * n)
    res = {}
    for name, fn in (("quantize", q), ("dequantize", d)):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        res[name] = {"us_per_launch": ms * 1e3, "gbs": bytes_per_launch / ms / 1e6}
    return res, bytes_per_launch, f"{count} matrices of order {n}, 4-bit diagreal, block {bs}"


def gemm_roofline(torch, device, iters=20):
    """tcgen05 product on the step's most common shape: 125 matrices of order 768 (V V^T), operands
    as the optimizer carries them (scaled fp16 plane pairs, 128-k accumulation chains)."""
    from optimizers import _gemm
    n, count = 768, 125
    A = torch.randn(count, n, n, device=device)
    P = _gemm.split(A)
    out = torch.empty(count, n, n, device=device)
    fn = lambda: _gemm.matmul(P, P, trans_b=True, out=out)
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    flops = 2.0 * count * n ** 3
    # context: the vendor library's own bf16 product on the same batched shape (one MMA per product,
    # bf16 accuracy) - what a 768-order batch reaches at all, next to the 8192^3 figure the peak comes from
    Ab = A.bfloat16()
    lib_ms = _time_cuda(torch, lambda: torch.bmm(Ab, Ab.transpose(1, 2)), 3, iters)
    return {"us_per_launch": ms * 1e3, "tflops_algorithmic": flops / ms / 1e9, "tflops_executed": 3 * flops / ms / 1e9,
            "flops_per_launch": flops, "library_bf16_same_shape_tflops": flops / lib_ms / 1e9,
            "case": f"{count} x ({n} x {n}) @ ({n} x {n})^T, scaled fp16 hi/lo planes in, fp32 out"}


def _time_cuda(torch, fn, warmup, iters):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def kernel_sweep(torch, device, orders=(128, 512, 1200, 2048, 4096, 8192), count=64):
    """Kernel sweep of the fused statistics update L <- beta L + (1-beta) G G^T on 4-bit state
    (dequantize and quantize inside the GEMM epilogue) and of the inverse 4th root, 64 matrices
    per order.  G ~ N(0, 1/n) fp32; L = Q diag(lambda) Q^T with lambda log-uniform in [1e-6, 1],
    stored 4-bit diagreal, block 64, beta = 0.95.  One JSON line per order; every working set
    is far larger than L2.  Checks on the way: the fused bytes equal the unfused sequence's."""
    import qtensor.functional as F
    from optimizers import _gemm, matrix_functions as MF
    from optimizers import _engine as E
    hbm_peak, tensor_peak, _, peak_kind = measured_peaks()
    code = F.create_linear_map(True, 4, 2).to(device)
    gen = torch.Generator(device=device).manual_seed(0)
    beta = 0.95
    for n in orders:
        torch.cuda.empty_cache()
        nb = (n + 63) // 64
        Q = torch.linalg.qr(torch.randn(n, n, device=device, generator=gen)).Q
        arena = E.QuantArena(n, count, device, 4, 64, code, 4096, diagreal=True)
        step = max(1, min(count, (1 << 28) // (n * n)))
        for a in range(0, count, step):
            lam = torch.exp(torch.rand(min(step, count - a), n, device=device, generator=gen) * 13.8155 - 13.8155)
            L = (Q.unsqueeze(0) * lam.unsqueeze(1)) @ Q.t()
            arena.quantize(a, a + L.shape[0], (0.5 * (L + L.transpose(1, 2))).contiguous())
        del L, lam
        G = torch.randn(count, n, n, device=device, generator=gen) / n ** 0.5
        st = arena.state(0, count)
        out = tuple(None if t is None else torch.empty_like(t) for t in st)
        iters = 10 if n <= 1200 else 3
        # fused: split G once per update (part of the operation), product + state in the epilogue
        P = _gemm.split(G)
        t_split = _time_cuda(torch, lambda: _gemm.split(G), 1, iters)
        t_fused = _time_cuda(torch, lambda: _gemm.matmul_q4(P, P, code, out, trans_b=True, alpha=1 - beta, beta=beta, old=st),
                             2, iters)
        # unfused sequence with the same kernels: dequantize -> product (fp32 C and D) -> quantize
        want = E.QuantArena(n, count, device, 4, 64, code, 4096, diagreal=True)

        def unfused():
            Lf = arena.dequantize(0, count)
            D, _ = _gemm.matmul(P, P, trans_b=True, alpha=1 - beta, beta=beta, C=Lf, out=Lf)
            want.quantize(0, count, D)
        t_unfused = _time_cuda(torch, unfused, 1, iters)
        same = all(torch.equal(a_, b_) for a_, b_ in zip(out, want.state(0, count)))
        del want
        # inverse 4th root, factor form (functional.py:749-762): rows = kept half of a 4-bit
        # orthogonal factor, 4 Bjorck steps, rows^T diag((S + rho)^-1/4) rows quantized in the epilogue
        fac = E.QuantArena(n, count, device, 4, 64, code, 4096, diagreal=False)
        for a in range(0, count, step):
            fac.quantize(a, min(count, a + step), Q.t().contiguous().unsqueeze(0).expand(min(step, count - a), n, n).contiguous())
        S = torch.exp(torch.rand(count, n // 2, device=device, generator=gen) * 13.8155 - 13.8155)
        prec = E.QuantArena(n, count, device, 4, 64, code, 4096, diagreal=True)

        def factor_root():
            rows = E.Mat(fac.dequantize(0, count)[:, : n // 2, :])
            for _ in range(4):
                rows = E.op_bjorck(rows, want_planes=True)
            w = 1 / (S + 1e-6).pow(0.25)
            scaled = E.Mat(w.unsqueeze(2) * rows.f32)
            _gemm.matmul_q4(rows.planes, scaled.planes, code, prec.state(0, count), trans_a=True)
        t_root = _time_cuda(torch, factor_root, 1, iters)
        del fac, prec
        t_newton = None
        if n <= 4096:                                        # Schur-Newton (matrix_functions.py:80-141) inside the library
            Lf = arena.dequantize(0, count)
            v0 = MF.draw_start_vectors(count, n, device)
            t_newton = _time_cuda(torch, lambda: MF.ComputePower(Lf.clone(), 4, ridge_epsilon=1e-6, v0=v0), 1, 2)
            del Lf
        state_bytes = (n * n) // 2 + 4 * n * nb + 4 * n
        algo_bytes = count * (4 * n * n + 2 * state_bytes)               # read G, read + write the 4-bit state
        flops = 2.0 * count * n ** 3
        line = {"case": "fused statistics update on 4-bit state", "n": n, "matrices": count, "beta": beta,
                "fused_us": t_fused * 1e3, "split_us": t_split * 1e3, "unfused_us": t_unfused * 1e3,
                "fused_equals_unfused_bytes": bool(same),
                "algorithmic_bytes": algo_bytes, "gbs": algo_bytes / (t_fused + t_split) / 1e6,
                "gbs_frac_of_measured_copy": algo_bytes / (t_fused + t_split) / 1e6 / hbm_peak,
                "tflops_algorithmic": flops / t_fused / 1e9, "tflops_executed": 3 * flops / t_fused / 1e9,
                "tensor_frac_of_measured_burst": 3 * flops / t_fused / 1e9 / tensor_peak,
                "operand_planes": "scaled fp16 pairs (22 bits), three MMAs per k-slice, 128-k accumulation chains",
                "peaks": peak_kind, "factor_root_us": t_root * 1e3, "newton_root_us": None if t_newton is None else t_newton * 1e3}
        print(json.dumps(line), flush=True)
        del G, P, arena, out, st


def config1_gpu(torch, lib, device):
    """The 1024 x 1024 configuration on the GPU: one matrix (launch-latency bound: 4.8 MB is under
    a microsecond of HBM traffic) and a batch of 64 such matrices (306 MB per pass, larger than L2)."""
    import qtensor.functional as F
    n, bs = 1024, 64
    nb = n // bs
    code = F.create_linear_map(True, 4, 2).to(device)
    p = lambda t: ct.c_void_p(t.data_ptr())
    st = ct.c_void_p(torch.cuda.current_stream().cuda_stream)
    res = {"case": "1024^2 SPD fp32 (Q diag(lambda) Q^T, lambda log-uniform in [1e-6, 1]), 4-bit linear-2 code, block 64"}
    A1 = config1_matrix(torch, n).to(device)
    for count, tag in ((1, "single"), (64, "batch64")):
        A = A1.unsqueeze(0).expand(count, n, n).contiguous()
        packed = torch.empty(count, n * n // 2, dtype=torch.uint8, device=device)
        absmax = torch.empty(count, n * nb, device=device)
        out = torch.empty_like(A)
        q = lambda: lib.qt_quantize_blockwise(p(A), 0, n * n, p(code), n, count, p(absmax), n * nb, None, 0,
                                              p(packed), n * n // 2, bs, 4, st)
        d = lambda: lib.qt_dequantize_blockwise(p(packed), n * n // 2, p(code), n, count, p(absmax), n * nb, None, 0,
                                                p(out), 0, n * n, bs, 4, st)
        nbytes = count * (4 * n * n + n * n // 2 + 4 * n * nb)
        for name, fn in (("quantize", q), ("dequantize", d)):
            ms = _time_cuda(torch, fn, 3, 50 if count == 1 else 20)
            res[f"{tag}_{name}_us"] = ms * 1e3
            res[f"{tag}_{name}_gbs"] = nbytes / ms / 1e6
    return res


def reference_cuda_quantizer(torch, device):
    """Context figure: the reference's own CUDA quantizer (cudaC_python/csrc, compiled unmodified
    for sm_100a into oracle/_ref/) on the 125 x 768^2 class, one launch per matrix on the legacy
    default stream as the reference does.  It writes a different byte format; only its rate is used."""
    path = os.path.join(ROOT, "oracle", "_ref", "libqtensor_cuda_ref.so")
    if not os.path.isfile(path):
        return None
    try:
        ref = ct.CDLL(path)
        import qtensor.functional as F
        n, count, bs = 768, 125, 64
        nb = n // bs
        A = torch.randn(count, n, n, device=device)
        packed = torch.empty(count, n * n // 2, dtype=torch.uint8, device=device)
        absmax = torch.empty(count, n * nb, device=device)
        out = torch.empty_like(A)
        code = F.create_linear_map(True, 4, 2).to(device)
        vp = lambda t, off=0: ct.c_void_p(t.data_ptr() + off)

        def q():
            for m in range(count):
                ref.cquantize_blockwise_4bit_fp32(vp(A, 4 * m * n * n), vp(code), ct.c_int32(n), vp(absmax, 4 * m * n * nb),
                                                  vp(packed, m * n * n // 2), ct.c_int32(bs))

        def d():
            for m in range(count):
                ref.cdequantize_blockwise_4bit_fp32(vp(packed, m * n * n // 2), vp(code), ct.c_int32(n), vp(absmax, 4 * m * n * nb),
                                                    vp(out, 4 * m * n * n), ct.c_int32(bs))
        nbytes = count * (4 * n * n + n * n // 2 + 4 * n * nb)
        with torch.cuda.stream(torch.cuda.default_stream(device)):
            tq = _time_cuda(torch, q, 2, 5)
            td = _time_cuda(torch, d, 2, 5)
        return {"what": "reference CUDA quantizer compiled for sm_100a, 125 launches per pass (one per matrix)",
                "quantize_gbs": nbytes / tq / 1e6, "dequantize_gbs": nbytes / td / 1e6}
    except Exception as exc:                                  # context only: never fail the bench for it
        return {"unavailable": repr(exc)}


def run_ours(args):
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    use_package()
    import workloads
    from optimizers.shampoo2 import ShampooAdamW
    from qtensor.cextension import get_lib
    lib = get_lib()

    # every rank holds the same model and the same gradients (seed 0 everywhere, as after a
    # data-parallel all-reduce), so parameters - and the checksum below - do not depend on N
    torch.manual_seed(0)
    model = workloads.vit_base_patch32_224().to(device)
    params = [p for p in model.parameters()]
    kwargs = dict(HYPER)
    kwargs["cuda_graph"] = not args.no_graph   # the step is replayed as CUDA graphs (sharded: two, around an eager all-gather)
    if world > 1:
        kwargs["process_group"] = dist.group.WORLD
    opt = ShampooAdamW(params, **kwargs)
    loss = workloads.synthetic_gradients(model, 256, 224, 1000, device, autocast_bf16=True, seed=0)
    grads = [p.grad.detach().clone() for p in params]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        t = torch.tensor([ms], device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- kernel-level: device-resident inputs ------------------------------------------
    for _ in range(args.warmup):
        opt.step()
    barrier()
    launches0 = lib.qt_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        e0.record()
        for _ in range(args.steps):
            opt.step()
        e1.record()
        barrier()
    launches = lib.qt_launch_count() - launches0
    ms_step = max_over_ranks(e0.elapsed_time(e1)) / args.steps
    # sharded == single: the same number for every N (all ranks hold identical parameters)
    checksum = float(sum(p.detach().double().sum() for p in params))

    # ---- end to end: this rank's gradients arrive from pinned host memory, a scalar goes back.
    # A rank reads the gradients of the parameters whose preconditioners it owns and of those that
    # have none; the directions of the others reach it through the all-gather.
    # The loop is the one a training script would write around optimizer.step(): the gradients of
    # step i+1 are uploaded on a copy stream into the second of two device buffers while step i
    # computes (all K uploads lie inside the timed region; the first one is not overlapped with
    # anything), p.grad is pointed at the buffer that just arrived, and every step's scalar is
    # copied to pinned host memory and read by the host one step later (all K reads inside the
    # timed region too); events order the reuse of the buffers.
    consumed = opt.consumed_params()
    idx = [k for k, p in enumerate(params) if p in consumed]
    host = [torch.empty(grads[k].shape, dtype=grads[k].dtype).pin_memory() for k in idx]
    for h, k in zip(host, idx):
        h.copy_(grads[k])
    grad_bytes = sum(h.numel() * h.element_size() for h in host)
    bufs = [[torch.empty_like(grads[k]) for k in idx] for _ in range(2)]
    arrived = [torch.cuda.Event(), torch.cuda.Event()]
    copy_stream = torch.cuda.Stream(device)
    user_grads = {k: params[k].grad for k in idx}

    def upload(slot):
        with torch.cuda.stream(copy_stream):
            for h, b in zip(host, bufs[slot]):
                b.copy_(h, non_blocking=True)
            arrived[slot].record(copy_stream)

    barrier()
    copy_stream.wait_stream(torch.cuda.current_stream())
    main = torch.cuda.current_stream()
    consumed = [torch.cuda.Event(), torch.cuda.Event()]           # step i has finished with gradient buffer i & 1
    back_host = [torch.zeros((), dtype=torch.float32).pin_memory() for _ in range(2)]
    back_done = [torch.cuda.Event(), torch.cuda.Event()]
    backs = []
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    upload(0)
    for i in range(args.steps):
        if i + 1 < args.steps:
            if i >= 1:
                copy_stream.wait_event(consumed[(i + 1) & 1])      # its last reader was step i-1
            upload((i + 1) & 1)
        main.wait_event(arrived[i & 1])
        for k, b in zip(idx, bufs[i & 1]):
            params[k].grad = b
        opt.step()
        consumed[i & 1].record(main)
        # the step's scalar goes to pinned host memory asynchronously and is read one step later,
        # so the host enqueues step i+1 while step i runs (a logging loop, not a blocking read)
        back_host[i & 1].copy_(params[-1].detach().float().sum(), non_blocking=True)
        back_done[i & 1].record(main)
        if i >= 1:
            back_done[(i - 1) & 1].synchronize()
            backs.append(float(back_host[(i - 1) & 1]))
    back_done[(args.steps - 1) & 1].synchronize()
    backs.append(float(back_host[(args.steps - 1) & 1]))
    e3.record()
    barrier()
    assert len(backs) == args.steps
    for k in idx:
        params[k].grad = user_grads[k]
    e2e_ms = max_over_ranks(e2.elapsed_time(e3)) / args.steps
    gb = torch.tensor([float(grad_bytes), float(grad_bytes)], device=device)
    if world > 1:
        dist.all_reduce(gb[0:1], op=dist.ReduceOp.SUM)
        dist.all_reduce(gb[1:2], op=dist.ReduceOp.MAX)
    h2d_total, h2d_max = int(gb[0].item()), int(gb[1].item())

    # ---- steady-state step: no interval fires (the common step at T1=100, T2=500): only the
    # preconditioned direction P_L G P_R, grafting, the exchange and the AdamW tail run
    for g in opt.param_groups:
        g['stat_compute_steps'] = g['prec_compute_steps'] = 10 ** 9
    for _ in range(2):
        opt.step()
    barrier()
    e4, e5 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e4.record()
    for _ in range(args.steps):
        opt.step()
    e5.record()
    barrier()
    steady_ms = max_over_ranks(e4.elapsed_time(e5)) / args.steps
    opt._check_device_error()                                 # a bounded wait that ran out would have voided the numbers

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    hbm_peak, tf_burst, tf_sustained, peak_kind = measured_peaks()
    qres, qbytes, qdesc = quantizer_roofline(torch, lib, device)
    gres = gemm_roofline(torch, device)
    step_flops = step_algorithmic_flops([tuple(p.shape) for p in params])
    # dominant kernel of the step: the tcgen05 product, timed alone -> burst peak.  `achieved`
    # counts algorithmic flops (2 M N K per product); the kernel executes three bf16 MMAs per
    # product (hi*hi + hi*lo + lo*hi), so the tensor pipe runs at 3x that rate (`executed`).
    roof = {"bound": "tensor", "kernel": "k_gemm_bf16x3 (tcgen05 kind::f16 on scaled fp16 plane pairs: hi*hi + hi*lo + lo*hi, fp32 accumulate in TMEM)",
            "achieved": gres["tflops_algorithmic"], "peak": tf_burst, "unit": "TFLOP/s",
            "frac": gres["tflops_algorithmic"] / tf_burst, "peak_kind": f"of {peak_kind} (burst bf16: the kernel is timed alone)",
            "executed": gres["tflops_executed"], "frac_executed": gres["tflops_executed"] / tf_burst,
            "emulation_factor": 3, "traffic": ncu_traffic("k_gemm_bf16x3"),
            "flops_per_launch": gres["flops_per_launch"], "case": gres["case"],
            "us_per_launch": gres["us_per_launch"],
            "library_bf16_same_shape": {"tflops": gres["library_bf16_same_shape_tflops"],
                                        "executed_over_library": gres["tflops_executed"] / gres["library_bf16_same_shape_tflops"],
                                        "what": "torch.bmm on bf16 copies of the same 125 x 768^3 batch (bf16 accuracy, one MMA per product)"},
            "step": {"algorithmic_flops": step_flops, "achieved": step_flops / ms_step / 1e9 / world, "unit": "TFLOP/s per GPU",
                     "peak": tf_sustained, "frac": step_flops / ms_step / 1e9 / world / tf_sustained,
                     "peak_kind": f"of {peak_kind} (sustained bf16: timed inside the whole step)",
                     "counting": "17 n^3 of products + 8/3 n^3 of QR per preconditioner matrix, 4 (m^2 k + m k^2) per gradient block"},
            "quantize": {"bound": "hbm", "achieved": qres["quantize"]["gbs"], "peak": hbm_peak, "unit": "GB/s",
                         "frac": qres["quantize"]["gbs"] / hbm_peak, "frac_of_nominal_8000": qres["quantize"]["gbs"] / 8000.0,
                         "bytes_per_launch": qbytes, "case": qdesc, "traffic": ncu_traffic("k_quantize_vec")},
            "dequantize": {"bound": "hbm", "achieved": qres["dequantize"]["gbs"], "peak": hbm_peak, "unit": "GB/s",
                           "frac": qres["dequantize"]["gbs"] / hbm_peak, "frac_of_nominal_8000": qres["dequantize"]["gbs"] / 8000.0,
                           "bytes_per_launch": qbytes, "case": qdesc, "traffic": ncu_traffic("k_dequantize_vec")}}
    line = {"metric": METRIC, "value": ms_step, "unit": "ms/step", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": False, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32 arithmetic on 4-bit state", "data": "synthetic",
            "config": {"workload": WORKLOAD, "gradients": "one bf16-autocast cross-entropy backward, batch 256 of "
                       "N(0,1) 224x224 images, uniform labels, seed 0 on every rank (computed once, reused every step)",
                       "execution": "eager" if args.no_graph else ("whole step captured once per schedule phase and replayed as a CUDA graph (ShampooAdamW(cuda_graph=True))" if world == 1 else "CUDA graphs per schedule phase around the NCCL exchange (ShampooAdamW(cuda_graph=True))"),
                       "l2": "per-step working set (4-bit state 130 MB + fp32 temporaries > 2 GB) exceeds the 126 MB L2",
                       "hyper": {k: (list(v) if isinstance(v, tuple) else v) for k, v in HYPER.items()}},
            "clocks": clocks.summary(),
            "e2e": {"value": e2e_ms, "unit": "ms/step", "h2d_bytes_per_step": h2d_total, "h2d_bytes_per_step_rank_max": h2d_max,
                    "d2h_bytes_per_step": 4 * world,
                    "loop": "gradients of step i+1 uploaded from pinned host memory on a copy stream while step i computes "
                            "(two device buffers, p.grad re-pointed every step); each step's 4-byte result copied to pinned host memory and read one step later; "
                            "every upload and every read-back inside the timed region"},
            "gpu_launches": int(launches),
            "steady_state_step": {"value": steady_ms, "unit": "ms/step",
                                  "what": "same optimizer with no interval firing (apply + grafting + AdamW tail only)"},
            "param_checksum": checksum,
            "quant_gbs": qres["quantize"]["gbs"], "dequant_gbs": qres["dequantize"]["gbs"],
            "roofline": roof, "config1": config1_gpu(torch, lib, device), "loss": loss}
    refq = reference_cuda_quantizer(torch, device)
    if refq is not None:
        line["reference_gpu_quantizer"] = refq
    if world == 1 and not args.no_cpu_baseline:
        ref = cpu_baseline_subprocess()
        if ref is not None:
            line["cpu_baseline"] = ref["cpu_baseline"]
            line["config1"]["cpu"] = ref.get("config1")
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-graph", action="store_true", help="run the step eagerly instead of as a captured CUDA graph")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU leg of the N=1 run")
    ap.add_argument("--sweep", action="store_true",
                    help="kernel sweep of the fused 4-bit statistics update and the inverse 4th root over orders 128..8192")
    ap.add_argument("--sweep-orders", default="128,512,1200,2048,4096,8192")
    ap.add_argument("--profile-case", default=None, choices=["quant", "gemm", "step", "panel"],
                    help="run only one small kernel case (for an ncu capture) and print its rates")
    args = ap.parse_args()
    if args.impl != "reference":
        use_package()
    if args.sweep:
        import torch
        from qtensor.cextension import get_lib
        get_lib()
        kernel_sweep(torch, torch.device("cuda", 0), orders=tuple(int(x) for x in args.sweep_orders.split(",")))
        return
    if args.profile_case == "quant":
        import torch
        from qtensor.cextension import get_lib
        res, nbytes, desc = quantizer_roofline(torch, get_lib(), torch.device("cuda", 0), iters=3)
        print(json.dumps({"case": desc, "bytes_per_launch": nbytes, **res}))
        return
    if args.profile_case == "step":
        # one eager optimizer step between cudaProfilerStart/Stop, for a launch list:
        #   ncu --profile-from-start off --metrics gpu__time_duration.sum --clock-control none --csv ...
        import torch
        import workloads
        from optimizers.shampoo2 import ShampooAdamW
        device = torch.device("cuda", 0)
        torch.manual_seed(0)
        model = workloads.vit_base_patch32_224().to(device)
        opt = ShampooAdamW(list(model.parameters()), **HYPER)
        workloads.synthetic_gradients(model, 256, 224, 1000, device, autocast_bf16=True, seed=0)
        for _ in range(3):
            opt.step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.profiler.start()
        e0.record()
        opt.step()
        e1.record()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        print(json.dumps({"case": "one eager ShampooAdamW.step(), ViT-B/32, T1=T2=1", "ms": e0.elapsed_time(e1)}))
        return
    if args.profile_case == "panel":
        # four launches of the QR panel kernel (8 matrices of order 1200: panels of 96 and of 1008 rows)
        import torch
        from qtensor.cextension import get_lib
        lib = get_lib()
        n, count = 1200, 8
        A = torch.randn(count, n, n, device="cuda")
        V = torch.zeros_like(A)
        T = torch.zeros(count, 32, 32, device="cuda")
        p = lambda t: ct.c_void_p(t.data_ptr())
        st = ct.c_void_p(torch.cuda.current_stream().cuda_stream)
        times = {}
        for j0 in (1104, 192):
            fn = lambda: lib.qt_householder_panel_fused(p(A), n * n, n, count, j0, 32, p(V), n * n, p(T), 1024, 0, None,
                                                        min(n, (j0 // 128) * 128 + 128), st)
            times[f"rows_{n - j0}_us"] = _time_cuda(torch, fn, 1, 2) * 1e3
        print(json.dumps({"case": "k_householder_panel, 8 x 1200^2, 32-column panels", **times}))
        return
    if args.profile_case == "gemm":
        import torch
        from qtensor.cextension import get_lib
        get_lib()
        print(json.dumps(gemm_roofline(torch, torch.device("cuda", 0), iters=3)))
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
