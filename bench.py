#!/usr/bin/env python
"""Benchmark of the reproducible operator backend.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload W]

Headline workload (default): the bit-exact fp32 product of two 16384 x 16384 matrices drawn
U[-1,1) from seed 4, A partitioned by rows over the N GPUs and C all-gathered, so that every rank
ends with the full product.  A "step" is one such product.  One JSON line is printed by rank 0.

  value      whole-job GFLOP/s (2 M N K per step) with operands resident in HBM
  e2e        the same with HOST operands: pinned A panel and B copied in, C panel copied out,
             every step, inside the timed region
  roofline   the GEMM kernel against the FP32 FMA-pipe peak measured on this GPU by a pure-FFMA
             probe kernel (tensor cores are not used: their accumulation order is not bit-specified)
  cpu_baseline  the reference's own CPU backend on a bounded sample of rows, timed on the host cores
  extra      (N = 1 only) the HBM-bound kernels of the same backend: exp/log/div/sqrt over 2^28
             elements and the fixed-order sums, each with its own roofline against measured HBM

`--impl reference` times the reference's CPU backend alone (rank 0 only) on a bounded row sample.
"""
import argparse
import hashlib
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def _reference_arm_requested(argv):
    for i, a in enumerate(argv):
        if a == "--impl" and i + 1 < len(argv) and argv[i + 1] == "reference":
            return True
        if a == "--impl=reference":
            return True
    return False


if _reference_arm_requested(sys.argv):
    # The reference arm is the reference's OpenMP loop on the host cores.  Only rank 0 runs it, and
    # it must get every core: torch.distributed.run exports OMP_NUM_THREADS=1 to its workers, and
    # both OpenMP runtimes (torch's and the libgomp the reference extension links) read the
    # variable when they are loaded, i.e. before `import torch`.
    if int(os.environ.get("RANK", "0")) != 0:
        sys.exit(0)
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)

import torch  # noqa: E402


def env_int(name, default):
    return int(os.environ.get(name, default))


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0])), mx.append(float(r[1])), pw.append(float(r[2]))
            except ValueError:
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "samples": len(sm),
                "reasons": sorted(reasons)}


def event_ms(fn, stream=None):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    fn()
    e1.record(stream)
    e1.synchronize()
    return e0.elapsed_time(e1)


def ffma_peak_tflops(fp64=False):
    """FP32 (or FP64) FMA-pipe peak of the current GPU from the library's probe kernel."""
    import ctypes
    from repdl_b200._cabi import check
    from repdl_b200.build import PROBE_LIB
    lib = ctypes.CDLL(PROBE_LIB)  # the probe kernel is a benchmark helper, not part of the operator ABI
    lib.repdl_b200_probe_fma.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                                         ctypes.POINTER(ctypes.c_double), ctypes.c_void_p]
    out = torch.zeros(4, dtype=torch.float64, device="cuda")
    flops = ctypes.c_double(0)
    iters = 1 << (14 if fp64 else 16)

    def run():
        check(lib.repdl_b200_probe_fma(int(fp64), iters, 8, out.data_ptr(), ctypes.byref(flops), None),
              "probe")
    run()
    torch.cuda.synchronize()
    best = min(event_ms(run) for _ in range(5))
    return flops.value / best / 1e9


def load_reference_cpu():
    """The reference's CPU backend built into oracle/_ref (preferred), else the C oracle port."""
    import oracle
    ref = oracle.ref()
    if ref is not None:
        return "reference", ref.cpu.mm, torch.get_num_threads()
    return "port", lambda a, b, ta, tb: oracle.mm(a, b, ta, tb), oracle.num_threads()


def cpu_side(op, x, bytes_per_element):
    """The reference's CPU path for one of the streaming operators, timed on the host cores on the
    sample x (a CPU tensor): its own backend where oracle/_ref is built, else the C oracle port."""
    import oracle
    ref = oracle.ref()
    if ref is not None:
        kind, cores = "reference", torch.get_num_threads()
        fns = {"div10": lambda t: t.div(10.0),                                      # repdl/ops.py:98-103
               "sqrt": lambda t: t.to(torch.float64).sqrt().to(torch.float32),      # repdl/ops.py:122-123
               "exp": lambda t: ref.math.exp2d(t.view(1, -1)),
               "log": lambda t: ref.math.log1d(t),
               "sum_rows": lambda t: ref.cpu.sum2d_dim1(t, False, False),
               "sum1d": lambda t: ref.cpu.sum1d(t, False)}
    else:
        kind, cores = "port", oracle.num_threads()
        fns = {"div10": lambda t: oracle.div(t, 10.0), "sqrt": oracle.sqrt, "exp": oracle.exp,
               "log": oracle.log, "sum_rows": oracle.sum2d_dim1, "sum1d": oracle.sum1d}
    fn = fns[op]
    fn(x)
    t0 = time.perf_counter()
    fn(x)
    dt = time.perf_counter() - t0
    return {"value": bytes_per_element * x.numel() / dt / 1e9, "unit": "GB/s",
            "cores": 1 if op == "sum1d" else cores, "kind": kind,
            "sample": "%d elements (%.0f ms)" % (x.numel(), dt * 1e3)}


def time_cpu_mm(a, b, budget_s, rows0=4):
    """Times the CPU mm on the first rows of A; grows the sample until it fills the budget."""
    kind, fn, cores = load_reference_cpu()
    K, N = b.shape
    rows = rows0
    t = time.perf_counter()
    fn(a[:rows].contiguous(), b, False, False)
    dt = time.perf_counter() - t
    want = int(max(rows, min(a.shape[0], rows * budget_s / max(dt, 1e-3))))
    want = max(rows0, (want // rows0) * rows0)
    if want > rows * 2:
        rows = want
        t = time.perf_counter()
        fn(a[:rows].contiguous(), b, False, False)
        dt = time.perf_counter() - t
    gflops = 2.0 * rows * N * K / dt / 1e9
    return {"value": gflops, "unit": "GFLOP/s", "cores": cores, "kind": kind,
            "sample": "first %d of %d rows of A times the full B (%.1f s)" % (rows, a.shape[0], dt)}


def run_reference(args, rank):
    """--impl reference: the reference's own CPU implementation of the path, rank 0 only.  Each step
    multiplies a fixed sample of rows of A with the full B; the sample is shrunk, if need be, so that
    the whole run of warm-up and timed steps stays within --ref-budget seconds."""
    if rank != 0:
        return
    from repdl_b200 import workloads
    n = args.size
    a, b = workloads.mm_large(n, 4)
    kind, fn, cores = load_reference_cpu()
    torch.set_num_threads(os.cpu_count() or 1)
    cores = max(cores, torch.get_num_threads())
    # one probe row block decides how many rows a step can afford
    probe = min(4, args.ref_rows)
    t = time.perf_counter()
    fn(a[:probe].contiguous(), b, False, False)
    per_row = (time.perf_counter() - t) / probe
    calls = args.steps + args.warmup
    rows = int(max(1, min(args.ref_rows, args.ref_budget / max(calls, 1) / max(per_row, 1e-6))))
    sample = a[:rows].contiguous()
    for _ in range(args.warmup):
        fn(sample, b, False, False)
    t = time.perf_counter()
    for _ in range(args.steps):
        fn(sample, b, False, False)
    dt = time.perf_counter() - t
    gflops = 2.0 * rows * n * n * args.steps / dt / 1e9
    line = {
        "impl": "reference", "metric": "bit-exact fp32 mm GFLOP/s", "value": gflops,
        "unit": "GFLOP/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "mm M=N=K=%d (config 5), reference CPU backend on a row sample" % n,
                   "sample_rows": rows},
        "cpu_baseline": {"value": gflops, "unit": "GFLOP/s", "cores": cores, "kind": kind,
                         "sample": "each step = first %d of %d rows of A times the full B" % (rows, n)},
        "e2e": {"value": gflops, "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def sum1d_walk_stats(flat):
    """What the serial part of the chain sum had to do (the walker's counters, read back from the
    scratch buffer of one extra call)."""
    import ctypes
    from repdl_b200._cabi import check, lib
    nb = lib.repdl_b200_sum1d_scratch_bytes(flat.numel())
    if nb == 0:
        return None
    sc = torch.empty(nb, dtype=torch.uint8, device=flat.device)
    o = torch.zeros((), device=flat.device)
    check(lib.repdl_b200_sum1d(flat.data_ptr(), o.data_ptr(), flat.numel(), 1.0, sc.data_ptr(), nb, None), "sum1d")
    torch.cuda.synchronize()
    st = (ctypes.c_longlong * 12)()
    check(lib.repdl_b200_sum1d_stats(sc.data_ptr(), st), "sum1d_stats")
    names = ["items", "summaries_applied", "leaves_walked", "spans_walked", "leaves_in_spans",
             "soft_runs_not_valid", "robust_runs_not_valid"]
    return dict(zip(names, list(st)[:7]), scratch_bytes=nb)


def flush_l2(scratch):
    """Evicts the 126 MB L2 between timed iterations of a workload that would otherwise fit in it."""
    scratch.add_(1.0)


def extras_mm(peak_tflops):
    """Config 1 (M = N = K = 1024, seed 0) and a mid size (4096), each launch timed on its own with
    CUDA events.  Config 1's operands and result are 12 MiB and fit the L2, so the L2 is flushed
    between timed launches (a 256 MiB buffer is rewritten); the L2-warm time is reported next to it."""
    from repdl_b200 import ops, workloads
    import oracle
    out = {}
    gold_path = os.path.join(ROOT, "tests", "golden", "configs.json")
    gold = json.load(open(gold_path)) if os.path.exists(gold_path) else None
    scratch = torch.zeros(64 << 20, device="cuda")  # 256 MiB
    for n, seed, name in ((1024, 0, "mm 1024^3 (config 1)"), (4096, 0, "mm 4096^3")):
        a, b = workloads.mm_square(n, seed)
        ad, bd = a.cuda(), b.cuda()
        for _ in range(3):
            c = ops.mm(ad, bd)
        torch.cuda.synchronize()
        cold = []
        for _ in range(7):
            flush_l2(scratch)
            cold.append(event_ms(lambda: ops.mm(ad, bd)))
        warm = min(event_ms(lambda: ops.mm(ad, bd)) for _ in range(5))
        cold.sort()
        ms = cold[len(cold) // 2]
        tf = 2.0 * n ** 3 / ms / 1e9
        rec = {"ms": ms, "ms_l2_warm": warm, "TFLOP/s": tf, "frac_of_ffma_peak": tf / peak_tflops,
               "frac_of_nominal": tf / (148 * 128 * 2 * 1.965e9 / 1e12),
               "l2": "flushed between timed launches" if n == 1024 else "operands (192 MiB) exceed L2; also flushed"}
        if n == 1024 and gold:
            rec["sha256_equal_reference_cpu"] = (
                hashlib.sha256(c.cpu().numpy().tobytes()).hexdigest() == gold["c1_mm_1024"]["sha256"])
        if n == 4096:
            rows = 32  # the CPU oracle on a row sample (the whole product would take half a minute)
            rec["rows_0_32_equal_oracle"] = bool(torch.equal(
                c[:rows].cpu().view(torch.int32), oracle.mm(a[:rows].contiguous(), b).view(torch.int32)))
        out[name] = rec
        del ad, bd, c
    return out


def extras_sum1d_full(hbm_peak, peak_kind, steps=5, warmup=3):
    """Config 3's 1-D case at its full size: ONE chain over 2^30 elements (4 GiB)."""
    from repdl_b200 import ops, workloads
    n = 1 << 30
    x = torch.empty(n, device="cuda")
    o = 0
    for c in workloads.sum_chunks(n, 2):
        x[o:o + c.numel()] = c.cuda()
        o += c.numel()
    for _ in range(warmup):
        y = ops.sum1d(x)
    torch.cuda.synchronize()
    ms = min(event_ms(lambda: ops.sum1d(x)) for _ in range(steps))
    rec = {"ms": ms, "GB/s": 4.0 * n / ms / 1e6, "frac_of_%s_hbm" % peak_kind: 4.0 * n / ms / 1e6 / hbm_peak,
           "elements": n, "walk": sum1d_walk_stats(x)}
    gold_path = os.path.join(ROOT, "tests", "golden", "configs.json")
    if os.path.exists(gold_path):
        want = json.load(open(gold_path))["c3_sum1d_2p30"]["result_hex"]
        rec["bits_equal_reference_cpu"] = ("%08x" % (y.cpu().view(torch.int32).item() & 0xFFFFFFFF)) == want
    del x
    torch.cuda.empty_cache()
    return rec


def reference_cuda_bench():
    """The reference's OWN CUDA backend (backend/cuda/*, compiled unmodified for sm_100a into
    oracle/_ref by oracle/build_ref.sh) on the same inputs, timed with CUDA events: the existing GPU
    kernels this repository replaces.  Every result is also compared with the CPU backend's bits
    (golden hashes, or this repository's result where that has just been checked against them).
    Returns None where the reference is not built."""
    import glob
    import importlib.util
    import oracle
    from repdl_b200 import ops, workloads
    site = oracle.ref_site()
    cands = glob.glob(os.path.join(site, "repdl", "backend", "cuda*.so")) if site else []
    if not cands:
        return None
    spec = importlib.util.spec_from_file_location("cuda", cands[0])
    rc = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(rc)
    rmath = None
    mpath = os.path.join(ROOT, "oracle", "_ref", "refmath_cuda.so")
    if os.path.exists(mpath):
        spec = importlib.util.spec_from_file_location("refmath_cuda", mpath)
        rmath = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(rmath)
    gold_path = os.path.join(ROOT, "tests", "golden", "configs.json")
    gold = json.load(open(gold_path)) if os.path.exists(gold_path) else {}
    out = {}

    def timed(fn, reps=3):
        y = fn()
        torch.cuda.synchronize()
        return min(event_ms(fn) for _ in range(reps)), y

    def sha(t):
        return hashlib.sha256(t.cpu().numpy().tobytes()).hexdigest()

    def same(a, b):
        return bool(torch.equal(a.cpu().contiguous().view(torch.int32), b.cpu().contiguous().view(torch.int32)))

    try:
        # mm: config 1 and config 5
        a, b = workloads.mm_square(1024, 0)
        ad, bd = a.cuda(), b.cuda()
        ms, y = timed(lambda: rc.mm(ad, bd, False, False))
        out["mm 1024^3"] = {"ms": ms, "TFLOP/s": 2.0 * 1024 ** 3 / ms / 1e9,
                            "equal_reference_cpu": sha(y) == gold.get("c1_mm_1024", {}).get("sha256")}
        a, b = workloads.mm_large(16384, 4)
        ad, bd = a.cuda(), b.cuda()
        del a, b
        ms, y = timed(lambda: rc.mm(ad, bd, False, False), reps=1)
        g5 = os.path.join(ROOT, "tests", "golden", "mm16k.json")
        out["mm 16384^3"] = {"ms": ms, "TFLOP/s": 2.0 * 16384 ** 3 / ms / 1e9,
                             "equal_reference_cpu": os.path.exists(g5) and sha(y) == json.load(open(g5))["sha256"]}
        del ad, bd, y
        torch.cuda.empty_cache()
        # the three convolutions at the shapes of config 4 (second layer: the expensive one)
        g = torch.Generator().manual_seed(3)
        x = torch.rand(256, 32, 26, 26, generator=g).cuda()
        k = (torch.rand(64, 32, 3, 3, generator=g) - 0.5).cuda()
        go = (torch.rand(256, 64, 24, 24, generator=g) - 0.5).cuda()
        ms, y = timed(lambda: rc.conv2d(x, k, 1, 1, 0, 0, 1))
        out["conv2d [256,32,26,26]*[64,32,3,3]"] = {"ms": ms, "equal_this_repo": same(y, ops.conv2d(x, k, (1, 1), (0, 0), 1))}
        ms, y = timed(lambda: rc.conv2d_grad_input(go, k, 26, 26, 1, 1, 0, 0))
        out["conv2d_grad_input"] = {"ms": ms, "equal_this_repo": same(y, ops.conv2d_grad_input((256, 32, 26, 26), k, go, (1, 1), (0, 0)))}
        ms, y = timed(lambda: rc.conv2d_grad_kernel(go, x, 3, 3, 1, 1, 0, 0), reps=1)
        out["conv2d_grad_kernel"] = {"ms": ms, "equal_this_repo": same(y, ops.conv2d_grad_kernel(x, (64, 32, 3, 3), go, (1, 1), (0, 0)))}
        del x, k, go
        # row sums of config 3
        r = workloads.sum_rows(65536, 4096, 2).cuda()
        ms, y = timed(lambda: rc.sum2d_dim1(r, False, False))
        out["sum rows [65536,4096]"] = {"ms": ms, "GB/s": 4.0 * r.numel() / ms / 1e6,
                                        "equal_reference_cpu": sha(y) == gold.get("c3_sum_rows_65536x4096", {}).get("sha256")}
        # its one-chain sum: a single CTA walks the array, so only a short chain is timed (2^22 elements)
        flat = r.view(-1)[:1 << 22].contiguous()
        ms, y = timed(lambda: rc.sum1d(flat, False), reps=1)
        out["sum1d chain [4194304]"] = {"ms": ms, "GB/s": 4.0 * flat.numel() / ms / 1e6,
                                        "equal_this_repo": same(y, ops.sum1d(flat))}
        del r, flat
        torch.cuda.empty_cache()
        if rmath is not None:
            n = 1 << 28
            xs = torch.cat(list(workloads.crmath_chunks(n, 1)))
            xd, xad = xs.cuda(), xs.abs().cuda()
            del xs
            ms, y = timed(lambda: rmath.exp2d(xd.view(16384, 16384)))
            out["exp(x) 2^28"] = {"ms": ms, "GB/s": 8.0 * n / ms / 1e6,
                                  "equal_reference_cpu": sha(y) == gold.get("c2_crmath_2p28", {}).get("whole", {}).get("exp")}
            ms, y = timed(lambda: rmath.log1d(xad))
            out["log(|x|) 2^28"] = {"ms": ms, "GB/s": 8.0 * n / ms / 1e6,
                                    "equal_reference_cpu": sha(y) == gold.get("c2_crmath_2p28", {}).get("whole", {}).get("log_abs")}
            del xd, xad, y
    except Exception as e:  # a report next to the measurement, never part of it
        out["error"] = repr(e)[:300]
    torch.cuda.empty_cache()
    return out


def extras_hbm(hbm_peak, peak_kind, n=1 << 28, which="all", steps=5, warmup=3):
    """The HBM-bound kernels (configs 2 and 3) with their own rooflines, on one GPU.  At the full
    size (2^28 elements) the outputs are also hashed and compared with the reference's hashes."""
    from repdl_b200 import ops, workloads
    out = {}
    gold_path = os.path.join(ROOT, "tests", "golden", "configs.json")
    gold = json.load(open(gold_path)) if (os.path.exists(gold_path) and n == 1 << 28) else None

    def measure(fn):
        # Three launches back to back between the events, divided by three: the host-side cost of a
        # call (about 10 us of Python before a 0.4 ms kernel starts on an idle GPU) then overlaps the
        # previous launch instead of being timed as GPU time.  Every launch streams its operands from
        # HBM again: they are far larger than the L2.
        for _ in range(warmup):
            y = fn()
        torch.cuda.synchronize()

        def thrice():
            fn(), fn(), fn()
        return min(event_ms(thrice) for _ in range(steps)) / 3.0, y

    if which in ("all", "crmath"):
        x = torch.cat(list(workloads.crmath_chunks(n, 1)))
        xa = x.abs()  # on the CPU: torch's CUDA abs() would canonicalise NaN payloads
        xd, xad = x.cuda(), xa.cuda()
        cs = min(n, 1 << 24)  # CPU sample: the first 2^24 elements
        cpu = {"div(x,10)": cpu_side("div10", x[:cs].clone(), 8), "sqrt(|x|)": cpu_side("sqrt", xa[:cs].clone(), 8),
               "exp(x)": cpu_side("exp", x[:cs].clone(), 8), "log(|x|)": cpu_side("log", xa[:cs].clone(), 8)}
        del x, xa
        for name, fn, key in (("div(x,10)", lambda: ops.div(xd, 10.0), "div10"),
                              ("sqrt(|x|)", lambda: ops.sqrt(xad), "sqrt_abs"),
                              ("exp(x)", lambda: ops.exp(xd), "exp"),
                              ("log(|x|)", lambda: ops.log(xad), "log_abs")):
            ms, y = measure(fn)
            rec = {"ms": ms, "GB/s": 8.0 * n / ms / 1e6,
                   "frac_of_%s_hbm" % peak_kind: 8.0 * n / ms / 1e6 / hbm_peak, "elements": n,
                   "cpu_baseline": cpu[name]}
            if gold:
                rec["sha256_equal_reference_cpu"] = (
                    hashlib.sha256(y.cpu().numpy().tobytes()).hexdigest()
                    == gold["c2_crmath_2p28"]["whole"][key])
            out[name] = rec
            del y
        del xd, xad
        torch.cuda.empty_cache()
    if which in ("all", "sums"):
        # rows x 4096 matrix from the first n elements of the config-3 stream
        rows = n // 4096
        r_cpu = torch.cat(list(workloads.sum_chunks(rows * 4096, 2))).view(rows, 4096)
        crows = min(rows, 4096)  # CPU sample: the first 2^24 elements
        cpu_rows = cpu_side("sum_rows", r_cpu[:crows].clone(), 4)
        cpu_chain = cpu_side("sum1d", r_cpu[:crows].clone().view(-1), 4)
        r = r_cpu.cuda()
        del r_cpu
        ms, y = measure(lambda: ops.sum2d_dim1(r))
        rec = {"ms": ms, "GB/s": 4.0 * r.numel() / ms / 1e6,
               "frac_of_%s_hbm" % peak_kind: 4.0 * r.numel() / ms / 1e6 / hbm_peak,
               "cpu_baseline": cpu_rows}
        if gold:
            rec["sha256_equal_reference_cpu"] = (hashlib.sha256(y.cpu().numpy().tobytes()).hexdigest()
                                                 == gold["c3_sum_rows_65536x4096"]["sha256"])
        out["sum rows [%d,4096]" % rows] = rec
        # the same elements as ONE chain (config 3's 1-D case is this stream continued to 2^30)
        flat = r.view(-1)
        ms, y = measure(lambda: ops.sum1d(flat))
        rec = {"ms": ms, "GB/s": 4.0 * flat.numel() / ms / 1e6,
               "frac_of_%s_hbm" % peak_kind: 4.0 * flat.numel() / ms / 1e6 / hbm_peak,
               "elements": flat.numel(), "cpu_baseline": cpu_chain}
        if gold and flat.numel() % (1 << 24) == 0:
            want = gold["c3_sum1d_2p30"]["state_after_chunk_hex"][flat.numel() // (1 << 24) - 1]
            rec["bits_equal_reference_cpu"] = (
                "%08x" % (y.cpu().view(torch.int32).item() & 0xFFFFFFFF)) == want
        rec["walk"] = sum1d_walk_stats(flat)
        out["sum1d chain [%d]" % flat.numel()] = rec
    return out


def cnn_step_bench(steps, warmup):
    """Config 4: conv-relu-conv-relu-maxpool-flatten-linear-relu-linear-cross-entropy, batch 256, SGD
    lr 0.01, same batch every step.  Reports ms per training step and checks the parameter hashes
    of the first steps against the reference's CPU run."""
    from repdl_b200 import nn as rnn
    from repdl_b200 import workloads
    torch.manual_seed(3)
    # (the two ReLU modules behind the convolutions are folded into the convolutions' epilogues: same bits)
    model = rnn.from_torch_module(workloads.cnn_torch_model(), fuse_relu=True)
    x, y = workloads.cnn_batch(256)
    model, x, y = model.cuda(), x.cuda(), y.cuda()
    loss_fn = rnn.CrossEntropyLoss()

    def phash():
        h = hashlib.sha256()
        for p in model.parameters():
            h.update(p.data.cpu().numpy().tobytes())
        return h.hexdigest()

    from repdl_b200 import optim
    sgd = optim.SGD(model.parameters(), lr=0.01)  # one multi-tensor launch: p += g * -lr, two roundings

    def step():
        for p in model.parameters():
            p.grad = None
        loss = loss_fn(model(x), y)
        loss.backward()
        sgd.step()

    gpath = os.path.join(ROOT, "tests", "golden", "cnn_steps.json")
    parity = None
    if os.path.exists(gpath):
        want = {s["step"]: s["params"] for s in json.load(open(gpath))["steps"]}
        ok = True
        for i in range(3):
            step()
            ok = ok and phash() == want[i]
        parity = "parameter sha256 of steps 0-2 equal to reference CPU run" if ok else "MISMATCH"
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    # one event pair per step: the median is what a step costs, the mean also shows a stalled step
    # (e.g. the caching allocator growing a pool)
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    evs[0].record()
    for i in range(steps):
        step()
        evs[i + 1].record()
    evs[-1].synchronize()
    per = sorted(evs[i].elapsed_time(evs[i + 1]) for i in range(steps))
    ms = per[len(per) // 2]
    rec = {"workload": "cnn training step (config 4), batch 256", "ms_per_step": ms,
           "ms_per_step_mean": evs[0].elapsed_time(evs[-1]) / steps,
           "GFLOP/s": 18.3 / ms * 1e3, "steps": steps, "parity": parity}
    cpu = cnn_step_cpu_reference()
    if cpu:
        rec["cpu_baseline"] = cpu
    return rec


def cnn_step_cpu_reference():
    """One training step of the same model and batch through the reference's own Python layers on its
    CPU backend (oracle/_ref), timed on the host cores; None where the reference is not built."""
    import oracle
    site = oracle.ref_site()
    if site is None:
        return None
    try:
        if site not in sys.path:
            sys.path.insert(0, site)
        import repdl
        from repdl_b200 import workloads
        torch.manual_seed(3)
        model = repdl.from_torch_module(workloads.cnn_torch_model())
        x, y = workloads.cnn_batch(256)
        loss_fn = repdl.nn.CrossEntropyLoss()
        t0 = time.perf_counter()
        loss = loss_fn(model(x), y)
        loss.backward()
        with torch.no_grad():
            for p in model.parameters():
                p.add_(p.grad.mul(-0.01))
        dt = time.perf_counter() - t0
        return {"value": dt * 1e3, "unit": "ms per step", "cores": torch.get_num_threads(), "kind": "reference",
                "sample": "one step, batch 256"}
    except Exception as e:  # the baseline is a report, not part of the measurement
        return {"unavailable": repr(e)[:200]}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--size", type=int, default=16384, help="M = N = K of the headline product")
    ap.add_argument("--mode", default="auto", choices=["auto", "nccl", "p2p"])
    ap.add_argument("--ref-rows", type=int, default=16)
    ap.add_argument("--ref-budget", type=float, default=100.0,
                    help="seconds the reference arm may spend on its warm-up and timed steps")
    ap.add_argument("--cpu-budget", type=float, default=15.0)
    ap.add_argument("--workload", default="mm", choices=["mm", "crmath", "sums", "cnn", "mmsmall", "refcuda", "chain"],
                    help="mm: the headline product; crmath / sums: only the HBM-bound kernels of "
                         "configs 2 / 3 at --elements; cnn: the config-4 training step "
                         "(these three are used for profiling captures)")
    ap.add_argument("--elements", type=int, default=1 << 28)
    ap.add_argument("--no-extra", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = max(args.warmup, 0)

    rank, world = env_int("RANK", 0), env_int("WORLD_SIZE", 1)
    local_rank = env_int("LOCAL_RANK", 0)
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch.distributed as dist
    from repdl_b200 import workloads
    from repdl_b200.dist import ShardedMM, mm_from_host

    if args.workload == "cnn":
        if rank == 0:
            torch.cuda.set_device(local_rank)
            print(json.dumps(cnn_step_bench(args.steps, args.warmup)), flush=True)
        return
    if args.workload in ("mmsmall", "refcuda", "chain"):
        if rank == 0:
            torch.cuda.set_device(local_rank)
            hbm_peak, peak_kind = measured_peaks()
            res = (extras_mm(ffma_peak_tflops(False)) if args.workload == "mmsmall"
                   else reference_cuda_bench() if args.workload == "refcuda"
                   else extras_sum1d_full(hbm_peak, peak_kind, args.steps, args.warmup))
            print(json.dumps({"workload": args.workload, "results": res}), flush=True)
        return
    if args.workload != "mm":
        if rank == 0:
            torch.cuda.set_device(local_rank)
            hbm_peak, peak_kind = measured_peaks()
            print(json.dumps({"workload": args.workload, "elements": args.elements,
                              "results": extras_hbm(hbm_peak, peak_kind, args.elements, args.workload,
                                                    args.steps, args.warmup)}), flush=True)
        return

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    n = args.size
    Mp = n // world
    a, b = workloads.mm_large(n, 4)
    a_host = a[rank * Mp:(rank + 1) * Mp].contiguous().pin_memory()
    b_host = b.pin_memory()
    a_dev, b_dev = a_host.to(dev), b_host.to(dev)
    sh = ShardedMM(n, n, n, device=dev, mode=args.mode)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        sh(a_dev, b_dev)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    sh.kernel_launches = 0
    kern_ev = []
    cur = torch.cuda.current_stream()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(cur)
    for _ in range(args.steps):
        sh(a_dev, b_dev)
    e1.record(cur)
    barrier()
    ms_total = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    launches = sh.kernel_launches

    # kernel-only duration of this rank's GEMM launch (events on the launching stream)
    # (the local-panel kernel alone; in p2p mode the timed steps run the same kernel with the
    # peer stores added to its epilogue)
    scratch_rows = torch.empty((Mp, n), dtype=torch.float32, device=dev) if world > 1 else sh.my_rows()
    kms = []
    for _ in range(max(3, args.steps)):
        kms.append(event_ms(lambda: sh.mm_into(a_dev, b_dev, scratch_rows), cur))
    kernel_ms = sum(kms) / len(kms)
    del scratch_rows

    t = torch.tensor([ms_total, kernel_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, kernel_ms = float(t[0]), float(t[1])
    ms_step = ms_total / args.steps
    flops_step = 2.0 * n * n * n
    value = flops_step / ms_step / 1e6  # GFLOP/s

    # end to end with host operands
    e2e = None
    if not args.no_e2e:
        c_host = torch.empty((Mp, n), dtype=torch.float32).pin_memory()
        for _ in range(2):
            mm_from_host(sh, a_host, b_host, a_dev, b_dev, c_host)
        barrier()
        ke = args.steps
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record(cur)
        for _ in range(ke):
            mm_from_host(sh, a_host, b_host, a_dev, b_dev, c_host)
        t1.record(cur)
        barrier()
        t = torch.tensor([t0.elapsed_time(t1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t[0]) / ke
        e2e = {"value": flops_step / e2e_ms / 1e6, "unit": "GFLOP/s", "ms_per_step": e2e_ms,
               # several GPUs: every rank uploads its A panel and 1/world of B (the rest is gathered)
               "h2d_bytes_per_step": (world * a_host.numel() + b_host.numel()) * 4 if world > 1
               else (a_host.numel() + b_host.numel()) * 4,
               "d2h_bytes_per_step": world * c_host.numel() * 4}

    # parity of the timed result against the hashes of the reference CPU backend's own product
    # (tests/golden/mm16k.json): rank 0 hashes the whole gathered C; with several ranks every rank
    # also hashes the rows IT computed, as they lie in ITS copy of C, against the per-block hashes
    parity = None
    gpath = os.path.join(ROOT, "tests", "golden", "mm16k.json")
    if n == 16384 and os.path.exists(gpath):
        gold = json.load(open(gpath))
        mine_ok = 1
        if world > 1 and Mp % 2048 == 0:
            for blk in range(Mp // 2048):
                r0 = rank * Mp + blk * 2048
                h = hashlib.sha256(sh.C[r0:r0 + 2048].cpu().numpy().tobytes()).hexdigest()
                mine_ok &= int(h == gold["row_block_2048_sha256"][r0 // 2048])
            t = torch.tensor([mine_ok], dtype=torch.int32, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MIN)
            mine_ok = int(t[0])
        if rank == 0:
            h = hashlib.sha256(sh.C.cpu().numpy().tobytes()).hexdigest()
            ok = h == gold["sha256"] and mine_ok == 1
            if e2e is not None and world == 1:  # what the host-operand step brought back to the host
                ok = ok and hashlib.sha256(c_host.numpy().tobytes()).hexdigest() == gold["sha256"]
            parity = ("sha256 equal to reference CPU backend" + (
                "; every rank's own row blocks too" if world > 1 and Mp % 2048 == 0 else "")) if ok else "MISMATCH"

    if rank == 0:
        hbm_peak, peak_kind = measured_peaks()
        peak = ffma_peak_tflops(False)
        achieved = flops_step / world / kernel_ms / 1e9  # TFLOP/s of one rank's launch
        line = {
            "metric": "bit-exact fp32 mm GFLOP/s", "value": value, "unit": "GFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": "mm M=N=K=%d fp32, A,B~U[-1,1) seed 4 (config 5); A row-sharded, "
                                   "C all-gathered" % n,
                       "parallelism": "rows/%d" % world, "collective": sh.mode,
                       "l2": "operands (3 GiB) exceed the 126 MB L2"},
            "roofline": {"bound": "fp32_ffma", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak,
                         # DRAM bytes of one rank's launch: ncu captures of the 16384^3 launch (summarised
                         # under profiles/), 27.53 GB with the 192 x 128 tile that 1 and 2 ranks get and
                         # 35.58 GB with the 128 x 256 tile that 4 and 8 ranks get, scaled by the rows a
                         # rank computes (B is streamed once per group of 8 tile rows, so the traffic is
                         # proportional to the rows); null for other sizes
                         "traffic": ((27.53e9 if world <= 2 else 35.58e9) / world if n == 16384 else None),
                         "algorithmic_bytes": 4.0 * (n * n / world + n * n + n * n / world),
                         "peak_source": "FFMA-only probe kernel timed in this run",
                         "peak_nominal": 148 * 128 * 2 * 1.965e9 / 1e12,
                         "kernel_ms": kernel_ms},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches * world, "parity": parity,
        }
        if world == 1:
            line["cpu_baseline"] = time_cpu_mm(a, b, args.cpu_budget)
            if not args.no_extra:
                del a_dev, b_dev, sh
                torch.cuda.empty_cache()
                line["extra"] = extras_mm(peak)
                line["extra"].update(extras_hbm(hbm_peak, peak_kind))
                line["extra"]["sum1d chain [1073741824] (config 3)"] = extras_sum1d_full(hbm_peak, peak_kind)
                ref_cuda = reference_cuda_bench()
                if ref_cuda is not None:
                    line["extra"]["reference CUDA backend (sm_100a build)"] = ref_cuda
                # the callers' side of the path: one SGD step of the CNN workload on these operators
                line["extra"]["cnn training step"] = cnn_step_bench(steps=5, warmup=3)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
