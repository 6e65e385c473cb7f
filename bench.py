"""Benchmark of the log-linear Mamba-2 chunkwise forward+backward hot path.

    python bench.py --gpus N --steps K --warmup W            # CUDA path (this repository)
    python bench.py --impl reference --gpus N --steps K ...  # the reference's CPU implementation on host cores

Workload at every N (weak scaling, one process per GPU, batch sharded, no data-path collective):
the configuration the headline metric is quoted on, per GPU: B=2, T=16384, H=32, P=64, N=128,
G=1, chunk 64, L=15, bf16 inputs with fp32 accumulation, synthetic seeded inputs with the value
distributions of that configuration.  A step is one forward plus one backward of the operator
(drivers `chunkwise_fwd` + `chunkwise_bwd`, the functions the reference's autograd boundary calls).

Printed: one JSON line (rank 0).  `value` is tokens/s with inputs resident in HBM, from the median of
R back-to-back blocks of K steps (R chosen so that about a second is timed; every block is bracketed by
CUDA events; `repeats` gives the spread); `e2e` is the same metric with every step's inputs copied from
pinned host memory and every output copied back.  At N=1 the line also carries `cpu_baseline` (the
reference's own PyTorch chunkwise form on host cores), `cpu_baseline_recurrent` (its token recurrence,
forward only), `triton_reference` (the reference's Triton kernels on the same GPU, same inputs) and
`secondary` (other configurations on the same kernels).
"""
import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "log-linear-attention_b200")
for _p in (ROOT, PKG):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

WORKLOAD = dict(B=2, T=16384, H=32, P=64, N=128, G=1, L=15, chunk=64)
METRIC = "log-linear Mamba-2 chunkwise fwd+bwd tokens/s at T=16K"


def workload_name(w=None):
    w = w or WORKLOAD
    return (f"log-linear Mamba-2 chunkwise fwd+bwd, B={w['B']} T={w['T']} H={w['H']} P={w['P']} N={w['N']} G={w['G']} "
            f"chunk=64 L={w['L']} (per GPU)")


def fmin_flops(B, T, H, P, N, C=64, backward=True):
    """Necessary tensor flops of the chunkwise Fenwick-merge algorithm, dense per 64x64 tile:
    fwd = CK + CV + (1 + Lc/2) S ; bwd = 3 CK + 2 CV + (3 + Lc) S per (batch, head, chunk)."""
    NT = T // C
    Lc = max(0, (NT - 1).bit_length())
    CK, CV, S = 2 * C * C * N, 2 * C * C * P, 2 * C * N * P
    fwd = CK + CV + (1 + Lc / 2) * S
    bwd = 3 * CK + 2 * CV + (3 + Lc) * S
    return (fwd + (bwd if backward else 0)) * B * H * NT


def algorithmic_bytes(B, T, H, P, N, G, L):
    fwd = 2 * B * T * G * N * 2 + 2 * B * T * H * P * 2 + B * T * H * L * 2 + B * T * H * 4
    bwd = fwd + 2 * B * T * H * P * 2 + 2 * B * T * H * N * 2 + B * T * H * L * 4 + B * T * H * 4
    return fwd + bwd


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return dict(tflops=d.get("bf16_tflops_sustained", d.get("bf16_tflops")), tflops_burst=d.get("bf16_tflops"),
                    hbm=d.get("hbm_gbs"), source="measured")
    return dict(tflops=1400.0, tflops_burst=1590.0, hbm=6650.0, source="fallback")


def measured_traffic(w):
    """DRAM read + write bytes per launch of the dominant kernel, from the counter file that the ncu recipe in
    profiles/ writes (captured at batch 1; every CTA handles one (batch, head, segment), so traffic is
    proportional to the batch).  None when there is no capture for this shape."""
    path = os.path.join(ROOT, "profiles", "tc_counters_B1.json")
    if not os.path.exists(path):
        return None, None
    d = json.load(open(path))
    shape = d.get("shape", {})
    if (shape.get("T"), shape.get("H"), shape.get("P"), shape.get("N")) != (w["T"], w["H"], w["P"], w["N"]):
        return None, None
    k = d["kernels"][d["dominant"]]
    per_b = k["dram_read_bytes"] + k["dram_write_bytes"]
    return per_b * w["B"] / shape.get("B", 1), d["dominant"]


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, val in zip(names, f[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def make_inputs(seed, pin, w=None):
    """Seeded synthetic tensors with the value distributions of the configuration: X~N(0,1);
    B,C~N(0,1)/sqrt(N); dt=softplus(N(0,1)-2); A=-exp(U(0,ln16)) per head; lambda=softplus(N(0,1));
    dY~N(0,1).  Kernel-level inputs: q=C, k=B, v=X*dt, g=A*dt."""
    w = w or WORKLOAD
    B, T, H, P, N, G, L = (w[x] for x in ("B", "T", "H", "P", "N", "G", "L"))
    gen = torch.Generator().manual_seed(seed)
    X = torch.randn(B, T, H, P, generator=gen)
    Bm = torch.randn(B, T, G, N, generator=gen) / math.sqrt(N)
    Cm = torch.randn(B, T, G, N, generator=gen) / math.sqrt(N)
    dt = torch.nn.functional.softplus(torch.randn(B, T, H, generator=gen) - 2.0)
    A = -torch.exp(torch.rand(H, generator=gen) * math.log(16.0))
    lam = torch.nn.functional.softplus(torch.randn(B, T, H, L, generator=gen))
    do = torch.randn(B, T, H, P, generator=gen)
    ts = [Cm.bfloat16(), Bm.bfloat16(), (X * dt[..., None]).bfloat16(), (A[None, None] * dt).float(), lam.bfloat16(),
          do.bfloat16()]
    return [t.pin_memory() for t in ts] if pin else ts


# ----------------------------------------------------------------------------------------------
# the reference's CPU implementation of the path (reference arm, cpu_baseline)
# ----------------------------------------------------------------------------------------------
CPU_SLICE = dict(B=1, T=4096)       # one step of the CPU arm: this slice of the workload (cost is linear in B and ~T log T)


def _cpu_forms():
    """(kind, chunkwise fwd+bwd step function factory, recurrent forward function or None).  The reference's own
    hssd_minimal_discrete / hattention_recurrent when the copy made by baseline/make_ref.py is present, else
    the oracle's port of the same algorithms."""
    from oracle import loglinear_oracle as orc
    try:
        from baseline import ref_compat
        m = ref_compat.load_reference(triton_path=False, torch_forms=True)
        hm, rec, base = m["hssd_minimal"], m["recurrent"], m["base"]

        def chunk_fwd(q, k, v, g, l):
            H = v.shape[2]
            return hm.hssd_minimal_discrete(v, g, k.expand(-1, -1, H, -1), q.expand(-1, -1, H, -1), l, 2, base.HType.WEAK, 64)

        def recurrent_fwd(q, k, v, g, l):
            H = v.shape[2]
            return rec.hattention_recurrent(q.expand(-1, -1, H, -1).contiguous(), k.expand(-1, -1, H, -1).contiguous(), v,
                                            torch.exp(g), None, l, 2, base.HType.WEAK, base.HStruct.MAMBA2)[0]
        return "reference", chunk_fwd, recurrent_fwd
    except Exception:                       # no copy of the reference on this machine
        return "port", (lambda q, k, v, g, l: orc.mamba2_chunkwise(q, k, v, g, l, chunk=64)), \
            (lambda q, k, v, g, l: orc.recurrent(q, k, v, g, l)[0])


def cpu_chunkwise_steps(threads, steps, warmup, T=None):
    """fp32 chunkwise forward + autograd backward of the reference's PyTorch form on a slice of the workload."""
    from oracle import loglinear_oracle as orc
    torch.set_num_threads(threads)
    w = WORKLOAD
    T = T or min(CPU_SLICE["T"], w["T"])
    kind, chunk_fwd, _ = _cpu_forms()
    q, k, v, g, l = orc.make_mamba2_inputs(CPU_SLICE["B"], T, w["H"], w["P"], w["N"], w["G"], w["L"], seed=0)
    do = torch.randn(CPU_SLICE["B"], T, w["H"], w["P"], generator=torch.Generator().manual_seed(1))

    def step():
        ins = [x.clone().requires_grad_(True) for x in (q, k, v, g, l)]
        o = chunk_fwd(*ins)
        torch.autograd.grad((o * do).sum(), ins)

    for _ in range(warmup):
        step()
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    what = "hssd_minimal_discrete" if kind == "reference" else "oracle port of hssd_minimal_discrete"
    sample = (f"each step = B={CPU_SLICE['B']} T={T} H={w['H']} P={w['P']} N={w['N']} L={w['L']} slice of the workload, fp32, "
              f"{what} forward + autograd backward")
    return kind, T, times, sample


def cpu_recurrent_sample(threads, T=256):
    """The reference's token recurrence (forward only; it has no backward), truncated to T tokens."""
    from oracle import loglinear_oracle as orc
    torch.set_num_threads(threads)
    w = WORKLOAD
    kind, _, rec_fwd = _cpu_forms()
    q, k, v, g, l = orc.make_mamba2_inputs(1, T, w["H"], w["P"], w["N"], w["G"], w["L"], seed=0)
    with torch.no_grad():
        rec_fwd(q[:, :32], k[:, :32], v[:, :32], g[:, :32], l[:, :32])
        t0 = time.perf_counter()
        rec_fwd(q, k, v, g, l)
        dt = time.perf_counter() - t0
    what = "hattention_recurrent" if kind == "reference" else "oracle port of hattention_recurrent"
    return {"value": T / dt, "unit": "tokens/s", "cores": threads, "kind": kind,
            "sample": f"{what}, forward only, B=1 truncated to T={T} (cost is linear in T), H={w['H']} P={w['P']} N={w['N']} L={w['L']}, fp32"}


def run_reference(args, rank, world):
    """Reference arm: the reference's own CPU implementation of the path, all host threads, rank 0 only."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    warm = min(args.warmup, 2)
    steps = max(1, min(args.steps, 10))
    kind, T, times, sample = cpu_chunkwise_steps(threads, steps, warm)
    dt = sum(times) / len(times)
    val = CPU_SLICE["B"] * T / dt
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "tokens/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": warm, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"B={CPU_SLICE['B']} T={T} slice of: {workload_name()}", "timed_on": "host cores",
                   "note": "tokens/s of the slice; the algorithm's cost per token grows with log2(T) only"},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------
# CUDA-event timing helpers
# ----------------------------------------------------------------------------------------------
def time_blocks(step, K, barrier, min_total_ms=1000.0, max_blocks=40):
    """Times blocks of exactly K steps, each bracketed by CUDA events on the current stream and a barrier +
    synchronise on both sides; repeats until about `min_total_ms` have been timed.  Returns the block times (ms)."""
    times = []
    total = 0.0
    while True:
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(K):
            step()
        e1.record()
        barrier()
        t = e0.elapsed_time(e1)
        times.append(t)
        total += t
        if total >= min_total_ms or len(times) >= max_blocks:
            return times


def launches():
    from hattention_b200 import _lib
    return _lib.lib().llattn_kernel_launches()


# ----------------------------------------------------------------------------------------------
# secondary measurements (N = 1): other configurations on the same kernels
# ----------------------------------------------------------------------------------------------
def secondary_mamba2(dev, B, T, H, backward, steps, label):
    from hattention_b200.base import HType
    from hattention_b200.chunkwise import chunkwise_bwd, chunkwise_fwd
    w = dict(WORKLOAD, B=B, T=T, H=H, L=7 + max(0, (T // 64 - 1).bit_length()))
    q, k, v, g, l, do = [t.to(dev) for t in make_inputs(7, False, w)]

    def step():
        kept = [] if backward else None
        o, g_cum, _ = chunkwise_fwd(q, k, v, g, l, False, 2, HType.WEAK, 64, False, keep_workspace=kept)
        if backward:
            chunkwise_bwd(q, k, v, g_cum, l, do, False, 2, HType.WEAK, 64, fwd_workspace=kept[0])

    for _ in range(3):
        step()
    n0 = launches()
    times = time_blocks(step, steps, torch.cuda.synchronize, min_total_ms=300.0, max_blocks=10)
    nl = (launches() - n0) // len(times)
    ms = statistics.median(times) / steps
    flops = fmin_flops(B, T, H, w["P"], w["N"], backward=backward)
    pk = peaks()
    return {"workload": label, "ms_per_step": ms, "tokens_per_s": B * T / (ms * 1e-3), "steps": steps, "blocks": len(times),
            "algorithmic_tflops": flops / (ms * 1e-3) / 1e12, "frac_of_sustained_bf16_peak": flops / (ms * 1e-3) / 1e12 / pk["tflops"],
            "gpu_launches": nl}


def secondary_gdn(dev, steps, B=4):
    from hattention_b200.gated_delta_rule_apis import chunk_h_gated_delta_rule
    T, H, Dk, Dv, L = 8192, 16, 128, 128, 14
    gen = torch.Generator().manual_seed(11)
    q = torch.randn(B, T, H, Dk, generator=gen).bfloat16().to(dev)
    k = torch.randn(B, T, H, Dk, generator=gen).bfloat16().to(dev)
    v = torch.randn(B, T, H, Dv, generator=gen).bfloat16().to(dev)
    beta = torch.sigmoid(torch.randn(B, T, H, generator=gen)).bfloat16().to(dev)
    g = torch.nn.functional.logsigmoid(torch.randn(B, T, H, generator=gen) + 3.0).float().to(dev)
    lam = torch.nn.functional.softplus(torch.randn(B, T, H, L, generator=gen)).bfloat16().to(dev)
    do = torch.randn(B, T, H, Dv, generator=gen).bfloat16().to(dev)
    ins = [x.clone().requires_grad_(True) for x in (q, k, v, g, lam, beta)]

    def fwd():
        with torch.no_grad():
            chunk_h_gated_delta_rule(q, k, v, g, lam, beta, use_qk_l2norm_in_kernel=True)

    def fwdbwd():
        o = chunk_h_gated_delta_rule(*ins, use_qk_l2norm_in_kernel=True)[0]
        torch.autograd.grad(o, ins, do)

    out = {}
    for name, fn in (("forward", fwd), ("forward+backward", fwdbwd)):
        for _ in range(2):
            fn()
        n0 = launches()
        times = time_blocks(fn, steps, torch.cuda.synchronize, min_total_ms=300.0, max_blocks=10)
        out[name] = (statistics.median(times) / steps, (launches() - n0) // len(times))
    C, NT = 64, T // 64
    Lc = (NT - 1).bit_length()
    CK, CV, S = 2 * C * C * Dk, 2 * C * C * Dv, 2 * C * Dk * Dv
    flops_fwd = (5 * CK + 2 * CV + 2 * C ** 3 + Lc * 2.5 * S) * B * H * NT     # count of the reference's formulation
    ms_fb, nl = out["forward+backward"]
    return {"workload": f"log-linear Gated DeltaNet fwd+bwd through chunk_h_gated_delta_rule, B={B} T={T} H={H} Dk=Dv=128 chunk=64 L={L}",
            "ms_per_step": ms_fb, "tokens_per_s": B * T / (ms_fb * 1e-3), "steps": steps, "gpu_launches": nl,
            "forward_only_ms": out["forward"][0],
            "forward_tflops_reference_formulation": flops_fwd / (out["forward"][0] * 1e-3) / 1e12}


# ----------------------------------------------------------------------------------------------
# the reference's Triton kernels on this GPU (N = 1), run in a child process
# ----------------------------------------------------------------------------------------------
def triton_arm_child(args):
    """Child process: times the reference's own chunkwise_fwd + chunkwise_bwd (Triton) on the headline inputs
    after its autotune warm-up, and compares this repository's outputs with them.  Prints one JSON line."""
    os.environ.setdefault("TRITON_CACHE_DIR", os.path.join(ROOT, "baseline", "_ref", "triton_cache"))
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    try:
        from baseline import ref_compat
        m = ref_compat.load_reference()
        cw, HT = m["chunkwise"], m["base"].HType
        q, k, v, g, l, do = [t.to(dev) for t in make_inputs(0, False)]

        def ref_step():
            o, gc, _ = cw.chunkwise_fwd(q=q, k=k, v=v, g=g, l=l, head_first=False, level_base=2, htype=HT.WEAK, chunk_size=64,
                                        output_final_state=False)
            return (o,) + tuple(cw.chunkwise_bwd(q=q, k=k, v=v, g=gc, l=l, do=do, head_first=False, level_base=2, htype=HT.WEAK,
                                                 chunk_size=64))
        t0 = time.perf_counter()
        ref = ref_step()                       # compiles and autotunes
        torch.cuda.synchronize()
        compile_s = time.perf_counter() - t0
        for _ in range(max(args.warmup, 3)):
            ref_step()
        K = max(3, min(args.steps, 10))
        times = time_blocks(ref_step, K, torch.cuda.synchronize, min_total_ms=500.0, max_blocks=5)
        ms = statistics.median(times) / K
        from hattention_b200.base import HType
        from hattention_b200.chunkwise import chunkwise_bwd, chunkwise_fwd
        kept = []
        o, g_cum, _ = chunkwise_fwd(q, k, v, g, l, False, 2, HType.WEAK, 64, False, keep_workspace=kept)
        ours = (o,) + tuple(chunkwise_bwd(q, k, v, g_cum, l, do, False, 2, HType.WEAK, 64, fwd_workspace=kept[0]))
        torch.cuda.synchronize()
        err = {}
        for name, a, b in zip(("o", "dq", "dk", "dv", "dg", "dl"), ours, ref):
            a, b = a.float(), b.float()
            err[name] = {"max_abs": (a - b).abs().max().item(), "max_abs_triton": b.abs().max().item(),
                         "rel_frobenius": ((a - b).norm() / b.norm()).item()}
        w = WORKLOAD
        print(json.dumps({"status": "ok", "ms_per_step": ms, "tokens_per_s": w["B"] * w["T"] / (ms * 1e-3), "steps": K,
                          "blocks": len(times), "first_call_s": compile_s, "max_err_vs_triton": err,
                          "what": "hattention.chunkwise.chunkwise_fwd + chunkwise_bwd (Triton, autotuned), same inputs, same GPU"}),
              flush=True)
    except Exception as e:      # noqa: BLE001  (the first line of the error is the result)
        msg = (str(e).strip().splitlines() or [type(e).__name__])[0]
        print(json.dumps({"status": "unavailable", "error": f"{type(e).__name__}: {msg}"[:400]}), flush=True)


def triton_reference(args, timeout_s):
    if not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "hattention")):
        return {"status": "unavailable", "error": "baseline/_ref/hattention missing (python baseline/make_ref.py <reference checkout>)"}
    cmd = [sys.executable, os.path.abspath(__file__), "--triton-arm-child", "--steps", str(args.steps), "--warmup", str(args.warmup)]
    env = dict(os.environ)
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        env.pop(k, None)
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout_s, env=env)
    except subprocess.TimeoutExpired:
        return {"status": "unavailable", "error": f"no result within {timeout_s} s (Triton compile + autotune of the reference kernels)"}
    for line in reversed(r.stdout.strip().splitlines()):
        if line.startswith("{"):
            try:
                return json.loads(line)
            except ValueError:
                continue
    tail = (r.stderr.strip().splitlines() or ["no output"])[-1]
    return {"status": "unavailable", "error": f"child exited {r.returncode}: {tail}"[:400]}


def run_sequence_parallel(args, rank, world, local):
    """Secondary bench line: one sequence of world x T tokens split along T over the ranks (B=2, H=32,
    P=64, N=128 per rank, T = --seq-len per rank): in-shard part on the CUDA kernels, shard summaries
    all-gathered (reduce-scattered in the backward) over NCCL, cross-shard levels as torch products."""
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29655")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from hattention_b200.sequence_parallel import hattention_sequence_parallel
    w = dict(WORKLOAD)
    w["L"] = WORKLOAD["L"] + (world - 1).bit_length()
    B, T, H, P, N, G, L = w["B"], w["T"], w["H"], w["P"], w["N"], w["G"], w["L"]
    gen = torch.Generator().manual_seed(100 + rank)
    q = (torch.randn(B, T, G, N, generator=gen) / N ** 0.5).bfloat16().to(dev)
    k = (torch.randn(B, T, G, N, generator=gen) / N ** 0.5).bfloat16().to(dev)
    v = torch.randn(B, T, H, P, generator=gen).bfloat16().to(dev)
    g = (-torch.nn.functional.softplus(torch.randn(B, T, H, generator=gen) - 2.0)).float().to(dev)
    lam = torch.nn.functional.softplus(torch.randn(B, T, H, L, generator=gen)).bfloat16().to(dev)
    do = torch.randn(B, T, H, P, generator=gen).bfloat16().to(dev)
    ins = [x.requires_grad_(True) for x in (q, k, v, g, lam)]

    def step():
        o = hattention_sequence_parallel(*ins)
        torch.autograd.grad(o, ins, do)

    def barrier():
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()

    W, K = max(args.warmup, 3), args.steps
    for _ in range(W):
        step()
    sampler = ClockSampler(local)
    times = time_blocks(step, K, barrier, min_total_ms=500.0, max_blocks=10)
    clocks = sampler.stop()
    t = torch.tensor([statistics.median(times) / K], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = t.item()
    if rank == 0:
        print(json.dumps({
            "metric": "log-linear Mamba-2 sequence-parallel fwd+bwd tokens/s", "value": world * B * T / (ms * 1e-3),
            "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"one sequence of {world}x{T} tokens split along T, B={B} H={H} P={P} N={N} L={L}",
                       "note": "cross-shard levels: all-gather of shard final states + torch products"},
            "clocks": clocks}), flush=True)
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="only the headline measurement: no secondary configurations, no Triton reference, no CPU baselines")
    ap.add_argument("--triton-timeout", type=int, default=420, help="seconds allowed for the reference Triton measurement")
    ap.add_argument("--triton-arm-child", action="store_true", help=argparse.SUPPRESS)
    ap.add_argument("--timed-ms", type=float, default=1000.0,
                    help="blocks of K steps are repeated until this much device time has been measured (0: one block, "
                         "for profiler captures)")
    ap.add_argument("--gdn-batch", type=int, default=4, help="batch of --workload gdn (4 is the benchmark configuration; profiler captures use 1)")
    ap.add_argument("--workload", default="mamba2", choices=["mamba2", "gdn", "mamba2-sp"],
                    help="mamba2 = the headline workload (other configurations ride along under `secondary`); "
                         "gdn = only the Gated DeltaNet secondary measurement (B=4 T=8192 H=16 Dk=Dv=128 L=14); mamba2-sp = Mamba-2 with one sequence split along T over the ranks (run under torchrun)")
    ap.add_argument("--batch", type=int, default=WORKLOAD["B"],
                    help="per-GPU batch; the headline workload is 2, profiler captures use 1")
    ap.add_argument("--seq-len", type=int, default=WORKLOAD["T"],
                    help="sequence length; the headline workload is 16384 (65536 with --batch 1 is one GPU's share of the "
                         "multi-GPU scaling configuration); L follows as 7 + ceil(log2(T/64))")
    args = ap.parse_args()
    WORKLOAD["B"] = args.batch
    if args.seq_len != WORKLOAD["T"]:
        WORKLOAD["T"] = args.seq_len
        WORKLOAD["L"] = 7 + max(0, (args.seq_len // 64 - 1).bit_length())
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.triton_arm_child:
        triton_arm_child(args)
        return
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.workload == "mamba2-sp":
        run_sequence_parallel(args, rank, world, local)
        return
    if args.workload == "gdn":
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
        torch.cuda.set_device(local)
        print(json.dumps(secondary_gdn(torch.device("cuda", local), args.steps, args.gdn_batch)), flush=True)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    import torch.distributed as dist
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    from hattention_b200 import _lib
    from hattention_b200.base import HType
    from hattention_b200.chunkwise import chunkwise_bwd, chunkwise_fwd

    w = WORKLOAD
    host = make_inputs(seed=rank, pin=True)
    q, k, v, g, l, do = [t.to(dev) for t in host]
    last_ws = []

    def step(q=q, k=k, v=v, g=g, l=l, do=do):
        kept = []      # the forward's scratch stays alive until the backward, as the autograd function does
        o, g_cum, _ = chunkwise_fwd(q, k, v, g, l, False, 2, HType.WEAK, 64, False, keep_workspace=kept)
        grads = chunkwise_bwd(q, k, v, g_cum, l, do, False, 2, HType.WEAK, 64, fwd_workspace=kept[0])
        last_ws[:] = kept
        return (o,) + tuple(grads)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    W = max(args.warmup, 3)
    K = args.steps
    for _ in range(W):
        outs = step()
    barrier()
    # ---- device-resident timing: R blocks of exactly K steps
    sampler = ClockSampler(local) if rank == 0 else None
    n0 = launches()
    times = time_blocks(step, K, barrier, min_total_ms=args.timed_ms)
    launches_per_block = (launches() - n0) // len(times)
    clocks = sampler.stop() if sampler else None
    status = _lib.workspace_status(last_ws[0], torch.cuda.current_stream().cuda_stream)
    if status != 0:
        raise SystemExit("a kernel gave up on a bounded wait during the timed region (status word set): no valid measurement")
    ms_block = statistics.median(times)

    # ---- end to end: host buffers in, host buffers out, every step
    outs = step()
    host_out = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in outs]
    h2d = sum(t.numel() * t.element_size() for t in host)
    d2h = sum(t.numel() * t.element_size() for t in host_out)

    # Three streams: copy-in, compute (the current stream), copy-out, with two sets of device input buffers, so
    # that step i+1's host->device copy and step i-1's device->host read overlap step i's kernels (PCIe is full
    # duplex).  Every step still moves all of its inputs from pinned host memory and all of its results back.
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    s_comp = torch.cuda.current_stream(dev)
    dbuf = [[torch.empty(t.shape, dtype=t.dtype, device=dev) for t in host] for _ in range(2)]
    in_ready = [torch.cuda.Event() for _ in range(2)]
    comp_done = [torch.cuda.Event() for _ in range(2)]

    def e2e_run(n):
        for i in range(n):
            b_ = i % 2
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(comp_done[b_])          # step i-2 has finished reading this input set
                for dst, src in zip(dbuf[b_], host):
                    dst.copy_(src, non_blocking=True)
                in_ready[b_].record(s_in)
            s_comp.wait_event(in_ready[b_])
            res = step(*dbuf[b_])
            comp_done[b_].record(s_comp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(comp_done[b_])
                for dst, src in zip(host_out, res):
                    dst.copy_(src, non_blocking=True)
                    src.record_stream(s_out)
        s_comp.wait_stream(s_out)
        s_comp.wait_stream(s_in)

    e2e_run(2)
    barrier()
    Ke = max(4, min(K, 10))
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    e2e_run(Ke)
    f1.record()
    barrier()
    ms_e2e = f0.elapsed_time(f1)

    t_dev = torch.tensor([ms_block, ms_e2e, min(times), max(times)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t_dev, op=dist.ReduceOp.MAX)
    ms_block, ms_e2e, t_min, t_max = t_dev.tolist()

    if rank == 0:
        tokens = w["B"] * w["T"] * world
        per_step = ms_block / K
        value = tokens / (per_step * 1e-3)
        e2e_val = tokens / (ms_e2e / Ke * 1e-3)
        pk = peaks()
        flops = fmin_flops(w["B"], w["T"], w["H"], w["P"], w["N"])
        achieved = flops / (per_step * 1e-3) / 1e12
        traffic, traffic_kernel = measured_traffic(w)
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": workload_name(), "l2": "inputs_exceed_l2 (about 320 MB of inputs per step vs 126 MB L2)",
                       "sharding": f"batch x {world}, no collective"},
            "repeats": {"blocks": len(times), "steps_per_block": K, "ms_per_step_median": per_step,
                        "ms_per_step_min": t_min / K, "ms_per_step_max": t_max / K, "timed_ms_total": sum(times)},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": pk["tflops"], "unit": "TFLOP/s",
                         "frac": achieved / pk["tflops"], "frac_of_burst_peak": achieved / pk["tflops_burst"],
                         "traffic": traffic, "traffic_kernel": traffic_kernel,
                         "traffic_source": "profiles/tc_counters_B1.json (ncu, batch 1, scaled by the batch)" if traffic else None,
                         "peak_source": pk["source"],
                         "kernel": "whole fwd+bwd launch chain of one step (algorithmic flops F_min / step time)",
                         "algorithmic_flops_per_step": flops,
                         "algorithmic_bytes_per_step": algorithmic_bytes(w["B"], w["T"], w["H"], w["P"], w["N"], w["G"], w["L"])},
            "e2e": {"value": e2e_val, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": Ke},
            "gpu_launches": launches_per_block,
            "clocks": clocks,
        }
        extras = world == 1 and not args.no_extras
        if extras and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            kind, T, ctimes, sample = cpu_chunkwise_steps(threads, steps=3, warmup=1)
            line["cpu_baseline"] = {"value": CPU_SLICE["B"] * T / min(ctimes), "unit": "tokens/s", "cores": threads, "kind": kind,
                                    "sample": sample + ", best of 3"}
            line["cpu_baseline_recurrent"] = cpu_recurrent_sample(threads)
        if extras:
            torch.cuda.empty_cache()
            sec = []
            for fn, a in ((secondary_mamba2, (dev, 8, 4096, 24, False, 10, "log-linear Mamba-2 forward, B=8 T=4096 H=24 P=64 N=128 G=1 L=13")),
                          (secondary_mamba2, (dev, 1, 65536, 32, True, 5, "log-linear Mamba-2 fwd+bwd, B=1 T=65536 H=32 P=64 N=128 G=1 L=17 "
                                                                           "(one GPU's share of the long-context configuration)")),
                          (secondary_gdn, (dev, 5))):
                try:
                    sec.append(fn(*a))
                except Exception as e:      # noqa: BLE001
                    sec.append({"workload": a[-1] if isinstance(a[-1], str) else "log-linear Gated DeltaNet", "error": str(e)[:200]})
                torch.cuda.empty_cache()
            line["secondary"] = sec
            tr = triton_reference(args, args.triton_timeout)
            if tr.get("status") == "ok":
                tr["speedup"] = tr["ms_per_step"] / per_step
            line["triton_reference"] = tr
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
