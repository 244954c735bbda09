#!/usr/bin/env python
"""Benchmark of the quantized-matmul hot path (quantizeQ4/Q8 -> matmulQ4/Q8) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

A "step" is one pass of the hot path over R distinct, device-resident packed
weight matrices of the workload's shape (R chosen so that R x bytes is at least
four times the 126 MB L2: consecutive products never find their weights in
cache).  For GEMV shapes (M <= 4) on one GPU the R products of a step run as ONE
persistent launch (smith_qmatmul_list), the way a decode engine runs its layer
stack; `config.form` says so and `config.per_call` gives the same R products as
R separate launches replayed from a CUDA graph.  Other shapes, and several GPUs,
use the graph of separate launches.  Timing is CUDA events on the launching
stream, max over ranks, between barriers.  Before anything is timed, a column
window of one output is compared with the CPU oracle (`parity`).

`value`  : algorithmic bytes (M <= 16) or FLOPs (M >= 64) of all launches / device time.
`e2e`    : the same quantity through the operator API (smith_b200.matmulQ4 /
           matmulQ8 on host-resident activation tensors): every call copies the
           activations host->device from page-locked memory, runs the kernel,
           copies the result device->host and waits, exactly what the JS
           operator does per call.  Packed weights stay resident, as they do in
           the reference (they are a device buffer returned by quantizeQ4).
`roofline`: achieved/peak for the dominant kernel, peak from MEASURED_PEAKS.json.
`cpu_baseline`: the reference's own shader source compiled as C++ (oracle/_ref)
           or, failing that, this repository's C restatement, on the host cores.

With N > 1 (launched by torch.distributed.run) the weights are sharded along
the output dimension N, activations are replicated, and each step ends with an
all-gather of the output row slices (strong scaling of a fixed problem).

Synthetic data: weights ~N(0, 0.02), activations ~N(0, 1), generated on the
device by the bridge's counter-based generator, packed by the CUDA packers.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: kind, M, K, N, weight std
    "q4_decode_gemv_4096x14336_m1": dict(kind=4, M=1, K=4096, N=14336, std=0.02),   # the decode GEMV the 70 % HBM target is quoted on
    "q4_decode_4096x14336_m4": dict(kind=4, M=4, K=4096, N=14336, std=0.02),
    "q4_decode_4096x14336_m16": dict(kind=4, M=16, K=4096, N=14336, std=0.02),
    "q4_prefill_4096x14336_m64": dict(kind=4, M=64, K=4096, N=14336, std=0.02),
    "q4_prefill_4096x14336_m256": dict(kind=4, M=256, K=4096, N=14336, std=0.02),
    "q4_prefill_4096x14336_m512": dict(kind=4, M=512, K=4096, N=14336, std=0.02),   # the prefill GEMM the 50 % tensor target is quoted on
    "q8_prefill_gemm_4096x11008_m512": dict(kind=8, M=512, K=4096, N=11008, std=0.02),  # Q8 prefill GEMM 512 x 4096 x 11008
    "q4_gemv_4096x4096_m1": dict(kind=4, M=1, K=4096, N=4096, std=0.02),            # the single Q4 GEMV a CPU can also run in full
    "q4_lm_head_4096x128256_m1": dict(kind=4, M=1, K=4096, N=128256, std=0.02),
    "q8_decode_gemv_4096x14336_m1": dict(kind=8, M=1, K=4096, N=14336, std=0.02),
    # every Q4 projection of an 8B-Llama-shaped decode step (32 layers + lm_head, 5.63 GB)
    "q4_llama8b_step_m1": dict(kind=4, M=1, step=dict(layers=32, dim=4096, kv=1024, ffn=14336, vocab=128256), std=0.02,
                               K=4096, N=14336),
    "q4_llama8b_step_m16": dict(kind=4, M=16, step=dict(layers=32, dim=4096, kv=1024, ffn=14336, vocab=128256), std=0.02,
                                K=4096, N=14336),       # the same step at batch 16 (single GPU)
    # the projections of a 70B-Llama-shaped decode step (80 layers + lm_head, 52.1 GB)
    "q4_llama70b_step_m1": dict(kind=4, M=1, step=dict(layers=80, dim=8192, kv=1024, ffn=28672, vocab=128256), std=0.015,
                                K=8192, N=28672),
}
# The packers by themselves (quantizeQ4 / quantizeQ8 on a weight of the decode GEMV's shape and of the lm_head's)
WORKLOADS.update({
    "pack_q4_4096x14336": dict(kind=4, pack=True, M=0, K=4096, N=14336, std=0.02),
    "pack_q8_4096x14336": dict(kind=8, pack=True, M=0, K=4096, N=14336, std=0.02),
    "pack_q4_4096x128256": dict(kind=4, pack=True, M=0, K=4096, N=128256, std=0.02),
})
# The unquantised sibling (src/ops/matmul.js): one dense product per step
WORKLOADS.update({
    "dense_f32_4096x4096x4096": dict(dense="f32", M=4096, K=4096, N=4096, kind=0, std=1.0),
    "dense_f16_4096x4096x4096": dict(dense="f16", M=4096, K=4096, N=4096, kind=0, std=1.0),
    "dense_f32_512x4096x11008": dict(dense="f32", M=512, K=4096, N=11008, kind=0, std=1.0),
})
DEFAULT = "q4_decode_gemv_4096x14336_m1"
L2_BYTES = 126e6


def algorithmic(kind, M, K, N):
    bb = 24 if kind == 4 else 34
    nbytes = ((K + 31) // 32) * N * bb + 4 * M * K + 4 * M * N
    return nbytes, 2 * M * K * N


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm=d["hbm_gbs"], tensor=d["bf16_tflops"],
                    tensor_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]), source="measured")
    return dict(hbm=6650.0, tensor=1590.0, tensor_sustained=1400.0, source="fallback")


def traffic_for(name):
    """DRAM bytes per launch of the dominant kernel from the committed ncu summary, or None."""
    p = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(p):
        return json.load(open(p)).get(name)
    return None


class ClockSampler:
    """Samples nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm = [float(r[1]) for r in self.rows if len(r) >= 8 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 8 and r[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 8 for n, v in zip(names, r[4:8]) if v.lower() == "active"})
        pw = [float(r[3]) for r in self.rows if len(r) >= 8 and r[3].replace(".", "").isdigit()]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm), "power_w_max": max(pw) if pw else None}


# ----------------------------------------------------------------------------- CPU arms
def cpu_run(kind, M, K, N, seconds, threads=None):
    """Times the reference's CPU arithmetic on one packed matrix of the workload's shape.

    Uses oracle/_ref (the reference's shader source compiled as C++) when built,
    else the oracle port.  For shapes whose full run is long, a column window is
    timed and scaled; `sample` says what ran."""
    import numpy as np
    from oracle import oracle as O
    knd = "q4" if kind == 4 else "q8"
    threads = threads or O.host_threads()      # not omp_get_max_threads(): launchers export OMP_NUM_THREADS=1
    use_ref = O.have_ref()
    fn = O.ref_matmul if use_ref else O.matmul
    rng = np.random.default_rng(0)
    macs = M * K * N
    cols = N
    budget = 4e9 * threads / 8          # MACs that finish in a few seconds on these cores
    if macs > budget:
        cols = max(64, int(N * budget / macs) // 64 * 64)
    w = (rng.standard_normal((K, cols)) * 0.02).astype(np.float32)
    packed = O.quantize_q4(w) if kind == 4 else O.quantize_q8(w)
    a = rng.standard_normal((M, K)).astype(np.float32)
    fn(a, packed, K, cols, knd, threads=threads)   # warm
    reps, t0 = 0, time.perf_counter()
    while True:
        fn(a, packed, K, cols, knd, threads=threads)
        reps += 1
        el = time.perf_counter() - t0
        if el >= seconds:
            break
    per_call = el / reps * (N / cols)
    sample = (f"{reps} runs of {'all' if cols == N else str(cols) + ' of ' + str(N)} columns"
              f"{'' if cols == N else ' (time scaled to all columns)'}, {el:.1f} s of CPU work")
    return per_call, threads, ("reference" if use_ref else "port"), sample


def metric_of(kind, M, K, N, seconds_per_call):
    nbytes, flops = algorithmic(kind, M, K, N)
    if M <= 16:
        return nbytes / seconds_per_call / 1e9, "GB/s"
    return flops / seconds_per_call / 1e12, "TFLOP/s"


def metric_name(M):
    return ("Q4/Q8 matmul HBM GB/s (algorithmic bytes / time)" if M <= 16
            else "Q4/Q8 matmul TFLOP/s (2*M*K*N / time)")


def run_reference_arm(args, wl, name):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    if wl.get("pack"):
        print(json.dumps({"impl": "reference", "unavailable": "the reference's packer is JavaScript and no JS runtime is "
                          "installed; its C restatement is timed as cpu_baseline of the packer workload itself"}))
        return
    if wl.get("dense"):
        import numpy as np
        from oracle import oracle as O
        f16 = wl["dense"] == "f16"
        M, K, N, rows = wl["M"], wl["K"], wl["N"], 8
        rng = np.random.default_rng(5)
        a = rng.standard_normal((rows, K)).astype(np.float16 if f16 else np.float32)
        b = rng.standard_normal((K, N)).astype(a.dtype)
        times = []
        for i in range(args.warmup + args.steps):
            t0 = time.perf_counter()
            O.dense_matmul(a, b)
            if i >= args.warmup:
                times.append(time.perf_counter() - t0)
        per = sum(times) / len(times)
        value = 2.0 * rows * N * K / per / 1e12
        sample = f"{rows} of {M} rows per step (the sequential-sum restatement of shaders/matmul.metal, all host threads)"
        print(json.dumps({
            "impl": "reference", "metric": "dense matmul TFLOP/s (2 M N K / time)", "value": value, "unit": "TFLOP/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": per * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": name, "M": M, "K": K, "N": N, "note": "the reference's Metal path is unavailable on this box"},
            "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": O.max_threads(), "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}))
        return
    times = []
    info = None
    for i in range(args.warmup + args.steps):
        per_call, threads, kind, sample = cpu_run(wl["kind"], wl["M"], wl["K"], wl["N"], seconds=1.0)
        info = (threads, kind, sample)
        if i >= args.warmup:
            times.append(per_call)
    per_call = sum(times) / len(times)
    value, unit = metric_of(wl["kind"], wl["M"], wl["K"], wl["N"], per_call)
    threads, kind, sample = info
    line = {
        "impl": "reference", "metric": metric_name(wl["M"]), "value": value, "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_call * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": name, "kind": f"q{wl['kind']}", "M": wl["M"], "K": wl["K"], "N": wl["N"],
                   "note": "the reference's own CPU implementation of the path (its matmul shader source compiled "
                           "as C++ when oracle/_ref is built, else the C restatement), all host threads; "
                           "the reference's Metal path is unavailable on this box"},
        "cpu_baseline": {"value": value, "unit": unit, "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------- decode-step workload
def run_step_list(args, wl, ctxinfo, name=None, steps=None, with_cpu=True):
    """One GPU, M <= 4: the whole decode step's projections as ONE persistent launch with the
    reference's pointwise glue folded in (src/gguf_cache.js:121-171): per layer
        q, k, v = rmsnorm(x, ln1) W{q,k,v};   x2 = x + attn Wo;
        h = silu(rmsnorm(x2, ln2) Wgate) * (rmsnorm(x2, ln2) Wup);   x = x2 + h Wdown
    then logits = rmsnorm(x, lnF) Wlm_head.  Attention itself is outside the path: a fixed synthetic
    row stands in for its output.  Hazards between the items (x, x2, h are written and read by
    consecutive items) are resolved on the device."""
    import numpy as np
    import torch
    import smith_b200 as smith
    from oracle import oracle as O
    from smith_b200 import device as D
    kind, M, st = wl["kind"], wl["M"], wl["step"]
    dim, kv, ffn, vocab, layers = st["dim"], st["kv"], st["ffn"], st["vocab"], st["layers"]
    bb, eps = 24, 1e-5
    stream = ctxinfo[3]
    name = name or args.workload
    steps = steps or min(args.steps, 200)
    warm = max(min(args.warmup, 10), 3)
    owned = []                                        # every buffer made here, released before returning

    def alloc(n):
        b = D.alloc(n, D.PRIVATE)
        owned.append(b)
        return b

    wtmp = alloc(max(dim * ffn, dim * vocab) * 4)
    seed = [17]
    weight_bytes, alg_bytes = [0], [0]

    def make(k, n):
        D.fillNormal(wtmp, k * n, seed[0], wl["std"])
        seed[0] += 1
        pk = alloc((k // 32) * n * bb)
        D.q4Pack(wtmp, pk, k, n)
        weight_bytes[0] += (k // 32) * n * bb
        alg_bytes[0] += (k // 32) * n * bb + 4 * M * k + 4 * M * n
        return pk

    def vec(n, sd, value):
        b = alloc(n * 4)
        D.fillNormal(b, n, sd, 0.05)
        v = D.download(b, n * 4, np.float32) + value
        D.upload(b, v.astype(np.float32))
        return b

    xs = [alloc(M * dim * 4) for _ in range(2)]
    x2, attn = alloc(M * dim * 4), alloc(M * dim * 4)
    q, k_, v_, h = (alloc(M * n * 4) for n in (dim, kv, kv, ffn))
    logits = alloc(M * vocab * 4)
    x0 = alloc(M * dim * 4)
    D.fillNormal(x0, M * dim, 7, 1.0)
    D.fillNormal(attn, M * dim, 8, 1.0)
    items = []
    for l in range(layers):
        ln1, ln2 = vec(dim, 100 + 2 * l, 1.0), vec(dim, 101 + 2 * l, 1.0)
        x_in, x_out = (x0 if l == 0 else xs[l & 1]), xs[(l + 1) & 1]
        items += [D.listItem(x_in, make(dim, dim), q, dim, dim, gamma=ln1, eps=eps),
                  D.listItem(x_in, make(dim, kv), k_, kv, dim, gamma=ln1, eps=eps),
                  D.listItem(x_in, make(dim, kv), v_, kv, dim, gamma=ln1, eps=eps),
                  D.listItem(attn, make(dim, dim), x2, dim, dim, residual=x_in),
                  D.listItem(x2, make(dim, ffn), h, ffn, dim, b2=make(dim, ffn), gamma=ln2, eps=eps),
                  D.listItem(h, make(ffn, dim), x_out, dim, ffn, residual=x2)]
    lnf = vec(dim, 99, 1.0)
    x_last = xs[layers & 1]
    head = make(dim, vocab)
    items.append(D.listItem(x_last, head, logits, vocab, dim, gamma=lnf, eps=eps))
    D.synchronize()
    lst = D.qmatmulListCreate(kind, M, items)

    def sync():
        D.synchronize()
        torch.cuda.synchronize()

    D.qmatmulListRun(lst)
    sync()
    if D.kernelStatus() != 0:
        raise SystemExit("a bounded device-side wait gave up during warm-up")
    # ---- parity before timing: a window of the logits against the oracle on the device's own final row
    xf = D.download(x_last, M * dim * 4, np.float32).reshape(M, dim)
    gf = D.download(lnf, dim * 4, np.float32)
    c0 = (vocab // 2) // 8 * 8
    cols = np.concatenate([D.download(head, 48 * bb, np.uint8, offset=(g * vocab + c0) * bb) for g in range(dim // 32)])
    nrm = O.rmsnorm(xf, gf, eps)
    want = O.matmul(nrm, cols, dim, 48, "q4", threads=O.host_threads())
    got = D.download(logits, M * vocab * 4, np.float32).reshape(M, vocab)
    bound = O.tolerance_bound(nrm, O.dequant(cols, dim, 48, "q4"), 1e-3)
    worst = float((np.abs(got[:, c0:c0 + 48].astype(np.float64) - want) / np.maximum(bound, 1e-300)).max())
    parity = {"checked": True, "worst_err_over_bound": worst, "ok": bool(worst <= 1.0 and np.all(np.isfinite(got))),
              "what": "48 logits of the step (rmsnorm + lm_head on the residual row the device produced through "
                      "all layers) against the CPU oracle; bound = 1e-3 * ||x_m|| * ||w_deq[:,n]||"}
    if not parity["ok"]:
        raise SystemExit(f"parity check failed before timing: {parity}")
    for _ in range(warm):
        D.qmatmulListRun(lst)
    sync()
    sampler = ClockSampler(ctxinfo[2])
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(30 if layers <= 32 else 6):        # settle: some tens of ms, so the clock samples see load
        D.qmatmulListRun(lst)
    e0.record(stream)
    for _ in range(steps):
        D.qmatmulListRun(lst)
    e1.record(stream)
    sync()
    ms = e0.elapsed_time(e1)
    # ---- end to end: the step's input row from page-locked host memory, the launch, the logits back
    x_np = D.download(x0, M * dim * 4, np.float32)

    def e2e_pass():
        D.upload(x0, x_np)
        D.qmatmulListRun(lst)
        D.synchronize()
        return D.download(logits, M * vocab * 4, np.float32)

    for _ in range(2):
        e2e_pass()
    e2e_steps = max(3, min(steps, 50))
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_pass()
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop()
    if D.kernelStatus() != 0:
        raise SystemExit("a bounded device-side wait gave up: results invalid")
    step_s = ms * 1e-3 / steps
    peaks = measured_peaks()
    ach = alg_bytes[0] / step_s / 1e9
    line = {
        "metric": "Q4 decode step HBM GB/s (algorithmic bytes of all projections / time)",
        "value": ach, "unit": "GB/s", "n_gpus": 1, "steps": steps, "warmup": warm, "ms_per_step": step_s * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": DTYPE_NOTE["gemv"], "data": "synthetic",
        "config": {"workload": name, "kind": "q4", "M": M, "layers": layers, "dim": dim, "kv_dim": kv, "ffn": ffn,
                   "vocab": vocab, "matmuls_per_step": 7 * layers + 1, "launches_per_step": 1, "items_per_launch": len(items),
                   "form": "list: every projection of the step in ONE persistent launch; RMSNorm folded into the "
                           "q/k/v, gate/up and lm_head items, SwiGLU into the gate/up item, the residual adds into the "
                           "wo and down items; hazards between items resolved on the device",
                   "packed_bytes_per_gpu": weight_bytes[0], "tokens_per_s": M / step_s, "sharding": "single GPU",
                   "l2": "every item reads its own packed matrix; one step's weights are %d x the 126 MB L2"
                         % (weight_bytes[0] // L2_BYTES),
                   "timing": "CUDA events on the launch stream around the timed launches"},
        "parity": parity,
        "e2e": {"value": alg_bytes[0] / (e2e_s / e2e_steps) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": 4 * M * dim,
                "d2h_bytes_per_step": 4 * M * vocab, "steps": e2e_steps,
                "note": "per step: H2D of the input row from page-locked memory, the launch, wait, D2H of the logits"},
        "gpu_launches": int(steps + e2e_steps + warm + 3),
        "roofline": {"bound": "hbm", "achieved": ach, "peak": peaks["hbm"], "unit": "GB/s", "frac": ach / peaks["hbm"],
                     "traffic": None,
                     "peak_source": f"{peaks['source']} (MEASURED_PEAKS.json)" if peaks["source"] == "measured"
                     else "fallback (no MEASURED_PEAKS.json)",
                     "peak_kind": "copy bandwidth", "frac_of_nominal": ach / 8000.0,
                     "algorithmic_per_launch": alg_bytes[0], "launch_us": step_s * 1e6},
        "clocks": clocks,
    }
    if with_cpu and not args.no_cpu:
        per_call, threads, ckind, sample = cpu_run(kind, M, dim, ffn, seconds=args.cpu_seconds)
        gate_bytes = algorithmic(kind, M, dim, ffn)[0]
        line["cpu_baseline"] = {"value": gate_bytes / per_call / 1e9, "unit": "GB/s", "cores": threads, "kind": ckind,
                                "sample": "the step's gate projection (%d x %d): " % (dim, ffn) + sample}
    else:
        line["cpu_baseline"] = None
    D.qmatmulListDestroy(lst)
    for b in owned:
        D.releaseBuffer(b)
    return line


def run_step_workload(args, wl, ctxinfo, name=None, steps=None, with_cpu=True):
    """One decode step's projection list, one launch per projection group: per layer wq, wk, wv, wo,
    gate, up, down, then lm_head (wq/wk/wv share a launch, gate/up share one).  Several GPUs: tensor
    parallel -- wq/wk/wv/gate/up column-sharded (outputs stay sharded), wo/down sharded along K with the
    all-reduce fused into the GEMV kernel, lm_head column-sharded with the all-gather fused into the
    GEMV kernel.  On one GPU with M <= 4 the step runs as a list instead (run_step_list)."""
    import numpy as np
    import torch
    import torch.distributed as dist
    world, rank, local, stream = ctxinfo
    name = name or args.workload
    if world == 1 and wl["M"] <= 4 and not args.no_list:
        return run_step_list(args, wl, ctxinfo, name=name, steps=steps, with_cpu=with_cpu)
    import smith_b200 as smith
    from smith_b200 import device as D
    from smith_b200 import parallel as P
    kind, M, st = wl["kind"], wl["M"], wl["step"]
    if M > 4 and world > 1:
        raise SystemExit("the step workloads shard over GPUs with the GEMV kernel's fused collectives (M <= 4)")
    dim, kv, ffn, vocab, layers = st["dim"], st["kv"], st["ffn"], st["vocab"], st["layers"]
    bb = 24
    steps = steps or min(args.steps, 200)
    warm = max(min(args.warmup, 10), 3)

    def shard_n(N):
        a, b = P.column_shard(N, world, rank)
        return b - a

    def shard_k(K):
        g0, g1 = P.group_shard(K // 32, world, rank)
        return (g1 - g0) * 32

    # (name, K_local, N_local, K_full, N_full, collective)
    per_layer = [("wq", dim, shard_n(dim), dim, dim, None), ("wk", dim, shard_n(kv), dim, kv, None),
                 ("wv", dim, shard_n(kv), dim, kv, None), ("wo", shard_k(dim), dim, dim, dim, "reduce"),
                 ("gate", dim, shard_n(ffn), dim, ffn, None), ("up", dim, shard_n(ffn), dim, ffn, None),
                 ("down", shard_k(ffn), dim, ffn, dim, "reduce")]
    head = ("lm_head", dim, shard_n(vocab), dim, vocab, "gather")
    biggest = max(k * n for _, k, n, _, _, _ in per_layer + [head])
    wtmp = D.alloc(biggest * 4, D.PRIVATE)
    seed = [17 + rank]

    def make(kl, nl):
        D.fillNormal(wtmp, kl * nl, seed[0], wl["std"])
        seed[0] += world
        pk = D.alloc((kl // 32) * nl * bb, D.PRIVATE)
        D.q4Pack(wtmp, pk, kl, nl)
        return pk

    x_dim = D.alloc(M * dim * 4, D.PRIVATE)          # activations of width dim / ffn (synthetic, replicated)
    x_ffn = D.alloc(M * ffn * 4, D.PRIVATE)
    D.fillNormal(x_dim, M * dim, 7, 1.0)
    D.fillNormal(x_ffn, M * ffn, 8, 1.0)
    y = D.alloc(M * max(ffn, dim, shard_n(vocab)) * 4, D.PRIVATE)
    y2 = [D.alloc(M * max(ffn, dim) * 4, D.PRIVATE) for _ in range(2)]     # second and third output of a shared launch
    ops, weight_bytes, alg_bytes = [], 0, 0
    reducers = {}
    # projections that read the same activations go out as one launch (smith_qmatmul_multi)
    shared = {"wq": "qkv", "wk": "qkv", "wv": "qkv", "gate": "gate_up", "up": "gate_up"}
    for layer in range(layers):
        open_group = None
        for name, kl, nl, kf, nf, coll in per_layer:
            pk = make(kl, nl)
            weight_bytes += (kl // 32) * nl * bb
            alg_bytes += (kl // 32) * nl * bb + 4 * M * kl + 4 * M * nl
            grp = shared.get(name)
            if grp and open_group and open_group[0] == grp:
                open_group[1].append(pk)
                open_group[3].append(nl)
                continue
            open_group = (grp or name, [pk], kl, [nl], coll)
            ops.append(open_group)
    pk = make(head[1], head[2])
    weight_bytes += (head[1] // 32) * head[2] * bb
    alg_bytes += (head[1] // 32) * head[2] * bb + 4 * M * head[1] + 4 * M * head[2]
    ops.append((head[0], [pk], head[1], [head[2]], head[5]))
    D.synchronize()
    D.releaseBuffer(wtmp)
    if world > 1:
        reducers["wo"] = P.FusedReduce(kind, M, dim, shard_k(dim), world, rank)
        reducers["down"] = P.FusedReduce(kind, M, dim, shard_k(ffn), world, rank)
        gather = P.FusedGather(M, vocab, world, rank, deferred=True)

    def one_pass():
        for name, pks, kl, nls, coll in ops:
            src = x_ffn if name == "down" else x_dim       # the K-slice a rank reads is the head of the buffer
            if world > 1 and coll == "reduce":
                reducers[name].enqueue(src, pks[0], y)
            elif world > 1 and coll == "gather":
                gather.enqueue(kind, src, pks[0], kl)
            elif len(pks) > 1:
                D.qmatmulMulti(kind, src, pks, ([y] + y2)[:len(pks)], nls, M, kl, kl // 32)
            else:
                D.qmatmul(kind, src, pks[0], y, M, nls[0], kl, kl // 32, D.PATH_AUTO)
        if world > 1:
            gather.finish()

    def barrier():
        D.synchronize()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    one_pass()
    D.synchronize()
    if D.kernelStatus() != 0:
        raise SystemExit("a bounded device-side wait gave up during warm-up")
    # ---- parity before timing (values, not only "no wait gave up")
    from oracle import oracle as O
    parity = None

    def window(pk, kl, nl, c0, width=48):
        c1 = min(nl, c0 + width)
        return np.concatenate([D.download(pk, (c1 - c0) * bb, np.uint8, offset=(g * nl + c0) * bb)
                               for g in range(kl // 32)]), c1 - c0

    if world > 1:
        # (1) K-sharded product with the fused all-reduce: every rank forms the oracle's partial product of
        # its own shard on the CPU, the partials are summed over the ranks, and every rank compares the
        # row its kernel produced with that sum.
        nm, pks, kl, nls, _ = next(o for o in ops if o[4] == "reduce")
        src = x_ffn if nm == "down" else x_dim
        reducers[nm].enqueue(src, pks[0], y)
        D.synchronize()
        cols, wd = window(pks[0], kl, nls[0], 0)
        a_loc = D.download(src, M * kl * 4, np.float32).reshape(M, kl)
        part = torch.tensor(O.matmul(a_loc, cols, kl, wd, "q4", threads=O.host_threads()).astype(np.float64), device="cuda")
        wsq = torch.tensor((O.dequant(cols, kl, wd, "q4").astype(np.float64) ** 2).sum(0), device="cuda")
        asq = torch.tensor((a_loc.astype(np.float64) ** 2).sum(1), device="cuda")
        for t in (part, wsq, asq):
            dist.all_reduce(t)
        got = D.download(y, M * nls[0] * 4, np.float32).reshape(M, nls[0])[:, :wd]
        bound = 1e-3 * np.sqrt(asq.cpu().numpy())[:, None] * np.sqrt(wsq.cpu().numpy())[None, :]
        worst_r = float((np.abs(got.astype(np.float64) - part.cpu().numpy()) / np.maximum(bound, 1e-300)).max())
        # (2) the gathered logits: a window of this rank's own slice, read from the gathered row
        one_pass()
        D.synchronize()
        row = gather.read()
        nm, pks, kl, nls, _ = ops[-1]
        n0g = P.column_shard(vocab, world, rank)[0]
        c0 = (nls[0] // 2) // 8 * 8
        cols, wd = window(pks[0], kl, nls[0], c0)
        a_loc = D.download(x_dim, M * kl * 4, np.float32).reshape(M, kl)
        want = O.matmul(a_loc, cols, kl, wd, "q4", threads=O.host_threads())
        bnd = O.tolerance_bound(a_loc, O.dequant(cols, kl, wd, "q4"), 1e-3)
        worst_g = float((np.abs(row[:, n0g + c0:n0g + c0 + wd].astype(np.float64) - want) / np.maximum(bnd, 1e-300)).max())
        w = torch.tensor([worst_r, worst_g, 0.0 if np.all(np.isfinite(row)) else 2.0], device="cuda")
        dist.all_reduce(w, op=dist.ReduceOp.MAX)
        worst_r, worst_g, bad = (float(v) for v in w.cpu())
        parity = {"checked": True, "worst_err_over_bound": max(worst_r, worst_g, bad), "ok": bool(max(worst_r, worst_g, bad) <= 1.0),
                  "all_reduce_worst": worst_r, "all_gather_worst": worst_g,
                  "what": "max over ranks: 48 columns of a K-sharded product (fused all-reduce) against the sum of the ranks' "
                          "oracle partials, and 48 logits of each rank's slice read from its gathered row; bound = 1e-3 * ||a|| * ||w_deq[:,n]||"}
        if not parity["ok"]:
            raise SystemExit(f"parity check failed before timing: {parity}")
    D.graphBegin()
    one_pass()
    graph = D.graphEnd()
    for _ in range(warm):
        D.graphLaunch(graph)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        D.graphLaunch(graph)
    e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    # ---- end to end: the step's input row from page-locked host memory, all projections, the logits back
    x_host = smith.tensorFrom(D.download(x_dim, M * dim * 4, np.float32), [M, dim])
    x_np = smith.toNumpy(x_host)
    n_logits = M * (vocab if world > 1 else head[2])

    def e2e_pass():
        D.upload(x_dim, x_np)
        D.graphLaunch(graph)
        D.synchronize()
        if world > 1:
            return gather.read()
        return D.download(y, n_logits * 4, np.float32)

    for _ in range(2):
        e2e_pass()
    barrier()
    e2e_steps = max(3, min(steps, 50))
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_pass()
    barrier()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    clocks = sampler.stop() if rank == 0 else None
    if D.kernelStatus() != 0:
        raise SystemExit("a bounded device-side wait gave up: results invalid")
    if world > 1:
        tot = torch.tensor([float(alg_bytes)], device="cuda")
        dist.all_reduce(tot)
        alg_all = float(tot.item())
    else:
        alg_all = float(alg_bytes)
    if rank == 0:
        step_s = ms * 1e-3 / steps
        peaks = measured_peaks()
        ach = alg_bytes / step_s / 1e9                       # this rank's kernels against this GPU's HBM
        line = {
            "metric": "Q4 decode step HBM GB/s (algorithmic bytes of all projections / time)",
            "value": alg_all / step_s / 1e9, "unit": "GB/s", "n_gpus": world, "steps": steps, "warmup": warm,
            "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": DTYPE_NOTE["gemv" if M <= 4 else "decode"], "data": "synthetic",
            "config": {"workload": name, "kind": "q4", "M": M, "layers": layers, "dim": dim, "kv_dim": kv,
                       "ffn": ffn, "vocab": vocab, "matmuls_per_step": 7 * layers + 1, "launches_per_step": len(ops),
                       "packed_bytes_per_gpu": weight_bytes, "tokens_per_s": M / step_s,
                       "sharding": ("tensor parallel over %d GPUs: wq/wk/wv/gate/up column-sharded, wo/down K-sharded "
                                    "with the all-reduce fused into the GEMV kernel, lm_head column-sharded with the "
                                    "all-gather fused into the GEMV kernel" % world) if world > 1 else "single GPU",
                       "l2": "every launch reads its own packed matrix; one step's weights are %d x the 126 MB L2"
                             % (weight_bytes * world // L2_BYTES),
                       "timing": "CUDA events on the launch stream around replays of one CUDA graph per step, "
                                 "max over ranks"},
            "e2e": {"value": alg_all / (e2e_s / e2e_steps) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": 4 * M * dim * world,
                    "d2h_bytes_per_step": 4 * n_logits * world, "steps": e2e_steps,
                    "note": "per step: H2D of the input row from page-locked memory, graph launch, wait, D2H of the logits"},
            "parity": parity,
            "gpu_launches": int((steps + e2e_steps) * len(ops)),
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peaks["hbm"], "unit": "GB/s", "frac": ach / peaks["hbm"],
                         "traffic": None,
                         "peak_source": f"{peaks['source']} (MEASURED_PEAKS.json)" if peaks["source"] == "measured"
                         else "fallback (no MEASURED_PEAKS.json)",
                         "peak_kind": "copy bandwidth", "frac_of_nominal": ach / 8000.0,
                         "algorithmic_per_launch": alg_bytes / len(ops),
                         "note": "all %d launches of a step taken together" % len(ops)},
            "clocks": clocks,
        }
        if world == 1 and with_cpu and not args.no_cpu:
            per_call, threads, ckind, sample = cpu_run(kind, M, dim, ffn, seconds=args.cpu_seconds)
            gate_bytes = algorithmic(kind, M, dim, ffn)[0]
            line["cpu_baseline"] = {"value": gate_bytes / per_call / 1e9, "unit": "GB/s", "cores": threads, "kind": ckind,
                                    "sample": "the step's gate projection (%d x %d): " % (dim, ffn) + sample}
        else:
            line["cpu_baseline"] = None
        return line
    return None


# ----------------------------------------------------------------------------- GPU arm
DTYPE_NOTE = {
    "gemv": "f32 accumulate; activations rounded to 15-bit block fixed point (two int8 digits per group of 32), "
            "integer-exact group sums over u4/i8 codes",
    "decode": "f32 accumulate; activations rounded to 15-bit block fixed point, integer mma.sync over u4/i8 codes",
    "tensor4": "f32 accumulate (TMEM) over bf16 activations and bf16 de-quantised u4 weights",
    "tensor8": "f32 accumulate (TMEM) over f16 activations and f16 de-quantised i8 weights",
    "generic": "f32 sequential accumulate over u4/i8 codes",
}


def parity_window(D, O, kind, M, K, Nl, a_dev, pack, read_out, c0=None, width=48):
    """Compares columns [c0, c0 + width) of one product with the CPU oracle (same f32 activations, the
    packed bytes of those columns brought back from the device).  Returns worst err / bound, where
    bound = 1e-3 * ||a_m|| * ||w_deq[:, n]||."""
    import numpy as np
    bb = 24 if kind == 4 else 34
    G = K // 32
    c0 = ((Nl // 2) // 8 * 8) if c0 is None else c0
    c1 = min(Nl, c0 + width)
    cols = np.empty((G, (c1 - c0) * bb), np.uint8)
    for g in range(G):
        cols[g] = D.download(pack, (c1 - c0) * bb, np.uint8, offset=(g * Nl + c0) * bb)
    cols = cols.reshape(-1)
    a = D.download(a_dev, M * K * 4, np.float32).reshape(M, K)
    knd = "q4" if kind == 4 else "q8"
    want = O.matmul(a, cols, K, c1 - c0, knd, threads=O.host_threads())
    got = read_out(c0, c1)
    bound = O.tolerance_bound(a, O.dequant(cols, K, c1 - c0, knd), 1e-3)
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    return float((err / np.maximum(bound, 1e-300)).max())


SETTLE_S = float(os.environ.get("SMITH_BENCH_SETTLE_S", "0.06"))


def settle_steps(step_s, world, torch, dist):
    """How many untimed steps make SETTLE_S of load just before the timed region, so that the
    clock samples (one per 20 ms) see load even when the timed region itself is a few milliseconds."""
    n = int(min(200000, max(0, SETTLE_S / max(step_s, 1e-7))))
    if world > 1:
        t = torch.tensor([n], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        n = int(t.item())
    return n


def run_matrix_workload(args, name, wl, steps, warm, ctxinfo, with_cpu=True, with_e2e=True, sampler_on=True):
    """One workload of R products of one shape; returns the JSON line as a dict (rank 0) or None."""
    import numpy as np
    import torch
    import torch.distributed as dist
    import smith_b200 as smith
    from oracle import oracle as O
    from smith_b200 import device as D
    from smith_b200 import parallel as P
    world, rank, local, stream = ctxinfo
    kind, M, K, N = wl["kind"], wl["M"], wl["K"], wl["N"]
    bb = 24 if kind == 4 else 34
    G = K // 32
    n0, n1 = P.column_shard(N, world, rank)      # this rank's output columns
    Nl = n1 - n0
    wbytes_full = G * N * bb
    R = max(2, int(-(-4 * L2_BYTES // wbytes_full)))
    if M <= 4:
        R = max(R, 16)                           # a list of at least 16 products per step

    # ---- synthetic weights: generated and packed on the device, shard by shard
    wtmp = D.alloc(K * Nl * 4, D.PRIVATE)
    packs = []
    for i in range(R):
        D.fillNormal(wtmp, K * Nl, 1000 * (i + 1) + rank, wl["std"])
        pk = D.alloc(G * Nl * bb, D.PRIVATE)
        (D.q4Pack if kind == 4 else D.q8Pack)(wtmp, pk, K, Nl)
        packs.append(pk)
    D.synchronize()
    D.releaseBuffer(wtmp)
    a_dev = D.alloc(M * K * 4, D.PRIVATE)
    D.fillNormal(a_dev, M * K, 7, 1.0)            # same seed on every rank: replicated activations
    # Several GPUs: the list kernel gathers its own outputs over peer memory (M <= 4, ShardedList);
    # with --no-list every launch of the GEMV kernel does (FusedGather); wider M uses NCCL.
    shards_ok = all(D.qmatmulListSupports(kind, M, b - a, K) for a, b in (P.column_shard(N, world, r) for r in range(world)))
    use_list = M <= 4 and shards_ok and not args.no_list
    gather, fused, slist = None, False, None
    if world > 1 and use_list:
        slist = P.ShardedList(kind, M, K, N, packs, world, rank, a_dev)
    elif world > 1:
        fused = M <= 4 and all(D.qgemvTiles(kind, M, b - a, K) > 0
                               for a, b in (P.column_shard(N, world, r) for r in range(world)))
        gather = P.FusedGather(M, N, world, rank, deferred=True) if fused else P.OutputGather(M, N, world, rank)
    outs = [D.alloc(M * Nl * 4, D.PRIVATE) for _ in range(R)] if (use_list and not slist) else []
    c_dev = (outs[0] if outs else D.alloc(M * Nl * 4, D.PRIVATE)) if (not gather or fused) else gather.local_buf
    lst = D.qmatmulListCreate(kind, M, [D.listItem(a_dev, pk, c, Nl, K) for pk, c in zip(packs, outs)]) if outs else None

    def launches_pass():
        for pk in packs:
            if fused:
                gather.enqueue(kind, a_dev, pk, K)
            else:
                D.qmatmul(kind, a_dev, pk, c_dev, M, Nl, K, G, D.PATH_AUTO)
                if gather:
                    gather.enqueue()
        if fused:
            gather.finish()                       # the last launch's row is whole when the pass ends

    graph = None
    if not slist:
        launches_pass()                           # sizes scratch before capture
        D.synchronize()
        if D.kernelStatus() != 0:
            raise SystemExit("a bounded device-side wait gave up during warm-up")
        if not gather or gather.capturable:
            D.graphBegin()
            launches_pass()
            graph = D.graphEnd()

    def per_call_step():
        if graph:
            D.graphLaunch(graph)
        else:
            launches_pass()

    def list_step():
        if slist:
            slist.run()
        else:
            D.qmatmulListRun(lst)

    step = list_step if use_list else per_call_step

    def barrier():
        D.synchronize()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    # ---- parity before timing: a column window of the last product of a step against the oracle
    step()
    barrier()
    if D.kernelStatus() != 0:
        raise SystemExit("a bounded device-side wait gave up")
    parity = None
    if rank == 0:
        if slist:
            # the gathered row of the last product: this rank's window lies inside its own slice, and
            # every pair of the row (all ranks' slices) must carry the launch's tag
            row, tags = slist.read(R - 1)
            worst = parity_window(D, O, kind, M, K, Nl, a_dev, packs[-1], lambda c0, c1: row[:, n0 + c0:n0 + c1])
            whole = bool(np.all(np.isfinite(row)) and np.all(tags == tags[0]) and tags[0] > 0)
        elif gather and fused:
            # the gathered row (all ranks' slices): this rank's window lies inside its own slice
            row = gather.read()
            worst = parity_window(D, O, kind, M, K, Nl, a_dev, packs[-1], lambda c0, c1: row[:, n0 + c0:n0 + c1])
            whole = bool(np.all(np.isfinite(row)))
        elif gather:
            row = gather.full.cpu().numpy()
            worst = parity_window(D, O, kind, M, K, Nl, a_dev, packs[-1], lambda c0, c1: row[:, n0 + c0:n0 + c1])
            whole = bool(np.all(np.isfinite(row)))
        else:
            last = outs[-1] if use_list else c_dev
            full = D.download(last, M * Nl * 4, np.float32).reshape(M, Nl)
            worst = parity_window(D, O, kind, M, K, Nl, a_dev, packs[-1], lambda c0, c1: full[:, c0:c1])
            whole = bool(np.all(np.isfinite(full)))
        parity = {"checked": True, "worst_err_over_bound": worst, "ok": bool(worst <= 1.0 and whole),
                  "what": "48 columns of the last product of a step"
                          + (" (read from the gathered row)" if (gather or slist) else "") + " against the CPU oracle; "
                          "bound = 1e-3 * ||a_m|| * ||w_deq[:,n]||"}
        if not parity["ok"]:
            raise SystemExit(f"parity check failed before timing: {parity}")

    def timed(fn, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(n):
            fn()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for _ in range(warm):
        step()
    barrier()
    est = timed(step, 3) / 3 * 1e-3
    sampler = ClockSampler(local)
    if rank == 0 and sampler_on:
        sampler.start()
    settle = 0 if args.no_settle else settle_steps(est, world, torch, dist)
    for _ in range(settle):
        step()
    barrier()
    launches0 = D.launchCount()
    ms = timed(step, steps)
    launches_value = D.launchCount() - launches0
    if not use_list and graph:
        launches_value = steps * R * ((1 + gather.kernels_per_call) if gather else 1)
    # the same products as one launch each (graph replay), for comparison with the list form
    per_call = None
    if use_list and not slist:
        for _ in range(3):
            per_call_step()
        barrier()
        n_pc = max(3, min(steps, 200))
        ms_pc = timed(per_call_step, n_pc)
        launches_value += (3 + n_pc) * R
        pc_s = ms_pc * 1e-3 / (n_pc * R)
        per_call = {"us_per_matmul": pc_s * 1e6, "value": metric_of(kind, M, K, N, pc_s)[0],
                    "note": "the same R products as R launches replayed from one CUDA graph"}

    # ---- end to end through the operator API, host-resident activations and outputs
    e2e = None
    launches_e2e = 0
    if with_e2e:
        a_host = smith.tensorFrom(D.download(a_dev, M * K * 4, np.float32), [M, K])
        wqs = [smith.ops.quantize.Quantized(buffer=pk, K=K, N=Nl, groups=G, totalBytes=G * Nl * bb) for pk in packs]
        mm = smith.matmulQ4 if kind == 4 else smith.matmulQ8
        sharded = [P.ShardedMatmul(kind, K, N, pk, M, world, rank) for pk in packs] if world > 1 else None
        a_np = smith.toNumpy(a_host)

        def e2e_pass():
            if sharded:                       # multi-GPU: upload, shard matmul, all-gather, download full rows
                for sm in sharded:
                    sm.forward(a_np)
            else:                             # the reference's operator call
                for wq in wqs:
                    smith.dispose(mm(a_host, wq))

        for _ in range(2):
            e2e_pass()
        barrier()
        launches1 = D.launchCount()
        e2e_steps = max(3, min(steps, 100))
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_pass()
        barrier()
        e2e_s = time.perf_counter() - t0
        launches_e2e = D.launchCount() - launches1
        if world > 1:
            t = torch.tensor([e2e_s], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_s = float(t.item())
        e2e_value, e2e_unit = metric_of(kind, M, K, N, e2e_s / (e2e_steps * R))
        e2e = {"value": e2e_value, "unit": e2e_unit, "h2d_bytes_per_step": R * 4 * M * K * world,
               "d2h_bytes_per_step": R * 4 * M * (N if world > 1 else Nl) * world, "steps": e2e_steps,
               "us_per_call": e2e_s / (e2e_steps * R) * 1e6,
               "note": "operator API per call (matmulQ4 / matmulQ8 on host tensors): H2D activations from page-locked "
                       "memory, kernel, D2H result, wait"}
    clocks = sampler.stop() if (rank == 0 and sampler_on) else None
    if D.kernelStatus() != 0:
        raise SystemExit("a bounded device-side wait gave up: results invalid")

    line = None
    if rank == 0:
        per_launch_s = ms * 1e-3 / (steps * R)         # per product
        value, unit = metric_of(kind, M, K, N, per_launch_s)
        peaks = measured_peaks()
        nbytes_l, flops_l = algorithmic(kind, M, K, Nl)       # what this rank's kernel moves per product
        sustained = False
        if M <= 64:
            ach, peak, runit, bound = nbytes_l / per_launch_s / 1e9, peaks["hbm"], "GB/s", "hbm"
        else:
            # A long timed region runs under the power cap like the sustained cuBLAS loop the peak file
            # holds beside the burst figure; a short one is compared with the burst figure.
            sustained = ms > 100.0
            ach, peak, runit, bound = (flops_l / per_launch_s / 1e12,
                                       peaks["tensor_sustained"] if sustained else peaks["tensor"], "TFLOP/s", "tensor")
        pid = D.qmatmulPath(kind, M, Nl, K)
        path = {0: "auto", 1: "generic", 2: "decode_mma", 3: "tensor_tcgen05", 4: "gemv_dp4a"}[pid]
        dtype = DTYPE_NOTE[{1: "generic", 2: "decode", 3: "tensor4" if kind == 4 else "tensor8", 4: "gemv"}.get(pid, "generic")]
        per_kernel = R if use_list else 1                        # products one launch of the dominant kernel covers
        line = {
            "metric": metric_name(M), "value": value, "unit": unit, "n_gpus": world, "steps": steps,
            "warmup": warm, "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": dtype, "data": "synthetic",
            "config": {"workload": name, "kind": f"q{kind}", "M": M, "K": K, "N": N,
                       "products_per_step": R, "launches_per_step": 1 if use_list else R,
                       "form": ("list: the R products of a step run as ONE persistent launch (smith_qmatmul_list), "
                                "the ring of weight stages never drains between matrices") if use_list
                               else "one launch per product, R launches replayed from one CUDA graph",
                       "kernel": ("gemv_list_dp4a" if use_list else path), "per_call": per_call,
                       "sharding": (f"N-sharded over {world} GPU(s), all-gather of outputs "
                                    + ("fused into the list kernel: every item's epilogue stores its columns as {value, launch tag} "
                                       "pairs into every rank's row over peer memory (NVLink); the ranks meet once per launch, "
                                       "when each waits until its own rows are whole" if slist else
                                       ("fused into the GEMV kernel (peer stores over NVLink; each launch waits for its predecessor's "
                                        "tiles after its own weight stream has started, a final wait closes the step)" if fused
                                        else "by NCCL")))
                       if world > 1 else "single GPU",
                       "l2": f"defeated by rotating over {R} distinct packed matrices per step "
                             f"({R * wbytes_full / 1e6:.0f} MB > 4 x 126 MB L2)",
                       "settle_steps": settle,
                       "timing": "CUDA events on the launch stream around the timed steps, max over ranks; "
                                 "settle_steps untimed steps run just before, so the clock samples see load"},
            "parity": parity,
            "e2e": e2e,
            "gpu_launches": int(launches_value + launches_e2e),
            "roofline": {"bound": bound, "achieved": ach, "peak": peak, "unit": runit, "frac": ach / peak,
                         "traffic": (traffic_for(name + ("#list" if use_list else "")) if world == 1 else None),
                         "peak_source": f"{peaks['source']} (MEASURED_PEAKS.json)" if peaks["source"] == "measured"
                         else "fallback (no MEASURED_PEAKS.json)",
                         "peak_kind": ("copy bandwidth" if bound == "hbm" else
                                       ("sustained cuBLAS bf16 (timed region %.0f ms)" % ms if sustained
                                        else "burst cuBLAS bf16 (timed region %.0f ms)" % ms)),
                         "frac_of_nominal": ach / (8000.0 if bound == "hbm" else 2250.0),
                         "algorithmic_per_launch": (nbytes_l if bound == "hbm" else flops_l) * per_kernel,
                         "launch_us": per_launch_s * per_kernel * 1e6},
            "clocks": clocks,
        }
        if world == 1 and with_cpu and not args.no_cpu:
            per_call_cpu, threads, ckind, sample = cpu_run(kind, M, K, N, seconds=args.cpu_seconds)
            cv, cu = metric_of(kind, M, K, N, per_call_cpu)
            line["cpu_baseline"] = {"value": cv, "unit": cu, "cores": threads, "kind": ckind, "sample": sample}
        else:
            line["cpu_baseline"] = None
    # ---- give the memory back (secondary workloads follow in the same process)
    if lst:
        D.qmatmulListDestroy(lst)
    if graph:
        D.graphDestroy(graph)
    if slist:
        slist.close()
    for b in packs + outs + [a_dev] + ([] if (outs or (gather and not fused)) else [c_dev]):
        D.releaseBuffer(b)
    return line


def run_pack_workload(args, name, wl, ctxinfo):
    """quantizeQ4 / quantizeQ8 alone: f32 [K, N] on the device -> packed blocks.  A step packs one of three
    distinct weight matrices (each larger than L2).  Algorithmic bytes: 4 K N read + groups N block-bytes
    written.  The CPU arm is the packer's C restatement on ONE thread -- the reference's own execution model
    (src/ops/quantize.js:14-68 runs on the single JS thread) -- on a column window, scaled."""
    import numpy as np
    import torch
    import smith_b200 as smith
    from oracle import oracle as O
    from smith_b200 import device as D
    world, rank, local, stream = ctxinfo
    kind, K, N = wl["kind"], wl["K"], wl["N"]
    bb = 24 if kind == 4 else 34
    G = K // 32
    nbytes = 4 * K * N + G * N * bb
    pack = D.q4Pack if kind == 4 else D.q8Pack
    R = 3
    ws = [D.alloc(K * N * 4, D.PRIVATE) for _ in range(R)]
    for i, w in enumerate(ws):
        D.fillNormal(w, K * N, 50 + i, wl["std"])
    out = D.alloc(G * N * bb, D.PRIVATE)
    steps, warm = min(args.steps, 200), max(min(args.warmup, 10), 3)
    pack(ws[0], out, K, N)
    D.synchronize()
    # parity before timing: 64 columns of the packed matrix, bit for bit against the CPU packer
    c0 = (N // 2) // 8 * 8
    w_cols = np.stack([D.download(ws[0], 64 * 4, np.float32, offset=(k * N + c0) * 4) for k in range(K)])
    got = np.concatenate([D.download(out, 64 * bb, np.uint8, offset=(g * N + c0) * bb) for g in range(G)])
    want = O.quantize_q4(w_cols) if kind == 4 else O.quantize_q8(w_cols)
    parity = {"checked": True, "ok": bool(np.array_equal(got, want)), "what": "64 columns of packed blocks, bit-exact against the CPU packer"}
    if not parity["ok"]:
        raise SystemExit("packed bytes differ from the CPU packer")
    for i in range(warm):
        pack(ws[i % R], out, K, N)
    D.synchronize()
    sampler = ClockSampler(local)
    sampler.start()
    for i in range(30):
        pack(ws[i % R], out, K, N)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(steps):
        pack(ws[i % R], out, K, N)
    e1.record(stream)
    D.synchronize()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    # end to end through the operator: weights in page-locked host memory -> quantizeQ4 -> a read of the result's head
    w_host = smith.tensorFrom(D.download(ws[0], K * N * 4, np.float32), [K, N])
    quant = smith.quantizeQ4 if kind == 4 else smith.quantizeQ8
    e2e_steps = 3

    def e2e_pass():
        q = quant(w_host)
        head = D.download(q.buffer, 4096, np.uint8)
        D.releaseBuffer(q.buffer)
        return head

    e2e_pass()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_pass()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    clocks = sampler.stop()
    step_s = ms * 1e-3 / steps
    peaks = measured_peaks()
    ach = nbytes / step_s / 1e9
    line = {
        "metric": "quantizeQ4/Q8 packer HBM GB/s (4 K N read + packed bytes written / time)", "value": ach, "unit": "GB/s",
        "n_gpus": 1, "steps": steps, "warmup": warm, "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f64 arithmetic (the reference packs with JS numbers), u4/i8 codes, f32/f16 scales",
        "data": "synthetic",
        "config": {"workload": name, "kind": f"q{kind}", "K": K, "N": N, "launches_per_step": 1,
                   "l2": "three distinct f32 matrices of %d MB in rotation" % (K * N * 4 // 1000000),
                   "timing": "CUDA events on the launch stream"},
        "parity": parity,
        "e2e": {"value": nbytes / e2e_s / 1e9, "unit": "GB/s", "h2d_bytes_per_step": 4 * K * N, "d2h_bytes_per_step": 4096,
                "steps": e2e_steps, "ms_per_call": e2e_s * 1e3,
                "note": "operator API: quantizeQ4/Q8 on a host tensor (H2D of the f32 weights from page-locked memory, the "
                        "kernel, wait); the packed result stays on the device by design, its first 4 KB are read back"},
        "gpu_launches": int(steps + warm + 31 + e2e_steps + 1),
        "roofline": {"bound": "hbm", "achieved": ach, "peak": peaks["hbm"], "unit": "GB/s", "frac": ach / peaks["hbm"],
                     "traffic": traffic_for(name), "peak_source": peaks["source"], "peak_kind": "copy bandwidth",
                     "frac_of_nominal": ach / 8000.0, "algorithmic_per_launch": nbytes, "launch_us": step_s * 1e6},
        "clocks": clocks,
    }
    if not args.no_cpu:
        cols = 256
        rng = np.random.default_rng(0)
        wc = (rng.standard_normal((K, cols)) * wl["std"]).astype(np.float32)
        fn = O.quantize_q4 if kind == 4 else O.quantize_q8
        fn(wc)
        reps, t0 = 0, time.perf_counter()
        while time.perf_counter() - t0 < min(args.cpu_seconds, 5.0):
            fn(wc)
            reps += 1
        el = time.perf_counter() - t0
        per_matrix = el / reps * (N / cols)
        line["cpu_baseline"] = {"value": nbytes / per_matrix / 1e9, "unit": "GB/s", "cores": 1, "kind": "port",
                                "sample": f"{reps} runs of {cols} of {N} columns on one thread (time scaled to all columns), {el:.1f} s of CPU work"}
    else:
        line["cpu_baseline"] = None
    for b in ws + [out]:
        D.releaseBuffer(b)
    return line


def run_dense_workload(args, name, wl, ctxinfo, steps=None, with_cpu=True, with_e2e=True):
    """The dense matmul c = a @ b through smith_matmul on device-resident operands; a step is one product
    (f32 storage: two split launches + the tcgen05 kernel; f16 storage: one transposition + the kernel).
    b alternates between two matrices, so a step's operands (>= 128 MB) do not fit L2.  Algorithmic flops
    2 M N K; the f32 path executes six bf16 products per f32 product, so its ceiling is a sixth of the
    bf16 peak and the line says so."""
    import numpy as np
    import torch
    import smith_b200 as smith
    from oracle import oracle as O
    from smith_b200 import device as D
    world, rank, local, stream = ctxinfo
    f16 = wl["dense"] == "f16"
    M, K, N = wl["M"], wl["K"], wl["N"]
    dt, es, npdt = (D.DTYPE_F16, 2, np.float16) if f16 else (D.DTYPE_F32, 4, np.float32)
    rng = np.random.default_rng(5)
    a_h = rng.standard_normal((M, K)).astype(npdt)
    b_h = [rng.standard_normal((K, N)).astype(npdt) for _ in range(2)]
    a = D.alloc(M * K * es, D.PRIVATE)
    bs = [D.alloc(K * N * es, D.PRIVATE) for _ in range(2)]
    c = D.alloc(M * N * es, D.PRIVATE)
    D.upload(a, a_h)
    for buf, h in zip(bs, b_h):
        D.upload(buf, h)
    steps = min(args.steps, 50) if steps is None else steps
    warm = max(min(args.warmup, 5), 3)
    D.matmul(dt, a, bs[0], c, M, N, K)
    D.synchronize()
    if D.kernelStatus() != 0:
        raise SystemExit("a bounded device-side wait gave up")
    # parity before timing: 16 rows of the product against the CPU restatement
    r0, nr = (M // 2) // 8 * 8, 16
    got = D.download(c, nr * N * es, npdt, offset=r0 * N * es).reshape(nr, N).astype(np.float64)
    if f16:
        want = a_h[r0:r0 + nr].astype(np.float64) @ b_h[0].astype(np.float64)
        bound = 2.0 ** -10 * np.abs(want) + 4e-6 * np.linalg.norm(a_h[r0:r0 + nr].astype(np.float64), axis=1)[:, None] * \
            np.linalg.norm(b_h[0].astype(np.float64), axis=0)[None, :]
        what = "16 rows against the exact product: 2^-10 |c| (one rounding to half) + 4e-6 ||a_m|| ||b_n||"
    else:
        want = O.dense_matmul(a_h[r0:r0 + nr], b_h[0]).astype(np.float64)
        bound = 4e-6 * np.linalg.norm(a_h[r0:r0 + nr].astype(np.float64), axis=1)[:, None] * \
            np.linalg.norm(b_h[0].astype(np.float64), axis=0)[None, :]
        what = "16 rows against the sequential f32 sums of the shaders: 4e-6 ||a_m|| ||b_n||"
    worst = float((np.abs(got - want) / bound).max())
    parity = {"checked": True, "ok": bool(worst <= 1.0), "worst_err_over_bound": worst, "what": what}
    if not parity["ok"]:
        raise SystemExit(f"dense product outside its tolerance: worst err/bound = {worst}")
    for i in range(warm):
        D.matmul(dt, a, bs[i % 2], c, M, N, K)
    D.synchronize()
    sampler = ClockSampler(local)
    sampler.start()
    n0 = D.launchCount()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(steps):
        D.matmul(dt, a, bs[i % 2], c, M, N, K)
    e1.record(stream)
    D.synchronize()
    torch.cuda.synchronize()
    launches = D.launchCount() - n0
    step_s = e0.elapsed_time(e1) * 1e-3 / steps
    e2e = None
    if with_e2e:
        ta, tb = smith.tensorFrom(a_h.ravel(), [M, K], "f32") if not f16 else None, None
        if f16:                                   # f16 tensors are filled through their views (tensorFrom converts element by element)
            ta, tb = smith.create([M, K], "f16"), smith.create([K, N], "f16")
            ta.data[:] = a_h.view(np.uint16).ravel()
            tb.data[:] = b_h[0].view(np.uint16).ravel()
        else:
            tb = smith.tensorFrom(b_h[0].ravel(), [K, N], "f32")
        out = smith.matmul(ta, tb)
        smith.tensor.release(out)
        n_e2e = 3
        t0 = time.perf_counter()
        for _ in range(n_e2e):
            out = smith.matmul(ta, tb)
            head = float(out.data[0])
            smith.tensor.release(out)
        e2e_s = (time.perf_counter() - t0) / n_e2e
        e2e = {"value": 2.0 * M * N * K / e2e_s / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": (M * K + K * N) * es,
               "d2h_bytes_per_step": M * N * es, "steps": n_e2e, "ms_per_call": e2e_s * 1e3,
               "note": "operator API: matmul(a, b) on host tensors (H2D of both operands from page-locked memory, "
                       "the launches, D2H of the whole product, wait)"}
        for t in (ta, tb):
            smith.tensor.release(t)
    clocks = sampler.stop()
    peaks = measured_peaks()
    ach = 2.0 * M * N * K / step_s / 1e12
    products = 1 if f16 else 6
    line = {
        "metric": "dense matmul TFLOP/s (2 M N K / time)", "value": ach, "unit": "TFLOP/s", "n_gpus": 1, "steps": steps,
        "warmup": warm, "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16 storage, f32 sums" if f16 else "f32 storage as three bf16 planes, six partial products, f32 sums",
        "data": "synthetic",
        "config": {"workload": name, "M": M, "K": K, "N": N, "launches_per_step": launches // steps,
                   "kernel": "dense_tc_kernel (tcgen05)", "l2": "b alternates between two matrices; operands of a step exceed L2",
                   "timing": "CUDA events on the launch stream, split / transposition launches included"},
        "parity": parity, "e2e": e2e, "gpu_launches": int(launches),
        "roofline": {"bound": "tensor", "achieved": ach, "peak": peaks["tensor"], "unit": "TFLOP/s", "frac": ach / peaks["tensor"],
                     "traffic": traffic_for(name), "peak_source": peaks["source"], "peak_kind": "cuBLAS bf16 burst",
                     "frac_of_nominal": ach / 2250.0, "algorithmic_per_launch": 2 * M * N * K, "launch_us": step_s * 1e6,
                     "bf16_products_per_product": products, "mma_tflops_executed": ach * products,
                     "frac_mma_executed": ach * products / peaks["tensor"]},
        "clocks": clocks,
    }
    if with_cpu and not args.no_cpu:
        rows = 8
        O.dense_matmul(a_h[:rows], b_h[0])
        reps, t0 = 0, time.perf_counter()
        while time.perf_counter() - t0 < min(args.cpu_seconds, 5.0):
            O.dense_matmul(a_h[:rows], b_h[0])
            reps += 1
        el = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": 2.0 * rows * N * K * reps / el / 1e12, "unit": "TFLOP/s", "cores": O.max_threads(),
                                "kind": "port", "sample": f"{reps} runs of {rows} of {M} rows, {el:.1f} s of CPU work"}
    else:
        line["cpu_baseline"] = None
    for x in [a, c] + bs:
        D.releaseBuffer(x)
    return line


SECONDARY = ["q4_prefill_4096x14336_m512", "q8_prefill_gemm_4096x11008_m512", "q4_gemv_4096x4096_m1"]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--workload", default=DEFAULT, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-list", action="store_true", help="time one launch per product instead of the list form")
    ap.add_argument("--no-secondary", action="store_true", help="skip the secondary workloads of the default run")
    ap.add_argument("--no-settle", action="store_true", help="no untimed load before the timed region (for profiler captures)")
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]
    if args.impl == "reference":
        return run_reference_arm(args, wl, args.workload)

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from smith_b200 import device as D
    D.ctx()
    stream = torch.cuda.ExternalStream(D.stream())
    ctxinfo = (world, rank, local, stream)
    warm = max(args.warmup, 3)
    if wl.get("pack"):
        if world != 1:
            raise SystemExit("the packer workloads run on one GPU")
        line = run_pack_workload(args, args.workload, wl, ctxinfo)
    elif wl.get("dense"):
        if world != 1:
            raise SystemExit("the dense workloads run on one GPU")
        line = run_dense_workload(args, args.workload, wl, ctxinfo)
    elif "step" in wl:
        line = run_step_workload(args, wl, ctxinfo)
    else:
        line = run_matrix_workload(args, args.workload, wl, args.steps, warm, ctxinfo)
    if args.workload == DEFAULT and not args.no_secondary:
        sec = []
        # The default single-GPU run also times, in the same process, the shapes the other stated targets
        # are quoted on (short runs: they are records, the headline is the line's own value).
        for nm in (SECONDARY if world == 1 else []):
            w2 = WORKLOADS[nm]
            st2 = 20 if w2["M"] > 64 else 300
            l2 = run_matrix_workload(args, nm, w2, st2, 5, ctxinfo, with_cpu=False, with_e2e=False, sampler_on=True)
            is_list = l2["config"]["kernel"] == "gemv_list_dp4a"
            sec.append({"workload": nm, "value": l2["value"], "unit": l2["unit"], "steps": st2,
                        "us_per_product": l2["roofline"]["launch_us"] / (l2["config"]["products_per_step"] if is_list else 1),
                        "form": "list" if is_list else "one launch per product",
                        "kernel": l2["config"]["kernel"], "per_call": l2["config"]["per_call"],
                        "roofline": {k: l2["roofline"][k] for k in ("bound", "achieved", "peak", "unit", "frac",
                                                                     "frac_of_nominal", "peak_kind")},
                        "frac_of_sustained_peak": (l2["roofline"]["achieved"] / measured_peaks()["tensor_sustained"]
                                                   if l2["roofline"]["bound"] == "tensor" else None),
                        "parity": l2["parity"], "clocks": l2["clocks"]})
        for nm in (["dense_f32_4096x4096x4096", "dense_f16_4096x4096x4096"] if world == 1 else []):
            try:
                l4 = run_dense_workload(args, nm, WORKLOADS[nm], ctxinfo, steps=10, with_cpu=False, with_e2e=False)
                sec.append({"workload": nm, "value": l4["value"], "unit": l4["unit"], "steps": l4["steps"],
                            "ms_per_step": l4["ms_per_step"], "kernel": l4["config"]["kernel"], "roofline": l4["roofline"],
                            "parity": l4["parity"], "clocks": l4["clocks"]})
            except (SystemExit, Exception) as e:
                sec.append({"workload": nm, "error": str(e)[:300]})
        # ... and, at every GPU count, the 70B-shaped decode step: the workload on which sharding pays
        # (52 GB of packed weights; several GPUs: tensor parallel with the all-reduce after wo / down and
        # the all-gather of the logits fused into the GEMV kernel).
        nm = "q4_llama70b_step_m1"
        try:
            l3 = run_step_workload(args, WORKLOADS[nm], ctxinfo, name=nm, steps=10, with_cpu=False)
            if rank == 0:
                sec.append({"workload": nm, "value": l3["value"], "unit": l3["unit"], "steps": l3["steps"],
                            "ms_per_step": l3["ms_per_step"], "n_gpus": world, "form": l3["config"].get("form", "one launch per projection group"),
                            "sharding": l3["config"]["sharding"], "launches_per_step": l3["config"]["launches_per_step"],
                            "roofline": {k: l3["roofline"][k] for k in ("bound", "achieved", "peak", "unit", "frac", "frac_of_nominal")},
                            "e2e": l3["e2e"], "parity": l3.get("parity"), "clocks": l3["clocks"]})
        except (SystemExit, Exception) as e:      # a record, not the headline: say what happened and go on
            if rank == 0:
                sec.append({"workload": nm, "error": str(e)[:300]})
        if rank == 0:
            line["secondary"] = sec
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
