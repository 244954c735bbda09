"""Per-kernel GPU timing -- the role of src/profile.js in the reference.

When profiling is on, dispatch.run ends each dispatch with the bridge's timed
submit and reports the kernel's device milliseconds here (src/dispatch.js:42-44,
src/profile.js:35-55).  ``profile(fn)`` and ``benchmark(name, fn)`` keep the
reference's result shapes (src/profile.js:103-175).

Added to the reference's report: for the kernels of the quantized path the
dispatcher also passes the ALGORITHMIC bytes and flops of the call (weights
read once, activations read once, output written once; 2 M K N), and every
kernel entry then carries ``gbs``, ``tflops`` and the fraction of the HBM or
tensor roofline it reached (``pctRoofline``, against ``setPeaks``' figures:
by default the nominal 8 000 GB/s and 2 250 TFLOP/s of a B200).
"""
import math
import time

from . import device

_enabled = False
_kernelStats = {}
_totalDispatches = 0
_totalGpuMs = 0.0
_peakMemory = 0
_startMemory = 0
_peaks = {"hbmGBs": 8000.0, "tensorTFlops": 2250.0, "source": "nominal"}


def setPeaks(hbmGBs=None, tensorTFlops=None, source="caller"):
    """Roofline denominators of ``report()`` (e.g. figures measured on the machine)."""
    if hbmGBs:
        _peaks["hbmGBs"] = float(hbmGBs)
    if tensorTFlops:
        _peaks["tensorTFlops"] = float(tensorTFlops)
    _peaks["source"] = source


def algorithmicCost(kernelName, params):
    """(bytes, flops) of one dispatch of a kernel from its parameter block, else None.
    matmul_q4 / matmul_q8: params = [M, N, K, groups]; quantize_q4 / quantize_q8: params = [K, N];
    matmul_f32 / matmul_f16 / matmul_simple[_f16] / matmul_batched[_f16]: params = [M, N, K(, batch)]."""
    if params is None:
        return None
    p = [int(v) for v in params]
    if kernelName in ("matmul_q4", "matmul_q8") and len(p) >= 4:
        M, N, K, groups = p[:4]
        bb = 24 if kernelName == "matmul_q4" else 34
        return groups * N * bb + 4 * M * K + 4 * M * N, 2 * M * K * N
    if kernelName in ("quantize_q4", "quantize_q8") and len(p) >= 2:
        K, N = p[:2]
        bb = 24 if kernelName == "quantize_q4" else 34
        return 4 * K * N + ((K + 31) // 32) * N * bb, 0
    if kernelName.startswith("matmul_") and len(p) >= 3:
        # the dense family: [M, N, K] or [M, N, K, batch]; f16 storage in the names that end in _f16
        M, N, K = p[:3]
        batch = p[3] if len(p) >= 4 and "batched" in kernelName else 1
        es = 2 if kernelName.endswith("_f16") else 4
        return batch * es * (M * K + K * N + M * N), batch * 2 * M * K * N
    return None


def _round(v):
    return math.floor(v * 1000 + 0.5) / 1000


def enableProfiling():
    global _enabled, _startMemory, _peakMemory
    _enabled = True
    _startMemory = device.allocatedSize()
    _peakMemory = _startMemory


def disableProfiling():
    global _enabled
    _enabled = False


def isProfilingEnabled():
    return _enabled


def recordKernel(kernelName, gpuMs, cost=None):
    global _totalDispatches, _totalGpuMs, _peakMemory
    _totalDispatches += 1
    _totalGpuMs += gpuMs
    s = _kernelStats.setdefault(kernelName, {"calls": 0, "totalGpuMs": 0.0, "minMs": math.inf, "maxMs": 0.0,
                                             "samples": [], "bytes": 0, "flops": 0, "costedMs": 0.0})
    s["calls"] += 1
    s["totalGpuMs"] += gpuMs
    if cost:
        s["bytes"] += cost[0]
        s["flops"] += cost[1]
        s["costedMs"] += gpuMs
    s["minMs"] = min(s["minMs"], gpuMs)
    s["maxMs"] = max(s["maxMs"], gpuMs)
    if len(s["samples"]) < 100:
        s["samples"].append(gpuMs)
    else:
        s["samples"][s["calls"] % 100] = gpuMs
    mem = device.allocatedSize()
    if mem > _peakMemory:
        _peakMemory = mem


def report():
    entries = []
    for name, s in _kernelStats.items():
        avg = s["totalGpuMs"] / s["calls"] if s["calls"] else 0
        pct = s["totalGpuMs"] / _totalGpuMs * 100 if _totalGpuMs > 0 else 0
        e = {"kernel": name, "calls": s["calls"], "totalMs": _round(s["totalGpuMs"]),
             "avgMs": _round(avg), "minMs": _round(0 if s["minMs"] == math.inf else s["minMs"]),
             "maxMs": _round(s["maxMs"]), "pct": _round(pct)}
        if s.get("costedMs", 0) > 0:
            sec = s["costedMs"] * 1e-3
            gbs, tfl = s["bytes"] / sec / 1e9, s["flops"] / sec / 1e12
            hbm, tensor = gbs / _peaks["hbmGBs"], tfl / _peaks["tensorTFlops"]
            e.update({"gbs": _round(gbs), "tflops": _round(tfl), "bound": "hbm" if hbm >= tensor else "tensor",
                      "pctRoofline": _round(100 * max(hbm, tensor))})
        entries.append(e)
    entries.sort(key=lambda e: -e["totalMs"])
    return {"dispatches": _totalDispatches, "totalGpuMs": _round(_totalGpuMs),
            "peaks": dict(_peaks),
            "memory": {"startBytes": _startMemory, "peakBytes": _peakMemory,
                       "currentBytes": device.allocatedSize(), "deltaBytes": _peakMemory - _startMemory},
            "kernels": entries}


def resetProfile():
    global _totalDispatches, _totalGpuMs, _peakMemory, _startMemory
    _kernelStats.clear()
    _totalDispatches = 0
    _totalGpuMs = 0.0
    _peakMemory = device.allocatedSize()
    _startMemory = _peakMemory


def profile(fn):
    was = _enabled
    enableProfiling()
    resetProfile()
    t0 = time.perf_counter()
    result = fn()
    cpuMs = (time.perf_counter() - t0) * 1000
    rep = report()
    if not was:
        disableProfiling()
    return {"result": result, "cpuMs": _round(cpuMs), "gpuMs": rep["totalGpuMs"], "dispatches": rep["dispatches"],
            "memory": rep["memory"], "kernels": rep["kernels"]}


def computeStats(sortedTimes):
    n = len(sortedTimes)
    if n == 0:
        return {"mean": 0, "median": 0, "min": 0, "max": 0, "p95": 0, "stddev": 0}
    mean = sum(sortedTimes) / n
    median = (sortedTimes[n // 2 - 1] + sortedTimes[n // 2]) / 2 if n % 2 == 0 else sortedTimes[n // 2]
    p95 = sortedTimes[min(math.ceil(n * 0.95) - 1, n - 1)]
    var = sum((v - mean) ** 2 for v in sortedTimes) / n
    return {"mean": _round(mean), "median": _round(median), "min": _round(sortedTimes[0]),
            "max": _round(sortedTimes[-1]), "p95": _round(p95), "stddev": _round(math.sqrt(var))}


def benchmark(name, fn, warmup=3, iterations=10):
    for _ in range(warmup):
        fn()
    cpu, gpu = [], []
    for _ in range(iterations):
        p = profile(fn)
        cpu.append(p["cpuMs"])
        gpu.append(p["gpuMs"])
    return {"name": name, "iterations": iterations, "cpu": computeStats(sorted(cpu)),
            "gpu": computeStats(sorted(gpu))}
