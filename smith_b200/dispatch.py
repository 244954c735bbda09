"""Kernel dispatch helper -- the role of src/dispatch.js in the reference.

``run`` replays the reference's encode-and-wait sequence (src/dispatch.js:17-48):
pipeline lookup, begin, set pipeline, bind buffers, copy the inline parameter
bytes, dispatch, then either a timed submit (profiling on) or a blocking one.
"""
import numpy as np

from . import device
from .profile import algorithmicCost, isProfilingEnabled, recordKernel

GROUP_1D = 256


def run(kernel, buffers, grid, group=None, params=None):
    pso = device.pipeline(kernel)
    if not isProfilingEnabled():
        # Same sequence (src/dispatch.js:17-48) through the bridge's one-call form
        # (native/gpu_bridge.h:104-108): one trip across the FFI instead of nine.
        data = np.ascontiguousarray(params["data"]) if params is not None else None
        gx, gy, gz = grid.get("x") or 1, grid.get("y") or 1, grid.get("z") or 1
        g = group or {}
        device.dispatchSync(pso, [b["buffer"] for b in buffers], [b["index"] for b in buffers], data,
                            params["index"] if params is not None else 0, (gx, gy, gz),
                            (g.get("x") or min(gx, GROUP_1D), g.get("y") or 1, g.get("z") or 1))
        return
    enc = device.begin()
    device.setPipeline(enc, pso)
    for b in buffers:
        device.setBuffer(enc, b["buffer"], b["index"])
    if params is not None:
        data = np.ascontiguousarray(params["data"])
        device.setBytes(enc, data, data.nbytes, params["index"])
    gx = grid.get("x") or 1
    gy = grid.get("y") or 1
    gz = grid.get("z") or 1
    group = group or {}
    grpX = group.get("x") or min(gx, GROUP_1D)
    grpY = group.get("y") or 1
    grpZ = group.get("z") or 1
    device.dispatch(enc, gx, gy, gz, grpX, grpY, grpZ)
    if isProfilingEnabled():
        timing = device.endTimed(enc)
        recordKernel(kernel, timing["gpuMs"], algorithmicCost(kernel, params["data"] if params is not None else None))
    else:
        device.endSync(enc)
