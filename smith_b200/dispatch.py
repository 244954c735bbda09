"""Kernel dispatch helper -- the role of src/dispatch.js in the reference.

``run`` replays the reference's encode-and-wait sequence (src/dispatch.js:17-48):
pipeline lookup, begin, set pipeline, bind buffers, copy the inline parameter
bytes, dispatch, then either a timed submit (profiling on) or a blocking one.
"""
import numpy as np

from . import device
from .profile import isProfilingEnabled, recordKernel

GROUP_1D = 256


def run(kernel, buffers, grid, group=None, params=None):
    pso = device.pipeline(kernel)
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
        recordKernel(kernel, timing["gpuMs"])
    else:
        device.endSync(enc)
