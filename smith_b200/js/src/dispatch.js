// dispatch.js -- encode one kernel dispatch and wait for it.
// run(kernel, buffers, grid, group, params): look the pipeline up by name, bind buffers and the
// inline parameter bytes, dispatch, then submit (timed when a profiler hook is installed).
import * as device from './device.js'

const GROUP_1D = 256
let _onKernelTime = null          // (kernelName, gpuMs) => void, set by a profiler

function setProfilerHook(fn) { _onKernelTime = fn }

function run(kernel, buffers, grid, group, params) {
  const enc = device.begin()
  device.setPipeline(enc, device.pipeline(kernel))
  for (const b of buffers) device.setBuffer(enc, b.buffer, b.index)
  if (params) device.setBytes(enc, params.data, params.data.byteLength, params.index)
  const gx = grid.x || 1, gy = grid.y || 1, gz = grid.z || 1
  device.dispatch(enc, gx, gy, gz,
    group?.x || Math.min(gx, GROUP_1D), group?.y || 1, group?.z || 1)
  if (_onKernelTime) _onKernelTime(kernel, device.endTimed(enc).gpuMs)
  else device.endSync(enc)
}

export { run, setProfilerHook, GROUP_1D }
