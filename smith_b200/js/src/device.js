// device.js -- bun:ffi binding of libsmith_cuda.so (the CUDA bridge for NVIDIA B200).
// Same exported names as the Metal-era device layer, so dispatch / tensor / pool code above it
// does not change.  Additions: lastError(), makeResident(), qmatmul(), graph capture.
import { dlopen, FFIType as T, toArrayBuffer, CString } from 'bun:ffi'
import { resolve, dirname } from 'path'

const LIB_PATH = process.env.SMITH_CUDA_LIB ||
  resolve(dirname(import.meta.dir), 'native', 'libsmith_cuda.so')

const { symbols: lib } = dlopen(LIB_PATH, {
  // lifecycle / info
  smith_init: { returns: T.ptr, args: [] },
  smith_destroy: { returns: T.void, args: [T.ptr] },
  smith_device_name: { returns: T.ptr, args: [T.ptr] },
  smith_max_threadgroup_memory: { returns: T.u64, args: [T.ptr] },
  smith_max_threads_per_threadgroup: { returns: T.u64, args: [T.ptr] },
  // buffers
  smith_alloc: { returns: T.ptr, args: [T.ptr, T.u64, T.u32] },
  smith_buffer_contents: { returns: T.ptr, args: [T.ptr] },
  smith_buffer_length: { returns: T.u64, args: [T.ptr] },
  smith_release_buffer: { returns: T.void, args: [T.ptr] },
  smith_buffer_retain_count: { returns: T.i64, args: [T.ptr] },
  smith_test_release: { returns: T.i64, args: [T.ptr] },
  smith_test_release_after_use: { returns: T.i64, args: [T.ptr] },
  // kernel registry
  smith_load_library: { returns: T.ptr, args: [T.ptr, T.cstring] },
  smith_compile_source: { returns: T.ptr, args: [T.ptr, T.cstring, T.ptr] },
  smith_create_pipeline: { returns: T.ptr, args: [T.ptr, T.ptr, T.cstring] },
  // encoder
  smith_begin: { returns: T.ptr, args: [T.ptr] },
  smith_set_buffer: { returns: T.void, args: [T.ptr, T.ptr, T.u32] },
  smith_set_bytes: { returns: T.void, args: [T.ptr, T.ptr, T.u32, T.u32] },
  smith_set_threadgroup_memory: { returns: T.void, args: [T.ptr, T.u64, T.u32] },
  smith_set_pipeline: { returns: T.void, args: [T.ptr, T.ptr] },
  smith_dispatch: { returns: T.void, args: [T.ptr, T.u64, T.u64, T.u64, T.u64, T.u64, T.u64] },
  smith_end_sync: { returns: T.void, args: [T.ptr] },
  smith_end_async: { returns: T.ptr, args: [T.ptr] },
  smith_wait: { returns: T.void, args: [T.ptr] },
  smith_end_timed: { returns: T.ptr, args: [T.ptr] },
  smith_allocated_size: { returns: T.u64, args: [T.ptr] },
  // additions of the CUDA bridge
  smith_last_error: { returns: T.cstring, args: [] },
  smith_clear_error: { returns: T.void, args: [] },
  smith_synchronize: { returns: T.i32, args: [T.ptr] },
  smith_buffer_device_ptr: { returns: T.ptr, args: [T.ptr] },
  smith_buffer_make_resident: { returns: T.i32, args: [T.ptr] },
  smith_buffer_evict: { returns: T.i32, args: [T.ptr] },
  smith_qmatmul: { returns: T.i32, args: [T.ptr, T.u32, T.ptr, T.ptr, T.ptr, T.u64, T.u64, T.u64, T.u64, T.u32] },
  // dense matmul on device-side buffers: (ctx, dtype 0 = f32 / 1 = f16, a, b, c, M, N, K, batch, path)
  smith_matmul: { returns: T.i32, args: [T.ptr, T.u32, T.ptr, T.ptr, T.ptr, T.u64, T.u64, T.u64, T.u64, T.u32] },
  smith_kernel_status: { returns: T.i32, args: [T.ptr] },
  smith_graph_begin: { returns: T.i32, args: [T.ptr] },
  smith_graph_end: { returns: T.ptr, args: [T.ptr] },
  smith_graph_launch: { returns: T.i32, args: [T.ptr, T.ptr] },
  smith_graph_destroy: { returns: T.void, args: [T.ptr] },
})

const SHARED = 0   // page-locked host memory, staged to the device around each dispatch
const PRIVATE = 1  // device memory only

function lastError() {
  const e = lib.smith_last_error()
  return e ? e.toString() : ''
}
function failIfError(what) {
  const e = lastError()
  if (e.length) { lib.smith_clear_error(); throw new Error(`smith: ${what}: ${e}`) }
}

const ctx = lib.smith_init()
if (!ctx) throw new Error('smith: failed to initialize CUDA device (NVIDIA B200 required): ' + lastError())

let _kernels = null
function shaderLib() {
  if (!_kernels) {
    _kernels = lib.smith_load_library(ctx, Buffer.from('builtin\0'))
    if (!_kernels) throw new Error('smith: failed to open the kernel registry')
  }
  return _kernels
}
const _pipelines = new Map()
function pipeline(name) {
  let p = _pipelines.get(name)
  if (!p) {
    p = lib.smith_create_pipeline(ctx, shaderLib(), Buffer.from(name + '\0'))
    if (!p) throw new Error(`smith: kernel '${name}' not found in shader library`)
    _pipelines.set(name, p)
  }
  return p
}

const deviceName = () => new CString(lib.smith_device_name(ctx)).toString()
const maxThreadgroupMemory = () => Number(lib.smith_max_threadgroup_memory(ctx))
const maxThreadsPerThreadgroup = () => Number(lib.smith_max_threads_per_threadgroup(ctx))

function alloc(bytes, mode = SHARED) {
  const b = lib.smith_alloc(ctx, bytes, mode)
  if (!b) throw new Error(`smith: failed to allocate ${bytes} bytes (mode=${mode})`)
  return b
}
const bufferContents = (b) => lib.smith_buffer_contents(b)
const bufferLength = (b) => Number(lib.smith_buffer_length(b))
const releaseBuffer = (b) => lib.smith_release_buffer(b)
const bufferRetainCount = (b) => Number(lib.smith_buffer_retain_count(b))
function viewBuffer(buffer, byteLength, TypedArray = Float32Array) {
  const raw = lib.smith_buffer_contents(buffer)
  if (!raw) throw new Error('smith: buffer has no host-visible contents (PRIVATE buffer)')
  return new TypedArray(toArrayBuffer(raw, 0, byteLength))
}
function makeResident(buffer) {
  if (lib.smith_buffer_make_resident(buffer) !== 0) failIfError('make_resident')
}

const begin = () => lib.smith_begin(ctx)
const setBuffer = (enc, buffer, index) => lib.smith_set_buffer(enc, buffer, index)
const setBytes = (enc, data, length, index) => lib.smith_set_bytes(enc, data, length, index)
const setThreadgroupMemory = (enc, length, index) => lib.smith_set_threadgroup_memory(enc, length, index)
const setPipeline = (enc, pso) => lib.smith_set_pipeline(enc, pso)
const dispatch = (enc, gx, gy, gz, tx, ty, tz) => lib.smith_dispatch(enc, gx, gy, gz, tx, ty, tz)
function endSync(enc) {
  lib.smith_clear_error()
  lib.smith_end_sync(enc)
  failIfError('dispatch failed')
}
function endAsync(enc) {
  lib.smith_clear_error()
  const token = lib.smith_end_async(enc)
  if (!token) failIfError('dispatch failed')
  return token
}
function wait(token) {
  lib.smith_wait(token)
  failIfError('wait failed')
}
function endTimed(enc) {
  lib.smith_clear_error()
  const t = lib.smith_end_timed(enc)
  if (!t) { failIfError('dispatch failed'); return { gpuStart: 0, gpuEnd: 0, gpuMs: 0 } }
  const f64 = new Float64Array(toArrayBuffer(t, 0, 24))   // SmithTiming: three doubles
  return { gpuStart: f64[0], gpuEnd: f64[1], gpuMs: f64[2] }
}
const allocatedSize = () => Number(lib.smith_allocated_size(ctx))

// src/device.js:195-213 in the reference.  The CUDA bridge has no run-time kernel compiler: the call
// reaches the bridge, which reports that, and this throws with the bridge's message like the
// reference does on a compile error.
function compileSource(source) {
  const src = Buffer.from(source + '\0', 'utf-8')
  const errSlot = new BigUint64Array(1)
  const library = lib.smith_compile_source(ctx, src, errSlot)
  if (!library) {
    const msg = errSlot[0] ? new CString(Number(errSlot[0])).toString() : (lastError() || 'unknown error')
    throw new Error(`smith: shader compilation failed: ${msg}`)
  }
  return library
}

// src/device.js:217-256 in the reference: a pipeline by kernel name from a library handle.
function createPipeline(library, fnName) {
  const name = Buffer.from(fnName + '\0', 'utf-8')
  const p = lib.smith_create_pipeline(ctx, library, name)
  if (!p) throw new Error(`smith: kernel '${fnName}' not found`)
  return p
}

export {
  SHARED, PRIVATE, ctx, lib, lastError,
  deviceName, maxThreadgroupMemory, maxThreadsPerThreadgroup,
  alloc, bufferContents, bufferLength, releaseBuffer, bufferRetainCount, viewBuffer, makeResident,
  shaderLib, pipeline,
  begin, setBuffer, setBytes, setThreadgroupMemory, setPipeline, dispatch, endSync, endAsync, wait,
  endTimed, allocatedSize, compileSource, createPipeline,
}
