// ops/quantize.js -- block quantisation of weights and quantized matmul on the CUDA bridge.
//   quantizeQ4(weight) / quantizeQ8(weight) -> { buffer, K, N, groups, totalBytes }
//   matmulQ4(a, wq) / matmulQ8(a, wq)       -> tensor [M, N]
// Packing runs on the device (kernels 'quantize_q4' / 'quantize_q8'); the packed weights stay in
// device memory.  Q4: 32-element groups, 24 bytes (16 nibble bytes, f32 scale, f32 zero).
// Q8: 32-element blocks, 34 bytes (f16 scale, 32 int8).
import * as device from '../device.js'
import { run } from '../dispatch.js'

const GROUP_SIZE = 32
const GROUP_BYTES = 24
const Q8_BLOCK_SIZE = 32
const Q8_BLOCK_BYTES = 34

// Smallest tensor record the operators need: { buffer, data, shape, dtype }.
function createTensor(shape, dtype = 'f32') {
  const bytes = shape.reduce((a, b) => a * b, 1) * 4
  const buffer = device.alloc(Math.max(bytes, 256), device.SHARED)
  return { buffer, data: device.viewBuffer(buffer, bytes, Float32Array), shape: shape.slice(), dtype }
}

function quantize(weight, kernel, blockBytes) {
  const [K, N] = weight.shape
  const groups = Math.ceil(K / 32)
  const totalBytes = groups * N * blockBytes
  const buffer = device.alloc(totalBytes, device.PRIVATE)
  run(kernel, [{ buffer: weight.buffer, index: 0 }, { buffer, index: 1 }],
    { x: N, y: groups }, { x: Math.min(N, 256), y: 1 }, { data: new Uint32Array([K, N]), index: 2 })
  return { buffer, K, N, groups, totalBytes }
}
const quantizeQ4 = (weight) => quantize(weight, 'quantize_q4', GROUP_BYTES)
const quantizeQ8 = (weight) => quantize(weight, 'quantize_q8', Q8_BLOCK_BYTES)

function matmul(name, kernel, a, bQuant, create) {
  const M = a.shape[0]
  const { N, K, groups, buffer } = bQuant
  if (a.shape[1] !== K) throw new Error(`${name}: inner dims don't match: ${a.shape[1]} vs ${K}`)
  const out = (create || createTensor)([M, N], a.dtype)
  run(kernel, [{ buffer: a.buffer, index: 0 }, { buffer, index: 1 }, { buffer: out.buffer, index: 2 }],
    { x: N, y: M }, { x: Math.min(N, 16), y: Math.min(M, 16) },
    { data: new Uint32Array([M, N, K, groups]), index: 3 })
  return out
}
const matmulQ4 = (a, bQuant, create) => matmul('matmulQ4', 'matmul_q4', a, bQuant, create)
const matmulQ8 = (a, bQuant, create) => matmul('matmulQ8', 'matmul_q8', a, bQuant, create)

export { quantizeQ4, quantizeQ8, matmulQ4, matmulQ8, createTensor,
  GROUP_SIZE, GROUP_BYTES, Q8_BLOCK_SIZE, Q8_BLOCK_BYTES }
