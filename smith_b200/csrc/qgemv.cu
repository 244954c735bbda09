// qgemv.cu -- GEMV-shaped quantized matmul, M <= 4 rows of activations.
//
// C[M,N] = A[M,K] (f32) x dequant(B); B in Smith's Q4 (24-byte) or Q8 (34-byte)
// block layout, block (g, col) at (g*N + col) * block_bytes
// (shaders/matmul_q4.metal:47-55, shaders/matmul_q8.metal:40-48).
//
// One packed weight is touched by exactly one multiply-add per activation
// row, so at M = 1 the kernel has about two instructions per weight to spend
// before it stops being bound by HBM.  The design spends them like this:
//
//  * Activations are converted once per CTA into block fixed point: for each
//    group of 32 the values are scaled by a power of two so the largest fits
//    15 bits, rounded to an integer, and stored as two int8 digits
//    (x_int = hi * 128 + lo, hi signed, lo in 0..127).  The digits sit in
//    shared memory in the order the weight codes come out of a 32-bit word.
//  * The 4-bit codes of a word are split with two masks (even codes in place,
//    odd codes left multiplied by 16) and multiplied into the digit words
//    with dp4a: four codes per instruction, exact int32 sums.  Q8 codes are
//    already bytes.  The group's integer dot product is exact; it is converted
//    to f32 once per block and scaled:
//        Q4: acc += (scale * 2^-e) * (dot - zero * sum_k x_int)
//        Q8: acc += (scale * 2^-e) * dot
//    The only rounding beyond the f32 accumulation over groups is the 15-bit
//    rounding of the activations (relative to the largest value of its group).
//  * One CTA owns TN adjacent columns and all of K.  Thread t owns column
//    t % TN and the group-rows of phase t / TN, so the tile width is free to be
//    whatever spreads N evenly over the SMs (the last warp may be partly idle).  Packed
//    group-rows (TN * block_bytes contiguous bytes each) arrive through a ring
//    of shared-memory stages filled by 1-D bulk async copies from a producer
//    thread (full/empty mbarriers, no multicast); lanes read adjacent blocks.
//    Where a tile's row segment is short (narrow N: 4096 columns give 672-byte
//    segments) the per-copy cost of the copy engine, about 40 ns, would set the
//    pace, so such tiles fetch a whole stage as ONE 2-D tensor-map box
//    (cp.async.bulk.tensor.2d over the packed matrix seen as [groups][N * block
//    bytes / 8] 64-bit words; rows past the end are zero-filled).
//  * The phases of a column are summed through shared memory in fixed order
//    and each output is written once.  No atomics, no global scratch.
//  * One CTA per SM with a deep ring (about 190 KB) where the matrix fits one wave
//    of tiles, two per SM (more warps in flight, one CTA's start-up and tail
//    overlap the other's stream) where tiles come in several waves, and a
//    half-SM footprint where a tile's whole K-slice fits it.  Up to four
//    matrices that share the activations run as one launch (each owns a range
//    of the grid's tiles).  The kernel
//    is launched with programmatic stream serialisation: it lets its successor
//    start as CTAs retire (griddepcontrol.launch_dependents at entry), and
//    itself waits for its predecessor (griddepcontrol.wait) only before it
//    first reads the activations -- the producer warp streams weights, which no
//    kernel writes, from the first instruction.  Back-to-back launches (a
//    decode step's layer stack) thus overlap launch gap, ramp-up and tail.
//
//  * Multi-GPU (weights sharded along N): the same kernel can end in a fused
//    all-gather, in two forms.  Counted form: instead of writing its columns to a local C, each CTA stores
//    them into every rank's gathered row through peer-mapped pointers (plain
//    stores over NVLink), fences, and adds one arrival to every rank's counter.
//    The last CTA of the grid to finish then waits -- bounded -- until its own
//    counter shows the tiles of all ranks, so the launch completes only when
//    this rank's gathered row is whole.  Two output buffers and two counters
//    are used alternately (a rank can run at most one step ahead of another,
//    because its step cannot complete without the other's arrivals), and the
//    step number lives in device memory so that a captured graph can be replayed.
//    Low-latency form: every output travels as one 8-byte {value, step tag} store, nothing is
//    fenced, counted or awaited at the end of a launch, and the next launch on the same state checks
//    the tags of the previous row (see Params::defer).
//
//    With weights sharded along K the same kernel ends in a fused all-reduce: every thread pushes
//    its partial sums as tagged pairs into this rank's slot on every rank (remote 8-byte stores),
//    polls -- bounded -- the same elements of all ranks' slots in its own memory, adds them in rank
//    order (so every rank gets the same bits) and writes the finished outputs.  The ranks tile N
//    identically, so a CTA waits only for the CTAs that work on its columns elsewhere, which run at
//    the same time.  Slots are double-buffered by step parity; a rank writes them only after its
//    previous launch has completed (griddepcontrol.wait), so it cannot run further than one step
//    ahead of a peer that still reads them.  No system-scope fence anywhere: on this part one costs
//    several microseconds per CTA.
//
// Waits are time-bounded as in pipeline.cuh.
#include <cuda.h>
#include <cuda_fp16.h>

#include "kernels.h"
#include "pipeline.cuh"
#include "qgemv_common.cuh"

namespace smith {
namespace {

constexpr int kMaxRowsM = 4;
constexpr int kMaxPeers = 8;
constexpr int kMaxMats = 4;                // weight matrices that may share one launch
constexpr int kRowsPerPhase = 4;           // group-rows a phase handles per stage: fewer, larger stages measured
                                           // faster than more, smaller ones (4096 x 14336 Q4: 9.4 us at 4 rows,
                                           // 11.3 at 2, 16.4 at 1, ring depth in bytes equal); 3 where 4 would
                                           // leave fewer than four stages (Q8's wider rows: 12.3 -> 11.8 us)
constexpr int kMaxStages = 8;
constexpr int kHeader = 256;               // barriers + abort flag
constexpr int kSmemBudget = 110 * 1024;    // per CTA: two CTAs share an SM
constexpr int kSmemBudgetSolo = 220 * 1024;  // long K: the activations' digit form needs the room, one CTA per SM
constexpr int kMaxConsumerThreads = 448;      // per CTA (two CTAs of 480 threads fit an SM at 64 registers)
constexpr int kCtasPerSm = 2;

struct Params {
  const float* A;
  // Weight matrices that share the activations (wq/wk/wv, gate/up) run as ONE launch: matrix i
  // owns the tiles [tile0[i], tile0[i + 1]) of the grid and has its own width and output.  One
  // launch instead of several saves their start-up and tail, the GEMV's only idle HBM time.
  const uint8_t* B[kMaxMats];
  float* C[kMaxMats];
  int N[kMaxMats];
  int tile0[kMaxMats + 1];
  int nmat;
  int use_tma;            // stages arrive as one 2-D tensor-map box each instead of one bulk copy per group-row
  int M, K, G;
  int TN, phases, nthreads;  // consumer threads = TN * phases
  int row_pitch, stage_rows, stage_bytes, stages;
  int xdig_off, xsc_off, ring_off;  // byte offsets in dynamic shared memory
  int* status;
  // Fused all-gather of the output slice over peer memory (world == 0: plain store to C).
  // y[r]: rank r's gathered output, two buffers [2][M][n_total] used alternately;
  // state[r]: rank r's four control words {step, finished-CTA ticket, arrivals[0], arrivals[1]}.
  float* y[kMaxPeers];
  unsigned* state[kMaxPeers];
  int world, rank, n0, n_total;
  unsigned target;  // tiles that arrive per step, summed over all ranks
  // Fused all-reduce instead (weights sharded along K): y[r] holds rank r's slots [2][world][M][N] of
  // {value, step + 1} pairs, one slot per contributing rank; C gets the sum.
  int reduce;
  // All-gather only, deferred form.  A system-scope fence per CTA costs 4-6 us per launch on this
  // part (measured, even with local memory only), so this form has none: every output travels as
  // one 8-byte store {value bits, step + 1} into y[r] (then [2][M][n_total] such pairs), which a
  // reader accepts only when the tag is the step it expects.  No counters, no arrivals, no wait at
  // the end of the launch.  The NEXT launch on the same state (or the closing wait kernel) polls
  // the tags of the previous row: before it reads its activations if that row is its input (its
  // producer streams weights meanwhile, so the NVLink latency hides behind the stream), else
  // after its main loop and before its own stores.
  int defer;
  int a_prev;             // deferred form: the activations ARE the previous step's gathered row (K == n_total)
};


// Bounded wait until an arrival counter (written by peers with system-scope atomics) reaches `expected`.
__device__ __forceinline__ bool wait_arrivals(const unsigned* counter, unsigned expected) {
  const long long t0 = clock64();
  for (unsigned spin = 0;; spin++) {
    unsigned seen;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
    if (seen >= expected) return true;
    if ((spin & 63u) == 63u && clock64() - t0 > kWaitLimitCycles) return false;
  }
}

// Deferred all-gather: wait (bounded) until `count` {value, tag} pairs all carry `tag`; the calling
// threads share the work.  Returns false if some pair never got there.
__device__ __forceinline__ bool wait_tags(const uint2* row, int count, unsigned tag, int tid, int nthreads) {
  // two pairs per 16-byte load (count is even: n_total is a multiple of 8), eight loads in flight per thread
  const uint4* row4 = reinterpret_cast<const uint4*>(row);
  const int n4 = count >> 1;
  const long long t0 = clock64();
  bool ok = true;
  for (int base = tid; base < n4 && ok; base += 8 * nthreads) {
    uint4 v[8];
#pragma unroll
    for (int u = 0; u < 8; u++) {
      const int i = base + u * nthreads;
      if (i < n4)
        asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w) : "l"(row4 + i) : "memory");
    }
#pragma unroll
    for (int u = 0; u < 8; u++) {
      const int i = base + u * nthreads;
      if (i < n4) {
        for (unsigned spin = 0; v[u].y != tag || v[u].w != tag; spin++) {
          if ((spin & 63u) == 63u && clock64() - t0 > kWaitLimitCycles) {
            ok = false;
            break;
          }
          asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w) : "l"(row4 + i) : "memory");
        }
      }
    }
  }
  return ok;
}

// Closes a chain of deferred all-gathers: returns when the last step's row on this rank is whole.
__global__ void __launch_bounds__(256) gather_wait_kernel(const unsigned* state, const uint2* y, int count,
                                                          int* status) {
  const unsigned step = *reinterpret_cast<const volatile unsigned*>(state);
  if (step == 0) return;
  const unsigned prev = step - 1u;
  if (!wait_tags(y + (size_t)(prev & 1u) * count, count, step, threadIdx.x, blockDim.x)) atomicExch(status, 1);
}

struct alignas(64) TensorMaps {
  CUtensorMap m[kMaxMats];
};


// COLL: the multi-GPU epilogues and waits are compiled only into the instantiations that use them;
// inside the plain kernel they cost registers and broke the batching of the activation loads
// (measured: 9.44 -> 9.73 us at 4096 x 14336, 11.35 -> 12.74 us for Q8).
// WIDE (collective instantiations only): a CTA whose ring takes more than half an SM runs alone
// there anyway, so its threads may use up to 128 registers; at 64 the collective code spills.
template <int KIND, int MR, int RPP, bool COLL, bool WIDE>
__global__ void __launch_bounds__(kMaxConsumerThreads + 32, WIDE ? 1 : kCtasPerSm) qgemv_kernel(const Params p,
                                                                                     const __grid_constant__ TensorMaps tm) {
  constexpr int BB = (KIND == 4) ? kQ4Bytes : kQ8Bytes;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty = full + kMaxStages;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 2 * kMaxStages * 8);
  uint4* xdig = reinterpret_cast<uint4*>(smem + p.xdig_off);     // [MR][G][4] uint4
  float2* xsc = reinterpret_cast<float2*>(smem + p.xsc_off);     // [MR][G]
  uint8_t* ring = smem + p.ring_off;

  const int tid = threadIdx.x;
  int mat = 0;
  while (mat + 1 < p.nmat && (int)blockIdx.x >= p.tile0[mat + 1]) mat++;
  const uint8_t* __restrict__ Bm = p.B[mat];
  float* __restrict__ Cm = p.C[mat];
  const int Nm = p.N[mat];
  const int col0 = ((int)blockIdx.x - p.tile0[mat]) * p.TN;
  const int tn = min(p.TN, Nm - col0);
  const int nthr = tn * p.phases;                 // consumer threads with work in this CTA
  const int nwarps = (p.nthreads + 31) / 32;      // consumer warps launched
  const int nst = (p.G + p.stage_rows - 1) / p.stage_rows;
  const uint32_t row_bytes = (uint32_t)tn * BB;

  if (tid == 0) {
    for (int s = 0; s < p.stages; s++) {
      mbar_init(smem_u32(&full[s]), 1);
      mbar_init(smem_u32(&empty[s]), nwarps);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (tid >= nwarps * 32) {
    // ------------------------------------------------------------ producer warp
    // One lane per group-row: the rows of a stage are issued by the warp in
    // parallel (a single thread issuing them one by one is too slow to keep
    // the stream busy).  Lane 0 arms the barrier before any copy can complete.
    const int lane = tid & 31;
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    bool live = true;
    // slot and parity are carried along: a division by the run-time ring depth costs more
    // instructions than the rest of the loop body
    int slot = 0;
    uint32_t par = 0;                               // parity of this pass over the ring
    for (int st = 0; st < nst && live; st++, slot = (slot + 1 == p.stages) ? 0 : slot + 1, par ^= (slot == 0)) {
      if (st >= p.stages) {
        int okw = 1;
        if (lane == 0) okw = mbar_wait(smem_u32(&empty[slot]), par ^ 1u, abort_flag, p.status);
        live = __shfl_sync(0xffffffffu, okw, 0) != 0;
        if (!live) break;
      }
      const int rows = min(p.stage_rows, p.G - st * p.stage_rows);
      const uint32_t bar = smem_u32(&full[slot]);
      const uint32_t dst = smem_u32(ring + (size_t)slot * p.stage_bytes);
      if (p.use_tma) {
        // the box is always stage_rows x TN blocks: what lies beyond N or the last group-row is zero-filled
        if (lane == 0) {
          mbar_expect_tx(bar, (uint32_t)p.stage_rows * (uint32_t)p.row_pitch);
          tma_box_2d(dst, &tm.m[mat], (col0 * BB) >> 3, st * p.stage_rows, bar, policy);
        }
        continue;
      }
      if (lane == 0) mbar_expect_tx(bar, (uint32_t)rows * row_bytes);
      __syncwarp();
      const uint8_t* src = Bm + ((size_t)st * p.stage_rows * Nm + col0) * BB;
      for (int rr = lane; rr < rows; rr += 32)
        bulk_load(dst + rr * p.row_pitch, src + (size_t)rr * Nm * BB, row_bytes, bar, policy);
    }
    return;  // consumers observe every full barrier, so the copies land before the CTA ends
  }

  // -------------------------------------------------------------- consumers
  // The activations (and the output buffer) may belong to the launch before this one.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  unsigned step = 0;
  if (COLL && p.world > 0) step = *reinterpret_cast<volatile unsigned*>(p.state[p.rank]);  // advanced by the previous launch
  if (COLL && p.world > 0 && p.defer && step > 0 && p.a_prev) {
    // the previous step's gathered row is this launch's input and must be whole: every pair of it
    // carries the tag `step`
    const unsigned prev = step - 1u;
    const uint2* row = reinterpret_cast<const uint2*>(p.y[p.rank]) + (size_t)(prev & 1u) * p.M * p.n_total;
    if (!wait_tags(row, p.M * p.n_total, step, tid, nwarps * 32)) atomicExch(p.status, 1);
    asm volatile("bar.sync 1, %0;" ::"r"(nwarps * 32));
  }
  // Activations -> digit words (overlaps the first weight copies).
  // (row, group) pairs are laid out as [MR][G], which is also the order of A's 32-element chunks.
  // Four passes' loads are issued before the first is used: a pass is one L2 round trip long, and a
  // long K (14336: eight passes) would otherwise spend several microseconds here.
  {
    const int total = (MR * p.G * 8 + 31) & ~31, stride = nwarps * 32, last = MR * p.G - 1;
    for (int i0 = tid; i0 < total; i0 += 4 * stride) {
      float4 t[4];
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const int i = i0 + u * stride;
        // clamp keeps whole warps in the shuffles; duplicates rewrite equal bytes
        if (i < total) {
          if (COLL && p.a_prev && step > 0) {
            // four {value, tag} pairs of the previous row (its tags were checked above); volatile,
            // so that no line cached two steps ago is read
            const uint2* pairs = reinterpret_cast<const uint2*>(p.y[p.rank]) +
                                 (size_t)((step - 1u) & 1u) * p.M * p.n_total + (size_t)min(i >> 3, last) * 32 + (i & 7) * 4;
            uint4 a, b;
            asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w) : "l"(pairs) : "memory");
            asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(pairs + 2) : "memory");
            t[u] = make_float4(__uint_as_float(a.x), __uint_as_float(a.z), __uint_as_float(b.x), __uint_as_float(b.z));
          } else {
            t[u] = __ldg(reinterpret_cast<const float4*>(p.A + (size_t)min(i >> 3, last) * 32) + (i & 7));
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const int i = i0 + u * stride;            // warp-uniform: total and stride are multiples of 32
        if (i < total) {
          const int grp = min(i >> 3, last);
          quantise_quarter<KIND>(t[u], i & 7, reinterpret_cast<uint8_t*>(xdig + (size_t)grp * 4), xsc + grp);
        }
      }
    }
  }
  asm volatile("bar.sync 1, %0;" ::"r"(nwarps * 32));

  const bool active = tid < nthr;
  const int col = active ? (tid % tn) : 0;
  const int phase = active ? (tid / tn) : 0;
  float acc[MR];
#pragma unroll
  for (int m = 0; m < MR; m++) acc[m] = 0.f;

  bool ok = true;
  int slot = 0;
  uint32_t ring_par = 0;
  for (int st = 0; st < nst && ok; st++, slot = (slot + 1 == p.stages) ? 0 : slot + 1, ring_par ^= (slot == 0)) {
    ok = mbar_wait(smem_u32(&full[slot]), ring_par, abort_flag, p.status);
    if (ok && active) {
      // 32-bit shared-memory addresses throughout: a per-thread base plus strides
      const int g0 = st * p.stage_rows + phase;
      const uint32_t step = (uint32_t)p.phases * (uint32_t)p.row_pitch;
      uint32_t blk = smem_u32(ring) + (uint32_t)slot * (uint32_t)p.stage_bytes + (uint32_t)phase * (uint32_t)p.row_pitch +
                     (uint32_t)col * BB;
      uint32_t xd = smem_u32(xdig) + (uint32_t)g0 * 64u, xs = smem_u32(xsc) + (uint32_t)g0 * 8u;
      const uint32_t xd_step = (uint32_t)p.phases * 64u, xs_step = (uint32_t)p.phases * 8u;
      if (st * p.stage_rows + p.stage_rows <= p.G) {
#pragma unroll
        for (int rr = 0; rr < RPP; rr++) {
          block_dot_s<KIND, MR>(blk, xd, xs, p.G, acc);
          blk += step, xd += xd_step, xs += xs_step;
        }
      } else {
        for (int rr = 0; rr < RPP; rr++) {
          if (g0 + rr * p.phases < p.G) block_dot_s<KIND, MR>(blk, xd, xs, p.G, acc);
          blk += step, xd += xd_step, xs += xs_step;
        }
      }
    }
    __syncwarp();
    if ((tid & 31) == 0) mbar_arrive(smem_u32(&empty[slot]));
  }

  if (COLL && p.world > 0 && p.defer && step > 0 && !p.a_prev) {
    // This launch does not read the previous step's row, but its own stores below may only go out
    // once that row is whole everywhere it is still being read: a rank must not run further ahead
    // than that.  Checked here rather than at the start, the tags have long arrived and the check
    // costs one pass over the row instead of a wait for the peers.
    const unsigned prev = step - 1u;
    const uint2* row = reinterpret_cast<const uint2*>(p.y[p.rank]) + (size_t)(prev & 1u) * p.M * p.n_total;
    if (!wait_tags(row, p.M * p.n_total, step, tid, nwarps * 32)) atomicExch(p.status, 1);
  }
  if (COLL && p.world > 0 && p.defer && tid == 0) {
    // Count this CTA as past its main loop.  The last one to get here knows that every CTA of the
    // launch has read `step`, so it may already advance it for the next launch (which reads it only
    // after this launch has completed); the round trip of the atomic overlaps the phase reduction.
    unsigned* mine = p.state[p.rank];
    if (atomicAdd(mine + 1, 1u) == gridDim.x - 1) {
      mine[1] = 0u;
      *reinterpret_cast<volatile unsigned*>(mine) = step + 1u;
    }
  }
  // ---------------------------------------------- sum the phases, fixed order
  asm volatile("bar.sync 1, %0;" ::"r"(nwarps * 32));  // every consumer is done with the ring
  float* red = reinterpret_cast<float*>(ring);        // [phases][MR][TN]
  if (active) {
#pragma unroll
    for (int m = 0; m < MR; m++) red[((size_t)phase * MR + m) * p.TN + col] = acc[m];
  }
  asm volatile("bar.sync 1, %0;" ::"r"(nwarps * 32));
  if (*abort_flag) return;
  if (!COLL || p.world == 0) {
    for (int i = tid; i < p.M * tn; i += nwarps * 32) {
      const int m = i / tn, c = i - m * tn;
      float sum = 0.f;
      for (int ph = 0; ph < p.phases; ph++) sum += red[((size_t)ph * MR + m) * p.TN + c];
      Cm[(size_t)m * Nm + col0 + c] = sum;
    }
    return;
  }
  const unsigned par = step & 1u;
  if (p.reduce) {
    // -------------------------------------------- fused all-reduce over peer memory
    // y[r]: rank r's slots [2][world][M][N] of {value, step + 1} pairs.  Each thread pushes its partial
    // sums into this rank's slot on every rank (one 8-byte store each: no fence is needed, a pair is
    // valid exactly when its tag is this step's), then polls the same elements of all slots in its
    // OWN memory and adds them in rank order, so every rank ends with the same bits.
    const size_t slot = (size_t)p.M * Nm;
    for (int i = tid; i < p.M * tn; i += nwarps * 32) {       // push everything first
      const int m = i / tn, c = i - m * tn;
      float sum = 0.f;
      for (int ph = 0; ph < p.phases; ph++) sum += red[((size_t)ph * MR + m) * p.TN + c];
      const size_t mine_at = ((size_t)par * p.world + p.rank) * slot + (size_t)m * Nm + col0 + c;
      for (int r = 0; r < p.world; r++)
        asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(reinterpret_cast<uint2*>(p.y[r]) + mine_at),
                     "r"(__float_as_uint(sum)), "r"(step + 1u)
                     : "memory");
    }
    bool there = true;
    const long long t0 = clock64();
    for (int i = tid; i < p.M * tn && there; i += nwarps * 32) {  // then collect
      const int m = i / tn, c = i - m * tn;
      const uint2* local = reinterpret_cast<const uint2*>(p.y[p.rank]) + (size_t)par * p.world * slot +
                           (size_t)m * Nm + col0 + c;
      float total = 0.f;
      for (int r = 0; r < p.world && there; r++) {
        unsigned v = 0, t;
        for (unsigned spin = 0;; spin++) {
          asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v), "=r"(t) : "l"(local + (size_t)r * slot) : "memory");
          if (t == step + 1u) break;
          if ((spin & 63u) == 63u && clock64() - t0 > kWaitLimitCycles) {
            there = false;                                // a peer never arrived: the result is not valid
            break;
          }
        }
        total += __uint_as_float(v);
      }
      if (there) Cm[(size_t)m * Nm + col0 + c] = total;
    }
    if (!there) atomicExch(p.status, 1);
    asm volatile("bar.sync 1, %0;" ::"r"(nwarps * 32));
    if (tid == 0) {
      unsigned* mine = p.state[p.rank];
      const unsigned ticket = atomicAdd(mine + 1, 1u);
      if (ticket == gridDim.x - 1) {                      // last CTA of this rank's grid
        mine[1] = 0u;
        __threadfence();
        *reinterpret_cast<volatile unsigned*>(mine) = step + 1u;
      }
    }
    return;
  }
  // ---------------------------------------------- fused all-gather over peer memory
  if (p.defer) {
    for (int i = tid; i < p.M * tn; i += nwarps * 32) {
      const int m = i / tn, c = i - m * tn;
      float sum = 0.f;
      for (int ph = 0; ph < p.phases; ph++) sum += red[((size_t)ph * MR + m) * p.TN + c];
      const size_t at = ((size_t)par * p.M + m) * p.n_total + p.n0 + col0 + c;
      for (int r = 0; r < p.world; r++)
        asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(reinterpret_cast<uint2*>(p.y[r]) + at),
                     "r"(__float_as_uint(sum)), "r"(step + 1u)
                     : "memory");
    }
    return;
  }
  for (int i = tid; i < p.M * tn; i += nwarps * 32) {
    const int m = i / tn, c = i - m * tn;
    float sum = 0.f;
    for (int ph = 0; ph < p.phases; ph++) sum += red[((size_t)ph * MR + m) * p.TN + c];
    const size_t at = ((size_t)par * p.M + m) * p.n_total + p.n0 + col0 + c;
    for (int r = 0; r < p.world; r++) p.y[r][at] = sum;
  }
  asm volatile("bar.sync 1, %0;" ::"r"(nwarps * 32));  // every store of this CTA is issued
  if (tid == 0) {
    __threadfence_system();                             // ... and ordered before the arrivals
    for (int r = 0; r < p.world; r++) atomicAdd_system(p.state[r] + 2 + par, 1u);
    unsigned* mine = p.state[p.rank];
    const unsigned ticket = atomicAdd(mine + 1, 1u);
    if (ticket == gridDim.x - 1) {                      // last CTA of this rank's grid
      // a peer that never arrives leaves the row invalid: the status word says so
      if (!wait_arrivals(mine + 2 + par, (step / 2u + 1u) * p.target)) atomicExch(p.status, 1);
      mine[1] = 0u;
      __threadfence();
      *reinterpret_cast<volatile unsigned*>(mine) = step + 1u;
    }
  }
}

struct Plan {
  Params p;
  int tiles;
  int rpp;                // group-rows per phase and stage (template argument of the kernel)
  size_t smem;
  bool ok;
};

Plan make_plan(int kind, int64_t M, const int64_t* Ns, int count, int64_t K) {
  const int BB = (kind == 4) ? kQ4Bytes : kQ8Bytes;
  const int sms = device_sm_count();
  Plan pl{};
  Params& p = pl.p;
  const int MR = (int)M;
  int64_t N = 0;                                   // all matrices' columns together
  for (int i = 0; i < count; i++) N += Ns[i];
  p.M = (int)M, p.K = (int)K, p.G = (int)(K / 32), p.nmat = count;
  const int xdig_bytes = MR * p.G * 64, xsc_bytes = MR * p.G * 8;
  // One CTA per SM with a deep ring when the whole matrix fits one wave of 128-column tiles
  // (nothing follows a CTA on its SM, so depth beats overlap); two per SM when tiles come in
  // several waves (one CTA's start-up and tail then overlap its neighbour's stream) -- unless the
  // activations' digit form alone takes most of a half SM.
  const bool solo = (xdig_bytes + xsc_bytes) > 48 * 1024 || N <= (int64_t)sms * 128;
  const int slots = solo ? sms : sms * kCtasPerSm;
  int budget = solo ? kSmemBudgetSolo : kSmemBudget;
  // Tile width: the smallest width that covers N in a whole number of waves of resident CTAs.
  // A tile's group-row span must start and end on 16 bytes: any even width for 24-byte blocks,
  // a multiple of 8 for 34-byte blocks.
  const int64_t q = (kind == 4) ? 2 : 8;
  int TN = 0;
  auto tiles_at = [&](int tn) {
    int64_t t = 0;
    for (int i = 0; i < count; i++) t += (Ns[i] + tn - 1) / tn;
    return t;
  };
  for (int64_t waves = 1;; waves++) {
    TN = (int)(q * ((N + q * slots * waves - 1) / (q * slots * waves)));
    while (tiles_at(TN) > slots * waves) TN += (int)q;   // several matrices: each one's last tile is partial
    if (TN <= (solo ? 128 : 112)) break;
  }
  p.TN = TN;
  p.tile0[0] = 0;
  for (int i = 0; i < count; i++) {
    p.N[i] = (int)Ns[i];
    p.tile0[i + 1] = p.tile0[i] + (int)((Ns[i] + TN - 1) / TN);
  }
  pl.tiles = p.tile0[count];
  // Phases: a multiple of 4 (so TN * phases fills whole warps), aiming at kMaxConsumerThreads.
  int phases = 0, stages = 0;
  for (pl.rpp = kRowsPerPhase; pl.rpp >= kRowsPerPhase - 1; pl.rpp--) {
    phases = (kMaxConsumerThreads / TN) & ~3;
    if (phases < 4) phases = 4;
    while (phases > 4 && (phases * pl.rpp > p.G * 2)) phases -= 4;  // short K: do not over-split
    p.phases = phases;
    p.nthreads = TN * phases;
    p.row_pitch = TN * BB;
    p.stage_rows = phases * pl.rpp;
    p.stage_bytes = ((p.stage_rows * p.row_pitch + 127) / 128) * 128;   // 128: alignment of a tensor-map box in shared memory
    p.xdig_off = kHeader;
    p.xsc_off = p.xdig_off + xdig_bytes;
    p.ring_off = ((p.xsc_off + xsc_bytes + 1023) / 1024) * 1024;
    // A one-CTA-per-SM tile whose whole K-slice fits a half-SM ring needs no more than that: the
    // smaller footprint lets the next launch's CTA move in beside it (programmatic dependent launch),
    // so start-up and tail of back-to-back launches overlap (4096 x 4096: 6.6 -> 5.6 us).
    int budget_here = budget;
    if (solo && (int64_t)p.G * p.row_pitch <= (int64_t)(kSmemBudget - p.ring_off - 64) &&
        (kSmemBudget - p.ring_off - 64) / p.stage_bytes >= 2)
      budget_here = kSmemBudget;
    const int room = budget_here - p.ring_off - 64;
    stages = room / p.stage_bytes;
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages >= 4 || (int64_t)stages * p.stage_rows >= p.G) break;   // deep enough, or the ring holds all of K
  }
  if (pl.rpp < kRowsPerPhase - 1) pl.rpp = kRowsPerPhase - 1;
  p.stages = stages;
  // Boxes pay where the per-copy cost of row-by-row bulk copies sets the pace: short row segments and
  // many of them.  Measured (M = 1, Q4): 14336 x 4096 (672-byte rows, 448 group-rows) 18.2 -> 12.2 us,
  // 8192 x 8192 (1344, 256) 13.1 -> 11.5 us; but 4096 x 4096 (672, 128) 5.6 -> 6.1 us and
  // 4096 x 11008 (1824, 128) 9.1 -> 10.1 us.  (A box side holds at most 256 64-bit words.)
  p.use_tma = (p.row_pitch <= 1408 && p.G >= 192 && p.stage_rows <= 256) ? 1 : 0;
  const size_t red = (size_t)phases * MR * TN * 4;
  const size_t ring = (size_t)(stages > 0 ? stages : 0) * p.stage_bytes + 64;
  pl.smem = p.ring_off + (ring > red ? ring : red);
  pl.ok = stages >= 2 && p.nthreads <= kMaxConsumerThreads && pl.smem <= 227 * 1024;
  return pl;
}

// Tensor maps of the plan's matrices: each packed matrix as [G][N * block bytes / 8] 64-bit words,
// box = one stage of one tile.  Leaves the plan on plain bulk copies if the driver entry is missing.
void make_tensor_maps(Plan& pl, int kind, TensorMaps& tm) {
  if (!pl.p.use_tma) return;
  EncodeTiledFn enc = encode_fn();
  const int BB = (kind == 4) ? kQ4Bytes : kQ8Bytes;
  for (int i = 0; i < pl.p.nmat && enc; i++) {
    const cuuint64_t dims[2] = {(cuuint64_t)pl.p.N[i] * BB / 8, (cuuint64_t)pl.p.G};
    const cuuint64_t strides[1] = {(cuuint64_t)pl.p.N[i] * BB};
    const cuuint32_t box[2] = {(cuuint32_t)pl.p.row_pitch / 8, (cuuint32_t)pl.p.stage_rows};
    const cuuint32_t estr[2] = {1, 1};
    if (enc(&tm.m[i], CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<uint8_t*>(pl.p.B[i]), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      enc = nullptr;
  }
  if (!enc) pl.p.use_tma = 0;
}

template <int KIND, int MR, int RPP, bool COLL, bool WIDE>
cudaError_t launch_one_mode(Plan& pl, cudaStream_t s) {
  static PerDeviceFlag configured;              // the attribute belongs to a device, not to the process
  bool* set = configured.here();
  if (!set) return cudaErrorInvalidDevice;
  if (!*set) {
    cudaError_t e =
        cudaFuncSetAttribute(qgemv_kernel<KIND, MR, RPP, COLL, WIDE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    *set = true;
  }
  const int threads = ((pl.p.nthreads + 31) / 32) * 32 + 32;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)pl.tiles);
  cfg.blockDim = dim3((unsigned)threads);
  cfg.dynamicSmemBytes = pl.smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  TensorMaps tm{};
  make_tensor_maps(pl, KIND, tm);
  const cudaError_t e = cudaLaunchKernelEx(&cfg, qgemv_kernel<KIND, MR, RPP, COLL, WIDE>, pl.p, tm);
  count_launch();
  return e;
}

template <int KIND, int MR, int RPP>
cudaError_t launch_one(Plan& pl, cudaStream_t s) {
  if (pl.p.world == 0) return launch_one_mode<KIND, MR, RPP, false, false>(pl, s);
  return pl.smem > 113 * 1024 ? launch_one_mode<KIND, MR, RPP, true, true>(pl, s)
                              : launch_one_mode<KIND, MR, RPP, true, false>(pl, s);
}

}  // namespace

int qgemv_tiles(int kind, int64_t M, int64_t N, int64_t K) {
  const Plan pl = make_plan(kind, M, &N, 1, K);
  return pl.ok ? pl.tiles : -1;
}

bool qgemv_supports(int kind, int64_t M, int64_t N, int64_t K, int64_t groups) {
  if (kind != 4 && kind != 8) return false;
  if (M < 1 || M > kMaxRowsM) return false;
  if (N < 8 || (N % 8) != 0) return false;  // 16-byte alignment of every group-row span
  if (K < 32 || (K % 32) != 0 || groups != K / 32) return false;
  if (N > (1 << 30) || K > (1 << 22)) return false;
  return make_plan(kind, M, &N, 1, K).ok;    // activations' digit form must fit beside the ring
}

bool qgemv_supports_multi(int kind, int64_t M, const int64_t* Ns, int count, int64_t K, int64_t groups) {
  if (count < 1 || count > kMaxMats) return false;
  for (int i = 0; i < count; i++)
    if (!qgemv_supports(kind, M, Ns[i], K, groups)) return false;
  return make_plan(kind, M, Ns, count, K).ok;
}

cudaError_t launch_qgemv_multi(int kind, const float* A, int count, const uint8_t* const* Bs, float* const* Cs,
                               const int64_t* Ns, int64_t M, int64_t K, int64_t groups, cudaStream_t s) {
  (void)groups;
  if (count < 1 || count > kMaxMats) return cudaErrorInvalidValue;
  if (reinterpret_cast<uintptr_t>(A) & 15) return cudaErrorMisalignedAddress;
  Plan pl = make_plan(kind, M, Ns, count, K);
  if (!pl.ok) return cudaErrorInvalidValue;
  pl.p.A = A;
  for (int i = 0; i < count; i++) {
    if (reinterpret_cast<uintptr_t>(Bs[i]) & 15) return cudaErrorMisalignedAddress;
    pl.p.B[i] = Bs[i], pl.p.C[i] = Cs[i];
  }
  pl.p.status = kernel_status_ptr();
  if (!pl.p.status) return cudaErrorUnknown;
  pl.p.world = 0;
#define SMITH_GEMV_CASE(KD, MRV) \
  if (kind == KD && M == MRV) return pl.rpp == 3 ? launch_one<KD, MRV, 3>(pl, s) : launch_one<KD, MRV, 4>(pl, s);
  SMITH_GEMV_CASE(4, 1) SMITH_GEMV_CASE(4, 2) SMITH_GEMV_CASE(4, 3) SMITH_GEMV_CASE(4, 4)
  SMITH_GEMV_CASE(8, 1) SMITH_GEMV_CASE(8, 2) SMITH_GEMV_CASE(8, 3) SMITH_GEMV_CASE(8, 4)
#undef SMITH_GEMV_CASE
  return cudaErrorInvalidValue;
}

cudaError_t launch_qgemv(int kind, const float* A, const uint8_t* B, float* C, int64_t M, int64_t N, int64_t K,
                         int64_t groups, cudaStream_t s) {
  return launch_qgemv_gather(kind, A, B, C, M, N, K, groups, nullptr, s);
}

cudaError_t launch_qgemv_gather(int kind, const float* A, const uint8_t* B, float* C, int64_t M, int64_t N,
                                int64_t K, int64_t groups, const GemvGather* g, cudaStream_t s) {
  (void)groups;
  if ((reinterpret_cast<uintptr_t>(B) & 15) || (reinterpret_cast<uintptr_t>(A) & 15)) return cudaErrorMisalignedAddress;
  Plan pl = make_plan(kind, M, &N, 1, K);
  if (!pl.ok) return cudaErrorInvalidValue;
  pl.p.A = A, pl.p.B[0] = B, pl.p.C[0] = C;
  pl.p.status = kernel_status_ptr();
  if (!pl.p.status) return cudaErrorUnknown;
  pl.p.world = 0;
  if (g) {
    if (g->world < 1 || g->world > kMaxPeers || g->rank < 0 || g->rank >= g->world) return cudaErrorInvalidValue;
    pl.p.world = g->world, pl.p.rank = g->rank, pl.p.n0 = (int)g->n0, pl.p.n_total = (int)g->n_total;
    pl.p.target = g->target;
    pl.p.reduce = g->reduce;
    pl.p.defer = (g->defer && !g->reduce) ? 1 : 0;
    pl.p.a_prev = (pl.p.defer && g->a_prev) ? 1 : 0;
    if (pl.p.a_prev && (K != g->n_total)) return cudaErrorInvalidValue;
    if (g->reduce && !C) return cudaErrorInvalidValue;
    for (int r = 0; r < g->world; r++) {
      pl.p.y[r] = g->y[r];
      pl.p.state[r] = g->state[r];
      if (!pl.p.y[r] || !pl.p.state[r]) return cudaErrorInvalidValue;
    }
  }
#define SMITH_GEMV_CASE(KD, MRV) \
  if (kind == KD && M == MRV) return pl.rpp == 3 ? launch_one<KD, MRV, 3>(pl, s) : launch_one<KD, MRV, 4>(pl, s);
  SMITH_GEMV_CASE(4, 1) SMITH_GEMV_CASE(4, 2) SMITH_GEMV_CASE(4, 3) SMITH_GEMV_CASE(4, 4)
  SMITH_GEMV_CASE(8, 1) SMITH_GEMV_CASE(8, 2) SMITH_GEMV_CASE(8, 3) SMITH_GEMV_CASE(8, 4)
#undef SMITH_GEMV_CASE
  return cudaErrorInvalidValue;
}

cudaError_t launch_gather_wait(const unsigned* state, const void* y, int64_t M, int64_t n_total, cudaStream_t s) {
  int* status = kernel_status_ptr();
  if (!status) return cudaErrorUnknown;
  // an ordinary launch: it starts after its predecessor has completed
  gather_wait_kernel<<<1, 256, 0, s>>>(state, static_cast<const uint2*>(y), (int)(M * n_total), status);
  count_launch();
  return cudaGetLastError();
}

}  // namespace smith
