// qgemv_list.cu -- a list of GEMV-shaped quantized matmuls (M <= 4) as ONE persistent launch.
//
// A decode step is a fixed sequence of such products (src/gguf_cache.js:121-171: per layer wq, wk,
// wv, wo, gate, up, down, then the output projection).  Launched one by one, each pays a start-up
// (barrier set-up, the first copies' trip to HBM and back) and a tail (the last stage's dot
// products, the phase reduction, the CTAs leaving their SMs) during which HBM idles: at
// 4096 x 14336 that is 2.7 of every 9.0 us.  Here one grid of one CTA per SM walks the whole list:
//
//  * Every CTA keeps ONE ring of shared-memory stages alive for the whole launch.  Its producer
//    warp issues the bulk copies of item i + 1's first stages while the consumer warps still work
//    on item i, so the stream of packed weights from HBM never drains between matrices.
//  * Item i is cut into tiles of TN_i columns x all of K_i; tile t runs on CTA
//    (first_cta_i + t) mod grid, where first_cta_i continues where item i - 1 stopped, so items
//    whose tile count is not a multiple of the grid still load the SMs evenly.
//  * The arithmetic is the GEMV kernel's (qgemv_common.cuh): activations in block fixed point as
//    two int8 digits, dp4a against the codes, exact integer group sums, f32 scale-and-add.
//  * Hazards between items are resolved on the device.  An item that reads what an earlier item
//    writes (or writes what one reads or writes) waits -- bounded -- until that item's counter of
//    outstanding output warps has reached zero.  Only the consumers wait: the producer keeps
//    filling the ring with the dependent item's weights, which no item writes.
//  * The pointwise glue of the step is folded in (src/gguf_cache.js:121,156-163):
//      - RMSNorm on the way in (shaders/rmsnorm.metal:15-49): y = x * rsqrt(mean(x^2) + eps) * gamma
//        is applied while the activations are turned into digits;
//      - SwiGLU on the way out (shaders/swiglu.metal:12-22): an item with two packed matrices
//        (gate, up) accumulates both products for its columns and stores silu(g) * u;
//      - the residual add (A.add(x, projected)): C = residual + product.
//
// Counters: done[i] starts a launch at the number of tiles of item i and drops by one per finished
// tile.  The fence that must separate a tile's stores from that count, and the atomic itself,
// cost the consumer warps a microsecond per tile when they issue them (measured: 8.2 -> 6.8 us per
// 4096 x 14336 matrix without them), so a warp of its own does it: the consumers hand each
// finished tile to it through a small mailbox ring of mbarriers and go on with the next tile.
// The last CTA to leave restores all counters, also after a give-up, so the next launch starts clean.
//
// Every wait is bounded (pipeline.cuh); one that gives up raises the status word.
#include <cuda.h>

#include <cstdarg>
#include <cstddef>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "kernels.h"
#include "pipeline.cuh"
#include "qgemv_common.cuh"

namespace smith {
namespace {

constexpr int kListMaxThreads = 448;   // consumer threads per CTA: 28 warps, plus a producer and a signalling warp,
                                       // at 64 registers a thread
constexpr int kListMaxStages = 8;
constexpr int kListHeader = 1536;      // barriers, abort flag, mailbox of finished tiles, three copies of an item
constexpr int kListDescOff = 512;
constexpr int kListSmem = 226 * 1024;     // dynamic part; the kernel's static shared memory takes up to 1 KB of the 227
constexpr int kListMaxDeps = 4;
constexpr int kListCounterStride = 32;  // words between two items' counters: one 128-byte line each, so that the
                                       // pollers of one item do not queue up with the decrements of another
constexpr int kListSigSlots = 4;       // finished tiles in flight to the signalling warp
constexpr int kListMaxTN = 112;        // widest tile: two panels of 56 columns (34-byte blocks) still fit a box

// What the kernel needs to know about one item: 64 words.
struct alignas(128) ItemHot {
  const float* A;
  const uint8_t* B0;
  const uint8_t* B1;        // second packed matrix of a gate/up pair, else null
  float* C;
  const float* gamma;       // RMSNorm weights [K], or null
  const float* residual;    // [M, N] added to the product, or null (may be C itself)
  int N, K, G, TN;
  int tiles, first_cta, phases, rpp;
  int stage_rows, row_pitch, nst;
  int c0;                   // 0: one bulk copy per group-row; else stages arrive as tensor-map boxes and c0 = columns of the first panel
  int nB, a_id;             // a_id: items with equal a_id read the same activations in the same state
  float eps;
  int ndeps;
  int dep[kListMaxDeps];    // earlier items that must be complete before this one touches its operands
  // Channels: tagged copies [M][N] of {value bits, launch tag} pairs through which an item hands its
  // output to the items that read it, element by element, without any fence or counter in between.
  const uint2* a_chan;      // read the activations from this channel instead of A (null: from A)
  const uint2* r_chan;      // read the residual from this channel instead of `residual`
  uint2* c_chan;            // also store the output here (null: no later item reads it whole)
  // Fused all-gather (weights sharded along N over several GPUs): the output is this rank's columns
  // [g_n0, g_n0 + N) of a row of g_n_total, stored as tagged pairs into every rank's row buffer
  // ([2][M][g_n_total] pairs, the half chosen by the launch tag's parity).
  int g_world, g_n0, g_n_total, g_pad;
  uint2* const* g_rows;     // [g_world] row buffers, rank by rank (device array)
  int pad[20];
};
static_assert(sizeof(ItemHot) == 256, "ItemHot is 64 words");
// 32-bit word offsets of ItemHot's fields (the consumers read them from a copy in shared memory)
enum : int {
  kW_A = 0, kW_B0 = 2, kW_B1 = 4, kW_C = 6, kW_gamma = 8, kW_residual = 10, kW_N = 12, kW_K = 13, kW_G = 14, kW_TN = 15,
  kW_tiles = 16, kW_first_cta = 17, kW_phases = 18, kW_rpp = 19, kW_stage_rows = 20, kW_row_pitch = 21, kW_nst = 22,
  kW_c0 = 23, kW_nB = 24, kW_a_id = 25, kW_eps = 26, kW_ndeps = 27, kW_dep = 28, kW_a_chan = 32, kW_r_chan = 34, kW_c_chan = 36,
  kW_g_world = 38, kW_g_n0 = 39, kW_g_n_total = 40, kW_g_rows = 42
};
static_assert(offsetof(ItemHot, N) == 4 * kW_N && offsetof(ItemHot, tiles) == 4 * kW_tiles &&
              offsetof(ItemHot, stage_rows) == 4 * kW_stage_rows && offsetof(ItemHot, nB) == 4 * kW_nB &&
              offsetof(ItemHot, eps) == 4 * kW_eps && offsetof(ItemHot, dep) == 4 * kW_dep && offsetof(ItemHot, C) == 4 * kW_C &&
              offsetof(ItemHot, residual) == 4 * kW_residual && offsetof(ItemHot, a_chan) == 4 * kW_a_chan &&
              offsetof(ItemHot, c_chan) == 4 * kW_c_chan && offsetof(ItemHot, g_world) == 4 * kW_g_world &&
              offsetof(ItemHot, g_rows) == 4 * kW_g_rows, "word offsets follow the struct");

struct RowCheck {
  const uint2* row;         // [2][count] pairs
  int count;                // M * n_total
  int pad;
};

struct ListParams {
  const ItemHot* items;
  const CUtensorMap* maps;  // [4 * nitems]: per item {B0 panel 0, B0 panel 1, B1 panel 0, B1 panel 1}
  unsigned* done;           // [nitems * kListCounterStride] outstanding tiles per item
  const unsigned* done_init;  // [nitems]
  unsigned* ticket;         // CTAs that have left
  unsigned* epoch;          // launch tag of the channels: starts at 1, advanced by the last CTA to leave
  // rows this rank gathers: before the launch ends, every pair of them must carry the launch's tag
  const RowCheck* checks;
  int nchecks;
#ifdef SMITH_LIST_TRACE
  unsigned long long* trace;   // [nitems][grid][8] global-timer stamps (measurement builds only)
#endif
  int* status;
  int nitems;
  int M;
  int nwarps;               // consumer warps per CTA
  int slots, slot_bytes;
  int xdig_off, xsc_off, rms_off, red_off, red_half, ring_off;  // byte offsets in dynamic shared memory
};

// What the producer warp needs of an item; loaded field by field so that it lives in registers.
struct ProdItem {
  const uint8_t* B0;
  const uint8_t* B1;
  int N, G, TN, tiles, first_cta, stage_rows, row_pitch, nst, c0, nB;
};
__device__ __forceinline__ ProdItem load_prod_item(const ItemHot* p) {
  const uint32_t* w = reinterpret_cast<const uint32_t*>(p);
  const uint4 a = __ldg(reinterpret_cast<const uint4*>(w)), b = __ldg(reinterpret_cast<const uint4*>(w + 4));
  const uint4 c = __ldg(reinterpret_cast<const uint4*>(w + 12)), d = __ldg(reinterpret_cast<const uint4*>(w + 16));
  const uint4 e = __ldg(reinterpret_cast<const uint4*>(w + 20));
  ProdItem it;
  it.B0 = reinterpret_cast<const uint8_t*>(((uint64_t)a.w << 32) | a.z);
  it.B1 = reinterpret_cast<const uint8_t*>(((uint64_t)b.y << 32) | b.x);
  it.N = (int)c.x, it.G = (int)c.z, it.TN = (int)c.w;
  it.tiles = (int)d.x, it.first_cta = (int)d.y;
  it.stage_rows = (int)e.x, it.row_pitch = (int)e.y, it.nst = (int)e.z, it.c0 = (int)e.w;
  it.nB = (int)__ldg(w + kW_nB);
  return it;
}

#ifdef SMITH_LIST_TRACE
__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define TRACE(ev) do { if (tid == 0 && p.trace) p.trace[((size_t)i * gridDim.x + blockIdx.x) * 8 + (ev)] = gtime(); } while (0)
#else
#define TRACE(ev) do { } while (0)
#endif

__device__ __forceinline__ uint4 ld_volatile_v4(const uint2* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint2 ld_volatile_v2(const uint2* p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_volatile_v2(uint2* p, uint32_t a, uint32_t b) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}

// Bounded wait until item `dep` is complete everywhere (its counter of outstanding tiles is zero).
__device__ __forceinline__ bool wait_item(const unsigned* counter, const int* status) {
  const long long t0 = clock64();
  for (unsigned spin = 0;; spin++) {
    unsigned seen;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
    if (seen == 0u) return true;
    if ((spin & 63u) == 63u) {
      if (*reinterpret_cast<const volatile int*>(status)) return false;   // someone else gave up: do not sit out the limit
      if (clock64() - t0 > kWaitLimitCycles) return false;
    }
  }
}

// Barrier over the consumer threads that also tells every one of them whether any has given up, so
// that they all leave together and none is left waiting at a later barrier.
__device__ __forceinline__ bool consumers_sync_any(int nct, bool mine) {
  uint32_t any;
  asm volatile(
      "{\n.reg .pred p, q;\n"
      "setp.ne.u32 q, %2, 0;\n"
      "bar.red.or.pred p, 1, %1, q;\n"
      "selp.u32 %0, 1, 0, p;\n}"
      : "=r"(any)
      : "r"(nct), "r"(mine ? 1u : 0u)
      : "memory");
  return any != 0;
}

// One stage against the digits: this thread's column (at byte `base` of a stage row of its panel,
// rows `pitch` bytes apart), group-rows phase, phase + phases, ... of the stage.
template <int KIND, int MR>
__device__ __forceinline__ void consume_stage(const uint8_t* stage, int st, int stage_rows, int rpp, int G, int phases,
                                              int phase, uint32_t base, uint32_t pitch, const uint4* xdig,
                                              const float2* xsc, float (&acc)[MR]) {
  // 32-bit shared-memory addresses throughout: a per-thread base plus strides
  const int g0 = st * stage_rows + phase;
  const uint32_t step = (uint32_t)phases * pitch;
  uint32_t blk = smem_u32(stage) + base + (uint32_t)phase * pitch;
  uint32_t xd = smem_u32(xdig) + (uint32_t)g0 * 64u, xs = smem_u32(xsc) + (uint32_t)g0 * 8u;
  const uint32_t xd_step = (uint32_t)phases * 64u, xs_step = (uint32_t)phases * 8u;
  if (st * stage_rows + stage_rows <= G) {
    int rr = 0;
    for (; rr + 4 <= rpp; rr += 4) {
#pragma unroll
      for (int u = 0; u < 4; u++) {
        block_dot_s<KIND, MR>(blk, xd, xs, G, acc);
        blk += step, xd += xd_step, xs += xs_step;
      }
    }
    for (; rr < rpp; rr++) {
      block_dot_s<KIND, MR>(blk, xd, xs, G, acc);
      blk += step, xd += xd_step, xs += xs_step;
    }
  } else {
    for (int rr = 0; rr < rpp; rr++) {
      if (g0 + rr * phases < G) block_dot_s<KIND, MR>(blk, xd, xs, G, acc);
      blk += step, xd += xd_step, xs += xs_step;
    }
  }
}

// CHAN: the list has channels.  Lists without them (independent products) run an instantiation that
// carries none of that code: inside the plain kernel it cost 0.4 to 0.6 us per tile.
template <int KIND, int MR, bool CHAN>
__global__ void __launch_bounds__(kListMaxThreads + 64, 1) qgemv_list_kernel(const ListParams p) {
  constexpr int BB = (KIND == 4) ? kQ4Bytes : kQ8Bytes;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty = full + kListMaxStages;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 2 * kListMaxStages * 8);
  uint64_t* sig_full = reinterpret_cast<uint64_t*>(smem + 256);                 // a finished tile is posted
  uint64_t* sig_empty = sig_full + kListSigSlots;                               // ... and has been counted
  volatile int* sig_item = reinterpret_cast<volatile int*>(smem + 256 + 2 * kListSigSlots * 8);
  uint4* xdig = reinterpret_cast<uint4*>(smem + p.xdig_off);     // [MR][G][4] uint4
  float2* xsc = reinterpret_cast<float2*>(smem + p.xsc_off);     // [MR][G]
  float* rms_part = reinterpret_cast<float*>(smem + p.rms_off);  // [MR][nwarps]
  uint8_t* ring = smem + p.ring_off;

  const int tid = threadIdx.x;
  const int nwarps = p.nwarps;
  const int ncta = (int)gridDim.x, cta = (int)blockIdx.x;
  const int nct = nwarps * 32;                    // consumer threads

  if (tid == 0) {
    for (int s = 0; s < p.slots; s++) {
      mbar_init(smem_u32(&full[s]), 1);
      mbar_init(smem_u32(&empty[s]), nwarps);
    }
    for (int s = 0; s < kListSigSlots; s++) {
      mbar_init(smem_u32(&sig_full[s]), nwarps);
      mbar_init(smem_u32(&sig_empty[s]), 1);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (tid >= nct + 32) {
    // ------------------------------------------------------------ signalling warp
    // Counts finished tiles: waits for the consumers to post one, fences (their stores to C become
    // visible device-wide before the count) and decrements the item's counter.  An item index of -1
    // ends it.
    if ((tid & 31) == 0) {
      int slot = 0;
      uint32_t par = 0;
      for (;;) {
        if (!mbar_wait(smem_u32(&sig_full[slot]), par, abort_flag, p.status)) break;
        const int item = sig_item[slot];
        if (item >= 0)   // release at device scope: the tile's stores (seen through the mailbox barrier) come first
          asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p.done + (size_t)item * kListCounterStride), "r"(0xFFFFFFFFu)
                       : "memory");
        mbar_arrive(smem_u32(&sig_empty[slot]));
        if (item < 0) break;
        slot = (slot + 1 == kListSigSlots) ? 0 : slot + 1;
        par ^= (slot == 0);
      }
    }
  } else if (tid >= nct) {
    // ------------------------------------------------------------ producer warp
    // Walks items, tiles and stages in the consumers' order, one ring slot per stage, and never
    // waits for anything but a free slot.
    const int lane = tid & 31;
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    bool live = true;
    int slot = 0;
    uint32_t par = 0;                               // parity of this pass over the ring
    int issued = 0;                                 // stages issued so far, saturating at the ring depth
    ProdItem nxt = load_prod_item(p.items);
    for (int i = 0; i < p.nitems && live; i++) {
      const ProdItem it = nxt;
      if (i + 1 < p.nitems) nxt = load_prod_item(p.items + i + 1);
      int t = cta - it.first_cta;
      if (t < 0) t += ncta;
      for (; t < it.tiles && live; t += ncta) {
        const int col0 = t * it.TN;
        const int tn = min(it.TN, it.N - col0);
        const uint32_t row_bytes = (uint32_t)tn * BB;
        for (int bi = 0; bi < it.nB && live; bi++) {
          const uint8_t* __restrict__ Bm = bi ? it.B1 : it.B0;
          const CUtensorMap* map = p.maps + 4 * i + 2 * bi;
          for (int st = 0; st < it.nst; st++) {
            if (issued >= p.slots) {
              int okw = 1;
              if (lane == 0) okw = mbar_wait(smem_u32(&empty[slot]), par ^ 1u, abort_flag, p.status);
              live = __shfl_sync(0xffffffffu, okw, 0) != 0;
              if (!live) break;
            } else {
              issued++;
            }
            const int rows = min(it.stage_rows, it.G - st * it.stage_rows);
            const uint32_t bar = smem_u32(&full[slot]);
            const uint32_t dst = smem_u32(ring + (size_t)slot * p.slot_bytes);
            if (it.c0) {
              // One box per panel, always stage_rows x panel columns: what lies beyond N or the last
              // group-row is zero-filled.  The second panel starts on the next 128 bytes.
              if (lane == 0) mbar_expect_tx(bar, (uint32_t)it.stage_rows * (uint32_t)it.row_pitch);
              __syncwarp();
              const int c1 = it.TN - it.c0;
              if (lane == 0) tma_box_2d(dst, map, (col0 * BB) >> 3, st * it.stage_rows, bar, policy);
              if (lane == 1 && c1 > 0)
                tma_box_2d(dst + (((uint32_t)it.stage_rows * it.c0 * BB + 127u) & ~127u), map + 1, ((col0 + it.c0) * BB) >> 3,
                           st * it.stage_rows, bar, policy);
            } else {
              if (lane == 0) mbar_expect_tx(bar, (uint32_t)rows * row_bytes);
              __syncwarp();
              const uint8_t* src = Bm + ((size_t)st * it.stage_rows * it.N + col0) * BB;
              for (int rr = lane; rr < rows; rr += 32)
                bulk_load(dst + rr * it.row_pitch, src + (size_t)rr * it.N * BB, row_bytes, bar, policy);
            }
            slot = (slot + 1 == p.slots) ? 0 : slot + 1;
            par ^= (slot == 0);
          }
        }
      }
    }
    // consumers observe every full barrier they were promised, so all copies have landed before the CTA ends
  } else {
    // -------------------------------------------------------------- consumers
    // `ok` is a thread's own view (a wait of its warp gave up); `quit` is what all consumers learn
    // together at a barrier, so that every barrier below is reached by all of them or by none.
    //
    // The consumers keep the current item in shared memory, not in registers (28 warps leave 64
    // registers a thread).  Three copies rotate: while item i is worked on, warp 0 fetches item
    // i + 1 and stores it before the first barrier it meets in item i, so every thread finds it
    // after that barrier; the copy it overwrites belonged to item i - 2, which no thread reads
    // any more once warp 0 has left item i - 1.
    const int lane = tid & 31, warp = tid >> 5;
    bool ok = true, quit = false;
    int slot = 0;
    uint32_t par = 0;
    int cur_a = -1;                                 // a_id whose digits are in shared memory
    int red_buf = 0;
    int sig_slot = 0, sig_used = 0;                 // mailbox slot of the next finished tile
    uint32_t sig_par = 0;
    // Hands a finished tile (or the end mark) to the signalling warp.  Thread 0 first makes sure the
    // slot's previous tile has been counted; its warp's arrival is the last a phase can get, so the
    // item index is in place when the phase completes.
    auto post = [&](int item) {
      if (tid == 0) {
        if (sig_used >= kListSigSlots) mbar_wait(smem_u32(&sig_empty[sig_slot]), sig_par ^ 1u, abort_flag, p.status);
        sig_item[sig_slot] = item;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sig_full[sig_slot]));
      if (sig_used < kListSigSlots) sig_used++;
      sig_slot = (sig_slot + 1 == kListSigSlots) ? 0 : sig_slot + 1;
      sig_par ^= (sig_slot == 0);
    };
    volatile uint32_t* dring = reinterpret_cast<volatile uint32_t*>(smem + kListDescOff);
    if (warp == 0) {
      const uint2 w = __ldg(reinterpret_cast<const uint2*>(p.items) + lane);
      dring[2 * lane] = w.x, dring[2 * lane + 1] = w.y;
    }
    const unsigned tag = CHAN ? *reinterpret_cast<const volatile unsigned*>(p.epoch) : 0u;   // the last CTA to leave advances it
    quit = consumers_sync_any(nct, false);
    int db = 0;                                     // which copy holds item i
    for (int i = 0; i < p.nitems && !quit; i++, db = (db == 2) ? 0 : db + 1) {
      // plain loads: an item's copy does not change while it is read, and every barrier below is a compiler fence
      const uint32_t* D = const_cast<const uint32_t*>(dring) + db * 64;
      auto ptr_of = [&](int w) { return ((uint64_t)D[w + 1] << 32) | D[w]; };
      uint2 pre = make_uint2(0u, 0u);
      if (warp == 0 && i + 1 < p.nitems) pre = __ldg(reinterpret_cast<const uint2*>(p.items + i + 1) + lane);
      bool published = false;
      auto publish = [&]() {                        // call before a barrier
        if (warp == 0 && !published) {
          volatile uint32_t* nd = dring + ((db == 2) ? 0 : db + 1) * 64;
          nd[2 * lane] = pre.x, nd[2 * lane + 1] = pre.y;
        }
        published = true;
      };
      const int tiles = (int)D[kW_tiles];
      int t = cta - (int)D[kW_first_cta];
      if (t < 0) t += ncta;
      if (t >= tiles) {                             // no tile of this item runs here
        publish();
        quit = consumers_sync_any(nct, !ok);
        continue;
      }
      // ---- hazards: every earlier item this one depends on must be complete everywhere.  One thread
      // polls (a couple of thousand pollers on one line of L2 delay the very decrements they wait for).
      const int ndeps = (int)D[kW_ndeps];
      if (ndeps > 0) {
        if (tid == 0 && ok) {
          bool there = true;
          for (int d = 0; d < ndeps && there; d++)
            there = wait_item(p.done + (size_t)D[kW_dep + d] * kListCounterStride, p.status);
          if (!there) {
            *abort_flag = 1;
            atomicExch(p.status, 1);
            ok = false;
          }
        }
        publish();
        quit = consumers_sync_any(nct, !ok);
        if (quit) break;
      }
      const int G = (int)D[kW_G];
      TRACE(0);                                     // hazards resolved
      // ---- activations -> digit words (skipped when the previous item left the same ones)
      if ((int)D[kW_a_id] != cur_a) {
        cur_a = (int)D[kW_a_id];
        // (row, group) pairs are laid out as [MR][G], which is also the order of A's 32-element chunks.
        // RMSNorm (shaders/rmsnorm.metal:33-48: y = x * rsqrt(mean(x^2) + eps) * gamma) costs no second pass
        // over x: the digits are taken of x * gamma and the row's 1/rms goes into the groups' scale factors.
        const float* A = reinterpret_cast<const float*>(ptr_of(kW_A));
        const uint2* achan = CHAN ? reinterpret_cast<const uint2*>(ptr_of(kW_a_chan)) : nullptr;
        const float* gamma = reinterpret_cast<const float*>(ptr_of(kW_gamma));
        const long long t_chan = clock64();
        float ss[MR];
#pragma unroll
        for (int m = 0; m < MR; m++) ss[m] = 0.f;
        const bool norm = gamma != nullptr;
        // Eight threads per (row, group), four quarters in flight per thread.
        const int total = (MR * G * 8 + 31) & ~31, last = MR * G - 1;
        for (int i0 = tid; i0 < total; i0 += 4 * nct) {
          float4 tv[4], gm[4];
          if (achan) {
            // Four {value, tag} pairs per quarter.  A pair counts once it carries this launch's tag: the
            // producing item's threads store value and tag as one 8-byte word, so no fence and no
            // counter stands between their store and this load.
            uint4 pa[4], pb[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
              const int q = i0 + u * nct;
              if (q < total) {     // clamp keeps whole warps in the shuffles; duplicates rewrite equal bytes
                const uint2* src = achan + (size_t)min(q >> 3, last) * 32 + (q & 7) * 4;
                pa[u] = ld_volatile_v4(src), pb[u] = ld_volatile_v4(src + 2);
              }
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
              const int q = i0 + u * nct;
              if (q < total) {
                const uint2* src = achan + (size_t)min(q >> 3, last) * 32 + (q & 7) * 4;
                for (unsigned spin = 0; ok && (pa[u].y != tag || pa[u].w != tag || pb[u].y != tag || pb[u].w != tag); spin++) {
                  if ((spin & 15u) == 15u && (clock64() - t_chan > kWaitLimitCycles || *abort_flag)) {
                    *abort_flag = 1;
                    atomicExch(p.status, 1);
                    ok = false;
                  }
                  pa[u] = ld_volatile_v4(src), pb[u] = ld_volatile_v4(src + 2);
                }
                tv[u] = make_float4(__uint_as_float(pa[u].x), __uint_as_float(pa[u].z), __uint_as_float(pb[u].x),
                                    __uint_as_float(pb[u].z));
              }
            }
          } else {
#pragma unroll
            for (int u = 0; u < 4; u++) {
              const int q = i0 + u * nct;
              if (q < total) tv[u] = __ldcg(reinterpret_cast<const float4*>(A + (size_t)min(q >> 3, last) * 32) + (q & 7));
            }
          }
          if (norm) {
#pragma unroll
            for (int u = 0; u < 4; u++) {
              const int q = i0 + u * nct;
              if (q < total) gm[u] = __ldg(reinterpret_cast<const float4*>(gamma + (size_t)(min(q >> 3, last) % G) * 32) + (q & 7));
            }
          }
#pragma unroll
          for (int u = 0; u < 4; u++) {
            const int q = i0 + u * nct;             // warp-uniform: total and nct are multiples of 32
            if (q < total) {
              const int grp = min(q >> 3, last);
              float4 v = tv[u];
              if (norm) {
                if ((q >> 3) <= last) {             // a clamped duplicate must not be counted twice
                  const float s2 = v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                  const int row = grp / G;
#pragma unroll
                  for (int m = 0; m < MR; m++) ss[m] += (row == m) ? s2 : 0.f;
                }
                v = make_float4(v.x * gm[u].x, v.y * gm[u].y, v.z * gm[u].z, v.w * gm[u].w);
              }
              quantise_quarter<KIND>(v, q & 7, reinterpret_cast<uint8_t*>(xdig + (size_t)grp * 4), xsc + grp);
            }
          }
        }
        TRACE(1);                                   // activations loaded and turned into digits (this thread)
        publish();
        if (norm) {
          // the row sums in a fixed order, so that every CTA normalises with the same bits
#pragma unroll
          for (int m = 0; m < MR; m++) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss[m] += __shfl_xor_sync(0xffffffffu, ss[m], o);
            if (lane == 0) rms_part[m * nwarps + warp] = ss[m];
          }
          quit = consumers_sync_any(nct, !ok);
          if (quit) break;
          const float K = (float)(int)D[kW_K], eps = __uint_as_float(D[kW_eps]);
          for (int g = tid; g < MR * G; g += nct) {
            const int row = g / G;
            float tot = 0.f;
            for (int w = 0; w < nwarps; w++) tot += rms_part[row * nwarps + w];
            xsc[g].x *= 1.0f / sqrtf(tot / K + eps);
          }
        }
        quit = consumers_sync_any(nct, !ok);
        if (quit) break;
      }

      TRACE(2);                                     // digits ready for everyone
      const int TN = (int)D[kW_TN], N = (int)D[kW_N], phases = (int)D[kW_phases], nB = (int)D[kW_nB];
      for (; t < tiles && !quit; t += ncta) {
        const int col0 = t * TN;
        const int tn = min(TN, N - col0);
        const bool active = tid < tn * phases;
        const int col = active ? (tid % tn) : 0;
        const int phase = active ? (tid / tn) : 0;
        float acc[MR], gate[MR];
#pragma unroll
        for (int m = 0; m < MR; m++) acc[m] = 0.f, gate[m] = 0.f;
        {
          const int stage_rows = (int)D[kW_stage_rows], rpp = (int)D[kW_rpp], nst = (int)D[kW_nst], c0 = (int)D[kW_c0];
          // where this thread's column sits in a stage: boxes land as one or two dense panels
          uint32_t base = (uint32_t)col * BB, pitch = D[kW_row_pitch];
          if (c0) {
            pitch = (uint32_t)c0 * BB;
            if (col >= c0) {
              base = (((uint32_t)stage_rows * c0 * BB + 127u) & ~127u) + (uint32_t)(col - c0) * BB;
              pitch = (uint32_t)(TN - c0) * BB;
            }
          }
          for (int bi = 0; bi < nB && ok; bi++) {
            if (bi == 1) {
#pragma unroll
              for (int m = 0; m < MR; m++) gate[m] = acc[m], acc[m] = 0.f;
            }
            for (int st = 0; st < nst && ok; st++) {
              ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&full[slot]), par, abort_flag, p.status));   // warp-uniform
              if (bi == 0 && st == 0) TRACE(3);             // first stage of the tile is there
              if (ok && active)
                consume_stage<KIND, MR>(ring + (size_t)slot * p.slot_bytes, st, stage_rows, rpp, G, phases, phase, base, pitch,
                                        xdig, xsc, acc);
              __syncwarp();
              if (lane == 0) mbar_arrive(smem_u32(&empty[slot]));
              slot = (slot + 1 == p.slots) ? 0 : slot + 1;
              par ^= (slot == 0);
            }
          }
        }
        TRACE(4);                                   // main loop done (this thread)
        // ---- sum the phases in fixed order; the scratch alternates between tiles, so one barrier per tile
        float* red = reinterpret_cast<float*>(smem + p.red_off + red_buf * p.red_half);   // [nB][phases][MR][TN]
        red_buf ^= 1;
        const int plane = phases * MR * TN;
        if (active) {
#pragma unroll
          for (int m = 0; m < MR; m++) {
            red[(phase * MR + m) * TN + col] = acc[m];
            if (nB == 2) red[plane + (phase * MR + m) * TN + col] = gate[m];
          }
        }
        publish();
        quit = consumers_sync_any(nct, !ok);
        if (quit) break;
        TRACE(5);                                   // partial sums of all phases in place
        if (tid < p.M * tn) {
          const int m = tid / tn, c = tid - m * tn;
          float v = 0.f;
          for (int ph = 0; ph < phases; ph++) v += red[(ph * MR + m) * TN + c];
          if (nB == 2) {
            // SwiGLU (shaders/swiglu.metal:18-20): the first matrix is the gate, the second is up
            float g = 0.f;
            for (int ph = 0; ph < phases; ph++) g += red[plane + (ph * MR + m) * TN + c];
            v = (g / (1.0f + expf(-g))) * v;
          }
          const size_t at = (size_t)m * N + col0 + c;
          const float* residual = reinterpret_cast<const float*>(ptr_of(kW_residual));
          const uint2* rchan = CHAN ? reinterpret_cast<const uint2*>(ptr_of(kW_r_chan)) : nullptr;
          if (rchan) {
            // the residual element as its producer left it in the channel: valid once it carries this launch's tag
            const long long t0 = clock64();
            uint2 pr = ld_volatile_v2(rchan + at);
            for (unsigned spin = 0; ok && pr.y != tag; spin++) {
              if ((spin & 15u) == 15u && (clock64() - t0 > kWaitLimitCycles || *abort_flag)) {
                *abort_flag = 1;
                atomicExch(p.status, 1);
                ok = false;
              }
              pr = ld_volatile_v2(rchan + at);
            }
            v = __uint_as_float(pr.x) + v;
          } else if (residual) {
            v = __ldcg(residual + at) + v;
          }
          reinterpret_cast<float*>(ptr_of(kW_C))[at] = v;
          uint2* cchan = CHAN ? reinterpret_cast<uint2*>(ptr_of(kW_c_chan)) : nullptr;
          if (cchan) st_volatile_v2(cchan + at, __float_as_uint(v), tag);
          if (CHAN && D[kW_g_world]) {
            // this rank's slice of the gathered row, into every rank's memory: one 8-byte store per
            // element and rank (plain stores over NVLink for the peers), valid by its tag, no fence
            uint2* const* rows = reinterpret_cast<uint2* const*>(ptr_of(kW_g_rows));
            const int gw = (int)D[kW_g_world], nt = (int)D[kW_g_n_total];
            const size_t gat = ((size_t)(tag & 1u) * p.M + m) * nt + (int)D[kW_g_n0] + col0 + c;
            for (int r = 0; r < gw; r++) st_volatile_v2(rows[r] + gat, __float_as_uint(v), tag);
          }
        }
        TRACE(6);                                   // outputs stored (this thread)
        post(i);
      }
    }
    if (CHAN && p.nchecks > 0 && !quit) {
      // The launch may end only when the rows this rank gathers are whole: every pair carries the tag.
      // (This also keeps the ranks within one launch of each other, which is what lets the two halves
      // of a row buffer alternate.)
      const long long t0 = clock64();
      for (int k = 0; k < p.nchecks && ok; k++) {
        const RowCheck ck = p.checks[k];
        const uint2* row = ck.row + (size_t)(tag & 1u) * ck.count;
        for (int e = cta * nct + tid; e < ck.count && ok; e += ncta * nct) {
          uint2 pr = ld_volatile_v2(row + e);
          for (unsigned spin = 0; pr.y != tag; spin++) {
            if ((spin & 15u) == 15u && (clock64() - t0 > kWaitLimitCycles || *abort_flag ||
                                       *reinterpret_cast<const volatile int*>(p.status))) {
              *abort_flag = 1;
              atomicExch(p.status, 1);
              ok = false;
              break;
            }
            pr = ld_volatile_v2(row + e);
          }
        }
      }
    }
    post(-1);
  }

  // ------------------------------------------------ leave: the last CTA restores the counters
  __syncthreads();
  __shared__ unsigned last_flag;
  if (tid == 0) {
    __threadfence();
    last_flag = (atomicAdd(p.ticket, 1u) == gridDim.x - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (last_flag) {
    __threadfence();
    for (int j = tid; j < p.nitems; j += blockDim.x) p.done[(size_t)j * kListCounterStride] = p.done_init[(size_t)j * kListCounterStride];
    if (tid == 0) {
      *p.ticket = 0u;
      *p.epoch = *p.epoch + 1u;
    }
  }
}

// ---------------------------------------------------------------------------------------- host side

// Planner knobs, overridable from the environment for measurements.
struct Tuning {
  int tma;          // 1: stages arrive as tensor-map boxes (default), 0: one bulk copy per group-row
  int stage_bytes;  // target size of a stage
  int max_tn;
};

Tuning tuning() {
  // Measured on B200 with a stand-alone ring (no arithmetic), 4096 x 14336 tiles: 16 bulk copies of
  // 2.3 KB per 37 KB stage, 5 slots: 6.1 TB/s; the same stage as two boxes: 6.2-6.4; 74 KB stages of
  // two boxes, 2-3 slots: 6.6-6.8.  Per-row bulk copies of 656 bytes: 2.4-2.9 TB/s; boxes: 6.4-6.8.
  Tuning t{1, 72 * 1024, kListMaxTN};
  if (const char* v = getenv("SMITH_LIST_TMA")) t.tma = atoi(v) ? 1 : 0;
  if (const char* v = getenv("SMITH_LIST_STAGE_BYTES")) t.stage_bytes = max(4096, min(100 * 1024, atoi(v)));
  if (const char* v = getenv("SMITH_LIST_MAX_TN")) t.max_tn = max(8, min(kListMaxTN, atoi(v)));
  return t;
}

bool overlap(const void* a, size_t an, const void* b, size_t bn) {
  if (!a || !b || !an || !bn) return false;
  const uintptr_t a0 = (uintptr_t)a, b0 = (uintptr_t)b;
  return a0 < b0 + bn && b0 < a0 + an;
}

int list_fail(const char** why, const char* fmt, ...) {
  static thread_local char buf[256];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (why) *why = buf;
  return 1;
}

// Tiling of one item for a grid of `ncta` CTAs.
void plan_item(int kind, int M, const ListItemDesc& d, int ncta, int stage_bytes, const Tuning& tu, ItemHot& h) {
  const int BB = (kind == 4) ? kQ4Bytes : kQ8Bytes;
  const int64_t q = (kind == 4) ? 2 : 8;          // a tile's group-row span starts and ends on 16 bytes
  h.N = (int)d.N, h.K = (int)d.K, h.G = (int)(d.K / 32);
  int TN = 0;
  for (int64_t waves = 1;; waves++) {
    TN = (int)(q * ((d.N + q * ncta * waves - 1) / (q * ncta * waves)));
    if (TN <= tu.max_tn) break;
  }
  h.TN = TN;
  h.tiles = (int)((d.N + TN - 1) / TN);
  // K-phases: as many as fill the consumer threads, no more than there are group-rows
  int phases = kListMaxThreads / TN;
  if (phases > h.G) phases = h.G;
  if (phases < 1) phases = 1;
  h.phases = phases;
  h.row_pitch = TN * BB;
  // group-rows per phase and stage: large stages stream best, but none larger than K needs
  int rpp = stage_bytes / (phases * h.row_pitch);
  const int need = (h.G + phases - 1) / phases;
  if (rpp > need) rpp = need;
  if (rpp * phases > 256) rpp = 256 / phases;     // a box side holds at most 256 rows
  if (rpp < 1) rpp = 1;
  h.rpp = rpp;
  h.stage_rows = phases * rpp;
  h.nst = (h.G + h.stage_rows - 1) / h.stage_rows;
  // Boxes: a box side holds at most 256 elements of 8 bytes, so tiles wider than 2 KB arrive as two
  // panels; each panel's first column must start on 16 bytes (any even column for 24-byte blocks, a
  // multiple of 8 for 34-byte blocks).
  h.c0 = 0;
  if (tu.tma) {
    int c0 = TN;
    if (c0 * BB > 2048) c0 = (int)(q * ((TN / 2 + q - 1) / q));
    if (c0 * BB <= 2048 && (TN - c0) * BB <= 2048) h.c0 = c0;
  }
  h.nB = d.B2 ? 2 : 1;
  (void)M;
}

}  // namespace

struct ListProgram {
  int kind = 0, M = 0, nitems = 0, ncta = 0, device = 0;
  size_t smem = 0;
  int threads = 0;
  ListParams p{};
  void* dev_block = nullptr;    // one allocation: items, maps, counters
  size_t dev_bytes = 0;
  uint64_t weight_bytes = 0;
  bool channels = false;
};

size_t list_device_bytes(const ListProgram* lp) { return lp ? lp->dev_bytes : 0; }
int list_grid(const ListProgram* lp) { return lp ? lp->ncta : 0; }

namespace {

template <int KIND, int MR, bool CHAN>
cudaError_t launch_list_as(const ListProgram* lp, cudaStream_t s) {
  static PerDeviceFlag configured;              // the attribute belongs to a device, not to the process
  bool* set = configured.here();
  if (!set) return cudaErrorInvalidDevice;
  cudaError_t e;
  if (!*set) {
    e = cudaFuncSetAttribute(qgemv_list_kernel<KIND, MR, CHAN>, cudaFuncAttributeMaxDynamicSharedMemorySize, kListSmem);
    if (e != cudaSuccess) return e;
    *set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)lp->ncta);
  cfg.blockDim = dim3((unsigned)lp->threads);
  cfg.dynamicSmemBytes = lp->smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;   // the CTAs wait on one another: all of them must be resident
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, qgemv_list_kernel<KIND, MR, CHAN>, lp->p);
  count_launch();
  return e;
}

}  // namespace

bool qgemv_list_supports(int kind, int64_t M, int64_t N, int64_t K) {
  if (kind != 4 && kind != 8) return false;
  if (M < 1 || M > 4) return false;
  if (N < 8 || (N % 8) != 0) return false;
  if (K < 32 || (K % 32) != 0 || K > (1 << 22) || N > (1 << 30)) return false;
  return (size_t)M * (K / 32) * 72 <= 96 * 1024;   // the activations' digit form must leave room for the ring
}

ListProgram* qgemv_list_create(int kind, int64_t M, const ListItemDesc* items, int count, int rank, unsigned flags,
                               const char** why) {
  if (why) *why = "";
  if (count < 1 || count > 65536) {
    list_fail(why, "a list holds 1 to 65536 items, got %d", count);
    return nullptr;
  }
  if (kind != 4 && kind != 8) {
    list_fail(why, "kind must be 4 or 8, got %d", kind);
    return nullptr;
  }
  int dev = 0, sms = 0, coop = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev) != cudaSuccess || sms < 1 || !coop) {
    cudaGetLastError();
    list_fail(why, "no device with cooperative launch");
    return nullptr;
  }
  const int BB = (kind == 4) ? kQ4Bytes : kQ8Bytes;
  const Tuning tu = tuning();
  for (int i = 0; i < count; i++) {
    const ListItemDesc& d = items[i];
    if (!qgemv_list_supports(kind, M, d.N, d.K)) {
      list_fail(why, "item %d: M=%lld N=%lld K=%lld is not a shape the list kernel takes (M <= 4, N %% 8 == 0, K %% 32 == 0)", i,
                (long long)M, (long long)d.N, (long long)d.K);
      return nullptr;
    }
    if (!d.A || !d.B || !d.C) {
      list_fail(why, "item %d: null operand", i);
      return nullptr;
    }
    if (((uintptr_t)d.A & 15) || ((uintptr_t)d.B & 15) || ((uintptr_t)d.B2 & 15) || ((uintptr_t)d.gamma & 15)) {
      list_fail(why, "item %d: activations, weights and norm weights must be 16-byte aligned", i);
      return nullptr;
    }
    if (overlap(d.A, (size_t)M * d.K * 4, d.C, (size_t)M * d.N * 4)) {
      list_fail(why, "item %d: output overlaps its own activations", i);
      return nullptr;
    }
    if (d.g_world) {
      if (d.g_world < 1 || d.g_world > 8 || rank < 0 || rank >= d.g_world || d.g_n0 < 0 || d.g_n0 + d.N > d.g_n_total ||
          2 * M * d.g_n_total > 0x7FFFFFFFll) {
        list_fail(why, "item %d: gather of columns [%lld, %lld) into a row of %lld over %d ranks (this is rank %d) is out of range", i,
                  (long long)d.g_n0, (long long)(d.g_n0 + d.N), (long long)d.g_n_total, d.g_world, rank);
        return nullptr;
      }
      for (int r = 0; r < d.g_world; r++)
        if (!d.g_rows[r] || ((uintptr_t)d.g_rows[r] & 7)) {
          list_fail(why, "item %d: row buffer of rank %d is null or not 8-byte aligned", i, r);
          return nullptr;
        }
    }
  }
  ListProgram* lp = new ListProgram();
  lp->kind = kind, lp->M = (int)M, lp->nitems = count, lp->ncta = sms, lp->device = dev;
  std::vector<ItemHot> hot(count);
  int slots = 0, slot_bytes = 0, nthreads = 0, ring_off = 0, xdig_off = 0, xsc_off = 0, rms_off = 0, red_off = 0, red_half = 0;
  // Three slots of the target stage size where they fit beside the activations' digit form;
  // smaller stages otherwise.
  for (int stage_bytes = tu.stage_bytes; stage_bytes >= 4096; stage_bytes = stage_bytes * 3 / 4) {
    int gmax = 0, red_max = 0;
    slot_bytes = 0, nthreads = 0;
    for (int i = 0; i < count; i++) {
      ItemHot& h = hot[i];
      memset(&h, 0, sizeof h);
      plan_item(kind, (int)M, items[i], sms, stage_bytes, tu, h);
      gmax = max(gmax, h.G);
      int bytes = h.stage_rows * h.row_pitch;
      if (h.c0 && h.c0 < h.TN)
        bytes = ((h.stage_rows * h.c0 * BB + 127) & ~127) + h.stage_rows * (h.TN - h.c0) * BB;
      slot_bytes = max(slot_bytes, ((bytes + 127) / 128) * 128);
      nthreads = max(nthreads, max(h.TN * h.phases, (int)M * h.TN));   // the epilogue gives every output its own thread
      red_max = max(red_max, h.phases * (int)M * h.TN * 4 * h.nB);
    }
    xdig_off = kListHeader;
    xsc_off = xdig_off + (int)M * gmax * 64;
    rms_off = xsc_off + (int)M * gmax * 8;
    red_off = rms_off + 4 * 32 * 4;
    red_half = (red_max + 15) & ~15;
    ring_off = ((red_off + 2 * red_half + 1023) / 1024) * 1024;
    slots = (kListSmem - 64 - ring_off) / slot_bytes;   // 64: the Q8 dot reads whole words around a block
    if (slots > kListMaxStages) slots = kListMaxStages;
    if (slots >= 3) break;
  }
  if (slots < 2 || nthreads > kListMaxThreads) {
    list_fail(why, "the list does not fit shared memory (%d ring slots of %d bytes, %d threads)", slots, slot_bytes, nthreads);
    delete lp;
    return nullptr;
  }
  // ---- operands, activation versions, rotation of the tiles over the grid
  int next_cta = 0, a_id = 0;
  for (int i = 0; i < count; i++) {
    const ListItemDesc& d = items[i];
    ItemHot& h = hot[i];
    h.A = d.A, h.B0 = d.B, h.B1 = d.B2, h.C = d.C, h.gamma = d.gamma, h.residual = d.residual, h.eps = d.eps;
    h.first_cta = next_cta;
    next_cta = (next_cta + h.tiles) % sms;
    bool same = i > 0 && items[i - 1].A == d.A && items[i - 1].K == d.K && items[i - 1].gamma == d.gamma &&
                items[i - 1].eps == d.eps &&
                !overlap(items[i - 1].C, (size_t)M * items[i - 1].N * 4, d.A, (size_t)M * d.K * 4);
    if (!same) a_id++;
    h.a_id = a_id;
    lp->weight_bytes += (uint64_t)h.G * d.N * BB * h.nB;
  }
  // ---- channels.  An item whose activations (or residual) are exactly the output of an earlier item
  // reads them from that item's channel: no counter, no fence, the tag of each pair says it is there.
  std::vector<int> a_src(count, -1), r_src(count, -1);
  std::vector<char> has_chan(count, 0);
  // Measured on one GPU (a chain of 4096 x 4096 items, an 8B-shaped decode step): 7.2 us per item and
  // 1.78 ms per step through channels against 6.8 us and 1.65 ms through the counters, because the
  // instantiation that carries the channel code is slower per tile.  So local hazards use the counters
  // unless SMITH_LIST_CHANNELS is set; gathered rows (several GPUs) always travel as tagged pairs.
  const bool use_chan = getenv("SMITH_LIST_CHANNELS") != nullptr;
  for (int i = 0; i < count && use_chan; i++) {
    const ListItemDesc& d = items[i];
    for (int j = i - 1; j >= 0; j--)
      if (overlap(items[j].C, (size_t)M * items[j].N * 4, d.A, (size_t)M * d.K * 4)) {
        if (items[j].C == d.A && items[j].N == d.K) a_src[i] = j, has_chan[j] = 1;
        break;                                       // the latest writer decides
      }
    for (int j = i - 1; j >= 0 && d.residual; j--)
      if (overlap(items[j].C, (size_t)M * items[j].N * 4, d.residual, (size_t)M * d.N * 4)) {
        if (items[j].C == d.residual && items[j].N == d.N && d.residual != d.C) r_src[i] = j, has_chan[j] = 1;
        break;
      }
  }
  // ---- hazards.  closure[i] = every item known to be complete once item i is.
  const int words = (count + 63) / 64;
  std::vector<uint64_t> closure((size_t)count * words, 0);
  auto bit = [&](int i, int j) -> bool { return (closure[(size_t)i * words + j / 64] >> (j % 64)) & 1; };
  for (int i = 0; i < count; i++) {
    const ListItemDesc& d = items[i];
    const size_t an = (size_t)M * d.K * 4, cn = (size_t)M * d.N * 4;
    ItemHot& h = hot[i];
    uint64_t* mine = &closure[(size_t)i * words];
    auto implies = [&](int j) {
      mine[j / 64] |= 1ull << (j % 64);
      const uint64_t* theirs = &closure[(size_t)j * words];
      for (int w = 0; w < words; w++) mine[w] |= theirs[w];
    };
    for (int j = i - 1; j >= 0; j--) {
      if (bit(i, j)) continue;                     // already implied by a dependency taken
      const ListItemDesc& e = items[j];
      const size_t ean = (size_t)M * e.K * 4, ecn = (size_t)M * e.N * 4;
      const bool raw_a = overlap(e.C, ecn, d.A, an) && j != a_src[i];
      const bool raw_r = overlap(e.C, ecn, d.residual, cn) && j != r_src[i];
      const bool war = overlap(d.C, cn, e.A, ean) || overlap(d.C, cn, e.residual, ecn);
      const bool waw = overlap(d.C, cn, e.C, ecn);
      if (!(raw_a || raw_r || war || waw)) {
        // every CTA that works on item i reads the WHOLE row of its activations' channel, so item j is
        // complete by then; a residual read through a channel sees single elements and implies nothing
        if (j == a_src[i]) implies(j);
        continue;
      }
      if (h.ndeps == kListMaxDeps) {
        list_fail(why, "item %d conflicts with more than %d earlier items that do not imply one another", i, kListMaxDeps);
        delete lp;
        return nullptr;
      }
      h.dep[h.ndeps++] = j;
      implies(j);
    }
  }
  // ---- device block: items | maps | done_init | done | ticket, epoch | channels
  const size_t items_bytes = (size_t)count * sizeof(ItemHot);
  const size_t maps_bytes = (size_t)count * 4 * sizeof(CUtensorMap);
  const size_t cnt_bytes = (size_t)count * kListCounterStride * 4;
  int ngather = 0;
  for (int i = 0; i < count; i++) ngather += items[i].g_world ? 1 : 0;
  const size_t rows_bytes = (size_t)ngather * 8 * sizeof(void*);          // per gathered item: its ranks' row buffers
  const size_t checks_bytes = (((size_t)ngather * sizeof(RowCheck) + 127) / 128) * 128;
  const size_t fixed_bytes = items_bytes + maps_bytes + 2 * cnt_bytes + 128 + rows_bytes + checks_bytes;
  std::vector<size_t> chan_at(count, 0);
  size_t chan_bytes = 0;
  for (int i = 0; i < count; i++)
    if (has_chan[i]) {
      chan_at[i] = fixed_bytes + chan_bytes;
      chan_bytes += (((size_t)M * items[i].N * 8 + 255) / 256) * 256;
    }
  lp->dev_bytes = fixed_bytes + chan_bytes;
  lp->channels = chan_bytes > 0 || ngather > 0;
  if (cudaMalloc(&lp->dev_block, lp->dev_bytes) != cudaSuccess) {
    cudaGetLastError();
    list_fail(why, "device allocation of %zu bytes for the list failed", lp->dev_bytes);
    lp->dev_block = nullptr;
    delete lp;
    return nullptr;
  }
  uint8_t* base = static_cast<uint8_t*>(lp->dev_block);
  for (int i = 0; i < count; i++) {
    ItemHot& h = hot[i];
    if (has_chan[i]) h.c_chan = reinterpret_cast<uint2*>(base + chan_at[i]);
    if (a_src[i] >= 0) h.a_chan = reinterpret_cast<const uint2*>(base + chan_at[a_src[i]]);
    if (r_src[i] >= 0) h.r_chan = reinterpret_cast<const uint2*>(base + chan_at[r_src[i]]);
  }
  std::vector<uint8_t> host(fixed_bytes, 0);
  {
    const size_t rows_at = items_bytes + maps_bytes + 2 * cnt_bytes + 128, checks_at = rows_at + rows_bytes;
    void** rows = reinterpret_cast<void**>(host.data() + rows_at);
    RowCheck* checks = reinterpret_cast<RowCheck*>(host.data() + checks_at);
    int g = 0;
    for (int i = 0; i < count; i++) {
      const ListItemDesc& d = items[i];
      if (!d.g_world) continue;
      ItemHot& h = hot[i];
      h.g_world = d.g_world, h.g_n0 = (int)d.g_n0, h.g_n_total = (int)d.g_n_total;
      h.g_rows = reinterpret_cast<uint2* const*>(base + rows_at + (size_t)g * 8 * sizeof(void*));
      for (int r = 0; r < d.g_world; r++) rows[g * 8 + r] = d.g_rows[r];
      checks[g].row = static_cast<const uint2*>(d.g_rows[rank]);
      checks[g].count = (int)(M * d.g_n_total);
      g++;
    }
    lp->p.checks = reinterpret_cast<const RowCheck*>(base + checks_at);
    lp->p.nchecks = (flags & kListNoClosingWait) ? 0 : ngather;
  }
  CUtensorMap* maps = reinterpret_cast<CUtensorMap*>(host.data() + items_bytes);
  unsigned* init = reinterpret_cast<unsigned*>(host.data() + items_bytes + maps_bytes);
  unsigned* done = reinterpret_cast<unsigned*>(host.data() + items_bytes + maps_bytes + cnt_bytes);
  reinterpret_cast<unsigned*>(host.data() + items_bytes + maps_bytes + 2 * cnt_bytes)[1] = 1u;   // the first launch's tag
  EncodeTiledFn enc = encode_fn();
  for (int i = 0; i < count; i++) {
    ItemHot& h = hot[i];
    if (h.c0) {
      // each packed matrix as [G][N * block bytes / 8] 64-bit words; box = one stage of one panel of a tile
      const cuuint64_t dims[2] = {(cuuint64_t)h.N * BB / 8, (cuuint64_t)h.G};
      const cuuint64_t strides[1] = {(cuuint64_t)h.N * BB};
      const cuuint32_t estr[2] = {1, 1};
      bool good = enc != nullptr;
      for (int b = 0; b < h.nB && good; b++)
        for (int pn = 0; pn < 2 && good; pn++) {
          const int cols = pn ? h.TN - h.c0 : h.c0;
          if (cols == 0) continue;
          const cuuint32_t box[2] = {(cuuint32_t)(cols * BB / 8), (cuuint32_t)h.stage_rows};
          good = enc(&maps[4 * i + 2 * b + pn], CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<uint8_t*>(b ? h.B1 : h.B0), dims,
                     strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
        }
      if (!good) {
        list_fail(why, "item %d: the driver refused the tensor map of a %d x %d tile", i, h.stage_rows, h.TN);
        qgemv_list_destroy(lp);
        return nullptr;
      }
    }
    init[(size_t)i * kListCounterStride] = done[(size_t)i * kListCounterStride] = (unsigned)h.tiles;
  }
  memcpy(host.data(), hot.data(), items_bytes);
  // channels start at zero: no pair carries a launch's tag (tags start at 1)
  if (cudaMemcpy(lp->dev_block, host.data(), fixed_bytes, cudaMemcpyHostToDevice) != cudaSuccess ||
      (chan_bytes && cudaMemset(base + fixed_bytes, 0, chan_bytes) != cudaSuccess)) {
    cudaGetLastError();
    list_fail(why, "upload of the list failed");
    qgemv_list_destroy(lp);
    return nullptr;
  }
  ListParams& p = lp->p;
  p.items = reinterpret_cast<const ItemHot*>(base);
  p.maps = reinterpret_cast<const CUtensorMap*>(base + items_bytes);
  p.done_init = reinterpret_cast<const unsigned*>(base + items_bytes + maps_bytes);
  p.done = reinterpret_cast<unsigned*>(base + items_bytes + maps_bytes + cnt_bytes);
  p.ticket = reinterpret_cast<unsigned*>(base + items_bytes + maps_bytes + 2 * cnt_bytes);
  p.epoch = p.ticket + 1;
#ifdef SMITH_LIST_TRACE
  p.trace = nullptr;
  if (getenv("SMITH_LIST_TRACE_OUT")) {
    cudaMalloc(&p.trace, (size_t)count * sms * 64);
    cudaMemset(p.trace, 0, (size_t)count * sms * 64);
  }
#endif
  p.nitems = count, p.M = (int)M;
  p.nwarps = (nthreads + 31) / 32;
  p.slots = slots, p.slot_bytes = slot_bytes;
  p.xdig_off = xdig_off, p.xsc_off = xsc_off, p.rms_off = rms_off, p.red_off = red_off, p.red_half = red_half;
  p.ring_off = ring_off;
  if (getenv("SMITH_LIST_VERBOSE")) {
    fprintf(stderr, "smith list: %d items, grid %d, %d consumer warps, %d slots x %d bytes, ring at %d, channels %zu bytes\n", count, sms,
            p.nwarps, slots, slot_bytes, ring_off, chan_bytes);
    for (int i = 0; i < count && i < 16; i++)
      fprintf(stderr, "  item %d: N=%d K=%d TN=%d tiles=%d phases=%d rpp=%d stage_rows=%d nst=%d c0=%d deps=%d a_chan=%d r_chan=%d c_chan=%d\n", i,
              hot[i].N, hot[i].K, hot[i].TN, hot[i].tiles, hot[i].phases, hot[i].rpp, hot[i].stage_rows, hot[i].nst, hot[i].c0,
              hot[i].ndeps, hot[i].a_chan != nullptr, hot[i].r_chan != nullptr, hot[i].c_chan != nullptr);
  }
  lp->threads = p.nwarps * 32 + 64;              // consumers, producer warp, signalling warp
  lp->smem = (size_t)ring_off + (size_t)slots * slot_bytes + 64;
  return lp;
}

cudaError_t qgemv_list_launch(const ListProgram* lp, cudaStream_t s) {
  if (!lp) return cudaErrorInvalidValue;
  ListProgram* m = const_cast<ListProgram*>(lp);
  m->p.status = kernel_status_ptr();
  if (!m->p.status) return cudaErrorUnknown;
#define SMITH_LIST_CASE(KD, MRV) \
  if (lp->kind == KD && lp->M == MRV) return lp->channels ? launch_list_as<KD, MRV, true>(lp, s) : launch_list_as<KD, MRV, false>(lp, s);
  SMITH_LIST_CASE(4, 1) SMITH_LIST_CASE(4, 2) SMITH_LIST_CASE(4, 3) SMITH_LIST_CASE(4, 4)
  SMITH_LIST_CASE(8, 1) SMITH_LIST_CASE(8, 2) SMITH_LIST_CASE(8, 3) SMITH_LIST_CASE(8, 4)
#undef SMITH_LIST_CASE
  return cudaErrorInvalidValue;
}

void qgemv_list_destroy(ListProgram* lp) {
  if (!lp) return;
#ifdef SMITH_LIST_TRACE
  if (lp->p.trace) {   // measurement builds: dump the stamps of the last launch
    std::vector<unsigned long long> h((size_t)lp->nitems * lp->ncta * 8);
    cudaDeviceSynchronize();
    cudaMemcpy(h.data(), lp->p.trace, h.size() * 8, cudaMemcpyDeviceToHost);
    if (FILE* f = fopen(getenv("SMITH_LIST_TRACE_OUT"), "wb")) {
      int hdr[2] = {lp->nitems, lp->ncta};
      fwrite(hdr, 4, 2, f);
      fwrite(h.data(), 8, h.size(), f);
      fclose(f);
    }
    cudaFree(lp->p.trace);
  }
#endif
  if (lp->dev_block) cudaFree(lp->dev_block);
  delete lp;
}

uint64_t qgemv_list_weight_bytes(const ListProgram* lp) { return lp ? lp->weight_bytes : 0; }

unsigned qgemv_list_next_tag(const ListProgram* lp) {
  unsigned t = 0;
  if (!lp || cudaDeviceSynchronize() != cudaSuccess || cudaMemcpy(&t, lp->p.epoch, 4, cudaMemcpyDeviceToHost) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return t;
}

}  // namespace smith
