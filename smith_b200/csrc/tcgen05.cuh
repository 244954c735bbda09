// tcgen05.cuh -- PTX wrappers for the 5th-generation tensor cores: tensor-map loads, tensor memory,
// tcgen05.mma on 16-bit K-major operands with 128-byte swizzle, commit, accumulator loads.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace smith {

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void bulk_load_plain(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// D[tmem] (+)= A[smem] x B[smem], 128 x N x 16 per tcgen05.mma, 16-bit inputs, f32 accumulate.
// The four MMAs of one 64-wide k-block in one go: k-step j reads both operands 32 bytes (two
// descriptor address units) further along the swizzled 128-byte rows.  The descriptors' high
// words are equal (same stride, version and layout) and only the first step may overwrite D.
__device__ __forceinline__ void umma_f16_kblock(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi,
                                                uint32_t idesc, uint32_t accumulate_first) {
  asm volatile(
      "{\n"
      ".reg .pred p, q;\n"
      ".reg .b32 ta, tb;\n"
      ".reg .b64 da, db;\n"
      "setp.ne.b32 p, %5, 0;\n"
      "setp.ne.b32 q, %4, 0;\n"          // the instruction descriptor is never zero: q = true
      "mov.b64 da, {%1, %3};\n"
      "mov.b64 db, {%2, %3};\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n"
      "add.u32 ta, %1, 2;\n"
      "add.u32 tb, %2, 2;\n"
      "mov.b64 da, {ta, %3};\n"
      "mov.b64 db, {tb, %3};\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, q;\n"
      "add.u32 ta, %1, 4;\n"
      "add.u32 tb, %2, 4;\n"
      "mov.b64 da, {ta, %3};\n"
      "mov.b64 db, {tb, %3};\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, q;\n"
      "add.u32 ta, %1, 6;\n"
      "add.u32 tb, %2, 6;\n"
      "mov.b64 da, {ta, %3};\n"
      "mov.b64 db, {tb, %3};\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, q;\n"
      "}\n" ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate_first)
      : "memory");
}
// mbarrier arrive once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of
// 128 bytes, groups of 8 rows 1024 bytes apart.  Fields (bit positions):
//   [0,14)  start address >> 4        [16,30) leading byte offset >> 4 (unused here)
//   [32,46) stride byte offset >> 4   [46,48) descriptor version = 1
//   [49,52) base offset = 0 (tiles are 1024-byte aligned)   [61,64) layout: 2 = 128-byte swizzle
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(1024u >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// ---------------------------------------------------------------- CTA pairs (cta_group::2)
// Two CTAs of a cluster (ranks 2i and 2i+1) act as one MMA unit: D has 256 rows, rows 0-127 in the
// even ("leader") CTA's tensor memory and rows 128-255 in the odd one's; each CTA stages its own 128
// rows of A and its own half of the N columns of B, at the same shared-memory offsets in both; one
// thread of the leader issues the MMAs and the commits.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_u32(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ uint32_t ld_cluster_u32(uint32_t caddr) {
  uint32_t v;
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(caddr) : "memory");
  return v;
}
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t cbar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.release.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(cbar), "r"(bytes) : "memory");
}
// tensor-map load into this CTA's shared memory whose bytes are counted on a barrier that may live in the peer CTA
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t cbar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.cta_group::2 [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(cbar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// The four MMAs (256 x N x 16 each) of one 64-wide k-block, as umma_f16_kblock.
__device__ __forceinline__ void umma_f16_kblock_pair(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi,
                                                     uint32_t idesc, uint32_t accumulate_first) {
  asm volatile(
      "{\n"
      ".reg .pred p, q;\n"
      ".reg .b32 ta, tb;\n"
      ".reg .b64 da, db;\n"
      "setp.ne.b32 p, %5, 0;\n"
      "setp.ne.b32 q, %4, 0;\n"
      "mov.b64 da, {%1, %3};\n"
      "mov.b64 db, {%2, %3};\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, p;\n"
      "add.u32 ta, %1, 2;\n"
      "add.u32 tb, %2, 2;\n"
      "mov.b64 da, {ta, %3};\n"
      "mov.b64 db, {tb, %3};\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, q;\n"
      "add.u32 ta, %1, 4;\n"
      "add.u32 tb, %2, 4;\n"
      "mov.b64 da, {ta, %3};\n"
      "mov.b64 db, {tb, %3};\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, q;\n"
      "add.u32 ta, %1, 6;\n"
      "add.u32 tb, %2, 6;\n"
      "mov.b64 da, {ta, %3};\n"
      "mov.b64 db, {tb, %3};\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, q;\n"
      "}\n" ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate_first)
      : "memory");
}
// mbarrier arrive (on a barrier of this or of the peer CTA, by its shared::cluster address) once every
// MMA issued so far by this thread has completed
__device__ __forceinline__ void umma_commit_pair(uint32_t cbar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cbar) : "memory");
}

}  // namespace smith
