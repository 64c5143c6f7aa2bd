// Blackwell tensor-core plumbing shared by the tcgen05 kernels: shared-memory matrix descriptors for the
// 128-byte-swizzled operand layout, the instruction descriptor, tensor-memory allocation / load / store,
// mbarriers with BOUNDED waits, and the cp.async fill of operand tiles in that layout.
//
// Operand tiles in shared memory: a [rows x D] bf16 tile is stored as D/64 "slabs" of [rows x 64] (128 B per row);
// inside a slab, 8 consecutive rows form a 1024-byte swizzle atom and the 16-byte chunk c of row r sits at chunk
// (c ^ (r & 7)).  Read with a K-major descriptor this is an operand whose contraction index runs along the row
// (Q, K for Q.K^T); read with an MN-major descriptor it is an operand whose contraction index is the ROW number
// (V for P.V, K for dS.K): the same bytes serve both uses.
#pragma once
#include "nsa_common.cuh"

namespace nsa {
namespace tc {

// ------------------------------------------------------------------ tile addressing
__device__ __forceinline__ uint32_t slab_off(int rows, int r, int c16) {  // c16: 16-byte chunk index along the row, 0..D/8-1
  return static_cast<uint32_t>((c16 >> 3) * rows * 128 + r * 128 + (((c16 & 7) ^ (r & 7)) << 4));
}

// ------------------------------------------------------------------ descriptors
// K-major, 128B swizzle: rows 128 B apart, 8-row groups SBO = 1024 B apart.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3fff);
  d |= (uint64_t)1 << 16;                  // leading byte offset: unused for swizzled K-major
  d |= (uint64_t)(1024 >> 4) << 32;        // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                  // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                  // 128-byte swizzle
  return d;
}
// MN-major, 128B swizzle: 64 contiguous MN elements per row, next 64 MN elements LBO bytes away (= one slab),
// 8-row (K) groups SBO = 1024 B apart.
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t saddr, uint32_t slab_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3fff);
  d |= (uint64_t)((slab_bytes >> 4) & 0x3fff) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// 16-bit x 16-bit -> fp32, M x N tile; each operand K-major (contraction index contiguous) or MN-major.  Operand format
// fields (bits 7-9 for A, 10-12 for B): 1 = bf16, 0 = IEEE half (the NSA_F16 build).
#ifdef NSA_F16
constexpr uint32_t kOperandFormat = 0u;
#else
constexpr uint32_t kOperandFormat = 1u;
#endif
__host__ __device__ constexpr uint32_t make_idesc(int M, int N, bool b_mn_major, bool a_mn_major = false) {
  return (1u << 4) | (kOperandFormat << 7) | (kOperandFormat << 10) | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
         ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// ------------------------------------------------------------------ MMA issue (one thread)
__device__ __forceinline__ void mma_ss(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}\n" ::"r"(tmem_d),
      "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// arrive on an mbarrier when every MMA issued so far by this thread has completed
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}

// ------------------------------------------------------------------ tensor memory
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(dst_smem), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
// make shared-memory writes done through the generic proxy (cp.async, st.shared) visible to the tensor core
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
// the same for global memory: plain stores of this thread become visible to bulk tensor loads issued after a barrier
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;\n" ::: "memory"); }

// each thread of a warp reads 32 consecutive fp32 columns of ITS lane (lane = 32*(warp%4) + laneid)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n" ::
          "r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
      "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
      "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
      "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n" ::"r"(taddr),
               "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
               "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
               : "memory");
}

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }
// Bounded wait.  Returns false when the phase did not complete within the poll budget; the caller records that in the
// status word and carries on (results are then garbage, but every thread still reaches the end of the kernel and the
// tensor memory is released).  After the first failure *budget is cut to a few polls so the kernel drains quickly.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* budget) {
  {   // a phase that is already complete (the common case for the MMA and TMA lanes) is seen by the non-blocking test in
      // ~14 cycles; the first try_wait of the loop below takes ~70 even then
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  for (int i = 0; i < *budget; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  *budget = 8;
  return false;
}
constexpr int kWaitBudget = 1 << 18;  // polls (a few milliseconds); a healthy wait takes a few hundred
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}\n" ::"r"(bar) : "memory");
}
// barrier among the `count` threads that use id `id` (warp-group scoped synchronisation)
__device__ __forceinline__ void named_barrier(int id, int count) {
  asm volatile("bar.sync %0, %1;\n" ::"r"(id), "r"(count) : "memory");
}

// ------------------------------------------------------------------ operand tile fill (all threads of the CTA)
// rows x D bf16 from global rows (row i at base + i*stride elements) into slab layout; rows >= valid zero-filled
template <int D>
__device__ __forceinline__ void fill_tile_async(uint32_t tile, const __nv_bfloat16* base, int64_t stride, int rows, int valid,
                                                int tid, int nthreads) {
  constexpr int CH = D / 8;
  for (int i = tid; i < rows * CH; i += nthreads) {
    int r = i / CH, c = i % CH;
    bool ok = r < valid;
    cp_async16(tile + slab_off(rows, r, c), base + (ok ? (int64_t)r * stride : 0) + c * 8, ok);
  }
}

// same, for rows of a sequence's K/V (or compressed K/V) that may live in a paged cache: logical rows row0.. of the piece
template <int D, bool CMP>
__device__ __forceinline__ void fill_kv_tile_async(uint32_t tile, const __nv_bfloat16* base, int64_t stride, const Piece& pc, int row0,
                                                   int rows, int valid, int tid, int nthreads) {
  constexpr int CH = D / 8;
  if ((CMP ? pc.y_tab : pc.x_tab) == nullptr) {  // contiguous rows: plain strided fill
    fill_tile_async<D>(tile, base + ((int64_t)(CMP ? pc.y_bos : pc.x_bos) + row0) * stride, stride, rows, valid, tid, nthreads);
    return;
  }
  for (int i = tid; i < rows * CH; i += nthreads) {
    int r = i / CH, c = i % CH;
    bool ok = r < valid;
    int64_t phys = ok ? (CMP ? cmp_row(pc, row0 + r) : tok_row(pc, row0 + r)) : 0;
    cp_async16(tile + slab_off(rows, r, c), base + phys * stride + c * 8, ok);
  }
}

}  // namespace tc
}  // namespace nsa
