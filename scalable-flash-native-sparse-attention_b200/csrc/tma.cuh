// TMA (bulk tensor copy) helpers: tensor-map creation on the host through the driver entry point, and the device-side
// load + transaction-count barrier instructions.  Only plain per-CTA loads and reductions are used (no cluster multicast).
#pragma once
#include <cuda.h>
#include "tc_common.cuh"

namespace nsa {
namespace tma {

__device__ __forceinline__ void load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
      : "memory");
}
// fetch the descriptor itself ahead of its first use
__device__ __forceinline__ void prefetch_map(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
// ask for a box to be brought into L2 (no shared-memory destination, no completion to wait for)
__device__ __forceinline__ void prefetch_3d(const CUtensorMap* map, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];\n" ::"l"(reinterpret_cast<uint64_t>(map)), "r"(c0),
               "r"(c1), "r"(c2)
               : "memory");
}
// add a box of shared memory into the tensor (element-wise, in the tensor's type); completion is tracked by the
// thread's bulk async-group.  Coordinates must not be negative, and c0 * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void reduce_add_3d(const CUtensorMap* map, int c0, int c1, int c2, uint32_t src) {
  asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2, %3}], [%4];\n" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(c0), "r"(c1), "r"(c2), "r"(src)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory"); }   // sources read
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory"); }         // writes done
__device__ __forceinline__ void expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}\n" ::"r"(bar), "r"(bytes) : "memory");
}

// Map of a [rows, heads, D] bf16 tensor (row stride given in elements) with a box of box_rows x box_heads x 64 elements and
// the 128-byte swizzle: the box lands in shared memory as (box_rows*box_heads) rows of 128 bytes, row-major over
// (row, head), in the operand layout of tc_common.cuh.  Out-of-range rows read as zero.  Returns false on failure.
bool make_map(CUtensorMap* m, const void* base, int64_t rows, int heads, int D, int64_t row_stride_elems, int box_rows, int box_heads);

}  // namespace tma
}  // namespace nsa
