// Shared device helpers for the NSA sm_100a kernels: error plumbing, piece (varlen / context-parallel)
// metadata lookup, bf16 packing, cp.async, ldmatrix, and the warp-level m16n8k16 bf16 MMA.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include "../../include/nsa_sm100.h"

// NSA_F16: the second build of the library (libnsa_sm100_f16.so), the same kernels with IEEE half as the 16-bit element
// type.  Every kernel touches its 16-bit data through the helpers below, the two scalar conversions and the element type
// named here; the MMA operand formats and the tensor-map element type follow the same switch (tc_common.cuh, abi.cu).
#ifdef NSA_F16
#define __nv_bfloat16 __half
#define __float2bfloat16 __float2half_rn
#define __bfloat162float __half2float
#define NSA_MMA_ELEM "f16"
#else
#define NSA_MMA_ELEM "bf16"
#endif

namespace nsa {

// ------------------------------------------------------------------ host-side error plumbing
void set_error(const char* fmt, ...);
int check_launch(const char* what);

#define NSA_REQUIRE(cond, code, ...)            \
  do {                                          \
    if (!(cond)) {                              \
      ::nsa::set_error(__VA_ARGS__);            \
      return (code);                            \
    }                                           \
  } while (0)

// launch description of the 64-row-tile dK/dV kernel of the dense branches (dkdv_tc.cu)
struct DkdvLaunch {
  int q_chunk;   // compressed branch: query tokens per CTA slice
};

// ------------------------------------------------------------------ piece lookup
// A "piece" is a run of local query rows that belongs to one sequence.  Without context parallelism
// a piece is a whole sequence (offset 0); with it, a piece is the part of a sequence that lies in one
// of the rank's chunks, and `off` is the position of its first token inside the sequence.
struct Piece {
  int q_start;   // first local row (q / o / lse / dq side)
  int len;       // number of local rows
  int off;       // position of row 0 within its sequence
  int seq;       // sequence id
  int x_bos;     // first row of the sequence in the K/V-side tensors
  int x_len;     // sequence length
  int y_bos;     // first compressed row of the sequence
  int y_len;     // compressed rows of the sequence
  const int32_t* x_tab;  // paged mode: this sequence's page list for token rows (else null)
  const int32_t* y_tab;  // paged mode: this sequence's page list for compressed rows (else null)
  int page_shift;        // log2(page size); page sizes are powers of two
};

// flat row index (in the K/V-side tensor) of token row r / compressed row j of the piece's sequence
__device__ __forceinline__ int64_t tok_row(const Piece& p, int r) {
  if (!p.x_tab) return (int64_t)p.x_bos + r;
  return ((int64_t)p.x_tab[r >> p.page_shift] << p.page_shift) + (r & ((1 << p.page_shift) - 1));
}
__device__ __forceinline__ int64_t cmp_row(const Piece& p, int j) {
  if (!p.y_tab) return (int64_t)p.y_bos + j;
  return ((int64_t)p.y_tab[j >> p.page_shift] << p.page_shift) + (j & ((1 << p.page_shift) - 1));
}

__device__ __forceinline__ Piece load_piece(const NsaSeqMeta& m, int b) {
  Piece p;
  p.q_start = m.piece_cu[b];
  p.len = m.piece_cu[b + 1] - p.q_start;
  p.seq = m.piece_seq ? m.piece_seq[b] : b;
  p.off = m.piece_off ? m.piece_off[b] : 0;
  p.x_bos = m.x_cu[p.seq];
  p.x_len = m.x_cu[p.seq + 1] - p.x_bos;
  if (m.y_cu) {
    p.y_bos = m.y_cu[p.seq];
    p.y_len = m.y_cu[p.seq + 1] - p.y_bos;
  } else {
    p.y_bos = 0;
    p.y_len = 0;
  }
  p.page_shift = 31 - __clz(max(m.page_size, 1));
  p.x_tab = m.kv_table ? m.kv_table + (int64_t)p.seq * m.kv_table_stride : nullptr;
  p.y_tab = m.cmp_table ? m.cmp_table + (int64_t)p.seq * m.cmp_table_stride : nullptr;
  return p;
}

// ------------------------------------------------------------------ small math / packing
// two floats -> one word of two 16-bit elements (low half first), and back ("bf16" in the names: the element type of the build)
#ifdef NSA_F16
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __low2float(*reinterpret_cast<const __half2*>(&v)); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __high2float(*reinterpret_cast<const __half2*>(&v)); }
#else
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
#endif

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ------------------------------------------------------------------ async copies (16 B)
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
// copies 16 bytes, or writes 16 zero bytes when !valid (src must still be a mapped address)
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

// ------------------------------------------------------------------ swizzled bf16 tiles in shared memory
// A tile is [rows][D] bf16, each row D*2 bytes = D/8 chunks of 16 B; chunk c of row r is stored at
// chunk (c ^ (r & 7)), which makes every ldmatrix phase (8 rows, same chunk) hit 8 different banks.
template <int D>
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
  return static_cast<uint32_t>(row * (D * 2) + ((chunk ^ (row & 7)) << 4));
}

__device__ __forceinline__ void ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}

// A fragment (16 rows x 16 k) of a row-major tile: rows row0.., k-step ks (16 elements = 2 chunks)
template <int D>
__device__ __forceinline__ void load_a_frag(uint32_t (&a)[4], uint32_t tile, int row0, int ks, int lane) {
  int r = row0 + (lane & 7) + ((lane >> 3) & 1) * 8;
  int c = ks * 2 + (lane >> 4);
  ldsm_x4(a[0], a[1], a[2], a[3], tile + tile_off<D>(r, c));
}
// B fragments of an operand stored [n][k] row-major (e.g. K for Q.K^T): two n-tiles (n0..n0+15), k-step ks.
// b[0],b[1] = n-tile 0; b[2],b[3] = n-tile 1.
template <int D>
__device__ __forceinline__ void load_b_frag_nk(uint32_t (&b)[4], uint32_t tile, int n0, int ks, int lane) {
  int r = n0 + (lane & 7) + (lane >> 4) * 8;
  int c = ks * 2 + ((lane >> 3) & 1);
  ldsm_x4(b[0], b[1], b[2], b[3], tile + tile_off<D>(r, c));
}
// B fragments of an operand stored [k][n] row-major (e.g. V for P.V): k rows k0..k0+15, two n-tiles at
// columns n0..n0+15.  b[0],b[1] = n-tile 0; b[2],b[3] = n-tile 1.
template <int D>
__device__ __forceinline__ void load_b_frag_kn(uint32_t (&b)[4], uint32_t tile, int k0, int n0, int lane) {
  int r = k0 + (lane & 7) + ((lane >> 3) & 1) * 8;
  int c = (n0 >> 3) + (lane >> 4);
  ldsm_x4_t(b[0], b[1], b[2], b[3], tile + tile_off<D>(r, c));
}

// D(16x8, fp32) += A(16x16, bf16) * B(16x8, bf16)
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32." NSA_MMA_ELEM "." NSA_MMA_ELEM ".f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32." NSA_MMA_ELEM "." NSA_MMA_ELEM ".f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// copy `rows` rows of D bf16 (global row i at base + i*stride elements) into a swizzled tile; rows for which
// i >= valid_rows are zero-filled.  All `nthreads` threads of the CTA take part.
template <int D>
__device__ __forceinline__ void load_tile_async(uint32_t tile, const __nv_bfloat16* base, int64_t stride, int rows,
                                                int valid_rows, int tid, int nthreads) {
  constexpr int CH = D / 8;
  for (int i = tid; i < rows * CH; i += nthreads) {
    int r = i / CH, c = i % CH;
    bool ok = r < valid_rows;
    const __nv_bfloat16* src = base + (ok ? (int64_t)r * stride : 0) + c * 8;
    cp_async16(tile + tile_off<D>(r, c), src, ok);
  }
}

__device__ __forceinline__ float warp_max4(float v) {  // reduce over the 4 lanes that share a fragment row
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
  return v;
}
__device__ __forceinline__ float warp_sum4(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  return v;
}

}  // namespace nsa
