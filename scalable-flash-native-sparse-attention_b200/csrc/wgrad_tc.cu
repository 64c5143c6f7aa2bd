// Weight gradient of the learned K/V compression, accumulated straight into the trainer's fp32 buffer:
//     main_grad[out, in] += dY[rows, out]^T  X[rows, in]          (dY, X bf16; main_grad fp32)
// One tcgen05 GEMM with the accumulate fused in: no fp32 [out, in] temporary and no second pass that adds it.
//
// Both operands are read "MN-major": the contraction index is the ROW of dY and of X, so a TMA box of (64 rows) x (64
// columns) lands in shared memory as the operand tile of tc_common.cuh without any transposition (A = dY^T, B = X).
// CTA = one 128 x 128 tile of main_grad and one slice of the rows (split-K: the result is added with fp32 atomics anyway, so
// slices simply add their partial tiles).  Warp 0 (one lane) feeds a 4-stage ring with TMA, warp 1 (one lane) issues the
// MMAs into a 128-column tensor-memory accumulator, warps 2-5 read it out (thread = row of main_grad) and add 16-byte
// vectors.  Rows past the end of the tensors are zero-filled by TMA and contribute nothing.
#include "tma.cuh"

namespace nsa {

constexpr int WG_STAGES = 4, WG_BK = 64;

__global__ void __launch_bounds__(192, 1)
    wgrad_tc_kernel(float* __restrict__ out, int64_t out_stride, int n_out, int n_in, int rows, int rows_per_cta, int32_t* status,
                    const __grid_constant__ CUtensorMap tma_dy, const __grid_constant__ CUtensorMap tma_x) {
  using namespace tc;
  constexpr uint32_t SLAB = WG_BK * 128, TILE = 2 * SLAB;   // [64 rows x 64 cols] slabs, two per 128-wide operand tile
  constexpr uint32_t IDESC = make_idesc(128, 128, true, true);
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  const uint32_t sA = base, sB = base + WG_STAGES * TILE;
  const uint32_t bars = sB + WG_STAGES * TILE;
  const uint32_t full = bars, empty = bars + 8 * WG_STAGES, done = empty + 8 * WG_STAGES, tm_slot = done + 8;

  const int tid = threadIdx.x, warp = tid >> 5;
  const int m0 = blockIdx.y * 128, n0 = blockIdx.x * 128;
  const int r0 = blockIdx.z * rows_per_cta, r1 = min(rows, r0 + rows_per_cta);
  if (r0 >= r1) return;
  if (base & 1023u) {
    if (tid == 0 && status) atomicOr(status, 8);
    return;
  }
  const int n_k = (r1 - r0 + WG_BK - 1) / WG_BK;

  if (tid == 0) {
    for (int s = 0; s < WG_STAGES; ++s) {
      mbar_init(full + 8 * s, 1);
      mbar_init(empty + 8 * s, 1);
    }
    mbar_init(done, 1);
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc(tm_slot, 128);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  uint32_t tmem;
  asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(tmem) : "r"(tm_slot));
  int budget = kWaitBudget;
  bool timed_out = false;

  if (warp == 0) {
    if ((tid & 31) == 0) {
      for (int i = 0; i < n_k; ++i) {
        const int s = i % WG_STAGES;
        if (i >= WG_STAGES && !mbar_wait(empty + 8 * s, ((i / WG_STAGES) - 1) & 1, &budget)) timed_out = true;
        tma::expect_tx(full + 8 * s, 2 * TILE);
        const int row = r0 + i * WG_BK;   // slices are whole k-steps; only the last one can reach past `rows` (zero-filled)
#pragma unroll
        for (int sl = 0; sl < 2; ++sl) {
          tma::load_3d(sA + s * TILE + sl * SLAB, &tma_dy, 0, m0 / 64 + sl, row, full + 8 * s);
          tma::load_3d(sB + s * TILE + sl * SLAB, &tma_x, 0, n0 / 64 + sl, row, full + 8 * s);
        }
      }
    }
  } else if (warp == 1) {
    if ((tid & 31) == 0) {
      for (int i = 0; i < n_k; ++i) {
        const int s = i % WG_STAGES;
        if (!mbar_wait(full + 8 * s, (i / WG_STAGES) & 1, &budget)) timed_out = true;
        fence_after_sync();
#pragma unroll
        for (int u = 0; u < WG_BK / 16; ++u)
          mma_ss(tmem, desc_mnmajor(sA + s * TILE + u * 2048, SLAB), desc_mnmajor(sB + s * TILE + u * 2048, SLAB), IDESC, (i > 0 || u > 0));
        mma_commit(empty + 8 * s);   // the stage may be refilled once these products have read it
      }
      mma_commit(done);
    }
  } else {
    if (!mbar_wait(done, 0, &budget)) timed_out = true;
    fence_after_sync();
    const uint32_t src = tmem + ((uint32_t)((warp & 3) * 32) << 16);   // a warp may only read the 32 lanes of its quarter
    const int lane_row = (warp & 3) * 32 + (tid & 31);
    float* dst = out + (int64_t)(m0 + lane_row) * out_stride + n0;
    const bool row_ok = m0 + lane_row < n_out;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t v[32];
      tmem_ld32(src + c * 32, v);
      wait_ld();
      if (row_ok) {
#pragma unroll
        for (int q4 = 0; q4 < 8; ++q4) {
          const int col = n0 + c * 32 + q4 * 4;
          if (col + 3 < n_in)
            atomicAdd(reinterpret_cast<float4*>(dst + c * 32 + q4 * 4),
                      make_float4(__uint_as_float(v[q4 * 4]), __uint_as_float(v[q4 * 4 + 1]), __uint_as_float(v[q4 * 4 + 2]),
                                  __uint_as_float(v[q4 * 4 + 3])));
        }
      }
    }
  }
  if (timed_out && status) atomicOr(status, 1024);
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 128);
}

}  // namespace nsa

using namespace nsa;

extern "C" int nsa_wgrad_accum(const NsaWgradParams* p, void* stream) {
  NSA_REQUIRE(p && p->dy && p->x && p->main_grad, NSA_ERR_BAD_ARG, "wgrad_accum: null pointer");
  NSA_REQUIRE(p->rows >= 0 && p->n_out > 0 && p->n_in > 0, NSA_ERR_BAD_ARG, "wgrad_accum: bad sizes");
  NSA_REQUIRE(p->n_out % 128 == 0 && p->n_in % 128 == 0, NSA_ERR_UNSUPPORTED_SHAPE,
              "wgrad_accum: n_out=%d and n_in=%d must be multiples of 128", p->n_out, p->n_in);
  NSA_REQUIRE((((uintptr_t)p->dy | (uintptr_t)p->x | (uintptr_t)p->main_grad) & 15) == 0 && (p->dy_stride * 2) % 16 == 0 &&
                  (p->x_stride * 2) % 16 == 0 && p->grad_stride % 4 == 0,
              NSA_ERR_BAD_ARG, "wgrad_accum: tensors must be 16-byte aligned with 16-byte-multiple row strides");
  if (p->rows == 0) return NSA_OK;
  // a [rows, cols] bf16 matrix seen as [rows, cols / 64 "heads", 64]: one box = 64 rows x 1 head x 64 columns
  CUtensorMap tdy, tx;
  if (!tma::make_map(&tdy, p->dy, p->rows, p->n_out / 64, 64, p->dy_stride, WG_BK, 1) ||
      !tma::make_map(&tx, p->x, p->rows, p->n_in / 64, 64, p->x_stride, WG_BK, 1)) {
    set_error("wgrad_accum: cuTensorMapEncodeTiled failed or is unavailable");
    return NSA_ERR_CUDA;
  }
  const int tiles = (p->n_out / 128) * (p->n_in / 128);
  int splits = max(1, min((2 * 148 + tiles - 1) / tiles, (int)((p->rows + 4 * WG_BK - 1) / (4 * WG_BK))));
  int rows_per_cta = (int)(((p->rows + splits - 1) / splits + WG_BK - 1) / WG_BK * WG_BK);   // slices are whole k-steps
  splits = (int)((p->rows + rows_per_cta - 1) / rows_per_cta);
  const size_t smem = (size_t)2 * WG_STAGES * 2 * WG_BK * 128 + 16 * WG_STAGES + 64;
  cudaError_t e = cudaFuncSetAttribute(wgrad_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_error("wgrad_accum: cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
    return NSA_ERR_CUDA;
  }
  dim3 grid(p->n_in / 128, p->n_out / 128, splits);
  wgrad_tc_kernel<<<grid, 192, smem, (cudaStream_t)stream>>>(p->main_grad, p->grad_stride, p->n_out, p->n_in, (int)p->rows, rows_per_cta,
                                                             p->status, tdy, tx);
  return check_launch("wgrad_accum");
}
