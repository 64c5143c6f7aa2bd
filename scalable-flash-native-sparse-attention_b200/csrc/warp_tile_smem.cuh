// Warp-level attention over one 64-key tile staged in shared memory: the 16 MMA rows are the query heads of one kv
// head for ONE token.  The warp copies the tile's 64 rows (any row addresses: pages, clamped rows) into its private
// buffer with 16-byte cp.async copies that are ALL in flight at once, and takes the MMA fragments with ldmatrix.
// Operand-direct global loads (as in slc_fwd.cu) are consumed n-tile by n-tile and leave a warp with a few hundred bytes in
// flight, so a tile costs a dozen dependent memory round trips; here it costs one (K) plus one that overlaps the
// softmax (V, into the same buffer once the scores are done).
#pragma once
#include "tc_common.cuh"

namespace nsa {
namespace wts {

constexpr int kTileRows = 64;

template <int D>
struct Acc {  // running softmax state of 16 rows x D columns in MMA accumulator layout: o[nt] = columns 8nt + 2c_, +1
  float o[D / 8][4];
  float m_lo, m_hi, l_lo, l_hi;
  __device__ __forceinline__ void init() {
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    m_lo = m_hi = -INFINITY;
    l_lo = l_hi = 0.f;
  }
};

// A fragments of the token's [G heads x D] query rows (rows >= G clamped to the last head)
template <int D>
__device__ __forceinline__ void load_q(uint32_t (&a)[D / 16][4], const __nv_bfloat16* base, int G, int lane) {
  const int g_ = lane >> 2, c_ = lane & 3;
  const __nv_bfloat16* r0 = base + min(g_, G - 1) * D + 2 * c_;
  const __nv_bfloat16* r1 = base + min(g_ + 8, G - 1) * D + 2 * c_;
#pragma unroll
  for (int k = 0; k < D / 16; ++k) {
    a[k][0] = *reinterpret_cast<const uint32_t*>(r0 + 16 * k);
    a[k][1] = *reinterpret_cast<const uint32_t*>(r1 + 16 * k);
    a[k][2] = *reinterpret_cast<const uint32_t*>(r0 + 16 * k + 8);
    a[k][3] = *reinterpret_cast<const uint32_t*>(r1 + 16 * k + 8);
  }
}

// start copying 64 rows of D bf16 into the warp's buffer (slab layout of tc_common.cuh); row(i) = flat tensor row
template <int D, class RowFn>
__device__ __forceinline__ void fill_async(uint32_t buf, const __nv_bfloat16* base, int64_t stride, RowFn row, int lane) {
  constexpr int CH = D / 8;
#pragma unroll 4
  for (int i = 0; i < kTileRows * CH / 32; ++i) {
    const int idx = i * 32 + lane, r = idx / CH, c = idx - r * CH;
    cp_async16(buf + tc::slab_off(kTileRows, r, c), base + row(r) * stride + c * 8, true);
  }
  cp_async_commit();
}
__device__ __forceinline__ void fill_wait() {
  cp_async_wait<0>();
  __syncwarp();
}

__device__ __forceinline__ void ldb_nk(uint32_t (&b)[4], uint32_t tile, int n0, int ks, int lane) {
  const int r = n0 + (lane & 7) + (lane >> 4) * 8;
  const int c = ks * 2 + ((lane >> 3) & 1);
  ldsm_x4(b[0], b[1], b[2], b[3], tile + tc::slab_off(kTileRows, r, c));
}
__device__ __forceinline__ void ldb_kn(uint32_t (&b)[4], uint32_t tile, int k0, int n0, int lane) {
  const int r = k0 + (lane & 7) + ((lane >> 3) & 1) * 8;
  const int c = (n0 >> 3) + (lane >> 4);
  ldsm_x4_t(b[0], b[1], b[2], b[3], tile + tc::slab_off(kTileRows, r, c));
}

// raw scores of 16 heads x 64 keys from the K tile in `buf`: s[nt][0..1] = row g_, keys 8nt + 2c_, +1; [2..3] = row g_+8
template <int D>
__device__ __forceinline__ void scores64(float (&s)[8][4], const uint32_t (&qf)[D / 16][4], uint32_t buf, int lane) {
#pragma unroll
  for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
    for (int np = 0; np < 4; ++np) {
      uint32_t b[4];
      ldb_nk(b, buf, np * 16, kk, lane);
      mma_bf16(s[2 * np], qf[kk], b[0], b[1]);
      mma_bf16(s[2 * np + 1], qf[kk], b[2], b[3]);
    }
  }
}

// online-softmax update of the state with the raw scores of one 64-key tile; on return s holds the probabilities
// exp2(s*c2 - new max) (0 for keys that do not take part) and the accumulator is rescaled, ready for P.V
template <int D, class VisFn>
__device__ __forceinline__ void softmax64(Acc<D>& a, float (&s)[8][4], VisFn vis, float c2, int lane) {
  const int c_ = lane & 3;
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    const int i = nt * 8 + 2 * c_;
    const bool v0 = vis(i), v1 = vis(i + 1);
    s[nt][0] = v0 ? s[nt][0] * c2 : -INFINITY;
    s[nt][1] = v1 ? s[nt][1] * c2 : -INFINITY;
    s[nt][2] = v0 ? s[nt][2] * c2 : -INFINITY;
    s[nt][3] = v1 ? s[nt][3] * c2 : -INFINITY;
  }
  float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    mx_lo = fmaxf(mx_lo, fmaxf(s[nt][0], s[nt][1]));
    mx_hi = fmaxf(mx_hi, fmaxf(s[nt][2], s[nt][3]));
  }
  mx_lo = warp_max4(mx_lo);
  mx_hi = warp_max4(mx_hi);
  const float mn_lo = fmaxf(a.m_lo, mx_lo), mn_hi = fmaxf(a.m_hi, mx_hi);
  const float mu_lo = (mn_lo == -INFINITY) ? 0.f : mn_lo, mu_hi = (mn_hi == -INFINITY) ? 0.f : mn_hi;
  const float al_lo = fast_exp2(a.m_lo - mu_lo), al_hi = fast_exp2(a.m_hi - mu_hi);
  float rs_lo = 0.f, rs_hi = 0.f;
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    s[nt][0] = fast_exp2(s[nt][0] - mu_lo);
    s[nt][1] = fast_exp2(s[nt][1] - mu_lo);
    s[nt][2] = fast_exp2(s[nt][2] - mu_hi);
    s[nt][3] = fast_exp2(s[nt][3] - mu_hi);
    rs_lo += s[nt][0] + s[nt][1];
    rs_hi += s[nt][2] + s[nt][3];
  }
  a.l_lo = a.l_lo * al_lo + rs_lo;   // per-lane partial sums; reduce over the quad when the state is read out
  a.l_hi = a.l_hi * al_hi + rs_hi;
  a.m_lo = mn_lo;
  a.m_hi = mn_hi;
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    a.o[i][0] *= al_lo; a.o[i][1] *= al_lo; a.o[i][2] *= al_hi; a.o[i][3] *= al_hi;
  }
}

// a.o += P V with the probabilities of softmax64 and the 64-row V tile in `buf`
template <int D>
__device__ __forceinline__ void pv64(Acc<D>& a, const float (&s)[8][4], uint32_t buf, int lane) {
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const uint32_t a0 = pack_bf16(s[2 * u][0], s[2 * u][1]), a1 = pack_bf16(s[2 * u][2], s[2 * u][3]);
    const uint32_t a2 = pack_bf16(s[2 * u + 1][0], s[2 * u + 1][1]), a3 = pack_bf16(s[2 * u + 1][2], s[2 * u + 1][3]);
#pragma unroll
    for (int np = 0; np < D / 16; ++np) {
      uint32_t b[4];
      ldb_kn(b, buf, u * 16, np * 16, lane);
      mma_bf16(a.o[2 * np], a0, a1, a2, a3, b[0], b[1]);
      mma_bf16(a.o[2 * np + 1], a0, a1, a2, a3, b[2], b[3]);
    }
  }
}

// one online-softmax step over a 64-key tile: row(i) gives the tensor row of key i (already clamped to valid
// rows), vis(i) says whether key i takes part.  The buffer holds K first, then V.
template <int D, class RowFn, class VisFn>
__device__ __forceinline__ void attend64(Acc<D>& a, const uint32_t (&qf)[D / 16][4], uint32_t buf, const __nv_bfloat16* kbase,
                                         const __nv_bfloat16* vbase, int64_t kstride, int64_t vstride, RowFn row, VisFn vis, float c2,
                                         int lane) {
  fill_async<D>(buf, kbase, kstride, row, lane);
  fill_wait();
  float s[8][4];
  scores64<D>(s, qf, buf, lane);
  __syncwarp();                                         // every lane has read K: the buffer takes V while the softmax runs
  fill_async<D>(buf, vbase, vstride, row, lane);
  softmax64<D>(a, s, vis, c2, lane);
  fill_wait();
  pv64<D>(a, s, buf, lane);
  __syncwarp();                                         // the buffer may be refilled by the next tile
}

// the same step for K and V tiles that are already in shared memory (filled by TMA): rows >= n_rows of the tiles may hold
// anything (cache rows past the sequence's end), so their V rows are cleared first: 0 * garbage must not reach the sums
template <int D, class VisFn>
__device__ __forceinline__ void attend64_smem(Acc<D>& a, const uint32_t (&qf)[D / 16][4], uint32_t buf_k, uint32_t buf_v, VisFn vis,
                                              int n_rows, float c2, int lane) {
  constexpr int CH = D / 8;
  if (n_rows < kTileRows) {
    for (int idx = n_rows * CH + lane; idx < kTileRows * CH; idx += 32) {
      const int r = idx / CH, c = idx - r * CH;
      asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};\n" ::"r"(buf_v + tc::slab_off(kTileRows, r, c)), "r"(0) : "memory");
    }
    __syncwarp();
  }
  float s[8][4];
  scores64<D>(s, qf, buf_k, lane);
  softmax64<D>(a, s, vis, c2, lane);
  pv64<D>(a, s, buf_v, lane);
}

// Dump a warp's state to shared memory as (m[16], l[16], o[16][D]) in plain row-major floats
template <int D>
__device__ __forceinline__ void store_state(const Acc<D>& a, float* dst, int lane) {
  const int g_ = lane >> 2, c_ = lane & 3;
  const float l_lo = warp_sum4(a.l_lo), l_hi = warp_sum4(a.l_hi);
  if (c_ == 0) {
    dst[g_] = a.m_lo;
    dst[g_ + 8] = a.m_hi;
    dst[16 + g_] = l_lo;
    dst[16 + g_ + 8] = l_hi;
  }
  float* o = dst + 32;
#pragma unroll
  for (int nt = 0; nt < D / 8; ++nt) {
    const int col = nt * 8 + 2 * c_;
    *reinterpret_cast<float2*>(o + g_ * D + col) = make_float2(a.o[nt][0], a.o[nt][1]);
    *reinterpret_cast<float2*>(o + (g_ + 8) * D + col) = make_float2(a.o[nt][2], a.o[nt][3]);
  }
}

}  // namespace wts
}  // namespace nsa
