// Warp-level attention over one 64-key tile with operands taken straight from global memory (no shared memory):
// the 16 MMA rows are the query heads of one kv head for ONE token.  Shared by the decode kernel; the fragment layouts
// are the ones of slc_fwd.cu (d-permuted fragments for Q.K^T, byte-permute transposition for P.V).
#pragma once
#include "nsa_common.cuh"

namespace nsa {
namespace wt {

__device__ __forceinline__ uint4 ld16(const __nv_bfloat16* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
__device__ __forceinline__ uint32_t u4(const uint4& v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

template <int D>
struct Acc {  // running softmax state of 16 rows x D columns, spread over the warp in MMA accumulator layout
  float o[D / 64][8][4];
  float m_lo, m_hi, l_lo, l_hi;
  __device__ __forceinline__ void init() {
#pragma unroll
    for (int h = 0; h < D / 64; ++h)
#pragma unroll
      for (int j = 0; j < 8; ++j) o[h][j][0] = o[h][j][1] = o[h][j][2] = o[h][j][3] = 0.f;
    m_lo = m_hi = -INFINITY;
    l_lo = l_hi = 0.f;
  }
};

// Q fragments of one token: rows g_ and g_+8 (clamped to the last real head), 8 contiguous d per 32-wide slab
template <int D>
__device__ __forceinline__ void load_q(uint4 (&qa)[D / 32], uint4 (&qb)[D / 32], const __nv_bfloat16* q_tok_kh, int G, int lane) {
  const int g_ = lane >> 2, c_ = lane & 3;
  const int h_lo = min(g_, G - 1), h_hi = min(g_ + 8, G - 1);
#pragma unroll
  for (int s = 0; s < D / 32; ++s) {
    qa[s] = ld16(q_tok_kh + h_lo * D + 32 * s + c_ * 8);
    qb[s] = ld16(q_tok_kh + h_hi * D + 32 * s + c_ * 8);
  }
}

// raw scores of 16 heads x 64 keys; row(i) gives the flat tensor row of key i of the tile (already clamped to a valid row)
template <int D, class RowFn>
__device__ __forceinline__ void scores64(float (&s)[8][4], const uint4 (&qa)[D / 32], const uint4 (&qb)[D / 32],
                                         const __nv_bfloat16* kbase, int64_t kstride, RowFn row, int lane) {
  const int g_ = lane >> 2, c_ = lane & 3;
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
    const __nv_bfloat16* kp = kbase + row(nt * 8 + g_) * kstride + c_ * 8;
    uint4 kk[D / 32];
#pragma unroll
    for (int ss = 0; ss < D / 32; ++ss) kk[ss] = ld16(kp + 32 * ss);
#pragma unroll
    for (int ss = 0; ss < D / 32; ++ss) {
      mma_bf16(s[nt], qa[ss].x, qb[ss].x, qa[ss].y, qb[ss].y, kk[ss].x, kk[ss].y);
      mma_bf16(s[nt], qa[ss].z, qb[ss].z, qa[ss].w, qb[ss].w, kk[ss].z, kk[ss].w);
    }
  }
}

// one online-softmax step over a 64-key tile: vis(i) says whether key i of the tile takes part
template <int D, class RowFn, class VisFn>
__device__ __forceinline__ void attend64(Acc<D>& a, const uint4 (&qa)[D / 32], const uint4 (&qb)[D / 32], const __nv_bfloat16* kbase,
                                         const __nv_bfloat16* vbase, int64_t kstride, int64_t vstride, RowFn row, VisFn vis, float c2,
                                         int lane) {
  const int g_ = lane >> 2, c_ = lane & 3;
  float s[8][4];
  scores64<D>(s, qa, qb, kbase, kstride, row, lane);
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
  for (int h = 0; h < D / 64; ++h)
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      a.o[h][j][0] *= al_lo; a.o[h][j][1] *= al_lo; a.o[h][j][2] *= al_hi; a.o[h][j][3] *= al_hi;
    }
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const uint32_t a0 = pack_bf16(s[2 * u][0], s[2 * u][1]), a1 = pack_bf16(s[2 * u][2], s[2 * u][3]);
    const uint32_t a2 = pack_bf16(s[2 * u + 1][0], s[2 * u + 1][1]), a3 = pack_bf16(s[2 * u + 1][2], s[2 * u + 1][3]);
    const int r0 = 16 * u + 2 * c_;
    const __nv_bfloat16* v0p = vbase + row(r0) * vstride + g_ * 8;
    const __nv_bfloat16* v1p = vbase + row(r0 + 1) * vstride + g_ * 8;
    const __nv_bfloat16* v2p = vbase + row(r0 + 8) * vstride + g_ * 8;
    const __nv_bfloat16* v3p = vbase + row(r0 + 9) * vstride + g_ * 8;
#pragma unroll
    for (int h = 0; h < D / 64; ++h) {
      const uint4 v0 = ld16(v0p + 64 * h), v1 = ld16(v1p + 64 * h), v2 = ld16(v2p + 64 * h), v3 = ld16(v3p + 64 * h);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t sel = (j & 1) ? 0x7632u : 0x5410u;
        mma_bf16(a.o[h][j], a0, a1, a2, a3, prmt(u4(v0, j >> 1), u4(v1, j >> 1), sel), prmt(u4(v2, j >> 1), u4(v3, j >> 1), sel));
      }
    }
  }
}

// Dump a warp's state to shared memory as (m[16], l[16], o[16][D]) in plain row-major floats.
// Thread (g_, c_) owns rows g_, g_+8 and columns 64h + 16c_ + {0..7 from element 0/2, 8..15 from element 1/3} of tile j.
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
  for (int h = 0; h < D / 64; ++h)
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int col = 64 * h + 16 * c_ + j;
      o[g_ * D + col] = a.o[h][j][0];
      o[g_ * D + col + 8] = a.o[h][j][1];
      o[(g_ + 8) * D + col] = a.o[h][j][2];
      o[(g_ + 8) * D + col + 8] = a.o[h][j][3];
    }
}

}  // namespace wt
}  // namespace nsa
