// Selected-block attention, forward.  One warp owns one (query token, kv head): its (<= 16) query heads are
// the 16 rows of the warp-level MMA tile, and it walks the token's own list of selected 64-key blocks.
// Every token has a different list, so nothing is staged in shared memory: operands go straight from
// global memory (L1/L2) into MMA fragments with 16-byte loads.
//   * Q.K^T contracts over the head dimension, which is contiguous for both operands, so the k index of the
//     fragments is a fixed permutation of d (thread c of a quad takes the 8 contiguous elements 32s+8c..+7 and
//     uses them for two k-steps) -- the same permutation on both sides leaves the dot product unchanged.
//   * P.V contracts over keys: a thread loads 4 key rows x 8 value columns and transposes 2x2 bf16 pairs with
//     byte permutes; the output column permutation this implies is undone when O is written.
#include "nsa_common.cuh"

namespace nsa {

__device__ __forceinline__ uint4 ldg_nc16(const __nv_bfloat16* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
__device__ __forceinline__ uint32_t u4_get(const uint4& v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

template <int D, bool PAGED>
__global__ void __launch_bounds__(128, 2) slc_fwd_kernel(NsaAttnParams p) {
  constexpr int SS = D / 32, HH = D / 64, BS = 64;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g_ = lane >> 2, c_ = lane & 3;
  // blockIdx.z = (kv head, group of 16 of its query heads): more than 16 query heads per kv head run as several groups
  const int Gall = p.QH / p.KH, HG = (Gall + 15) / 16;
  const int kh = blockIdx.z / HG, hg = blockIdx.z % HG;
  const int G = min(16, Gall - 16 * hg);
  const int64_t hbase = (int64_t)kh * Gall + 16 * hg;   // first query head of my group
  const Piece pc = load_piece(p.meta, blockIdx.y);
  const int tl = (gridDim.x - 1 - blockIdx.x) * 4 + warp;  // local row inside the piece
  if (tl >= pc.len) return;
  const int t_abs = pc.off + tl;
  const int64_t q_row = pc.q_start + tl;
  const int nk = t_abs >= 0 ? t_abs / BS : -1;  // a padded row (empty sequence) attends nothing
  const int n_valid = min(p.hp.top_n, nk + 1);
  const float c2 = p.sm_scale * 1.4426950408889634f;

  const int h_lo = min(g_, G - 1), h_hi = min(g_ + 8, G - 1);
  const __nv_bfloat16* qp = reinterpret_cast<const __nv_bfloat16*>(p.q) + q_row * p.q_stride_t + hbase * D + c_ * 8;
  uint4 qa[SS], qb[SS];
#pragma unroll
  for (int s = 0; s < SS; ++s) {
    qa[s] = ldg_nc16(qp + h_lo * D + 32 * s);
    qb[s] = ldg_nc16(qp + h_hi * D + 32 * s);
  }
  const __nv_bfloat16* kb = reinterpret_cast<const __nv_bfloat16*>(p.k) + kh * D + c_ * 8;
  const __nv_bfloat16* vb = reinterpret_cast<const __nv_bfloat16*>(p.v) + kh * D + g_ * 8;
  const int32_t* idx = p.topk + (int64_t)kh * p.topk_stride_h + q_row * p.hp.top_n;
  const int last_row = pc.x_len - 1;
  auto krow = [&](int r) -> int64_t { return PAGED ? tok_row(pc, r) : (int64_t)pc.x_bos + r; };

  float o[HH][8][4];
#pragma unroll
  for (int h = 0; h < HH; ++h)
#pragma unroll
    for (int j = 0; j < 8; ++j) o[h][j][0] = o[h][j][1] = o[h][j][2] = o[h][j][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

  for (int i = 0; i < n_valid; ++i) {
    const int blk = __ldg(idx + i);
    if (blk < 0 || blk > nk) continue;  // unused slot or out-of-range entry: nothing to attend
    const int key0 = blk * BS;
    // ---- S = Q K^T  (16 heads x 64 keys)
    float s[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
      const __nv_bfloat16* kp = kb + krow(min(key0 + nt * 8 + g_, last_row)) * p.k_stride_t;
      uint4 kk[SS];
#pragma unroll
      for (int ss = 0; ss < SS; ++ss) kk[ss] = ldg_nc16(kp + 32 * ss);
#pragma unroll
      for (int ss = 0; ss < SS; ++ss) {
        mma_bf16(s[nt], qa[ss].x, qb[ss].x, qa[ss].y, qb[ss].y, kk[ss].x, kk[ss].y);
        mma_bf16(s[nt], qa[ss].z, qb[ss].z, qa[ss].w, qb[ss].w, kk[ss].z, kk[ss].w);
      }
    }
    if (blk == nk) {
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        int key = key0 + nt * 8 + 2 * c_;
        bool v0 = key <= t_abs, v1 = key + 1 <= t_abs;
        s[nt][0] = v0 ? s[nt][0] * c2 : -INFINITY;
        s[nt][1] = v1 ? s[nt][1] * c2 : -INFINITY;
        s[nt][2] = v0 ? s[nt][2] * c2 : -INFINITY;
        s[nt][3] = v1 ? s[nt][3] * c2 : -INFINITY;
      }
    } else {
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        s[nt][0] *= c2; s[nt][1] *= c2; s[nt][2] *= c2; s[nt][3] *= c2;
      }
    }
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      mx_lo = fmaxf(mx_lo, fmaxf(s[nt][0], s[nt][1]));
      mx_hi = fmaxf(mx_hi, fmaxf(s[nt][2], s[nt][3]));
    }
    mx_lo = warp_max4(mx_lo);
    mx_hi = warp_max4(mx_hi);
    float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
    float mu_lo = (mn_lo == -INFINITY) ? 0.f : mn_lo, mu_hi = (mn_hi == -INFINITY) ? 0.f : mn_hi;
    float al_lo = fast_exp2(m_lo - mu_lo), al_hi = fast_exp2(m_hi - mu_hi);
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
    l_lo = l_lo * al_lo + rs_lo;
    l_hi = l_hi * al_hi + rs_hi;
    m_lo = mn_lo;
    m_hi = mn_hi;
#pragma unroll
    for (int h = 0; h < HH; ++h)
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        o[h][j][0] *= al_lo; o[h][j][1] *= al_lo; o[h][j][2] *= al_hi; o[h][j][3] *= al_hi;
      }
    // ---- O += P V
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      uint32_t a0 = pack_bf16(s[2 * u][0], s[2 * u][1]), a1 = pack_bf16(s[2 * u][2], s[2 * u][3]);
      uint32_t a2 = pack_bf16(s[2 * u + 1][0], s[2 * u + 1][1]), a3 = pack_bf16(s[2 * u + 1][2], s[2 * u + 1][3]);
      const int r0 = key0 + 16 * u + 2 * c_;
      const __nv_bfloat16* v0p = vb + krow(min(r0, last_row)) * p.v_stride_t;
      const __nv_bfloat16* v1p = vb + krow(min(r0 + 1, last_row)) * p.v_stride_t;
      const __nv_bfloat16* v2p = vb + krow(min(r0 + 8, last_row)) * p.v_stride_t;
      const __nv_bfloat16* v3p = vb + krow(min(r0 + 9, last_row)) * p.v_stride_t;
#pragma unroll
      for (int h = 0; h < HH; ++h) {
        uint4 v0 = ldg_nc16(v0p + 64 * h), v1 = ldg_nc16(v1p + 64 * h), v2 = ldg_nc16(v2p + 64 * h), v3 = ldg_nc16(v3p + 64 * h);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t sel = (j & 1) ? 0x7632u : 0x5410u;
          uint32_t b0 = prmt(u4_get(v0, j >> 1), u4_get(v1, j >> 1), sel);
          uint32_t b1 = prmt(u4_get(v2, j >> 1), u4_get(v3, j >> 1), sel);
          mma_bf16(o[h][j], a0, a1, a2, a3, b0, b1);
        }
      }
    }
  }

  l_lo = warp_sum4(l_lo);
  l_hi = warp_sum4(l_hi);
  float inv_lo = l_lo > 0.f ? 1.f / l_lo : 0.f, inv_hi = l_hi > 0.f ? 1.f / l_hi : 0.f;
  __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(p.o) + q_row * p.o_stride_t + hbase * D + 16 * c_;
#pragma unroll
  for (int h = 0; h < HH; ++h) {
    if (g_ < G) {
      uint4 w0, w1;  // columns 64h+16c .. +7 come from element 0 of tiles j=0..7, the next 8 from element 1
      w0.x = pack_bf16(o[h][0][0] * inv_lo, o[h][1][0] * inv_lo); w0.y = pack_bf16(o[h][2][0] * inv_lo, o[h][3][0] * inv_lo);
      w0.z = pack_bf16(o[h][4][0] * inv_lo, o[h][5][0] * inv_lo); w0.w = pack_bf16(o[h][6][0] * inv_lo, o[h][7][0] * inv_lo);
      w1.x = pack_bf16(o[h][0][1] * inv_lo, o[h][1][1] * inv_lo); w1.y = pack_bf16(o[h][2][1] * inv_lo, o[h][3][1] * inv_lo);
      w1.z = pack_bf16(o[h][4][1] * inv_lo, o[h][5][1] * inv_lo); w1.w = pack_bf16(o[h][6][1] * inv_lo, o[h][7][1] * inv_lo);
      *reinterpret_cast<uint4*>(op + g_ * D + 64 * h) = w0;
      *reinterpret_cast<uint4*>(op + g_ * D + 64 * h + 8) = w1;
    }
    if (g_ + 8 < G) {
      uint4 w0, w1;
      w0.x = pack_bf16(o[h][0][2] * inv_hi, o[h][1][2] * inv_hi); w0.y = pack_bf16(o[h][2][2] * inv_hi, o[h][3][2] * inv_hi);
      w0.z = pack_bf16(o[h][4][2] * inv_hi, o[h][5][2] * inv_hi); w0.w = pack_bf16(o[h][6][2] * inv_hi, o[h][7][2] * inv_hi);
      w1.x = pack_bf16(o[h][0][3] * inv_hi, o[h][1][3] * inv_hi); w1.y = pack_bf16(o[h][2][3] * inv_hi, o[h][3][3] * inv_hi);
      w1.z = pack_bf16(o[h][4][3] * inv_hi, o[h][5][3] * inv_hi); w1.w = pack_bf16(o[h][6][3] * inv_hi, o[h][7][3] * inv_hi);
      *reinterpret_cast<uint4*>(op + (g_ + 8) * D + 64 * h) = w0;
      *reinterpret_cast<uint4*>(op + (g_ + 8) * D + 64 * h + 8) = w1;
    }
  }
  if (c_ == 0 && p.lse) {
    if (g_ < G)
      p.lse[q_row * p.lse_stride_t + (hbase + g_) * p.lse_stride_h] = l_lo > 0.f ? m_lo + log2f(l_lo) : 0.f;
    if (g_ + 8 < G)
      p.lse[q_row * p.lse_stride_t + (hbase + g_ + 8) * p.lse_stride_h] = l_hi > 0.f ? m_hi + log2f(l_hi) : 0.f;
  }
}

int check_attn_common(const NsaAttnParams* p, const char* name, bool need_y);
int launch_slc_tma(const NsaAttnParams* p, cudaStream_t st, bool backward);   // slc_tma.cu

}  // namespace nsa

using namespace nsa;

extern "C" int nsa_slc_attn_fwd(const NsaAttnParams* p, void* stream) {
  int rc = check_attn_common(p, "slc_attn_fwd", false);
  if (rc) return rc;
  NSA_REQUIRE(p->topk, NSA_ERR_BAD_ARG, "slc_attn_fwd: topk is required");
  NSA_REQUIRE(p->hp.block_size == 64, NSA_ERR_UNSUPPORTED_SHAPE, "slc_attn_fwd: block_size=%d (only 64 is implemented)", p->hp.block_size);
  if (p->meta.n_pieces <= 0 || p->meta.max_piece_len <= 0) return NSA_OK;
  rc = launch_slc_tma(p, (cudaStream_t)stream, false);   // contiguous K/V: TMA-staged tiles
  if (rc != 1) return rc;
  dim3 grid((p->meta.max_piece_len + 3) / 4, p->meta.n_pieces, p->KH * ((p->QH / p->KH + 15) / 16));
  const bool paged = p->meta.kv_table != nullptr;
  if (p->D == 128) {
    if (paged) slc_fwd_kernel<128, true><<<grid, 128, 0, (cudaStream_t)stream>>>(*p);
    else slc_fwd_kernel<128, false><<<grid, 128, 0, (cudaStream_t)stream>>>(*p);
  } else {
    if (paged) slc_fwd_kernel<64, true><<<grid, 128, 0, (cudaStream_t)stream>>>(*p);
    else slc_fwd_kernel<64, false><<<grid, 128, 0, (cudaStream_t)stream>>>(*p);
  }
  return check_launch("slc_attn_fwd");
}
