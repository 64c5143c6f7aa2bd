// Selected-block attention, backward: the entry point and the token-major dQ kernel for paged / unaligned callers.
//   dK/dV (+ dQ): slc_bwd_tc_kernel (slc_bwd_tc.cu), persistent, over the work items of the key-block -> queries index.
//   dQ alone:     slc_tma.cu when its conditions hold, otherwise the kernel below: one warp per (query token, kv head),
//                 like the forward: recompute S and P for each selected block, dP = dO V^T, dS = P*(dP - delta),
//                 dQ += dS K.  Operands come straight from global memory into MMA fragments (see slc_fwd.cu).
#include <cstdlib>
#include "nsa_common.cuh"

namespace nsa {

int launch_slc_bwd_tc(const NsaAttnParams* p, cudaStream_t st, const char* name, int fuse);   // slc_bwd_tc.cu
int launch_slc_tma(const NsaAttnParams* p, cudaStream_t st, bool backward);   // slc_tma.cu
void launch_delta(const void* o, const void* dout, float* delta, int64_t T, int H, int D, int64_t o_stride_t,
                  int64_t do_stride_t, int64_t lse_stride_t, int64_t lse_stride_h, cudaStream_t st);
int check_attn_common(const NsaAttnParams* p, const char* name, bool need_y);

__device__ __forceinline__ uint4 ldg_nc16b(const __nv_bfloat16* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ uint32_t prmt_b(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
__device__ __forceinline__ uint32_t u4_at(const uint4& v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

template <int D>
__global__ void __launch_bounds__(128, 2) slc_dq_kernel(NsaAttnParams p) {
  constexpr int SS = D / 32, HH = D / 64, BS = 64;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g_ = lane >> 2, c_ = lane & 3;
  // blockIdx.z = (kv head, group of 16 of its query heads): more than 16 query heads per kv head run as several groups
  const int Gall = p.QH / p.KH, HG = (Gall + 15) / 16;
  const int kh = blockIdx.z / HG, hg = blockIdx.z % HG;
  const int G = min(16, Gall - 16 * hg);
  const int64_t hbase = (int64_t)kh * Gall + 16 * hg;   // first query head of my group
  const Piece pc = load_piece(p.meta, blockIdx.y);
  const int tl = (gridDim.x - 1 - blockIdx.x) * 4 + warp;
  if (tl >= pc.len) return;
  const int t_abs = pc.off + tl;
  const int64_t q_row = pc.q_start + tl;
  const int nk = t_abs / BS;
  const int n_valid = min(p.hp.top_n, nk + 1);
  const float c2 = p.sm_scale * 1.4426950408889634f;

  const int h_lo = min(g_, G - 1), h_hi = min(g_ + 8, G - 1);
  const __nv_bfloat16* qp = reinterpret_cast<const __nv_bfloat16*>(p.q) + q_row * p.q_stride_t + hbase * D + c_ * 8;
  const __nv_bfloat16* dop = reinterpret_cast<const __nv_bfloat16*>(p.dout) + q_row * p.do_stride_t + hbase * D + c_ * 8;
  uint4 qa[SS], qb[SS], oa[SS], ob[SS];
#pragma unroll
  for (int s = 0; s < SS; ++s) {
    qa[s] = ldg_nc16b(qp + h_lo * D + 32 * s);
    qb[s] = ldg_nc16b(qp + h_hi * D + 32 * s);
    oa[s] = ldg_nc16b(dop + h_lo * D + 32 * s);
    ob[s] = ldg_nc16b(dop + h_hi * D + 32 * s);
  }
  const int64_t la = q_row * p.lse_stride_t + (hbase + h_lo) * p.lse_stride_h;
  const int64_t lb = q_row * p.lse_stride_t + (hbase + h_hi) * p.lse_stride_h;
  const float lse_lo = p.lse[la], lse_hi = p.lse[lb], dl_lo = p.delta[la], dl_hi = p.delta[lb];

  const __nv_bfloat16* kb = reinterpret_cast<const __nv_bfloat16*>(p.k) + (int64_t)pc.x_bos * p.k_stride_t + kh * D;
  const __nv_bfloat16* vb = reinterpret_cast<const __nv_bfloat16*>(p.v) + (int64_t)pc.x_bos * p.v_stride_t + kh * D;
  const int32_t* idx = p.topk + (int64_t)kh * p.topk_stride_h + q_row * p.hp.top_n;
  const int last_row = pc.x_len - 1;

  float dq[HH][8][4];
#pragma unroll
  for (int h = 0; h < HH; ++h)
#pragma unroll
    for (int j = 0; j < 8; ++j) dq[h][j][0] = dq[h][j][1] = dq[h][j][2] = dq[h][j][3] = 0.f;

  for (int i = 0; i < n_valid; ++i) {
    const int blk = __ldg(idx + i);
    if (blk < 0 || blk > nk) continue;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int key0 = blk * BS + half * 32;
      float s[4][4], dp[4][4];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
        dp[nt][0] = dp[nt][1] = dp[nt][2] = dp[nt][3] = 0.f;
        const int64_t r = min(key0 + nt * 8 + g_, last_row);
        const __nv_bfloat16* kp = kb + r * p.k_stride_t + c_ * 8;
        const __nv_bfloat16* vp = vb + r * p.v_stride_t + c_ * 8;
        uint4 kk[SS], vv[SS];
#pragma unroll
        for (int ss = 0; ss < SS; ++ss) {
          kk[ss] = ldg_nc16b(kp + 32 * ss);
          vv[ss] = ldg_nc16b(vp + 32 * ss);
        }
#pragma unroll
        for (int ss = 0; ss < SS; ++ss) {
          mma_bf16(s[nt], qa[ss].x, qb[ss].x, qa[ss].y, qb[ss].y, kk[ss].x, kk[ss].y);
          mma_bf16(s[nt], qa[ss].z, qb[ss].z, qa[ss].w, qb[ss].w, kk[ss].z, kk[ss].w);
          mma_bf16(dp[nt], oa[ss].x, ob[ss].x, oa[ss].y, ob[ss].y, vv[ss].x, vv[ss].y);
          mma_bf16(dp[nt], oa[ss].z, ob[ss].z, oa[ss].w, ob[ss].w, vv[ss].z, vv[ss].w);
        }
      }
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const int key = key0 + nt * 8 + 2 * c_;
        const bool v0 = key <= t_abs, v1 = key + 1 <= t_abs;
        float p0 = v0 ? fast_exp2(fmaf(s[nt][0], c2, -lse_lo)) : 0.f;
        float p1 = v1 ? fast_exp2(fmaf(s[nt][1], c2, -lse_lo)) : 0.f;
        float p2 = v0 ? fast_exp2(fmaf(s[nt][2], c2, -lse_hi)) : 0.f;
        float p3 = v1 ? fast_exp2(fmaf(s[nt][3], c2, -lse_hi)) : 0.f;
        dp[nt][0] = p0 * (dp[nt][0] - dl_lo);
        dp[nt][1] = p1 * (dp[nt][1] - dl_lo);
        dp[nt][2] = p2 * (dp[nt][2] - dl_hi);
        dp[nt][3] = p3 * (dp[nt][3] - dl_hi);
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        uint32_t a0 = pack_bf16(dp[2 * u][0], dp[2 * u][1]), a1 = pack_bf16(dp[2 * u][2], dp[2 * u][3]);
        uint32_t a2 = pack_bf16(dp[2 * u + 1][0], dp[2 * u + 1][1]), a3 = pack_bf16(dp[2 * u + 1][2], dp[2 * u + 1][3]);
        const int r0 = key0 + 16 * u + 2 * c_;
        const __nv_bfloat16* k0p = kb + (int64_t)min(r0, last_row) * p.k_stride_t + g_ * 8;
        const __nv_bfloat16* k1p = kb + (int64_t)min(r0 + 1, last_row) * p.k_stride_t + g_ * 8;
        const __nv_bfloat16* k2p = kb + (int64_t)min(r0 + 8, last_row) * p.k_stride_t + g_ * 8;
        const __nv_bfloat16* k3p = kb + (int64_t)min(r0 + 9, last_row) * p.k_stride_t + g_ * 8;
#pragma unroll
        for (int h = 0; h < HH; ++h) {
          uint4 w0 = ldg_nc16b(k0p + 64 * h), w1 = ldg_nc16b(k1p + 64 * h), w2 = ldg_nc16b(k2p + 64 * h), w3 = ldg_nc16b(k3p + 64 * h);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint32_t sel = (j & 1) ? 0x7632u : 0x5410u;
            uint32_t b0 = prmt_b(u4_at(w0, j >> 1), u4_at(w1, j >> 1), sel);
            uint32_t b1 = prmt_b(u4_at(w2, j >> 1), u4_at(w3, j >> 1), sel);
            mma_bf16(dq[h][j], a0, a1, a2, a3, b0, b1);
          }
        }
      }
    }
  }

  __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(p.dq) + q_row * p.dq_stride_t + hbase * D + 16 * c_;
  const float sc = p.sm_scale;
#pragma unroll
  for (int h = 0; h < HH; ++h) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int g = g_ + 8 * half;
      if (g < G) {
        const int e0 = 2 * half, e1 = 2 * half + 1;
        float f[16];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          f[j] = dq[h][j][e0] * sc;
          f[8 + j] = dq[h][j][e1] * sc;
        }
        uint4* dst = reinterpret_cast<uint4*>(op + g * D + 64 * h);
        if (p.accumulate_dq) {
          uint4 o0 = dst[0], o1 = dst[1];
          f[0] += bf16_lo(o0.x); f[1] += bf16_hi(o0.x); f[2] += bf16_lo(o0.y); f[3] += bf16_hi(o0.y);
          f[4] += bf16_lo(o0.z); f[5] += bf16_hi(o0.z); f[6] += bf16_lo(o0.w); f[7] += bf16_hi(o0.w);
          f[8] += bf16_lo(o1.x); f[9] += bf16_hi(o1.x); f[10] += bf16_lo(o1.y); f[11] += bf16_hi(o1.y);
          f[12] += bf16_lo(o1.z); f[13] += bf16_hi(o1.z); f[14] += bf16_lo(o1.w); f[15] += bf16_hi(o1.w);
        }
        uint4 w0, w1;
        w0.x = pack_bf16(f[0], f[1]); w0.y = pack_bf16(f[2], f[3]); w0.z = pack_bf16(f[4], f[5]); w0.w = pack_bf16(f[6], f[7]);
        w1.x = pack_bf16(f[8], f[9]); w1.y = pack_bf16(f[10], f[11]); w1.z = pack_bf16(f[12], f[13]); w1.w = pack_bf16(f[14], f[15]);
        dst[0] = w0;
        dst[1] = w1;
      }
    }
  }
}

}  // namespace nsa

using namespace nsa;

extern "C" int nsa_slc_attn_bwd(const NsaAttnParams* p, void* stream) {
  int rc = check_attn_common(p, "slc_attn_bwd", false);
  if (rc) return rc;
  NSA_REQUIRE(p->topk && p->lse && p->dout && p->delta && p->dq && p->dk && p->dv, NSA_ERR_BAD_ARG,
              "slc_attn_bwd: topk, lse, dout, delta, dq, dk, dv are required");
  NSA_REQUIRE(p->k2q_tokens && p->k2q_blk_cu, NSA_ERR_BAD_ARG, "slc_attn_bwd: the k2q index is required");
  NSA_REQUIRE(!((p->phases ? p->phases : 7) & 2) || (p->k2q_items && p->k2q_n_items && p->k2q_items_cap > 0), NSA_ERR_BAD_ARG,
              "slc_attn_bwd: the k2q index must carry work items (build it with item_rows > 0)");
  NSA_REQUIRE((((uintptr_t)p->k2q_items) & 15) == 0, NSA_ERR_BAD_ARG, "slc_attn_bwd: k2q_items must be 16-byte aligned");
  NSA_REQUIRE((((uintptr_t)p->q | (uintptr_t)p->dout | (uintptr_t)p->k | (uintptr_t)p->v) & 15) == 0 && (p->q_stride_t * 2) % 16 == 0 &&
                  (p->do_stride_t * 2) % 16 == 0 && (p->k_stride_t * 2) % 16 == 0 && (p->v_stride_t * 2) % 16 == 0,
              NSA_ERR_BAD_ARG, "slc_attn_bwd: q, dout, k, v must be 16-byte aligned with 16-byte-multiple row strides (bulk tensor loads)");
  NSA_REQUIRE(!(p->meta.kv_table), NSA_ERR_UNSUPPORTED_SHAPE, "slc_attn_bwd: paged K/V is an inference layout; the backward takes contiguous K/V");
  NSA_REQUIRE(p->hp.block_size == 64, NSA_ERR_UNSUPPORTED_SHAPE, "slc_attn_bwd: block_size=%d (only 64 is implemented)", p->hp.block_size);
  NSA_REQUIRE(p->dk_stride_t % 2 == 0 && p->dv_stride_t % 2 == 0, NSA_ERR_BAD_ARG, "slc_attn_bwd: dk/dv row strides must be even");
  if (p->meta.n_pieces <= 0 || p->meta.max_piece_len <= 0 || p->n_q_rows <= 0) return NSA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int ph = p->phases ? p->phases : 7;
  if (ph & 1)
    launch_delta(p->o, p->dout, p->delta, p->n_q_rows, p->QH, p->D, p->o_stride_t, p->do_stride_t, p->lse_stride_t, p->lse_stride_h, st);
  // dK/dV and dQ asked for together: the block-major kernel also forms dS K per tile and adds it into dq with bf16
  // reductions in global memory (as the reference's dq kernel does, flash_nsa/ops/select_attn.py), so the token-major dQ
  // kernel and its second pass over K, V, q, dout are not needed.  NSA_SLC_BWD_UNFUSED=1 keeps the two-kernel form
  // (dq accumulated in fp32 per token, deterministic).
  static const bool unfused = [] { const char* e = getenv("NSA_SLC_BWD_UNFUSED"); return e && e[0] == '1'; }();
  // the bulk tensor reductions need dq 16-byte aligned with a row stride that is a multiple of 16 bytes
  const bool dq_tma_ok = (((uintptr_t)p->dq) & 15) == 0 && (p->dq_stride_t * 2) % 16 == 0;
  const bool fuse = (ph & 2) && (ph & 4) && !unfused && dq_tma_ok && p->n_blocks_total > 0;
  if (fuse && !p->accumulate_dq) {
    cudaError_t e = cudaMemset2DAsync(p->dq, (size_t)p->dq_stride_t * 2, 0, (size_t)p->QH * p->D * 2, (size_t)p->n_q_rows, st);
    if (e != cudaSuccess) {
      set_error("slc_attn_bwd: clearing dq failed: %s", cudaGetErrorString(e));
      return NSA_ERR_CUDA;
    }
  }
  if ((ph & 2) && p->n_blocks_total > 0) {
    rc = launch_slc_bwd_tc(p, st, "slc_attn_bwd(dkdv)", fuse ? 1 : 0);
    if (rc) return rc;
  }
  if (!(ph & 4) || fuse) return check_launch("slc_attn_bwd");
  rc = launch_slc_tma(p, st, true);
  if (rc != 1) return rc;
  dim3 grid((p->meta.max_piece_len + 3) / 4, p->meta.n_pieces, p->KH * ((p->QH / p->KH + 15) / 16));
  if (p->D == 128) slc_dq_kernel<128><<<grid, 128, 0, st>>>(*p);
  else slc_dq_kernel<64><<<grid, 128, 0, st>>>(*p);
  return check_launch("slc_attn_bwd(dq)");
}
