// Backward kernels on the warp-level tensor-core path.
//
//  dense_dq_kernel<D,MODE>   dQ of the compressed / sliding-window branch: one CTA per 128-row query tile
//                            (tokens x the G heads of a kv head), loops over its K/V tiles:
//                            S = QK^T, P = exp2(S*c - lse), dP = dO V^T, dS = P*(dP - delta), dQ += dS K.
//  (dK/dV of all three branches live in dkdv_tc.cu; this file launches them.)
// P and dS are rounded to bf16 before the second-stage products, as in the reference kernels
// (flash_nsa/ops/compress_attn.py:311-325, flash_nsa/ops/select_attn.py:262-280).
#include "nsa_common.cuh"

namespace nsa {

constexpr int MODE_CMP = 0;
constexpr int MODE_SWA = 1;
constexpr int MODE_SLC = 2;

void launch_delta(const void* o, const void* dout, float* delta, int64_t T, int H, int D, int64_t o_stride_t,
                  int64_t do_stride_t, int64_t lse_stride_t, int64_t lse_stride_h, cudaStream_t st);
int check_attn_common(const NsaAttnParams* p, const char* name, bool need_y);

// ------------------------------------------------------------------------------------------------ dQ
template <int D, int MODE>
__global__ void __launch_bounds__(256, 1) dense_dq_kernel(NsaAttnParams p) {
  constexpr int BM = 128, BN = 64, CH = D / 8, KS = D / 16, NT = D / 8;
  extern __shared__ __align__(128) unsigned char smem[];
  const uint32_t sQ = smem_u32(smem);             // Q staging, later the dQ staging tile
  const uint32_t sO = sQ + BM * D * 2;            // dO staging
  const uint32_t sK = sO + BM * D * 2;
  const uint32_t sV = sK + 2 * BN * D * 2;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = p.QH / p.KH;
  const int TOK = BM / G;
  const int tile = gridDim.x - 1 - blockIdx.x;
  const int kh = blockIdx.z;
  const Piece pc = load_piece(p.meta, blockIdx.y);
  const int t0 = tile * TOK;
  if (t0 >= pc.len) return;
  const int ntok = min(TOK, pc.len - t0);
  const int tabs_min = pc.off + t0, tabs_max = tabs_min + ntok - 1;
  const int ks = p.hp.kernel_size, st = p.hp.stride, W = p.hp.window;

  int kv_lo, kv_hi;
  const __nv_bfloat16 *kbase, *vbase;
  if (MODE == MODE_CMP) {
    kv_lo = 0;
    kv_hi = (tabs_max >= ks - 1) ? min(pc.y_len, (tabs_max - (ks - 1)) / st + 1) : 0;
    kbase = reinterpret_cast<const __nv_bfloat16*>(p.k) + (int64_t)pc.y_bos * p.k_stride_t + kh * D;
    vbase = reinterpret_cast<const __nv_bfloat16*>(p.v) + (int64_t)pc.y_bos * p.v_stride_t + kh * D;
  } else {
    kv_lo = max(0, tabs_min - W);
    kv_hi = min(tabs_max + 1, pc.x_len);
    kbase = reinterpret_cast<const __nv_bfloat16*>(p.k) + (int64_t)pc.x_bos * p.k_stride_t + kh * D;
    vbase = reinterpret_cast<const __nv_bfloat16*>(p.v) + (int64_t)pc.x_bos * p.v_stride_t + kh * D;
  }
  const int ntiles = (kv_hi > kv_lo) ? (kv_hi - kv_lo + BN - 1) / BN : 0;

  {
    const __nv_bfloat16* qb = reinterpret_cast<const __nv_bfloat16*>(p.q) + (int64_t)(pc.q_start + t0) * p.q_stride_t +
                              (int64_t)kh * G * D;
    const __nv_bfloat16* ob = reinterpret_cast<const __nv_bfloat16*>(p.dout) + (int64_t)(pc.q_start + t0) * p.do_stride_t +
                              (int64_t)kh * G * D;
    for (int i = tid; i < BM * CH; i += 256) {
      int r = i / CH, c = i % CH;
      int tok = r / G, g = r - tok * G;
      bool ok = tok < ntok;
      cp_async16(sQ + tile_off<D>(r, c), qb + (ok ? (int64_t)tok * p.q_stride_t + g * D : 0) + c * 8, ok);
      cp_async16(sO + tile_off<D>(r, c), ob + (ok ? (int64_t)tok * p.do_stride_t + g * D : 0) + c * 8, ok);
    }
    cp_async_commit();
  }
  auto load_kv = [&](int it) {
    int kv0 = kv_lo + it * BN;
    int valid = min(BN, kv_hi - kv0);
    load_tile_async<D>(sK + (it & 1) * BN * D * 2, kbase + (int64_t)kv0 * p.k_stride_t, p.k_stride_t, BN, valid, tid, 256);
    load_tile_async<D>(sV + (it & 1) * BN * D * 2, vbase + (int64_t)kv0 * p.v_stride_t, p.v_stride_t, BN, valid, tid, 256);
  };
  if (ntiles > 0) load_kv(0);
  cp_async_commit();
  cp_async_wait<1>();
  __syncthreads();

  uint32_t qf[KS][4], of[KS][4];
#pragma unroll
  for (int kk = 0; kk < KS; ++kk) {
    load_a_frag<D>(qf[kk], sQ, warp * 16, kk, lane);
    load_a_frag<D>(of[kk], sO, warp * 16, kk, lane);
  }

  const int g_ = lane >> 2, c_ = lane & 3;
  const int row_lo = warp * 16 + g_, row_hi = row_lo + 8;
  const int tok_lo = row_lo / G, tok_hi = row_hi / G;
  const int tabs_lo = tabs_min + tok_lo, tabs_hi = tabs_min + tok_hi;
  const float c2 = p.sm_scale * 1.4426950408889634f;
  float lse_lo = 0.f, lse_hi = 0.f, dl_lo = 0.f, dl_hi = 0.f;
  if (tok_lo < ntok) {
    int64_t a = (int64_t)(pc.q_start + t0 + tok_lo) * p.lse_stride_t + (int64_t)(kh * G + row_lo - tok_lo * G) * p.lse_stride_h;
    lse_lo = p.lse[a];
    dl_lo = p.delta[a];
  }
  if (tok_hi < ntok) {
    int64_t a = (int64_t)(pc.q_start + t0 + tok_hi) * p.lse_stride_t + (int64_t)(kh * G + row_hi - tok_hi * G) * p.lse_stride_h;
    lse_hi = p.lse[a];
    dl_hi = p.delta[a];
  }

  float dq[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) dq[i][0] = dq[i][1] = dq[i][2] = dq[i][3] = 0.f;

  for (int it = 0; it < ntiles; ++it) {
    if (it + 1 < ntiles) load_kv(it + 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const uint32_t tK = sK + (it & 1) * BN * D * 2, tV = sV + (it & 1) * BN * D * 2;
    const int kv0 = kv_lo + it * BN;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float s[4][4], dp[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
        dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.f;
      }
#pragma unroll
      for (int kk = 0; kk < KS; ++kk) {
#pragma unroll
        for (int np = 0; np < 2; ++np) {
          uint32_t b[4];
          load_b_frag_nk<D>(b, tK, half * 32 + np * 16, kk, lane);
          mma_bf16(s[2 * np], qf[kk], b[0], b[1]);
          mma_bf16(s[2 * np + 1], qf[kk], b[2], b[3]);
          load_b_frag_nk<D>(b, tV, half * 32 + np * 16, kk, lane);
          mma_bf16(dp[2 * np], of[kk], b[0], b[1]);
          mma_bf16(dp[2 * np + 1], of[kk], b[2], b[3]);
        }
      }
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          int col = kv0 + half * 32 + nt * 8 + 2 * c_ + (e & 1);
          int ta = (e < 2) ? tabs_lo : tabs_hi;
          bool vis;
          if (MODE == MODE_CMP)
            vis = (col * st + ks - 1 <= ta) && (col < kv_hi);
          else
            vis = (col <= ta) && (col >= ta - W) && (col < kv_hi);
          float pv = vis ? fast_exp2(fmaf(s[nt][e], c2, -((e < 2) ? lse_lo : lse_hi))) : 0.f;
          dp[nt][e] = pv * (dp[nt][e] - ((e < 2) ? dl_lo : dl_hi));
        }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        uint32_t a0 = pack_bf16(dp[2 * u][0], dp[2 * u][1]), a1 = pack_bf16(dp[2 * u][2], dp[2 * u][3]);
        uint32_t a2 = pack_bf16(dp[2 * u + 1][0], dp[2 * u + 1][1]), a3 = pack_bf16(dp[2 * u + 1][2], dp[2 * u + 1][3]);
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
          uint32_t b[4];
          load_b_frag_kn<D>(b, tK, half * 32 + u * 16, np * 16, lane);
          mma_bf16(dq[2 * np], a0, a1, a2, a3, b[0], b[1]);
          mma_bf16(dq[2 * np + 1], a0, a1, a2, a3, b[2], b[3]);
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

  __syncwarp();
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    uint32_t lo = pack_bf16(dq[nt][0] * p.sm_scale, dq[nt][1] * p.sm_scale);
    uint32_t hi = pack_bf16(dq[nt][2] * p.sm_scale, dq[nt][3] * p.sm_scale);
    asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(sQ + tile_off<D>(row_lo, nt) + c_ * 4), "r"(lo));
    asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(sQ + tile_off<D>(row_hi, nt) + c_ * 4), "r"(hi));
  }
  __syncwarp();
  {
    __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(p.dq) + (int64_t)(pc.q_start + t0) * p.dq_stride_t + (int64_t)kh * G * D;
    for (int i = lane; i < 16 * CH; i += 32) {
      int r = warp * 16 + i / CH, c = i % CH;
      int tok = r / G, g = r - tok * G;
      if (tok < ntok) {
        uint4 v;
        asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];\n"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                     : "r"(sQ + tile_off<D>(r, c)));
        uint4* dst = reinterpret_cast<uint4*>(ob + (int64_t)tok * p.dq_stride_t + g * D + c * 8);
        if (p.accumulate_dq) {
          uint4 old = *dst;
          v.x = pack_bf16(bf16_lo(v.x) + bf16_lo(old.x), bf16_hi(v.x) + bf16_hi(old.x));
          v.y = pack_bf16(bf16_lo(v.y) + bf16_lo(old.y), bf16_hi(v.y) + bf16_hi(old.y));
          v.z = pack_bf16(bf16_lo(v.z) + bf16_lo(old.z), bf16_hi(v.z) + bf16_hi(old.z));
          v.w = pack_bf16(bf16_lo(v.w) + bf16_lo(old.w), bf16_hi(v.w) + bf16_hi(old.w));
        }
        *dst = v;
      }
    }
  }
}

template <int D, int MODE>
int launch_dkdv(const NsaAttnParams* p, cudaStream_t st, const char* name, dim3 grid, DkdvLaunch L);  // dkdv_tc.cu

template <typename K>
static int set_smem(K kernel, size_t smem, const char* name) {
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_error("%s: cudaFuncSetAttribute failed: %s", name, cudaGetErrorString(e));
    return NSA_ERR_CUDA;
  }
  return NSA_OK;
}

template <int D, int MODE>
static int launch_dq(const NsaAttnParams* p, cudaStream_t st, const char* name) {
  const int G = p->QH / p->KH, TOK = 128 / G;
  size_t smem = (size_t)(2 * 128 + 4 * 64) * D * 2;
  int rc = set_smem(dense_dq_kernel<D, MODE>, smem, name);
  if (rc) return rc;
  dim3 grid((p->meta.max_piece_len + TOK - 1) / TOK, p->meta.n_pieces, p->KH);
  dense_dq_kernel<D, MODE><<<grid, 256, smem, st>>>(*p);
  return check_launch(name);
}

static int check_bwd(const NsaAttnParams* p, const char* name) {
  NSA_REQUIRE(p->lse && p->dout && p->delta && p->dq && p->dk && p->dv, NSA_ERR_BAD_ARG, "%s: lse, dout, delta, dq, dk, dv are required", name);
  NSA_REQUIRE(p->QH / p->KH <= 64, NSA_ERR_UNSUPPORTED_SHAPE, "%s: more than 64 query heads per kv head", name);
  NSA_REQUIRE(p->dk_stride_t % 2 == 0 && p->dv_stride_t % 2 == 0, NSA_ERR_BAD_ARG, "%s: dk/dv row strides must be even", name);
  return NSA_OK;
}

}  // namespace nsa

using namespace nsa;

extern "C" int nsa_cmp_attn_bwd(const NsaAttnParams* p, void* stream) {
  int rc = check_attn_common(p, "cmp_attn_bwd", true);
  if (rc) return rc;
  if ((rc = check_bwd(p, "cmp_attn_bwd"))) return rc;
  if (p->meta.n_pieces <= 0 || p->meta.max_piece_len <= 0 || p->n_q_rows <= 0) return NSA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int ph = p->phases ? p->phases : 7;
  if (ph & 1)
    launch_delta(p->o, p->dout, p->delta, p->n_q_rows, p->QH, p->D, p->o_stride_t, p->do_stride_t, p->lse_stride_t, p->lse_stride_h, st);
  if ((ph & 2) && p->meta.y_maxlen > 0) {
    DkdvLaunch L{2048, 1, nullptr};
    dim3 grid((p->meta.y_maxlen + 63) / 64, (p->meta.max_piece_len + L.q_chunk - 1) / L.q_chunk, p->meta.n_pieces * p->KH);
    rc = (p->D == 128) ? launch_dkdv<128, MODE_CMP>(p, st, "cmp_attn_bwd(dkdv)", grid, L)
                       : launch_dkdv<64, MODE_CMP>(p, st, "cmp_attn_bwd(dkdv)", grid, L);
    if (rc) return rc;
  }
  if (!(ph & 4)) return check_launch("cmp_attn_bwd");
  return (p->D == 128) ? launch_dq<128, MODE_CMP>(p, st, "cmp_attn_bwd(dq)") : launch_dq<64, MODE_CMP>(p, st, "cmp_attn_bwd(dq)");
}

extern "C" int nsa_swa_bwd(const NsaAttnParams* p, void* stream) {
  int rc = check_attn_common(p, "swa_bwd", false);
  if (rc) return rc;
  if ((rc = check_bwd(p, "swa_bwd"))) return rc;
  if (p->meta.n_pieces <= 0 || p->meta.max_piece_len <= 0 || p->n_q_rows <= 0) return NSA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int ph = p->phases ? p->phases : 7;
  if (ph & 1)
    launch_delta(p->o, p->dout, p->delta, p->n_q_rows, p->QH, p->D, p->o_stride_t, p->do_stride_t, p->lse_stride_t, p->lse_stride_h, st);
  if (ph & 2) {
    DkdvLaunch L{0, 1, nullptr};
    dim3 grid((p->meta.max_piece_len + p->hp.window + 63) / 64 + 1, 1, p->meta.n_pieces * p->KH);
    rc = (p->D == 128) ? launch_dkdv<128, MODE_SWA>(p, st, "swa_bwd(dkdv)", grid, L) : launch_dkdv<64, MODE_SWA>(p, st, "swa_bwd(dkdv)", grid, L);
    if (rc) return rc;
  }
  if (!(ph & 4)) return check_launch("swa_bwd");
  return (p->D == 128) ? launch_dq<128, MODE_SWA>(p, st, "swa_bwd(dq)") : launch_dq<64, MODE_SWA>(p, st, "swa_bwd(dq)");
}
