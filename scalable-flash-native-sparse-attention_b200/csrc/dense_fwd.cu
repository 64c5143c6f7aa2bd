// Forward of the two "dense range" attention branches on the warp-level tensor-core path:
//   MODE_CMP  query t attends compressed rows j with  stride*j + kernel_size - 1 <= t
//   MODE_SWA  query t attends keys  t-window .. t
// One CTA owns a 128-row tile = (128/G consecutive tokens) x (the G query heads of one kv head), so a K/V tile
// staged in shared memory is shared by all heads of the group.  8 warps x 16 rows, online softmax in base 2,
// K/V tiles of 64 rows double-buffered with cp.async.
#include "nsa_common.cuh"

namespace nsa {

constexpr int MODE_CMP = 0;
constexpr int MODE_SWA = 1;

template <int D, int MODE>
__global__ void __launch_bounds__(256, 1) dense_fwd_kernel(NsaAttnParams p) {
  constexpr int BM = 128, BN = 64, CH = D / 8, KS = D / 16, NT = D / 8;
  extern __shared__ __align__(128) unsigned char smem[];
  const uint32_t sQ = smem_u32(smem);
  const uint32_t sK = sQ + BM * D * 2;
  const uint32_t sV = sK + 2 * BN * D * 2;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = p.QH / p.KH;
  const int TOK = BM / G;
  const int tile = gridDim.x - 1 - blockIdx.x;  // long (late) tiles first
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

  // ---- stage Q (rows = token-major, head-minor)
  {
    const __nv_bfloat16* qb = reinterpret_cast<const __nv_bfloat16*>(p.q) + (int64_t)(pc.q_start + t0) * p.q_stride_t +
                              (int64_t)kh * G * D;
    for (int i = tid; i < BM * CH; i += 256) {
      int r = i / CH, c = i % CH;
      int tok = r / G, g = r - tok * G;
      bool ok = tok < ntok;
      const __nv_bfloat16* src = qb + (ok ? (int64_t)tok * p.q_stride_t + g * D : 0) + c * 8;
      cp_async16(sQ + tile_off<D>(r, c), src, ok);
    }
    cp_async_commit();
  }
  auto load_kv = [&](int it) {
    int kv0 = kv_lo + it * BN;
    int valid = min(BN, kv_hi - kv0);
    uint32_t dk = sK + (it & 1) * BN * D * 2, dv = sV + (it & 1) * BN * D * 2;
    load_tile_async<D>(dk, kbase + (int64_t)kv0 * p.k_stride_t, p.k_stride_t, BN, valid, tid, 256);
    load_tile_async<D>(dv, vbase + (int64_t)kv0 * p.v_stride_t, p.v_stride_t, BN, valid, tid, 256);
  };
  if (ntiles > 0) load_kv(0);
  cp_async_commit();
  cp_async_wait<1>();
  __syncthreads();

  uint32_t qf[KS][4];
#pragma unroll
  for (int kk = 0; kk < KS; ++kk) load_a_frag<D>(qf[kk], sQ, warp * 16, kk, lane);

  const int g_ = lane >> 2, c_ = lane & 3;
  const int row_lo = warp * 16 + g_, row_hi = row_lo + 8;
  const int tok_lo = row_lo / G, tok_hi = row_hi / G;
  const int tabs_lo = tabs_min + tok_lo, tabs_hi = tabs_min + tok_hi;
  const float c2 = p.sm_scale * 1.4426950408889634f;

  float o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

  for (int it = 0; it < ntiles; ++it) {
    if (it + 1 < ntiles) load_kv(it + 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const uint32_t tK = sK + (it & 1) * BN * D * 2, tV = sV + (it & 1) * BN * D * 2;
    const int kv0 = kv_lo + it * BN;

    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < KS; ++kk) {
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t b[4];
        load_b_frag_nk<D>(b, tK, np * 16, kk, lane);
        mma_bf16(s[2 * np], qf[kk], b[0], b[1]);
        mma_bf16(s[2 * np + 1], qf[kk], b[2], b[3]);
      }
    }
    // ---- scale + mask
    bool full;
    if (MODE == MODE_CMP)
      full = ((kv0 + BN - 1) * st + ks - 1 <= tabs_min) && (kv0 + BN <= kv_hi);
    else
      full = (kv0 + BN - 1 <= tabs_min) && (kv0 >= tabs_max - W) && (kv0 + BN <= kv_hi);
    if (full) {
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        s[nt][0] *= c2; s[nt][1] *= c2; s[nt][2] *= c2; s[nt][3] *= c2;
      }
    } else {
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          int col = kv0 + nt * 8 + 2 * c_ + (e & 1);
          int ta = (e < 2) ? tabs_lo : tabs_hi;
          bool vis;
          if (MODE == MODE_CMP)
            vis = (col * st + ks - 1 <= ta) && (col < kv_hi);
          else
            vis = (col <= ta) && (col >= ta - W) && (col < kv_hi);
          s[nt][e] = vis ? s[nt][e] * c2 : -INFINITY;
        }
      }
    }
    // ---- online softmax
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
    for (int i = 0; i < NT; ++i) {
      o[i][0] *= al_lo; o[i][1] *= al_lo; o[i][2] *= al_hi; o[i][3] *= al_hi;
    }
    // ---- O += P V
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      uint32_t a0 = pack_bf16(s[2 * u][0], s[2 * u][1]), a1 = pack_bf16(s[2 * u][2], s[2 * u][3]);
      uint32_t a2 = pack_bf16(s[2 * u + 1][0], s[2 * u + 1][1]), a3 = pack_bf16(s[2 * u + 1][2], s[2 * u + 1][3]);
#pragma unroll
      for (int np = 0; np < NT / 2; ++np) {
        uint32_t b[4];
        load_b_frag_kn<D>(b, tV, u * 16, np * 16, lane);
        mma_bf16(o[2 * np], a0, a1, a2, a3, b[0], b[1]);
        mma_bf16(o[2 * np + 1], a0, a1, a2, a3, b[2], b[3]);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

  // ---- epilogue: normalise, stage the bf16 tile in the (warp-private) Q rows, write out
  l_lo = warp_sum4(l_lo);
  l_hi = warp_sum4(l_hi);
  float inv_lo = l_lo > 0.f ? 1.f / l_lo : 0.f, inv_hi = l_hi > 0.f ? 1.f / l_hi : 0.f;
  float lse_lo = l_lo > 0.f ? m_lo + log2f(l_lo) : 0.f, lse_hi = l_hi > 0.f ? m_hi + log2f(l_hi) : 0.f;
  __syncwarp();
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    uint32_t lo = pack_bf16(o[nt][0] * inv_lo, o[nt][1] * inv_lo);
    uint32_t hi = pack_bf16(o[nt][2] * inv_hi, o[nt][3] * inv_hi);
    asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(sQ + tile_off<D>(row_lo, nt) + c_ * 4), "r"(lo));
    asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(sQ + tile_off<D>(row_hi, nt) + c_ * 4), "r"(hi));
  }
  __syncwarp();
  {
    __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(p.o) + (int64_t)(pc.q_start + t0) * p.o_stride_t +
                        (int64_t)kh * G * D;
    for (int i = lane; i < 16 * CH; i += 32) {
      int r = warp * 16 + i / CH, c = i % CH;
      int tok = r / G, g = r - tok * G;
      if (tok < ntok) {
        uint4 v;
        asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];\n"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                     : "r"(sQ + tile_off<D>(r, c)));
        *reinterpret_cast<uint4*>(ob + (int64_t)tok * p.o_stride_t + g * D + c * 8) = v;
      }
    }
  }
  if (c_ == 0 && p.lse) {
    if (tok_lo < ntok) {
      int g = row_lo - tok_lo * G;
      p.lse[(int64_t)(pc.q_start + t0 + tok_lo) * p.lse_stride_t + (int64_t)(kh * G + g) * p.lse_stride_h] = lse_lo;
    }
    if (tok_hi < ntok) {
      int g = row_hi - tok_hi * G;
      p.lse[(int64_t)(pc.q_start + t0 + tok_hi) * p.lse_stride_t + (int64_t)(kh * G + g) * p.lse_stride_h] = lse_hi;
    }
  }
}

template <int D, int MODE>
static int launch_dense_fwd(const NsaAttnParams* p, cudaStream_t st, const char* name) {
  const int G = p->QH / p->KH;
  const int TOK = 128 / G;
  size_t smem = (128 + 4 * 64) * D * 2;
  static bool attr_done = false;  // per template instance
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(dense_fwd_kernel<D, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
      set_error("%s: cudaFuncSetAttribute failed: %s", name, cudaGetErrorString(e));
      return NSA_ERR_CUDA;
    }
    attr_done = true;
  }
  dim3 grid((p->meta.max_piece_len + TOK - 1) / TOK, p->meta.n_pieces, p->KH);
  dense_fwd_kernel<D, MODE><<<grid, 256, smem, st>>>(*p);
  return check_launch(name);
}

int check_attn_common(const NsaAttnParams* p, const char* name, bool need_y) {
  NSA_REQUIRE(p && p->q && p->k && p->v && p->o, NSA_ERR_BAD_ARG, "%s: null tensor pointer", name);
  NSA_REQUIRE(p->meta.piece_cu && p->meta.x_cu && (!need_y || p->meta.y_cu), NSA_ERR_BAD_ARG, "%s: null metadata pointer", name);
  NSA_REQUIRE(p->D == 64 || p->D == 128, NSA_ERR_UNSUPPORTED_SHAPE, "%s: head dim %d not supported (64 or 128, qk dim == v dim)", name, p->D);
  NSA_REQUIRE(p->KH > 0 && p->QH % p->KH == 0, NSA_ERR_BAD_ARG, "%s: QH=%d must be a multiple of KH=%d", name, p->QH, p->KH);
  NSA_REQUIRE(p->QH / p->KH <= 128, NSA_ERR_UNSUPPORTED_SHAPE, "%s: more than 128 query heads per kv head", name);
  NSA_REQUIRE(p->hp.kernel_size > 0 && p->hp.stride > 0, NSA_ERR_BAD_ARG, "%s: bad kernel_size/stride", name);
  return NSA_OK;
}

}  // namespace nsa

using namespace nsa;

extern "C" int nsa_cmp_attn_fwd(const NsaAttnParams* p, void* stream) {
  int rc = check_attn_common(p, "cmp_attn_fwd", true);
  if (rc) return rc;
  NSA_REQUIRE(p->lse, NSA_ERR_BAD_ARG, "cmp_attn_fwd: lse is required");
  if (p->meta.n_pieces <= 0 || p->meta.max_piece_len <= 0) return NSA_OK;
  if (p->D == 128) return launch_dense_fwd<128, MODE_CMP>(p, (cudaStream_t)stream, "cmp_attn_fwd");
  return launch_dense_fwd<64, MODE_CMP>(p, (cudaStream_t)stream, "cmp_attn_fwd");
}

extern "C" int nsa_swa_fwd(const NsaAttnParams* p, void* stream) {
  int rc = check_attn_common(p, "swa_fwd", false);
  if (rc) return rc;
  NSA_REQUIRE(p->hp.window >= 0, NSA_ERR_BAD_ARG, "swa_fwd: negative window");
  if (p->meta.n_pieces <= 0 || p->meta.max_piece_len <= 0) return NSA_OK;
  if (p->D == 128) return launch_dense_fwd<128, MODE_SWA>(p, (cudaStream_t)stream, "swa_fwd");
  return launch_dense_fwd<64, MODE_SWA>(p, (cudaStream_t)stream, "swa_fwd");
}
