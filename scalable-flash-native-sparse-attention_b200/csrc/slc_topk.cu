// Block-importance scores and top-n selection, fused (no [KH,T,blocks] score tensor is materialised).
//
// One warp owns one query token; the query heads of one kv head are the 16 rows of an MMA tile, taken 16 at a time
// (HG head groups: the probabilities of all groups are summed before the pooling, so the selection is shared by every
// head of the kv head).  The 8 warps of a CTA (8 consecutive tokens) share the compressed-key tiles in shared memory.
// Per 64 compressed rows:  P_cmp[j] = sum_heads exp2(q.k_j*c - lse_head)  (0 where row j is not yet visible),
// pooled into 16 selection blocks  P_slc[b] = P_cmp[4b-1] + 2(P_cmp[4b]+P_cmp[4b+1]+P_cmp[4b+2]) + P_cmp[4b+3],
// and the warp keeps a running, descending list of the best free blocks (ties: lower block index first).
// The forced blocks (first num_init, last num_local up to the query's own block) never enter the list.
#include "nsa_common.cuh"

namespace nsa {

template <int D, int HG>
__global__ void __launch_bounds__(256, HG == 1 ? 2 : 1) slc_topk_kernel(NsaTopkParams p) {
  constexpr int BN = 64, CH = D / 8, KS = D / 16, TOK = 8;
  extern __shared__ __align__(128) unsigned char smem[];
  const uint32_t sQ = smem_u32(smem);                 // [HG][8 tokens x 16 heads][D]
  const uint32_t sK = sQ + HG * 128 * D * 2;
  float* pc_all = reinterpret_cast<float*>(smem + HG * 128 * D * 2 + 2 * BN * D * 2);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = p.QH / p.KH;
  const int tile = gridDim.x - 1 - blockIdx.x;
  const int kh = blockIdx.z;
  const Piece pc = load_piece(p.meta, blockIdx.y);
  const int t0 = tile * TOK;
  if (t0 >= pc.len) return;
  const int ntok = min(TOK, pc.len - t0);
  const int ks = p.hp.kernel_size, st = p.hp.stride, bs = p.hp.block_size;
  const int top_n = p.hp.top_n, ni = p.hp.num_init, nl = p.hp.num_local;
  const int tabs_max = pc.off + t0 + ntok - 1;
  const int nvis_max = (tabs_max >= ks - 1) ? min(pc.y_len, (tabs_max - (ks - 1)) / st + 1) : 0;
  const int ntiles = max(1, max((nvis_max + BN - 1) / BN, (max(tabs_max, 0) / bs + 1 + 15) / 16));

  const __nv_bfloat16* kbase = reinterpret_cast<const __nv_bfloat16*>(p.ck) + kh * D;
  {
    const __nv_bfloat16* qb = reinterpret_cast<const __nv_bfloat16*>(p.q) + (int64_t)(pc.q_start + t0) * p.q_stride_t +
                              (int64_t)kh * G * D;
    for (int i = tid; i < HG * 128 * CH; i += 256) {
      int hg = i / (128 * CH), j = i - hg * 128 * CH;
      int r = j / CH, c = j % CH;
      int tok = r >> 4, g = 16 * hg + (r & 15);
      bool ok = tok < ntok && g < G;
      const __nv_bfloat16* src = qb + (ok ? (int64_t)tok * p.q_stride_t + g * D : 0) + c * 8;
      cp_async16(sQ + hg * 128 * D * 2 + tile_off<D>(r, c), src, ok);
    }
    cp_async_commit();
  }
  auto load_k = [&](int it) {
    int kv0 = it * BN;
    int valid = max(0, min(BN, pc.y_len - kv0));
    const uint32_t dst = sK + (it & 1) * BN * D * 2;
    for (int i = tid; i < BN * CH; i += 256) {
      int r = i / CH, c = i % CH;
      bool ok = r < valid;
      cp_async16(dst + tile_off<D>(r, c), kbase + (ok ? cmp_row(pc, kv0 + r) : 0) * p.ck_stride_t + c * 8, ok);
    }
  };
  load_k(0);
  cp_async_commit();
  cp_async_wait<1>();
  __syncthreads();

  uint32_t qf[KS][4];   // one head group: loaded once; several: re-read from shared memory for every key tile
  if (HG == 1) {
#pragma unroll
    for (int kk = 0; kk < KS; ++kk) load_a_frag<D>(qf[kk], sQ, warp * 16, kk, lane);
  }

  const int g_ = lane >> 2, c_ = lane & 3;
  const bool tok_ok = warp < ntok;
  const int t_abs = pc.off + t0 + warp;
  const int64_t q_row = pc.q_start + t0 + warp;
  const int nvis = (tok_ok && t_abs >= ks - 1) ? min(pc.y_len, (t_abs - (ks - 1)) / st + 1) : 0;
  const int nk = t_abs >= 0 ? t_abs / bs : -1;  // a padded row (empty sequence) selects nothing
  const int n_free = tok_ok ? max(0, min(top_n, nk + 1) - ni - nl) : 0;
  const float c2 = p.sm_scale * 1.4426950408889634f;
  // -lse of this thread's two rows of every head group (heads 16hg + g_ and + 8); rows beyond G contribute nothing
  float nl_lo[HG], nl_hi[HG];
  bool h_lo[HG], h_hi[HG];
#pragma unroll
  for (int hg = 0; hg < HG; ++hg) {
    h_lo[hg] = tok_ok && 16 * hg + g_ < G;
    h_hi[hg] = tok_ok && 16 * hg + g_ + 8 < G;
    nl_lo[hg] = h_lo[hg] ? -p.lse[q_row * p.lse_stride_t + (int64_t)(kh * G + 16 * hg + g_) * p.lse_stride_h] : 0.f;
    nl_hi[hg] = h_hi[hg] ? -p.lse[q_row * p.lse_stride_t + (int64_t)(kh * G + 16 * hg + g_ + 8) * p.lse_stride_h] : 0.f;
  }

  float* pcw = pc_all + warp * 72;  // [0] = carry (compressed row kv0-1), [1..64] = this tile
  float my_v = -1.f;                // running list entry of this lane (lanes < n_free)
  int my_i = p.ignore_index;
  if (lane == 0) pcw[64] = 0.f;
  __syncwarp();

  for (int it = 0; it < ntiles; ++it) {
    if (it + 1 < ntiles) load_k(it + 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const uint32_t tK = sK + (it & 1) * BN * D * 2;
    const int kv0 = it * BN;
    if (tok_ok) {
      float v0s[8], v1s[8];   // per compressed row: probabilities summed over the heads of all groups
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) v0s[nt] = v1s[nt] = 0.f;
#pragma unroll
      for (int hg = 0; hg < HG; ++hg) {
        if (HG > 1) {
#pragma unroll
          for (int kk = 0; kk < KS; ++kk) load_a_frag<D>(qf[kk], sQ + hg * 128 * D * 2, warp * 16, kk, lane);
        }
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
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
          int col = kv0 + nt * 8 + 2 * c_;
          float e0 = (h_lo[hg] && col < nvis) ? fast_exp2(fmaf(s[nt][0], c2, nl_lo[hg])) : 0.f;
          float e1 = (h_lo[hg] && col + 1 < nvis) ? fast_exp2(fmaf(s[nt][1], c2, nl_lo[hg])) : 0.f;
          float e2 = (h_hi[hg] && col < nvis) ? fast_exp2(fmaf(s[nt][2], c2, nl_hi[hg])) : 0.f;
          float e3 = (h_hi[hg] && col + 1 < nvis) ? fast_exp2(fmaf(s[nt][3], c2, nl_hi[hg])) : 0.f;
          v0s[nt] += e0 + e2;
          v1s[nt] += e1 + e3;
        }
      }
      if (lane == 0) pcw[0] = pcw[64];
      __syncwarp();
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        float v0 = v0s[nt], v1 = v1s[nt];
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
          v0 += __shfl_xor_sync(0xffffffffu, v0, o);
          v1 += __shfl_xor_sync(0xffffffffu, v1, o);
        }
        if (g_ == nt) {
          pcw[1 + nt * 8 + 2 * c_] = v0;
          pcw[2 + nt * 8 + 2 * c_] = v1;
        }
      }
      __syncwarp();
      // ---- pool 4 -> 1 (+ the row before) and quantise
      float val = -1.f;
      int blk = it * 16 + lane;
      bool cand = false;
      if (lane < 16) {
        float a = pcw[4 * lane + 1], b2 = pcw[4 * lane + 2], c3 = pcw[4 * lane + 3], d4 = pcw[4 * lane + 4];
        float pv = pcw[4 * lane] + ((2.f * a + 2.f * b2) + (2.f * c3 + d4));
        if (p.quant == 1) pv = __half2float(__float2half_rn(pv));
        else if (p.quant == 2) pv = __half2float(__float2half_rn(pv * pv * pv));
        val = pv;
        cand = (blk >= ni) && (blk <= nk - nl);
        if (p.probs && blk < (int)p.probs_stride_t) {
          if (p.quant == 0)
            reinterpret_cast<float*>(p.probs)[((int64_t)kh * p.meta.piece_cu[p.meta.n_pieces] + q_row) * p.probs_stride_t + blk] = pv;
          else
            reinterpret_cast<__half*>(p.probs)[((int64_t)kh * p.meta.piece_cu[p.meta.n_pieces] + q_row) * p.probs_stride_t + blk] =
                __float2half_rn(pv);
        }
      }
      // ---- merge the candidates into the running list
      if (n_free > 0) {
        float thr = __shfl_sync(0xffffffffu, my_v, n_free - 1);
        unsigned mask = __ballot_sync(0xffffffffu, cand && val > thr);
        while (mask) {
          int j = __ffs(mask) - 1;
          mask &= mask - 1;
          float cv = __shfl_sync(0xffffffffu, val, j);
          int ci = __shfl_sync(0xffffffffu, blk, j);
          unsigned ge = __ballot_sync(0xffffffffu, lane < n_free && my_v >= cv);
          int pos = __popc(ge);
          float uv = __shfl_up_sync(0xffffffffu, my_v, 1);
          int ui = __shfl_up_sync(0xffffffffu, my_i, 1);
          if (pos < n_free) {
            if (lane > pos && lane < n_free) {
              my_v = uv;
              my_i = ui;
            } else if (lane == pos) {
              my_v = cv;
              my_i = ci;
            }
          }
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

  const int r = lane - ni - nl;
  const int li = __shfl_sync(0xffffffffu, my_i, r >= 0 ? r : 0);
  if (tok_ok && lane < top_n) {
    int out;
    if (lane < ni)
      out = (lane <= nk) ? lane : p.ignore_index;
    else if (lane < ni + nl)
      out = (lane <= nk) ? nk - (lane - ni) : p.ignore_index;
    else
      out = (r < n_free) ? li : p.ignore_index;
    int64_t Tq = p.meta.piece_cu[p.meta.n_pieces];
    p.topk[((int64_t)kh * Tq + q_row) * top_n + lane] = out;
  }
}

}  // namespace nsa

using namespace nsa;

namespace nsa {
int launch_slc_topk_tc(const NsaTopkParams* p, int64_t q_rows, int64_t ck_rows, cudaStream_t st);  // slc_topk_tc.cu
int launch_slc_topk_general(const NsaTopkParams* p, cudaStream_t st);                               // slc_topk_general.cu
}

extern "C" int nsa_slc_topk(const NsaTopkParams* p, void* stream) {
  NSA_REQUIRE(p && p->q && p->ck && p->lse && p->topk, NSA_ERR_BAD_ARG, "slc_topk: null tensor pointer");
  NSA_REQUIRE(p->meta.piece_cu && p->meta.x_cu && p->meta.y_cu, NSA_ERR_BAD_ARG, "slc_topk: null metadata pointer");
  NSA_REQUIRE(p->D == 64 || p->D == 128, NSA_ERR_UNSUPPORTED_SHAPE, "slc_topk: head dim %d not supported (64 or 128)", p->D);
  NSA_REQUIRE(p->KH > 0 && p->QH % p->KH == 0, NSA_ERR_BAD_ARG, "slc_topk: QH=%d must be a multiple of KH=%d", p->QH, p->KH);
  NSA_REQUIRE(p->hp.kernel_size > 0 && p->hp.stride > 0 && p->hp.block_size > 0, NSA_ERR_BAD_ARG,
              "slc_topk: kernel_size, stride, block_size must be positive (got %d/%d/%d)", p->hp.kernel_size, p->hp.stride, p->hp.block_size);
  NSA_REQUIRE(p->hp.top_n >= 1, NSA_ERR_UNSUPPORTED_SHAPE, "slc_topk: top_n=%d must be positive", p->hp.top_n);
  NSA_REQUIRE(p->hp.num_init >= 0 && p->hp.num_local >= 0 && p->hp.num_init + p->hp.num_local <= p->hp.top_n, NSA_ERR_BAD_ARG,
              "slc_topk: num_init + num_local exceeds top_n");
  NSA_REQUIRE(p->quant >= 0 && p->quant <= 3, NSA_ERR_BAD_ARG, "slc_topk: quant=%d", p->quant);
  NSA_REQUIRE(!p->meta.cmp_table || (p->meta.page_size > 0 && (p->meta.page_size & (p->meta.page_size - 1)) == 0),
              NSA_ERR_UNSUPPORTED_SHAPE, "slc_topk: page_size=%d must be a power of two", p->meta.page_size);
  if (p->meta.n_pieces <= 0 || p->meta.max_piece_len <= 0) return NSA_OK;
  const bool std_sizes = p->hp.kernel_size == 32 && p->hp.stride == 16 && p->hp.block_size == 64;
  if (!std_sizes || p->quant == 3 || p->hp.top_n > 32) {
    // any other compression / block geometry, the per-row rounding mode, or a long list: the general kernel
    return launch_slc_topk_general(p, (cudaStream_t)stream);
  }
  if (p->q_rows > 0 && p->ck_rows > 0 && p->QH / p->KH <= 64) {
    int rc = launch_slc_topk_tc(p, p->q_rows, p->ck_rows, (cudaStream_t)stream);
    if (rc <= 0) return rc;
  }
  const int G = p->QH / p->KH, HG = G <= 16 ? 1 : (G <= 32 ? 2 : 4);
  NSA_REQUIRE(G <= 64, NSA_ERR_UNSUPPORTED_SHAPE, "slc_topk: at most 64 query heads per kv head (got %d)", G);
  const int D = p->D;
  size_t smem = (size_t)HG * 128 * D * 2 + 2 * 64 * D * 2 + 8 * 72 * sizeof(float);
  dim3 grid((p->meta.max_piece_len + 7) / 8, p->meta.n_pieces, p->KH);
  auto go = [&](auto kernel) -> cudaError_t {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) kernel<<<grid, 256, smem, (cudaStream_t)stream>>>(*p);
    return e;
  };
  cudaError_t e;
  if (D == 128) e = HG == 1 ? go(slc_topk_kernel<128, 1>) : (HG == 2 ? go(slc_topk_kernel<128, 2>) : go(slc_topk_kernel<128, 4>));
  else e = HG == 1 ? go(slc_topk_kernel<64, 1>) : (HG == 2 ? go(slc_topk_kernel<64, 2>) : go(slc_topk_kernel<64, 4>));
  if (e != cudaSuccess) {
    set_error("slc_topk: cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
    return NSA_ERR_CUDA;
  }
  return check_launch("slc_topk");
}
