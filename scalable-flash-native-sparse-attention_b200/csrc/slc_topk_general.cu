// Block-importance scores and top-n selection for ANY kernel_size / stride / block_size (stride a power of two dividing
// both, block_size >= kernel_size), and for the per-row rounding mode of the reference's general path.
//
// The reference's general path is a kernel pair (flash_nsa/ops/topk.py:19-218): the first stores, per (kv head, token,
// compressed row), the probability summed over the kv head's query heads, in half precision unless fp32 was asked for; the
// second pools those rows into selection blocks in fp32 with the weights overlap(row window, block) / stride and picks the
// blocks by repeated arg-max (lowest index on ties).  Here both steps are one kernel and the [KH,T,rows] tensor is never
// written: one warp owns one query token and the query heads of one kv head as the 16 rows of an MMA tile (more than 16
// heads: HG groups of 16, their probabilities summed before the pooling), the 8
// warps of a CTA share the compressed-key tiles in shared memory, and each warp keeps the token's block scores in a
// shared-memory array while it walks the tiles; the selection then runs over that array.
//     quant 0: fp32 everywhere             quant 3: per-row sums rounded to half before pooling (the reference's default here)
//     quant 1 / 2: pooled score (or its cube) rounded to half, as in the 32/16/64 kernel pair
// This is the slow, general kernel: the 32/16/64 configuration that every module of the reference uses runs on the tcgen05
// kernel (slc_topk_tc.cu) or on slc_topk.cu.
#include "nsa_common.cuh"

namespace nsa {

template <int D, int HG>
__global__ void __launch_bounds__(256, 1) slc_topk_general_kernel(NsaTopkParams p, int blk_cap) {
  constexpr int BN = 64, CH = D / 8, KS = D / 16, TOK = 8;
  extern __shared__ __align__(128) unsigned char smem[];
  const uint32_t sQ = smem_u32(smem);
  const uint32_t sK = sQ + HG * 128 * D * 2;
  float* pc_all = reinterpret_cast<float*>(smem + HG * 128 * D * 2 + 2 * BN * D * 2);   // [8 warps][64]: per-row sums of a tile
  float* sc_all = pc_all + 8 * 64;                                                // [8 warps][blk_cap]: block scores

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
  const int ntiles = (nvis_max + BN - 1) / BN;

  const __nv_bfloat16* kbase = reinterpret_cast<const __nv_bfloat16*>(p.ck) + kh * D;
  {
    const __nv_bfloat16* qb = reinterpret_cast<const __nv_bfloat16*>(p.q) + (int64_t)(pc.q_start + t0) * p.q_stride_t + (int64_t)kh * G * D;
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
  if (ntiles > 0) load_k(0);
  cp_async_commit();
  cp_async_wait<0>();
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
  const int n_sel = tok_ok ? min(top_n, nk + 1) : 0;
  const float c2 = p.sm_scale * 1.4426950408889634f;
  float nl_lo[HG], nl_hi[HG];
  bool h_lo[HG], h_hi[HG];
#pragma unroll
  for (int hg = 0; hg < HG; ++hg) {
    h_lo[hg] = tok_ok && 16 * hg + g_ < G;
    h_hi[hg] = tok_ok && 16 * hg + g_ + 8 < G;
    nl_lo[hg] = h_lo[hg] ? -p.lse[q_row * p.lse_stride_t + (int64_t)(kh * G + 16 * hg + g_) * p.lse_stride_h] : 0.f;
    nl_hi[hg] = h_hi[hg] ? -p.lse[q_row * p.lse_stride_t + (int64_t)(kh * G + 16 * hg + g_ + 8) * p.lse_stride_h] : 0.f;
  }

  float* pcw = pc_all + warp * 64;
  float* sc = sc_all + (size_t)warp * blk_cap;
  const int n_blk = min(nk + 1, blk_cap);   // blocks 0..nk can hold visible keys
  for (int i = lane; i < n_blk; i += 32) sc[i] = 0.f;
  __syncwarp();
  const float inv_st = 1.f / (float)st;

  for (int it = 0; it < ntiles; ++it) {
    if (it + 1 < ntiles) load_k(it + 1);
    cp_async_commit();
    const uint32_t tK = sK + (it & 1) * BN * D * 2;
    const int kv0 = it * BN;
    if (tok_ok && kv0 < nvis) {
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
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        float v0 = v0s[nt], v1 = v1s[nt];
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
          v0 += __shfl_xor_sync(0xffffffffu, v0, o);
          v1 += __shfl_xor_sync(0xffffffffu, v1, o);
        }
        if (g_ == nt) {
          pcw[nt * 8 + 2 * c_] = v0;
          pcw[nt * 8 + 2 * c_ + 1] = v1;
        }
      }
      __syncwarp();
      // ---- pool the 64 per-row sums into the blocks their windows overlap (a window spans at most two blocks)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int r = lane + 32 * half, j = kv0 + r;
        if (j < nvis) {
          float v = pcw[r];
          if (p.quant == 3) v = __half2float(__float2half_rn(v));
          const int lo = st * j, hi = lo + ks;
          const int b0 = lo / bs, b1 = (hi - 1) / bs;
          for (int blk = b0; blk <= b1; ++blk) {
            const int ov = min(hi, (blk + 1) * bs) - max(lo, blk * bs);
            if (blk < n_blk) atomicAdd(sc + blk, v * ((float)ov * inv_st));
          }
        }
      }
      __syncwarp();
    }
    cp_async_wait<0>();
    __syncthreads();
  }

  if (!tok_ok) return;
  // ---- rounding of the pooled scores, optional output, forced blocks out of the running
  const int64_t Tq = p.meta.piece_cu[p.meta.n_pieces];
  for (int i = lane; i < n_blk; i += 32) {
    float pv = sc[i];
    if (p.quant == 1) pv = __half2float(__float2half_rn(pv));
    else if (p.quant == 2) pv = __half2float(__float2half_rn(pv * pv * pv));
    if (p.probs && i < (int)p.probs_stride_t) {
      if (p.quant == 0 || p.quant == 3) reinterpret_cast<float*>(p.probs)[((int64_t)kh * Tq + q_row) * p.probs_stride_t + i] = pv;
      else reinterpret_cast<__half*>(p.probs)[((int64_t)kh * Tq + q_row) * p.probs_stride_t + i] = __float2half_rn(pv);
    }
    const bool forced = i < ni || i > nk - nl;
    sc[i] = forced ? -1.f : pv;
  }
  __syncwarp();
  int32_t* out = p.topk + ((int64_t)kh * Tq + q_row) * top_n;
  for (int i = lane; i < top_n; i += 32) {
    int v = p.ignore_index;
    if (i < ni) v = (i <= nk) ? i : p.ignore_index;
    else if (i < ni + nl) v = (i <= nk) ? nk - (i - ni) : p.ignore_index;
    out[i] = v;
  }
  // ---- the free slots: repeated arg-max, ties to the lowest block index
  for (int i = ni + nl; i < n_sel; ++i) {
    float best = -2.f;
    int arg = 0x7fffffff;
    for (int b = lane; b < n_blk; b += 32) {
      const float v = sc[b];
      if (v > best) { best = v; arg = b; }   // ascending b within a lane: the first maximum is kept
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ov > best || (ov == best && oa < arg)) { best = ov; arg = oa; }
    }
    if (lane == 0) {
      out[i] = arg;
      sc[arg] = -1.f;
    }
    __syncwarp();
  }
}

// returns 0 on launch, < 0 on error
int launch_slc_topk_general(const NsaTopkParams* p, cudaStream_t st) {
  const int D = p->D;
  const int blk_cap = (p->meta.x_maxlen > 0 ? (p->meta.x_maxlen + p->hp.block_size - 1) / p->hp.block_size : 0);
  NSA_REQUIRE(blk_cap > 0, NSA_ERR_BAD_ARG, "slc_topk (general sizes): meta.x_maxlen must give the longest sequence");
  const int G = p->QH / p->KH, HG = G <= 16 ? 1 : (G <= 32 ? 2 : 4);
  NSA_REQUIRE(G <= 64, NSA_ERR_UNSUPPORTED_SHAPE, "slc_topk (general sizes): at most 64 query heads per kv head (got %d)", G);
  const size_t fixed = (size_t)HG * 128 * D * 2 + 2 * 64 * D * 2 + 8 * 64 * sizeof(float);
  const size_t smem = fixed + (size_t)8 * blk_cap * sizeof(float);
  NSA_REQUIRE(smem <= 227 * 1024, NSA_ERR_UNSUPPORTED_SHAPE,
              "slc_topk (general sizes): %d selection blocks per sequence exceed what the score arrays in shared memory hold (%d)",
              blk_cap, (int)((227 * 1024 - fixed) / (8 * sizeof(float))));
  dim3 grid((p->meta.max_piece_len + 7) / 8, p->meta.n_pieces, p->KH);
  auto go = [&](auto kernel) -> cudaError_t {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) kernel<<<grid, 256, smem, st>>>(*p, blk_cap);
    return e;
  };
  cudaError_t e;
  if (D == 128) e = HG == 1 ? go(slc_topk_general_kernel<128, 1>) : (HG == 2 ? go(slc_topk_general_kernel<128, 2>) : go(slc_topk_general_kernel<128, 4>));
  else e = HG == 1 ? go(slc_topk_general_kernel<64, 1>) : (HG == 2 ? go(slc_topk_general_kernel<64, 2>) : go(slc_topk_general_kernel<64, 4>));
  if (e != cudaSuccess) {
    set_error("slc_topk (general sizes): cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
    return NSA_ERR_CUDA;
  }
  return check_launch("slc_topk (general sizes)");
}

}  // namespace nsa
