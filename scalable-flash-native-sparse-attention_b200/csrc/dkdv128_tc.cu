// dK/dV of the compressed and sliding-window branches with 128-row K/V tiles (tcgen05 + tensor memory, TMA loads).
//
// These two branches read their queries from a CONTIGUOUS token range, so a query tile is one TMA box
// (64 d) x (G heads) x (64/G tokens) per 64-wide slab, and a 128-row K/V tile halves the number of times every Q/dO row is
// streamed compared with a 64-row tile.  The MMA M dimension is the K/V row, so thread i of the compute warp group owns
// K/V row i (tensor-memory lane i) and the gradients accumulate un-transposed:
//     S^T  = K Q^T           M = 128 keys, N = 64 query rows   (A = K tile, B = Q tile, both K-major from shared memory)
//     dP^T = V dO^T
//     P^T  = exp2(S^T*c - lse[col]),  dS^T = P^T * (dP^T - delta[col])  -> bf16, written over S^T / dP^T in tensor memory
//     dV  += P^T dO          A = P^T from tensor memory, B = dO tile read MN-major
//     dK  += dS^T Q
// S^T/dP^T are double-buffered in tensor memory (2 x 128 columns) next to dV and dK (2 x 128 columns); Q/dO tiles go
// through a 3-stage shared-memory ring filled by TMA.  Warp 8 (one lane) issues all TMA loads and MMAs; warps 0-3 and
// 4-7 are two compute groups that take the even and the odd query tiles, so the softmax arithmetic of one tile overlaps the
// tensor-memory round trips of the other.
#include "tma.cuh"

namespace nsa {

constexpr int MODE_CMP = 0;
constexpr int MODE_SWA = 1;

template <int D, int MODE>
__global__ void __launch_bounds__(288, 1)
    dkdv128_tc_kernel(NsaAttnParams p, DkdvLaunch L, const __grid_constant__ CUtensorMap tmq, const __grid_constant__ CUtensorMap tmo,
                      const __grid_constant__ CUtensorMap tmk, const __grid_constant__ CUtensorMap tmv) {
  using namespace tc;
  constexpr int BK = 128, BQ = 64, NS = 3, SLABS = D / 64;
  constexpr uint32_t KV_BYTES = BK * D * 2, Q_BYTES = BQ * D * 2, K_SLAB = BK * 128, Q_SLAB = BQ * 128;
  constexpr uint32_t IDESC_SD = make_idesc(BK, BQ, false), IDESC_KV = make_idesc(BK, D, true);
  constexpr uint32_t TM_DV = 256, TM_DK = 384;

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  const uint32_t sK = base, sV = sK + KV_BYTES;
  const uint32_t sQ = sV + KV_BYTES;            // NS stages
  const uint32_t sO = sQ + NS * Q_BYTES;        // NS stages
  const uint32_t meta_off = 2 * KV_BYTES + 2 * NS * Q_BYTES;
  float* sLse = reinterpret_cast<float*>(smem_raw + meta_off);   // [4][64]: two buffers per compute warp group
  float* sDl = sLse + 4 * BQ;
  int* sTa = reinterpret_cast<int*>(sDl + 4 * BQ);
  const uint32_t bars = base + meta_off + 12 * BQ * 4;
  const uint32_t kv_full = bars, q_full = bars + 8, q_free = q_full + 8 * NS, sd_full = q_free + 8 * NS, pds_full = sd_full + 16,
                 done = pds_full + 16, tm_slot = done + 8;

  const int tid = threadIdx.x, warp = tid >> 5;
  const int G = p.QH / p.KH;
  const int TOKQ = BQ / G;
  const int ks = p.hp.kernel_size, st = p.hp.stride, W = p.hp.window;
  const int kh = blockIdx.z % p.KH;
  const Piece pc = load_piece(p.meta, blockIdx.z / p.KH);
  int k0, kv_rows, r_lo, r_hi;
  int64_t kv_bos;
  if (MODE == MODE_CMP) {
    k0 = blockIdx.x * BK;
    kv_bos = pc.y_bos;
    kv_rows = min(BK, pc.y_len - k0);
    int first = max(0, k0 * st + ks - 1 - pc.off);
    r_lo = max(first, (int)blockIdx.y * L.q_chunk);
    r_hi = min(pc.len, ((int)blockIdx.y + 1) * L.q_chunk);
  } else {
    k0 = (max(0, pc.off - W) / BK) * BK + blockIdx.x * BK;
    kv_bos = pc.x_bos;
    kv_rows = min(BK, pc.x_len - k0);
    r_lo = max(k0, pc.off) - pc.off;
    r_hi = min(k0 + BK - 1 + W, pc.off + pc.len - 1) + 1 - pc.off;
  }
  if (kv_rows <= 0 || r_hi <= r_lo) return;
  if (base & 1023u) {
    if (tid == 0 && p.status) atomicOr(p.status, 8);
    return;
  }
  const int n_it = (r_hi - r_lo + TOKQ - 1) / TOKQ;

  if (tid == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < NS; ++s) {
      mbar_init(q_full + 8 * s, 1);
      mbar_init(q_free + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(sd_full + 8 * b, 1);
      mbar_init(pds_full + 8 * b, 128);
    }
    mbar_init(done, 1);
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc(tm_slot, 512);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  uint32_t tmem;
  asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(tmem) : "r"(tm_slot));
  int budget = kWaitBudget;
  bool timed_out = false;

  if (warp == 8) {
    if ((tid & 31) == 0) {
      // ============================================ producer: TMA loads + MMA issue
      tma::expect_tx(kv_full, 2 * KV_BYTES);
#pragma unroll
      for (int sl = 0; sl < SLABS; ++sl) {
        tma::load_3d(sK + sl * K_SLAB, &tmk, sl * 64, kh, (int)(kv_bos + k0), kv_full);
        tma::load_3d(sV + sl * K_SLAB, &tmv, sl * 64, kh, (int)(kv_bos + k0), kv_full);
      }
      int nl_ = 0;
      auto top_up = [&](int upto) {
        while (nl_ < n_it && nl_ < upto) {
          const int s = nl_ % NS;
          if (nl_ >= NS && !mbar_wait(q_free + 8 * s, ((nl_ / NS) - 1) & 1, &budget)) timed_out = true;
          tma::expect_tx(q_full + 8 * s, 2 * Q_BYTES);
          const int row = pc.q_start + r_lo + nl_ * TOKQ;
#pragma unroll
          for (int sl = 0; sl < SLABS; ++sl) {
            tma::load_3d(sQ + s * Q_BYTES + sl * Q_SLAB, &tmq, sl * 64, kh * G, row, q_full + 8 * s);
            tma::load_3d(sO + s * Q_BYTES + sl * Q_SLAB, &tmo, sl * 64, kh * G, row, q_full + 8 * s);
          }
          ++nl_;
        }
      };
      top_up(NS - 1);
      if (!mbar_wait(kv_full, 0, &budget)) timed_out = true;
      auto issue_kv = [&](int i) {  // dV += P^T dO, dK += dS^T Q for tile i
        const int s = i % NS, b = i & 1;
        if (!mbar_wait(pds_full + 8 * b, (i >> 1) & 1, &budget)) timed_out = true;
        fence_after_sync();
#pragma unroll
        for (int u = 0; u < BQ / 16; ++u)
          mma_ts(tmem + TM_DV, tmem + 128 * b + u * 8, desc_mnmajor(sO + s * Q_BYTES + u * 2048, Q_SLAB), IDESC_KV, (i > 0 || u > 0));
#pragma unroll
        for (int u = 0; u < BQ / 16; ++u)
          mma_ts(tmem + TM_DK, tmem + 128 * b + 64 + u * 8, desc_mnmajor(sQ + s * Q_BYTES + u * 2048, Q_SLAB), IDESC_KV, (i > 0 || u > 0));
        mma_commit(q_free + 8 * s);
      };
      for (int i = 0; i < n_it; ++i) {
        const int s = i % NS, b = i & 1;
        if (!mbar_wait(q_full + 8 * s, (i / NS) & 1, &budget)) timed_out = true;
        fence_after_sync();
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t ao = (k >> 2) * K_SLAB + (k & 3) * 32, bo = (k >> 2) * Q_SLAB + (k & 3) * 32;
          mma_ss(tmem + 128 * b, desc_kmajor(sK + ao), desc_kmajor(sQ + s * Q_BYTES + bo), IDESC_SD, k > 0);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t ao = (k >> 2) * K_SLAB + (k & 3) * 32, bo = (k >> 2) * Q_SLAB + (k & 3) * 32;
          mma_ss(tmem + 128 * b + 64, desc_kmajor(sV + ao), desc_kmajor(sO + s * Q_BYTES + bo), IDESC_SD, k > 0);
        }
        mma_commit(sd_full + 8 * b);
        if (i > 0) issue_kv(i - 1);
        top_up(i + NS);
      }
      issue_kv(n_it - 1);
      mma_commit(done);
    }
  } else {
    // ============================================ two compute warp groups: group w takes the tiles of parity w;
    // thread = K/V row (tensor-memory lane)
    const int t = tid & 127, wg = warp >> 2;
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const int key = k0 + t;
    const bool key_ok = t < kv_rows;
    const float c2 = p.sm_scale * 1.4426950408889634f;
    // column metadata of a tile: -lse, delta, absolute position (-1 = no such query row); loaded one tile ahead
    float m_lse = 0.f, m_dl = 0.f;
    int m_ta = -1;
    auto fetch_meta = [&](int i) {
      m_lse = 0.f; m_dl = 0.f; m_ta = -1;
      if (t < BQ && i < n_it) {
        const int n = t / G, g = t - n * G;
        const int tok = r_lo + i * TOKQ + n;
        if (n < TOKQ && tok < r_hi) {
          const int64_t q_row = (int64_t)pc.q_start + tok;
          const int64_t a = q_row * p.lse_stride_t + (int64_t)(kh * G + g) * p.lse_stride_h;
          m_lse = -p.lse[a];
          m_dl = p.delta[a];
          m_ta = pc.off + tok;
        }
      }
    };
    fetch_meta(wg);
    int j = 0;
    for (int i = wg; i < n_it; i += 2, ++j) {
      const int b = wg, mb = 2 * wg + (j & 1);   // mb: metadata buffer, last read two of this group's tiles ago
      if (t < BQ) {
        sLse[mb * BQ + t] = m_lse;
        sDl[mb * BQ + t] = m_dl;
        sTa[mb * BQ + t] = m_ta;
      }
      fetch_meta(i + 2);
      named_barrier(1 + wg, 128);
      // every (key, query) pair of the tile visible?  then the position test is skipped
      const int tok0 = r_lo + i * TOKQ, ta_min = pc.off + tok0, ta_max = ta_min + TOKQ - 1;
      bool full = kv_rows == BK && tok0 + TOKQ <= r_hi;
      if (MODE == MODE_CMP) full = full && ((k0 + BK - 1) * st + ks - 1 <= ta_min);
      else full = full && (k0 + BK - 1 <= ta_min) && (ta_max - k0 <= W);
      if (!mbar_wait(sd_full + 8 * b, (i >> 1) & 1, &budget)) timed_out = true;
      fence_after_sync();
      const float4* lse4 = reinterpret_cast<const float4*>(sLse + mb * BQ);
      const float4* dl4 = reinterpret_cast<const float4*>(sDl + mb * BQ);
      const int4* ta4 = reinterpret_cast<const int4*>(sTa + mb * BQ);
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t sv[32], dv[32], pp[16], dd[16];
        tmem_ld32(lane_base + 128 * b + half * 32, sv);
        tmem_ld32(lane_base + 128 * b + 64 + half * 32, dv);
        wait_ld();
        if (full) {
#pragma unroll
          for (int c = 0; c < 32; c += 4) {
            const float4 nl = lse4[half * 8 + (c >> 2)], dl = dl4[half * 8 + (c >> 2)];
            const float x0 = fast_exp2(fmaf(__uint_as_float(sv[c]), c2, nl.x));
            const float x1 = fast_exp2(fmaf(__uint_as_float(sv[c + 1]), c2, nl.y));
            const float x2 = fast_exp2(fmaf(__uint_as_float(sv[c + 2]), c2, nl.z));
            const float x3 = fast_exp2(fmaf(__uint_as_float(sv[c + 3]), c2, nl.w));
            pp[c >> 1] = pack_bf16(x0, x1);
            pp[(c >> 1) + 1] = pack_bf16(x2, x3);
            dd[c >> 1] = pack_bf16(x0 * (__uint_as_float(dv[c]) - dl.x), x1 * (__uint_as_float(dv[c + 1]) - dl.y));
            dd[(c >> 1) + 1] = pack_bf16(x2 * (__uint_as_float(dv[c + 2]) - dl.z), x3 * (__uint_as_float(dv[c + 3]) - dl.w));
          }
        } else {
          // visible iff lo <= ta <= hi for this thread's key
          int lo, hi;
          if (MODE == MODE_CMP) { lo = key * st + ks - 1; hi = 0x7fffffff; }
          else { lo = key; hi = key + W; }
          if (!key_ok) lo = 0x7fffffff;
#pragma unroll
          for (int c = 0; c < 32; c += 4) {
            const float4 nl = lse4[half * 8 + (c >> 2)], dl = dl4[half * 8 + (c >> 2)];
            const int4 ta = ta4[half * 8 + (c >> 2)];
            const float x0 = (ta.x >= lo && ta.x <= hi) ? fast_exp2(fmaf(__uint_as_float(sv[c]), c2, nl.x)) : 0.f;
            const float x1 = (ta.y >= lo && ta.y <= hi) ? fast_exp2(fmaf(__uint_as_float(sv[c + 1]), c2, nl.y)) : 0.f;
            const float x2 = (ta.z >= lo && ta.z <= hi) ? fast_exp2(fmaf(__uint_as_float(sv[c + 2]), c2, nl.z)) : 0.f;
            const float x3 = (ta.w >= lo && ta.w <= hi) ? fast_exp2(fmaf(__uint_as_float(sv[c + 3]), c2, nl.w)) : 0.f;
            pp[c >> 1] = pack_bf16(x0, x1);
            pp[(c >> 1) + 1] = pack_bf16(x2, x3);
            dd[c >> 1] = pack_bf16(x0 * (__uint_as_float(dv[c]) - dl.x), x1 * (__uint_as_float(dv[c + 1]) - dl.y));
            dd[(c >> 1) + 1] = pack_bf16(x2 * (__uint_as_float(dv[c + 2]) - dl.z), x3 * (__uint_as_float(dv[c + 3]) - dl.w));
          }
        }
        tmem_st16(lane_base + 128 * b + half * 16, pp);        // P^T over the consumed S^T columns
        tmem_st16(lane_base + 128 * b + 64 + half * 16, dd);   // dS^T over dP^T
      }
      wait_st();
      fence_before_sync();
      mbar_arrive(pds_full + 8 * b);
    }
    if (!mbar_wait(done, 0, &budget)) timed_out = true;
    fence_after_sync();
    // ---- my K/V row: group 0 adds dV, group 1 adds dK
    float* dst = (wg == 0 ? p.dv + (kv_bos + k0 + t) * p.dv_stride_t : p.dk + (kv_bos + k0 + t) * p.dk_stride_t) + kh * D;
    const float sc = wg == 0 ? 1.f : p.sm_scale;
    const uint32_t src = lane_base + (wg == 0 ? TM_DV : TM_DK);
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
      uint32_t v[32];
      tmem_ld32(src + c * 32, v);
      wait_ld();
      if (key_ok) {
#pragma unroll
        for (int q4 = 0; q4 < 8; ++q4)
          atomicAdd(reinterpret_cast<float4*>(dst + c * 32 + q4 * 4),
                    make_float4(__uint_as_float(v[q4 * 4]) * sc, __uint_as_float(v[q4 * 4 + 1]) * sc, __uint_as_float(v[q4 * 4 + 2]) * sc,
                                __uint_as_float(v[q4 * 4 + 3]) * sc));
      }
    }
  }
  if (timed_out && p.status) atomicOr(p.status, 64);
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

// returns 1 when the configuration is not covered (the 64-row-tile kernel then runs), 0 on launch, < 0 on error
template <int D, int MODE>
static int launch128(const NsaAttnParams* p, cudaStream_t st, const char* name, int q_chunk) {
  const int G = p->QH / p->KH;
  if (G > 64 || (64 % G) != 0) return 1;
  if (p->meta.kv_table || p->meta.cmp_table || p->n_k_rows <= 0 || p->n_q_rows <= 0) return 1;
  if (((uintptr_t)p->q | (uintptr_t)p->dout | (uintptr_t)p->k | (uintptr_t)p->v) & 15) return 1;
  if ((p->q_stride_t * 2) % 16 || (p->do_stride_t * 2) % 16 || (p->k_stride_t * 2) % 16 || (p->v_stride_t * 2) % 16) return 1;
  if ((p->dk_stride_t % 4) || (p->dv_stride_t % 4) || (((uintptr_t)p->dk | (uintptr_t)p->dv) & 15)) return 1;
  CUtensorMap tmq, tmo, tmk, tmv;
  const int TOKQ = 64 / G;
  if (!tma::make_map(&tmq, p->q, p->n_q_rows, p->QH, D, p->q_stride_t, TOKQ, G) ||
      !tma::make_map(&tmo, p->dout, p->n_q_rows, p->QH, D, p->do_stride_t, TOKQ, G) ||
      !tma::make_map(&tmk, p->k, p->n_k_rows, p->KH, D, p->k_stride_t, 128, 1) ||
      !tma::make_map(&tmv, p->v, p->n_k_rows, p->KH, D, p->v_stride_t, 128, 1)) {
    set_error("%s: cuTensorMapEncodeTiled failed or is unavailable", name);
    return NSA_ERR_CUDA;
  }
  size_t smem = (size_t)(2 * 128 + 6 * 64) * D * 2 + 12 * 64 * 4 + 256;
  cudaError_t e = cudaFuncSetAttribute(dkdv128_tc_kernel<D, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_error("%s: cudaFuncSetAttribute failed: %s", name, cudaGetErrorString(e));
    return NSA_ERR_CUDA;
  }
  DkdvLaunch L{q_chunk, 1, nullptr};
  dim3 grid;
  if (MODE == MODE_CMP) grid = dim3((p->meta.y_maxlen + 127) / 128, (p->meta.max_piece_len + q_chunk - 1) / q_chunk, p->meta.n_pieces * p->KH);
  else grid = dim3((p->meta.max_piece_len + p->hp.window + 127) / 128 + 1, 1, p->meta.n_pieces * p->KH);
  dkdv128_tc_kernel<D, MODE><<<grid, 288, smem, st>>>(*p, L, tmq, tmo, tmk, tmv);
  return check_launch(name);
}

int launch_dkdv128(const NsaAttnParams* p, cudaStream_t st, const char* name, bool cmp, int q_chunk) {
  if (p->D == 128) return cmp ? launch128<128, MODE_CMP>(p, st, name, q_chunk) : launch128<128, MODE_SWA>(p, st, name, q_chunk);
  return cmp ? launch128<64, MODE_CMP>(p, st, name, q_chunk) : launch128<64, MODE_SWA>(p, st, name, q_chunk);
}

}  // namespace nsa
