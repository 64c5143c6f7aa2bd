// dK/dV of the compressed and sliding-window branches with 128-row K/V tiles (tcgen05 + tensor memory, TMA loads).
//
// These two branches read their queries from a CONTIGUOUS token range, so a query tile is one TMA box
// (64 d) x (G heads) x (128/G tokens) per 64-wide slab.  The MMA M dimension is the K/V row, so thread i of a compute
// warp group owns K/V row i (tensor-memory lane i) and the gradients accumulate un-transposed:
//     S^T  = K Q^T           M = 128 keys, N = 128 query rows  (A = K tile, B = Q tile, both K-major from shared memory)
//     dP^T = V dO^T
//     P^T  = exp2(S^T*c - lse[col]),  dS^T = P^T * (dP^T - delta[col])  -> bf16, written over S^T / dP^T in tensor memory
//     dV  += P^T dO          A = P^T from tensor memory, B = dO tile read MN-major
//     dK  += dS^T Q
// N = 128 halves the shared-memory reads per query row of the two score products (the A tile is re-read by every MMA).
// Tensor memory holds S^T, dP^T, dV, dK (4 x 128 columns), so the products of one tile are ordered
//     S^T(i) | dK(i-1) | dP^T(i) | dV(i)     with exp2 of tile i running under dK(i-1) and dP^T(i), and dS^T under dV(i).
// Warp 8 (one lane) issues the MMAs, warp 9 (one lane) the TMA loads; warps 0-3 and 4-7 are two compute groups that take the query columns
// 0-63 and 64-127 of every tile.  Q/dO tiles go through a 2-stage shared-memory ring.
#include "tma.cuh"

namespace nsa {

constexpr int MODE_CMP = 0;
constexpr int MODE_SWA = 1;

template <int D, int MODE>
__global__ void __launch_bounds__(320, 1)
    dkdv128_tc_kernel(NsaAttnParams p, DkdvLaunch L, const __grid_constant__ CUtensorMap tmq, const __grid_constant__ CUtensorMap tmo,
                      const __grid_constant__ CUtensorMap tmk, const __grid_constant__ CUtensorMap tmv) {
  using namespace tc;
  constexpr int BK = 128, BQ = 128, NS = 2, SLABS = D / 64;
  constexpr uint32_t KV_BYTES = BK * D * 2, Q_BYTES = BQ * D * 2, K_SLAB = BK * 128, Q_SLAB = BQ * 128;
  constexpr uint32_t IDESC_SD = make_idesc(BK, BQ, false), IDESC_KV = make_idesc(BK, D, true);
  constexpr uint32_t TM_S = 0, TM_DP = 128, TM_DV = 256, TM_DK = 384;

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  const uint32_t sK = base, sV = sK + KV_BYTES;
  const uint32_t sQ = sV + KV_BYTES;            // NS stages
  const uint32_t sO = sQ + NS * Q_BYTES;        // NS stages
  const uint32_t meta_off = 2 * KV_BYTES + 2 * NS * Q_BYTES;
  float* sLse = reinterpret_cast<float*>(smem_raw + meta_off);   // [2][128]: -lse of the tile's query rows, two buffers
  float* sDl = sLse + 2 * BQ;
  int* sTa = reinterpret_cast<int*>(sDl + 2 * BQ);
  const uint32_t bars = base + meta_off + 6 * BQ * 4;
  const uint32_t kv_full = bars, q_full = bars + 8, s_full = q_full + 8 * NS, dp_full = s_full + 8, p_ready = dp_full + 8,
                 ds_ready = p_ready + 8, kv_done = ds_ready + 8, done = kv_done + 8, tm_slot = done + 8;

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
  // Order of the query tiles.  Sliding window: neighbouring key tiles see overlapping query ranges, and their CTAs run
  // at the same time; step i of every CTA takes the tile whose absolute tile number is i modulo the tile count, so the
  // CTAs that share a query tile read it at about the same time and it is served from L2.
  int rot = 0;
  if (MODE == MODE_SWA) {
    const int abs0 = (pc.off + r_lo) / TOKQ;
    rot = (n_it - abs0 % n_it) % n_it;
  }
  auto tile_of = [&](int i) { return MODE == MODE_SWA ? (i + rot) % n_it : i; };

  if (tid == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < NS; ++s) mbar_init(q_full + 8 * s, 1);
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(p_ready, 256);
    mbar_init(ds_ready, 256);
    mbar_init(kv_done, 1);
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

  if (warp == 9) {
    if ((tid & 31) == 0) {
      // ============================================ TMA producer: K/V once, then the Q/dO tiles through the 2-stage ring
      tma::expect_tx(kv_full, 2 * KV_BYTES);
#pragma unroll
      for (int sl = 0; sl < SLABS; ++sl) {
        tma::load_3d(sK + sl * K_SLAB, &tmk, sl * 64, kh, (int)(kv_bos + k0), kv_full);
        tma::load_3d(sV + sl * K_SLAB, &tmv, sl * 64, kh, (int)(kv_bos + k0), kv_full);
      }
      for (int i = 0; i < n_it; ++i) {
        const int s = i % NS;
        // the stage of tile i-2 is free once its dK product is done
        if (i >= NS && !mbar_wait(kv_done, (i - NS) & 1, &budget)) timed_out = true;
        tma::expect_tx(q_full + 8 * s, 2 * Q_BYTES);
        const int row = pc.q_start + r_lo + tile_of(i) * TOKQ;
#pragma unroll
        for (int sl = 0; sl < SLABS; ++sl) {
          tma::load_3d(sQ + s * Q_BYTES + sl * Q_SLAB, &tmq, sl * 64, kh * G, row, q_full + 8 * s);
          tma::load_3d(sO + s * Q_BYTES + sl * Q_SLAB, &tmo, sl * 64, kh * G, row, q_full + 8 * s);
        }
      }
    }
  } else if (warp == 8) {
    if ((tid & 31) == 0) {
      // ============================================ MMA issue
      if (!mbar_wait(kv_full, 0, &budget)) timed_out = true;
      auto issue_dk = [&](int i) {  // dK += dS^T Q of tile i; k-step u covers query rows 16u..16u+15, which group
        const int s = i % NS;       // w = u / 4 wrote at columns 64w + 32h + 8e of the dP^T region
        if (!mbar_wait(ds_ready, i & 1, &budget)) timed_out = true;
        fence_after_sync();
#pragma unroll
        for (int u = 0; u < BQ / 16; ++u)
          mma_ts(tmem + TM_DK, tmem + TM_DP + 64 * (u >> 2) + 32 * ((u >> 1) & 1) + 8 * (u & 1),
                 desc_mnmajor(sQ + s * Q_BYTES + u * 2048, Q_SLAB), IDESC_KV, (i > 0 || u > 0));
        mma_commit(kv_done);
      };
      // MMAs of one thread execute in issue order, so a product may overwrite a tensor-memory region that an earlier
      // product still reads as its A operand; barriers are needed only against the compute groups and the TMA loads.
      for (int i = 0; i < n_it; ++i) {
        const int s = i % NS, ph = i & 1;
        if (!mbar_wait(q_full + 8 * s, (i / NS) & 1, &budget)) timed_out = true;
        fence_after_sync();
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t ao = (k >> 2) * K_SLAB + (k & 3) * 32, bo = (k >> 2) * Q_SLAB + (k & 3) * 32;
          mma_ss(tmem + TM_S, desc_kmajor(sK + ao), desc_kmajor(sQ + s * Q_BYTES + bo), IDESC_SD, k > 0);
        }
        mma_commit(s_full);
        if (i > 0) issue_dk(i - 1);   // runs while the compute groups turn S^T of tile i into P^T
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t ao = (k >> 2) * K_SLAB + (k & 3) * 32, bo = (k >> 2) * Q_SLAB + (k & 3) * 32;
          mma_ss(tmem + TM_DP, desc_kmajor(sV + ao), desc_kmajor(sO + s * Q_BYTES + bo), IDESC_SD, k > 0);
        }
        mma_commit(dp_full);
        if (!mbar_wait(p_ready, ph, &budget)) timed_out = true;
        fence_after_sync();
#pragma unroll
        for (int u = 0; u < BQ / 16; ++u)
          mma_ts(tmem + TM_DV, tmem + TM_S + 64 * (u >> 2) + 32 * ((u >> 1) & 1) + 8 * (u & 1), desc_mnmajor(sO + s * Q_BYTES + u * 2048, Q_SLAB),
                 IDESC_KV, (i > 0 || u > 0));
      }
      issue_dk(n_it - 1);
      mma_commit(done);
    }
  } else {
    // ============================================ two compute warp groups: group w owns query columns 64w..64w+63 of
    // every tile; thread = K/V row (tensor-memory lane)
    const int t = tid & 127, wg = warp >> 2;
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16) + 64 * wg;
    const int key = k0 + t;
    const bool key_ok = t < kv_rows;
    const float c2 = p.sm_scale * 1.4426950408889634f;
    // visible iff lo <= ta <= hi for this thread's key
    int lo, hi;
    if (MODE == MODE_CMP) { lo = key * st + ks - 1; hi = 0x7fffffff; }
    else { lo = key; hi = key + W; }
    if (!key_ok) lo = 0x7fffffff;
    // column metadata of a tile: -lse, delta, absolute position (-1 = no such query row); loaded one tile ahead
    float m_lse = 0.f, m_dl = 0.f;
    int m_ta = -1;
    auto fetch_meta = [&](int i) {
      m_lse = 0.f; m_dl = 0.f; m_ta = -1;
      if (t < 64 && i < n_it) {
        const int col = 64 * wg + t;
        const int n = col / G, g = col - n * G;
        const int tok = r_lo + tile_of(i) * TOKQ + n;
        if (tok < r_hi) {
          const int64_t q_row = (int64_t)pc.q_start + tok;
          const int64_t a = q_row * p.lse_stride_t + (int64_t)(kh * G + g) * p.lse_stride_h;
          m_lse = -p.lse[a];
          m_dl = p.delta[a];
          m_ta = pc.off + tok;
        }
      }
    };
    fetch_meta(0);
    for (int i = 0; i < n_it; ++i) {
      const int ph = i & 1;
      const int mo = ph * BQ + 64 * wg;   // this group's 64 columns of metadata buffer ph
      if (t < 64) {
        sLse[mo + t] = m_lse;
        sDl[mo + t] = m_dl;
        sTa[mo + t] = m_ta;
      }
      fetch_meta(i + 1);
      named_barrier(1 + wg, 128);   // buffer ph was last read two tiles ago, before the previous tile's barrier
      // every (key, query) pair of the tile visible?  then the position test is skipped
      const int tok0 = r_lo + tile_of(i) * TOKQ, ta_min = pc.off + tok0, ta_max = ta_min + TOKQ - 1;
      bool full = kv_rows == BK && tok0 + TOKQ <= r_hi;
      if (MODE == MODE_CMP) full = full && ((k0 + BK - 1) * st + ks - 1 <= ta_min);
      else full = full && (k0 + BK - 1 <= ta_min) && (ta_max - k0 <= W);
      const float4* lse4 = reinterpret_cast<const float4*>(sLse + mo);
      const float4* dl4 = reinterpret_cast<const float4*>(sDl + mo);
      const int4* ta4 = reinterpret_cast<const int4*>(sTa + mo);
      float x[64];
      // ---- P^T = exp2(S^T c - lse), written over S^T while dP^T is being multiplied
      if (!mbar_wait(s_full, ph, &budget)) timed_out = true;
      fence_after_sync();
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t sv[32], pp[16];
        tmem_ld32(lane_base + TM_S + half * 32, sv);
        wait_ld();
        if (full) {
#pragma unroll
          for (int c = 0; c < 32; c += 4) {
            const float4 nl = lse4[half * 8 + (c >> 2)];
            x[half * 32 + c] = fast_exp2(fmaf(__uint_as_float(sv[c]), c2, nl.x));
            x[half * 32 + c + 1] = fast_exp2(fmaf(__uint_as_float(sv[c + 1]), c2, nl.y));
            x[half * 32 + c + 2] = fast_exp2(fmaf(__uint_as_float(sv[c + 2]), c2, nl.z));
            x[half * 32 + c + 3] = fast_exp2(fmaf(__uint_as_float(sv[c + 3]), c2, nl.w));
          }
        } else {
#pragma unroll
          for (int c = 0; c < 32; c += 4) {
            const float4 nl = lse4[half * 8 + (c >> 2)];
            const int4 ta = ta4[half * 8 + (c >> 2)];
            x[half * 32 + c] = (ta.x >= lo && ta.x <= hi) ? fast_exp2(fmaf(__uint_as_float(sv[c]), c2, nl.x)) : 0.f;
            x[half * 32 + c + 1] = (ta.y >= lo && ta.y <= hi) ? fast_exp2(fmaf(__uint_as_float(sv[c + 1]), c2, nl.y)) : 0.f;
            x[half * 32 + c + 2] = (ta.z >= lo && ta.z <= hi) ? fast_exp2(fmaf(__uint_as_float(sv[c + 2]), c2, nl.z)) : 0.f;
            x[half * 32 + c + 3] = (ta.w >= lo && ta.w <= hi) ? fast_exp2(fmaf(__uint_as_float(sv[c + 3]), c2, nl.w)) : 0.f;
          }
        }
#pragma unroll
        for (int c = 0; c < 32; c += 2) pp[c >> 1] = pack_bf16(x[half * 32 + c], x[half * 32 + c + 1]);
        tmem_st16(lane_base + TM_S + half * 32, pp);
      }
      wait_st();
      fence_before_sync();
      mbar_arrive(p_ready);
      // ---- dS^T = P^T (dP^T - delta), written over dP^T while dV is being accumulated
      if (!mbar_wait(dp_full, ph, &budget)) timed_out = true;
      fence_after_sync();
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t dv[32], dd[16];
        tmem_ld32(lane_base + TM_DP + half * 32, dv);
        wait_ld();
#pragma unroll
        for (int c = 0; c < 32; c += 4) {
          const float4 dl = dl4[half * 8 + (c >> 2)];
          dd[c >> 1] = pack_bf16(x[half * 32 + c] * (__uint_as_float(dv[c]) - dl.x), x[half * 32 + c + 1] * (__uint_as_float(dv[c + 1]) - dl.y));
          dd[(c >> 1) + 1] =
              pack_bf16(x[half * 32 + c + 2] * (__uint_as_float(dv[c + 2]) - dl.z), x[half * 32 + c + 3] * (__uint_as_float(dv[c + 3]) - dl.w));
        }
        tmem_st16(lane_base + TM_DP + half * 32, dd);
      }
      wait_st();
      fence_before_sync();
      mbar_arrive(ds_ready);
    }
    if (!mbar_wait(done, 0, &budget)) timed_out = true;
    fence_after_sync();
    // ---- my K/V row: group 0 adds dV, group 1 adds dK
    float* dst = (wg == 0 ? p.dv + (kv_bos + k0 + t) * p.dv_stride_t : p.dk + (kv_bos + k0 + t) * p.dk_stride_t) + kh * D;
    const float sc = wg == 0 ? 1.f : p.sm_scale;
    const uint32_t src = tmem + ((uint32_t)((warp & 3) * 32) << 16) + (wg == 0 ? TM_DV : TM_DK);
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
  if (G > 128 || (128 % G) != 0) return 1;
  if (p->meta.kv_table || p->meta.cmp_table || p->n_k_rows <= 0 || p->n_q_rows <= 0) return 1;
  if (((uintptr_t)p->q | (uintptr_t)p->dout | (uintptr_t)p->k | (uintptr_t)p->v) & 15) return 1;
  if ((p->q_stride_t * 2) % 16 || (p->do_stride_t * 2) % 16 || (p->k_stride_t * 2) % 16 || (p->v_stride_t * 2) % 16) return 1;
  if ((p->dk_stride_t % 4) || (p->dv_stride_t % 4) || (((uintptr_t)p->dk | (uintptr_t)p->dv) & 15)) return 1;
  CUtensorMap tmq, tmo, tmk, tmv;
  const int TOKQ = 128 / G;
  if (!tma::make_map(&tmq, p->q, p->n_q_rows, p->QH, D, p->q_stride_t, TOKQ, G) ||
      !tma::make_map(&tmo, p->dout, p->n_q_rows, p->QH, D, p->do_stride_t, TOKQ, G) ||
      !tma::make_map(&tmk, p->k, p->n_k_rows, p->KH, D, p->k_stride_t, 128, 1) ||
      !tma::make_map(&tmv, p->v, p->n_k_rows, p->KH, D, p->v_stride_t, 128, 1)) {
    set_error("%s: cuTensorMapEncodeTiled failed or is unavailable", name);
    return NSA_ERR_CUDA;
  }
  size_t smem = (size_t)(2 * 128 + 4 * 128) * D * 2 + 6 * 128 * 4 + 256;
  cudaError_t e = cudaFuncSetAttribute(dkdv128_tc_kernel<D, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_error("%s: cudaFuncSetAttribute failed: %s", name, cudaGetErrorString(e));
    return NSA_ERR_CUDA;
  }
  DkdvLaunch L{q_chunk};
  dim3 grid;
  if (MODE == MODE_CMP) grid = dim3((p->meta.y_maxlen + 127) / 128, (p->meta.max_piece_len + q_chunk - 1) / q_chunk, p->meta.n_pieces * p->KH);
  else grid = dim3((p->meta.max_piece_len + p->hp.window + 127) / 128 + 1, 1, p->meta.n_pieces * p->KH);
  dkdv128_tc_kernel<D, MODE><<<grid, 320, smem, st>>>(*p, L, tmq, tmo, tmk, tmv);
  return check_launch(name);
}

int launch_dkdv128(const NsaAttnParams* p, cudaStream_t st, const char* name, bool cmp, int q_chunk) {
  if (p->D == 128) return cmp ? launch128<128, MODE_CMP>(p, st, name, q_chunk) : launch128<128, MODE_SWA>(p, st, name, q_chunk);
  return cmp ? launch128<64, MODE_CMP>(p, st, name, q_chunk) : launch128<64, MODE_SWA>(p, st, name, q_chunk);
}

}  // namespace nsa
