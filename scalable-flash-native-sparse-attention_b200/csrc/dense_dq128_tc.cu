// dQ of the compressed and sliding-window branches over CONTIGUOUS K/V: one 128-row query tile per CTA, 128-row K/V
// tiles, TMA loads, warp-specialised (tcgen05 + tensor memory).
//
// A query tile is (128/G consecutive tokens) x (the G query heads of one kv head); thread i of a compute group owns
// row i (tensor-memory lane i).  Per K/V tile:
//     S  = Q K^T    (A = Q tile, B = K tile, K-major from shared memory; two S buffers in tensor memory)
//     dP = dO V^T
//     P  = exp2(S c - lse),  dS = P (dP - delta) -> bf16, written over dP
//     dQ += dS K    (A = dS from tensor memory, B = K tile read MN-major)
// Warp 8 (one lane) issues every MMA, warp 9 (one lane) the TMA loads (Q and dO once, K and V through 2-stage rings);
// warps 0-3 and 4-7 are two compute groups that take key columns 0-63 and 64-127 of every tile.  MMAs of one thread
// execute in issue order, so dP of the next tile may overwrite the dS that dQ of this tile still reads; the order
//     S(0) | dP(i) S(i+1) dQ(i) | ...
// lets exp2 of tile i+1 run under dQ(i) and dP(i+1), and dS of tile i under S(i+1).
#include <algorithm>
#include "tma.cuh"

namespace nsa {

namespace {
constexpr int MODE_CMP = 0;
constexpr int MODE_SWA = 1;
}  // namespace

template <int D, int MODE>
__global__ void __launch_bounds__(320, 1)
    dense_dq128_tc_kernel(NsaAttnParams p, int items, const __grid_constant__ CUtensorMap tmq, const __grid_constant__ CUtensorMap tmo,
                          const __grid_constant__ CUtensorMap tmk, const __grid_constant__ CUtensorMap tmv) {
  using namespace tc;
  constexpr int BM = 128, BN = 128, HN = BN / 2, SLABS = D / 64;
  constexpr uint32_t Q_BYTES = BM * D * 2, KV_BYTES = BN * D * 2, Q_SLAB = BM * 128, K_SLAB = BN * 128;
  constexpr uint32_t TM_S = 0, TM_DP = 256, TM_DQ = 384;   // S: two buffers of 128 columns
  constexpr uint32_t IDESC_S = make_idesc(BM, BN, false), IDESC_Q = make_idesc(BM, D, true);

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  const uint32_t sQ = base, sO = sQ + Q_BYTES;
  const uint32_t sK = sO + Q_BYTES;             // 2 stages
  const uint32_t sV = sK + 2 * KV_BYTES;        // 2 stages
  const uint32_t bars = sV + 2 * KV_BYTES;
  const uint32_t q_full = bars, k_full = bars + 8, v_full = k_full + 16, k_free = v_full + 16, v_free = k_free + 16,
                 s_full = v_free + 16, dp_full = s_full + 16, ds_ready = dp_full + 8, done = ds_ready + 8, q_free = done + 8,
                 dq_free = q_free + 8, tm_slot = dq_free + 8;

  const int tid = threadIdx.x, warp = tid >> 5;
  const int G = p.QH / p.KH;
  const int TOK = BM / G;
  const int kh = blockIdx.z;
  const Piece pc = load_piece(p.meta, blockIdx.y);
  const int ks = p.hp.kernel_size, st = p.hp.stride, W = p.hp.window;
  const int kv_bos = (MODE == MODE_CMP) ? pc.y_bos : pc.x_bos;
  // This CTA's query tiles: `items` consecutive ones.  All roles walk them with the same two running counters: qi (tiles
  // with work done so far) and gt (K/V tiles done so far), from which every barrier phase and ring stage is derived, so
  // the loads and the first MMAs of the next query tile run under the epilogue of the current one.
  const int tile0 = (gridDim.x - 1 - blockIdx.x) * items;
  struct Item {
    int t0, ntok, tabs_min, kv_lo, kv_hi, ntiles;
  };
  auto item_of = [&](int i, Item& it) -> bool {
    it.t0 = (tile0 + i) * TOK;
    if (it.t0 >= pc.len) return false;
    it.ntok = min(TOK, pc.len - it.t0);
    it.tabs_min = pc.off + it.t0;
    const int tabs_max = it.tabs_min + it.ntok - 1;
    if (MODE == MODE_CMP) {
      it.kv_lo = 0;
      it.kv_hi = (tabs_max >= ks - 1) ? min(pc.y_len, (tabs_max - (ks - 1)) / st + 1) : 0;
    } else {
      it.kv_lo = (max(0, it.tabs_min - W) / BN) * BN;   // tiles on a fixed grid of key positions: a row's result does not
      it.kv_hi = min(tabs_max + 1, pc.x_len);           // depend on which rows share its CTA (shards reproduce the full run)
    }
    it.ntiles = (it.kv_hi > it.kv_lo) ? (it.kv_hi - it.kv_lo + BN - 1) / BN : 0;
    return true;
  };
  {
    Item first;
    if (!item_of(0, first)) return;
  }
  if (base & 1023u) {
    if (tid == 0 && p.status) atomicOr(p.status, 8);
    return;
  }
  if (tid == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_free, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(k_full + 8 * s, 1);
      mbar_init(v_full + 8 * s, 1);
      mbar_init(k_free + 8 * s, 1);
      mbar_init(v_free + 8 * s, 1);
      mbar_init(s_full + 8 * s, 1);
    }
    mbar_init(dp_full, 1);
    mbar_init(ds_ready, 256);
    mbar_init(done, 1);
    mbar_init(dq_free, 256);
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
  int gt = 0, qi = 0;

  if (warp == 9) {
    if ((tid & 31) == 0) {
      // ============================================ TMA producer
      for (int i = 0; i < items; ++i) {
        Item im;
        if (!item_of(i, im)) break;
        if (im.ntiles == 0) continue;
        if (qi > 0 && !mbar_wait(q_free, (qi - 1) & 1, &budget)) timed_out = true;   // S and dP of the previous tile are done
        tma::expect_tx(q_full, 2 * Q_BYTES);
#pragma unroll
        for (int sl = 0; sl < SLABS; ++sl) {
          tma::load_3d(sQ + sl * Q_SLAB, &tmq, sl * 64, kh * G, pc.q_start + im.t0, q_full);
          tma::load_3d(sO + sl * Q_SLAB, &tmo, sl * 64, kh * G, pc.q_start + im.t0, q_full);
        }
        for (int it = 0; it < im.ntiles; ++it) {
          const int g = gt + it, s = g & 1, row = kv_bos + im.kv_lo + it * BN;
          if (g >= 2 && !mbar_wait(k_free + 8 * s, ((g >> 1) - 1) & 1, &budget)) timed_out = true;
          tma::expect_tx(k_full + 8 * s, KV_BYTES);
#pragma unroll
          for (int sl = 0; sl < SLABS; ++sl) tma::load_3d(sK + s * KV_BYTES + sl * K_SLAB, &tmk, sl * 64, kh, row, k_full + 8 * s);
          if (g >= 2 && !mbar_wait(v_free + 8 * s, ((g >> 1) - 1) & 1, &budget)) timed_out = true;
          tma::expect_tx(v_full + 8 * s, KV_BYTES);
#pragma unroll
          for (int sl = 0; sl < SLABS; ++sl) tma::load_3d(sV + s * KV_BYTES + sl * K_SLAB, &tmv, sl * 64, kh, row, v_full + 8 * s);
        }
        gt += im.ntiles;
        ++qi;
      }
    }
  } else if (warp == 8) {
    if ((tid & 31) == 0) {
      // ============================================ MMA issue
      auto issue_s = [&](int g) {   // S of K/V tile g = Q K^T into buffer g & 1
        const uint32_t tK = sK + (g & 1) * KV_BYTES;
        if (!mbar_wait(k_full + 8 * (g & 1), (g >> 1) & 1, &budget)) timed_out = true;
        fence_after_sync();
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t ao = (k >> 2) * Q_SLAB + (k & 3) * 32, bo = (k >> 2) * K_SLAB + (k & 3) * 32;
          mma_ss(tmem + TM_S + 128 * (g & 1), desc_kmajor(sQ + ao), desc_kmajor(tK + bo), IDESC_S, k > 0);
        }
        mma_commit(s_full + 8 * (g & 1));
      };
      for (int i = 0; i < items; ++i) {
        Item im;
        if (!item_of(i, im)) break;
        if (im.ntiles == 0) continue;
        if (!mbar_wait(q_full, qi & 1, &budget)) timed_out = true;
        issue_s(gt);
        for (int it = 0; it < im.ntiles; ++it) {
          const int g = gt + it, s = g & 1;
          const uint32_t tK = sK + s * KV_BYTES, tV = sV + s * KV_BYTES;
          if (!mbar_wait(v_full + 8 * s, (g >> 1) & 1, &budget)) timed_out = true;
          fence_after_sync();
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint32_t ao = (k >> 2) * Q_SLAB + (k & 3) * 32, bo = (k >> 2) * K_SLAB + (k & 3) * 32;
            mma_ss(tmem + TM_DP, desc_kmajor(sO + ao), desc_kmajor(tV + bo), IDESC_S, k > 0);
          }
          mma_commit(dp_full);
          mma_commit(v_free + 8 * s);
          if (it + 1 < im.ntiles) issue_s(g + 1);
          else mma_commit(q_free);   // every S and dP of this query tile has been issued: Q and dO may be replaced
          // dQ += dS K: k-step u covers keys 16u..16u+15; group h = u / 4 wrote them at columns 64h + 8(u % 4) of dP
          if (!mbar_wait(ds_ready, g & 1, &budget)) timed_out = true;
          if (it == 0 && qi > 0 && !mbar_wait(dq_free, (qi - 1) & 1, &budget)) timed_out = true;   // dQ of the previous tile read out
          fence_after_sync();
#pragma unroll
          for (int u = 0; u < BN / 16; ++u)
            mma_ts(tmem + TM_DQ, tmem + TM_DP + 64 * (u >> 2) + 8 * (u & 3), desc_mnmajor(tK + u * 2048, K_SLAB), IDESC_Q, (it > 0 || u > 0));
          mma_commit(k_free + 8 * s);
        }
        mma_commit(done);
        gt += im.ntiles;
        ++qi;
      }
    }
  } else {
    // ============================================ compute groups: column half h; thread = query row
    const int h = warp >> 2, row = tid & 127;
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16) + h * HN;
    const int tok = row / G, g_ = row % G;
    const float c2 = p.sm_scale * 1.4426950408889634f;
    const float sc = p.sm_scale;
    for (int i = 0; i < items; ++i) {
      Item im;
      if (!item_of(i, im)) break;
      const bool row_ok = tok < im.ntok;
      const int64_t q_row = pc.q_start + im.t0 + tok;
      __nv_bfloat16* dq_row = reinterpret_cast<__nv_bfloat16*>(p.dq) + q_row * p.dq_stride_t + (int64_t)(kh * G + g_) * D + h * (D / 2);
      if (im.ntiles == 0) {   // nothing visible for the whole tile: the gradient is zero
        if (row_ok && !p.accumulate_dq) {
#pragma unroll
          for (int c = 0; c < D / 16; ++c) reinterpret_cast<uint4*>(dq_row)[c] = make_uint4(0, 0, 0, 0);
        }
        continue;
      }
      const int t_abs = im.tabs_min + tok;
      // keys vis_lo..vis_hi (positions in the sequence's K/V rows) are visible to my row
      int vis_lo = 0, vis_hi = -1;
      float nlse = 0.f, dl = 0.f;
      if (row_ok) {
        if (MODE == MODE_CMP) vis_hi = (t_abs - ks + 1 >= 0) ? (t_abs - ks + 1) / st : -1;
        else { vis_hi = t_abs; vis_lo = t_abs - W; }
        vis_hi = min(vis_hi, im.kv_hi - 1);
        const int64_t a = q_row * p.lse_stride_t + (int64_t)(kh * G + g_) * p.lse_stride_h;
        nlse = -p.lse[a];
        dl = p.delta[a];
      }
      for (int it = 0; it < im.ntiles; ++it) {
        const int g = gt + it;
        const int kv0 = im.kv_lo + it * BN + h * HN;
        const int lo = vis_lo - kv0, hi = vis_hi - kv0;   // visible columns of my half of this tile
        const bool full = lo <= 0 && hi >= HN - 1;
        float x[HN];
        // ---- P = exp2(S c - lse)
        if (!mbar_wait(s_full + 8 * (g & 1), (g >> 1) & 1, &budget)) timed_out = true;
        fence_after_sync();
#pragma unroll
        for (int c = 0; c < HN / 32; ++c) {
          uint32_t sv[32];
          tmem_ld32(lane_base + TM_S + 128 * (g & 1) + c * 32, sv);
          wait_ld();
          if (full) {
#pragma unroll
            for (int e = 0; e < 32; ++e) x[c * 32 + e] = fast_exp2(fmaf(__uint_as_float(sv[e]), c2, nlse));
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const int col = c * 32 + e;
              x[col] = (col >= lo && col <= hi) ? fast_exp2(fmaf(__uint_as_float(sv[e]), c2, nlse)) : 0.f;
            }
          }
        }
        // ---- dS = P (dP - delta) -> bf16 over the first 32 of my 64 dP columns (already consumed)
        if (!mbar_wait(dp_full, g & 1, &budget)) timed_out = true;
        fence_after_sync();
#pragma unroll
        for (int c = 0; c < HN / 32; ++c) {
          uint32_t dv[32], dd[16];
          tmem_ld32(lane_base + TM_DP + c * 32, dv);
          wait_ld();
#pragma unroll
          for (int e = 0; e < 32; e += 2)
            dd[e >> 1] = pack_bf16(x[c * 32 + e] * (__uint_as_float(dv[e]) - dl), x[c * 32 + e + 1] * (__uint_as_float(dv[e + 1]) - dl));
          tmem_st16(lane_base + TM_DP + c * 16, dd);
        }
        wait_st();
        fence_before_sync();
        mbar_arrive(ds_ready);
      }
      // ---- epilogue: my half of my row of dQ; when adding into an existing dq its old values are fetched before the
      // wait for the last MMA, so that their latency is hidden
      uint4 old[D / 16];
#pragma unroll
      for (int c = 0; c < D / 16; ++c)
        old[c] = (p.accumulate_dq && row_ok) ? *reinterpret_cast<const uint4*>(dq_row + c * 8) : make_uint4(0, 0, 0, 0);
      if (!mbar_wait(done, qi & 1, &budget)) timed_out = true;
      fence_after_sync();
      const uint32_t acc = tmem + ((uint32_t)((warp & 3) * 32) << 16) + TM_DQ + h * (D / 2);
      uint32_t o[D / 2];
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        uint32_t t32[32];
        tmem_ld32(acc + c * 32, t32);
#pragma unroll
        for (int e = 0; e < 32; ++e) o[c * 32 + e] = t32[e];
      }
      wait_ld();
      fence_before_sync();
      mbar_arrive(dq_free);   // the accumulator may be overwritten by the next query tile's first dQ product
      if (row_ok) {
#pragma unroll
        for (int q8 = 0; q8 < D / 16; ++q8) {
          const uint4 od = old[q8];
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(o[q8 * 8 + e]) * sc;
          f[0] += bf16_lo(od.x); f[1] += bf16_hi(od.x); f[2] += bf16_lo(od.y); f[3] += bf16_hi(od.y);
          f[4] += bf16_lo(od.z); f[5] += bf16_hi(od.z); f[6] += bf16_lo(od.w); f[7] += bf16_hi(od.w);
          uint4 wv;
          wv.x = pack_bf16(f[0], f[1]); wv.y = pack_bf16(f[2], f[3]); wv.z = pack_bf16(f[4], f[5]); wv.w = pack_bf16(f[6], f[7]);
          *reinterpret_cast<uint4*>(dq_row + q8 * 8) = wv;
        }
      }
      gt += im.ntiles;
      ++qi;
    }
  }
  if (timed_out && p.status) atomicOr(p.status, 4);
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

// returns 1 when the configuration is not covered (the 64-row-tile kernel then runs), 0 on launch, < 0 on error
template <int D, int MODE>
static int launch128(const NsaAttnParams* p, cudaStream_t st, const char* name) {
  const int G = p->QH / p->KH;
  if (G > 128 || (128 % G) != 0) return 1;
  if (p->meta.kv_table || p->meta.cmp_table || p->n_k_rows <= 0 || p->n_q_rows <= 0) return 1;
  if (((uintptr_t)p->q | (uintptr_t)p->dout | (uintptr_t)p->k | (uintptr_t)p->v) & 15) return 1;
  if ((p->q_stride_t * 2) % 16 || (p->do_stride_t * 2) % 16 || (p->k_stride_t * 2) % 16 || (p->v_stride_t * 2) % 16) return 1;
  const int TOK = 128 / G;
  CUtensorMap tmq, tmo, tmk, tmv;
  if (!tma::make_map(&tmq, p->q, p->n_q_rows, p->QH, D, p->q_stride_t, TOK, G) ||
      !tma::make_map(&tmo, p->dout, p->n_q_rows, p->QH, D, p->do_stride_t, TOK, G) ||
      !tma::make_map(&tmk, p->k, p->n_k_rows, p->KH, D, p->k_stride_t, 128, 1) ||
      !tma::make_map(&tmv, p->v, p->n_k_rows, p->KH, D, p->v_stride_t, 128, 1)) {
    set_error("%s: cuTensorMapEncodeTiled failed or is unavailable", name);
    return NSA_ERR_CUDA;
  }
  const size_t smem = (size_t)6 * 128 * D * 2 + 256;
  cudaError_t e = cudaFuncSetAttribute(dense_dq128_tc_kernel<D, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_error("%s: cudaFuncSetAttribute failed: %s", name, cudaGetErrorString(e));
    return NSA_ERR_CUDA;
  }
  // consecutive query tiles per CTA (up to 8): the CTA's set-up, and the epilogue of one tile under the loads of the next,
  // are shared; fewer when the launch would not fill the GPU a few times over
  const int n_q_tiles = (p->meta.max_piece_len + TOK - 1) / TOK;
  const int64_t total = (int64_t)n_q_tiles * p->meta.n_pieces * p->KH;
  const int items = (int)std::max<int64_t>(1, std::min<int64_t>(8, total / (148 * 4)));
  dim3 grid((n_q_tiles + items - 1) / items, p->meta.n_pieces, p->KH);
  dense_dq128_tc_kernel<D, MODE><<<grid, 320, smem, st>>>(*p, items, tmq, tmo, tmk, tmv);
  return check_launch(name);
}

int launch_dq128(const NsaAttnParams* p, cudaStream_t st, const char* name, bool cmp) {
  if (p->D == 128) return cmp ? launch128<128, MODE_CMP>(p, st, name) : launch128<128, MODE_SWA>(p, st, name);
  return cmp ? launch128<64, MODE_CMP>(p, st, name) : launch128<64, MODE_SWA>(p, st, name);
}

}  // namespace nsa
