// Forward of the compressed and sliding-window branches over CONTIGUOUS K/V: two 128-row query tiles per CTA, 128-row
// K/V tiles, TMA loads, warp-specialised (tcgen05 + tensor memory).
//
// A query tile is (128/G consecutive tokens) x (the G query heads of one kv head); a CTA owns two consecutive tiles
// a and b that walk over the same K/V tiles, so every K/V tile is fetched once for 256 query rows.
//   warps 0-7 / 8-15  softmax of tile a / b: two groups of 128 threads per tile, thread i of a group owns row i
//                     (tensor-memory lane i) and one half of the 128 key columns; the row maximum and the final
//                     row sum cross the halves through shared memory
//   warp 16 (one lane) issues every MMA:   S = Q K^T   (A = Q tile, B = K tile, both K-major from shared memory)
//                                         O += P V    (A = P from tensor memory, B = V tile read MN-major)
//   warp 17 (one lane) issues the TMA loads: both Q tiles once, K and V tiles through 2-stage rings
// Tensor memory: S_a, S_b (128 fp32 columns each; the bf16 P of a column half is written over S columns of that half)
// and O_a, O_b.  MMAs of one thread execute in issue order, so S of the next K/V tile may be issued straight after
// the P.V product that still reads P from the same columns; the order
//     S_a(0) S_b(0) | PV_a(i) S_a(i+1) PV_b(i) S_b(i+1) | ...
// keeps the tensor core busy with one tile while the other tile's group does its softmax.
// The running maximum of a row is only raised when the tile maximum exceeds it by more than 2^8 (the row's thread then
// rescales its O row in tensor memory); l and the final normalisation use the same reference, so the result is exact.
#include <algorithm>
#include "tma.cuh"

namespace nsa {

namespace {
constexpr int MODE_CMP = 0;
constexpr int MODE_SWA = 1;
}  // namespace

template <int D, int MODE>
__global__ void __launch_bounds__(576, 1)
    dense_fwd128_tc_kernel(NsaAttnParams p, int items, const __grid_constant__ CUtensorMap tmq, const __grid_constant__ CUtensorMap tmk,
                           const __grid_constant__ CUtensorMap tmv) {
  using namespace tc;
  constexpr int BM = 128, BN = 128, SLABS = D / 64;
  constexpr uint32_t Q_BYTES = BM * D * 2, KV_BYTES = BN * D * 2, Q_SLAB = BM * 128, K_SLAB = BN * 128;
  constexpr uint32_t TM_S = 0, TM_O = 256;   // + 128 * tile
  constexpr uint32_t IDESC_S = make_idesc(BM, BN, false), IDESC_O = make_idesc(BM, D, true);

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  const uint32_t sQ = base;                     // 2 tiles
  const uint32_t sK = sQ + 2 * Q_BYTES;         // 2 stages
  const uint32_t sV = sK + 2 * KV_BYTES;        // 2 stages
  const uint32_t bars = sV + 2 * KV_BYTES;
  const uint32_t q_full = bars, k_full = bars + 8, v_full = k_full + 16, k_free = v_full + 16, v_free = k_free + 16,
                 s_full = v_free + 16, p_ready = s_full + 16, o_done = p_ready + 16, o_free = o_done + 16, q_free = o_free + 16, tm_slot = q_free + 8;
  float* sX = reinterpret_cast<float*>(smem_raw + 2 * Q_BYTES + 4 * KV_BYTES + 256);   // row maxima / sums crossing the two column halves

  const int tid = threadIdx.x, warp = tid >> 5;
  const int G = p.QH / p.KH;
  const int TOK = BM / G;
  const int kh = blockIdx.z;
  const Piece pc = load_piece(p.meta, blockIdx.y);
  const int ks = p.hp.kernel_size, st = p.hp.stride, W = p.hp.window;
  const int kv_bos = (MODE == MODE_CMP) ? pc.y_bos : pc.x_bos;
  // This CTA's query-tile pairs: `items` consecutive ones.  All roles walk them with the same two running counters: qi
  // (pairs with work done so far) and gt (K/V tiles done so far), from which every barrier phase and ring stage is
  // derived, so the loads and the first products of the next pair run under the epilogue of the current one.
  const int pair0 = (gridDim.x - 1 - blockIdx.x) * items;
  struct Item {
    int t0, ntok, tabs_min, kv_lo, kv_hi, ntiles;
  };
  auto item_of = [&](int i, Item& it) -> bool {
    it.t0 = (pair0 + i) * 2 * TOK;
    if (it.t0 >= pc.len) return false;
    it.ntok = min(2 * TOK, pc.len - it.t0);
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
      mbar_init(p_ready + 8 * s, 256);
      mbar_init(o_done + 8 * s, 1);
      mbar_init(o_free + 8 * s, 256);
    }
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

  if (warp == 17) {
    if ((tid & 31) == 0) {
      // ============================================ TMA producer
      for (int i = 0; i < items; ++i) {
        Item im;
        if (!item_of(i, im)) break;
        if (im.ntiles == 0) continue;
        if (qi > 0 && !mbar_wait(q_free, (qi - 1) & 1, &budget)) timed_out = true;   // every S of the previous pair is done
        tma::expect_tx(q_full, 2 * Q_BYTES);
#pragma unroll
        for (int w = 0; w < 2; ++w)
#pragma unroll
          for (int sl = 0; sl < SLABS; ++sl)
            tma::load_3d(sQ + w * Q_BYTES + sl * Q_SLAB, &tmq, sl * 64, kh * G, pc.q_start + im.t0 + w * TOK, q_full);
        for (int it = 0; it < im.ntiles; ++it) {
          const int g = gt + it, s = g & 1;
          // paged cache: a 128-row tile lies inside one page (page sizes are multiples of 128), one table look-up per tile
          const int row = (MODE == MODE_CMP) ? (pc.y_tab ? (int)cmp_row(pc, im.kv_lo + it * BN) : kv_bos + im.kv_lo + it * BN)
                                             : (pc.x_tab ? (int)tok_row(pc, im.kv_lo + it * BN) : kv_bos + im.kv_lo + it * BN);
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
  } else if (warp == 16) {
    if ((tid & 31) == 0) {
      // ============================================ MMA issue
      auto issue_s = [&](int w, int g) {   // S_w = Q_w K(g)^T
        const uint32_t tK = sK + (g & 1) * KV_BYTES;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t ao = (k >> 2) * Q_SLAB + (k & 3) * 32, bo = (k >> 2) * K_SLAB + (k & 3) * 32;
          mma_ss(tmem + TM_S + 128 * w, desc_kmajor(sQ + w * Q_BYTES + ao), desc_kmajor(tK + bo), IDESC_S, k > 0);
        }
        mma_commit(s_full + 8 * w);
      };
      auto issue_pv = [&](int w, int g, bool first) {  // O_w += P_w V(g); k-step u = keys 16u..16u+15; P of keys 64h.. starts at column 64h
        const uint32_t tV = sV + (g & 1) * KV_BYTES;
        if (!mbar_wait(p_ready + 8 * w, g & 1, &budget)) timed_out = true;
        // the first product of a pair overwrites O_w: the previous pair's epilogue must have read it
        if (first && qi > 0 && !mbar_wait(o_free + 8 * w, (qi - 1) & 1, &budget)) timed_out = true;
        fence_after_sync();
#pragma unroll
        for (int u = 0; u < BN / 16; ++u)
          mma_ts(tmem + TM_O + 128 * w, tmem + TM_S + 128 * w + 64 * (u >> 2) + 8 * (u & 3), desc_mnmajor(tV + u * 2048, K_SLAB), IDESC_O,
                 (!first || u > 0));
        mma_commit(o_done + 8 * w);
      };
      for (int i = 0; i < items; ++i) {
        Item im;
        if (!item_of(i, im)) break;
        if (im.ntiles == 0) continue;
        if (!mbar_wait(q_full, qi & 1, &budget)) timed_out = true;
        if (!mbar_wait(k_full + 8 * (gt & 1), (gt >> 1) & 1, &budget)) timed_out = true;
        fence_after_sync();
        issue_s(0, gt);
        issue_s(1, gt);
        mma_commit(k_free + 8 * (gt & 1));
        if (im.ntiles == 1) mma_commit(q_free);
        for (int it = 0; it < im.ntiles; ++it) {
          const int g = gt + it, s = g & 1;
          const bool more = it + 1 < im.ntiles;
          if (!mbar_wait(v_full + 8 * s, (g >> 1) & 1, &budget)) timed_out = true;
          issue_pv(0, g, it == 0);
          if (more) {
            if (!mbar_wait(k_full + 8 * (s ^ 1), ((g + 1) >> 1) & 1, &budget)) timed_out = true;
            fence_after_sync();
            issue_s(0, g + 1);
          }
          issue_pv(1, g, it == 0);
          mma_commit(v_free + 8 * s);
          if (more) {
            issue_s(1, g + 1);
            mma_commit(k_free + 8 * (s ^ 1));
            if (it + 2 == im.ntiles) mma_commit(q_free);   // the pair's last S products are issued: Q may be replaced
          }
        }
        gt += im.ntiles;
        ++qi;
      }
    }
  } else {
    // ============================================ softmax: tile w = a / b, column half h; thread = query row
    const int w = warp >> 3, h = (warp >> 2) & 1, row = tid & 127;
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16) + 128 * w;
    const float c2 = p.sm_scale * 1.4426950408889634f;
    float* xmax = sX + (w * 3) * 256;       // [2 maximum buffers + 1 sum buffer][2 halves][128 rows] of this tile
    constexpr int HN = BN / 2;
    for (int i = 0; i < items; ++i) {
      Item im;
      if (!item_of(i, im)) break;
      const int tok = w * TOK + row / G, g_ = row % G;
      const bool row_ok = tok < im.ntok;
      const int t_abs = im.tabs_min + tok;
      const int64_t q_row = pc.q_start + im.t0 + tok;
      __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.o) + q_row * p.o_stride_t + (int64_t)(kh * G + g_) * D + h * (D / 2);
      if (im.ntiles == 0) {  // nothing visible for the whole pair: zeros
        if (row_ok) {
#pragma unroll
          for (int c = 0; c < D / 16; ++c) reinterpret_cast<uint4*>(orow)[c] = make_uint4(0, 0, 0, 0);
          if (p.lse && h == 0) p.lse[q_row * p.lse_stride_t + (int64_t)(kh * G + g_) * p.lse_stride_h] = 0.f;
        }
        continue;
      }
      // keys vis_lo..vis_hi (positions in the sequence's K/V rows) are visible to my row
      int vis_lo = 0, vis_hi = -1;
      if (row_ok) {
        if (MODE == MODE_CMP) vis_hi = (t_abs - ks + 1 >= 0) ? (t_abs - ks + 1) / st : -1;
        else { vis_hi = t_abs; vis_lo = t_abs - W; }
        vis_hi = min(vis_hi, im.kv_hi - 1);
      }
      float m_ref = -INFINITY, l_run = 0.f;   // l_run: my half of the columns only

      for (int it = 0; it < im.ntiles; ++it) {
        const int g = gt + it;
        const int kv0 = im.kv_lo + it * BN + h * HN;
        const int lo = vis_lo - kv0, hi = vis_hi - kv0;   // visible columns of my half of this tile
        const bool full = lo <= 0 && hi >= HN - 1;
        if (!mbar_wait(s_full + 8 * w, g & 1, &budget)) timed_out = true;
        fence_after_sync();
        // ---- pass 1: row maximum over my 64 columns, then over both halves through shared memory
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // independent chains
#pragma unroll
        for (int c = 0; c < HN / 32; ++c) {
          uint32_t sv[32];
          tmem_ld32(lane_base + TM_S + h * HN + c * 32, sv);
          wait_ld();
          if (full) {
#pragma unroll
            for (int e = 0; e < 32; ++e) mx4[e & 3] = fmaxf(mx4[e & 3], __uint_as_float(sv[e]));
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if (c * 32 + e >= lo && c * 32 + e <= hi) mx4[e & 3] = fmaxf(mx4[e & 3], __uint_as_float(sv[e]));
          }
        }
        float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        float* xb = xmax + (g & 1) * 256;   // this buffer was last read two tiles ago, before the previous tile's barrier
        xb[h * 128 + row] = mx;
        named_barrier(1 + w, 256);
        mx = fmaxf(mx, xb[(h ^ 1) * 128 + row]) * c2;
        // ---- reference maximum: raise it only when the row maximum ran away by more than 2^8
        float alpha = 1.f;
        bool need = false;
        if (m_ref == -INFINITY) {
          m_ref = mx;  // nothing accumulated yet for this row (its O row is still exactly zero or unwritten)
        } else if (mx > m_ref + 8.f) {
          alpha = fast_exp2(m_ref - mx);
          m_ref = mx;
          need = true;
        }
        const float nmu = (m_ref == -INFINITY) ? 0.f : -m_ref;
        // ---- pass 2: P = exp2(S c - m) -> bf16, written over the first 32 of MY 64 S columns (already consumed)
        float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
        for (int c = 0; c < HN / 32; ++c) {
          uint32_t sv[32], pk[16];
          tmem_ld32(lane_base + TM_S + h * HN + c * 32, sv);
          wait_ld();
          if (full) {
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
              const float e0 = fast_exp2(fmaf(__uint_as_float(sv[e]), c2, nmu)), e1 = fast_exp2(fmaf(__uint_as_float(sv[e + 1]), c2, nmu));
              rs0 += e0;
              rs1 += e1;
              pk[e >> 1] = pack_bf16(e0, e1);
            }
          } else {
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
              const int col = c * 32 + e;
              const float e0 = (col >= lo && col <= hi) ? fast_exp2(fmaf(__uint_as_float(sv[e]), c2, nmu)) : 0.f;
              const float e1 = (col + 1 >= lo && col + 1 <= hi) ? fast_exp2(fmaf(__uint_as_float(sv[e + 1]), c2, nmu)) : 0.f;
              rs0 += e0;
              rs1 += e1;
              pk[e >> 1] = pack_bf16(e0, e1);
            }
          }
          tmem_st16(lane_base + TM_S + h * HN + c * 16, pk);
        }
        l_run = l_run * alpha + (rs0 + rs1);
        if (it > 0 && __any_sync(0xffffffffu, need)) {  // rescale my half of my O row (warp-uniform branch, per-lane
#pragma unroll                                          // factor); the previous P.V of this tile retired before this S
          for (int c = 0; c < D / 64; ++c) {
            uint32_t o[32];
            tmem_ld32(lane_base + TM_O + h * (D / 2) + c * 32, o);
            wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
            tmem_st32(lane_base + TM_O + h * (D / 2) + c * 32, o);
          }
        }
        wait_st();
        fence_before_sync();
        mbar_arrive(p_ready + 8 * w);
      }
      // the row's l: both halves (a buffer of its own: the maximum buffers belong to the tiles around this point)
      float* xl = xmax + 2 * 256;
      xl[h * 128 + row] = l_run;
      named_barrier(1 + w, 256);
      l_run += xl[(h ^ 1) * 128 + row];
      if (!mbar_wait(o_done + 8 * w, (gt + im.ntiles - 1) & 1, &budget)) timed_out = true;
      fence_after_sync();
      // ---- epilogue: my half of my row of O
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      uint32_t o[D / 2];
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        uint32_t t32[32];
        tmem_ld32(lane_base + TM_O + h * (D / 2) + c * 32, t32);
#pragma unroll
        for (int e = 0; e < 32; ++e) o[c * 32 + e] = t32[e];
      }
      wait_ld();
      fence_before_sync();
      mbar_arrive(o_free + 8 * w);   // O_w (and the sum buffer) may be overwritten by the next pair
      if (row_ok) {
#pragma unroll
        for (int q8 = 0; q8 < D / 16; ++q8) {
          uint4 x;
          x.x = pack_bf16(__uint_as_float(o[q8 * 8 + 0]) * inv, __uint_as_float(o[q8 * 8 + 1]) * inv);
          x.y = pack_bf16(__uint_as_float(o[q8 * 8 + 2]) * inv, __uint_as_float(o[q8 * 8 + 3]) * inv);
          x.z = pack_bf16(__uint_as_float(o[q8 * 8 + 4]) * inv, __uint_as_float(o[q8 * 8 + 5]) * inv);
          x.w = pack_bf16(__uint_as_float(o[q8 * 8 + 6]) * inv, __uint_as_float(o[q8 * 8 + 7]) * inv);
          *reinterpret_cast<uint4*>(orow + q8 * 8) = x;
        }
        if (p.lse && h == 0)
          p.lse[q_row * p.lse_stride_t + (int64_t)(kh * G + g_) * p.lse_stride_h] = l_run > 0.f ? m_ref + log2f(l_run) : 0.f;
      }
      gt += im.ntiles;
      ++qi;
    }
  }
  if (timed_out && p.status) atomicOr(p.status, 1);
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

// returns 1 when the configuration is not covered (the 64-row-tile kernel then runs), 0 on launch, < 0 on error
template <int D, int MODE>
static int launch128(const NsaAttnParams* p, cudaStream_t st, const char* name) {
  const int G = p->QH / p->KH;
  if (G > 128 || (128 % G) != 0) return 1;
  if (p->n_k_rows <= 0 || p->n_q_rows <= 0) return 1;
  // a paged cache: pages must hold whole 128-row tiles (the caller clears the rows past each sequence's end, nsa_paged_zero_tails)
  // (prefill chunks only: one-token pieces of a decode step are better served by the 64-row-tile kernel)
  if ((p->meta.kv_table || p->meta.cmp_table) &&
      (p->meta.page_size < 128 || (p->meta.page_size & (p->meta.page_size - 1)) || p->meta.max_piece_len < 64))
    return 1;
  if (((uintptr_t)p->q | (uintptr_t)p->k | (uintptr_t)p->v) & 15) return 1;
  if ((p->q_stride_t * 2) % 16 || (p->k_stride_t * 2) % 16 || (p->v_stride_t * 2) % 16) return 1;
  const int TOK = 128 / G;
  CUtensorMap tmq, tmk, tmv;
  if (!tma::make_map(&tmq, p->q, p->n_q_rows, p->QH, D, p->q_stride_t, TOK, G) ||
      !tma::make_map(&tmk, p->k, p->n_k_rows, p->KH, D, p->k_stride_t, 128, 1) ||
      !tma::make_map(&tmv, p->v, p->n_k_rows, p->KH, D, p->v_stride_t, 128, 1)) {
    set_error("%s: cuTensorMapEncodeTiled failed or is unavailable", name);
    return NSA_ERR_CUDA;
  }
  const size_t smem = (size_t)6 * 128 * D * 2 + 256 + 6 * 256 * 4;
  cudaError_t e = cudaFuncSetAttribute(dense_fwd128_tc_kernel<D, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_error("%s: cudaFuncSetAttribute failed: %s", name, cudaGetErrorString(e));
    return NSA_ERR_CUDA;
  }
  // consecutive query-tile pairs per CTA (up to 8): the CTA's set-up, and the epilogue of one pair under the loads of the
  // next, are shared; fewer when the launch would not fill the GPU a few times over
  const int n_pairs = (p->meta.max_piece_len + 2 * TOK - 1) / (2 * TOK);
  const int64_t total = (int64_t)n_pairs * p->meta.n_pieces * p->KH;
  const int items = (int)std::max<int64_t>(1, std::min<int64_t>(8, total / (148 * 4)));
  dim3 grid((n_pairs + items - 1) / items, p->meta.n_pieces, p->KH);
  dense_fwd128_tc_kernel<D, MODE><<<grid, 576, smem, st>>>(*p, items, tmq, tmk, tmv);
  return check_launch(name);
}

int launch_fwd128(const NsaAttnParams* p, cudaStream_t st, const char* name, bool cmp) {
  if (p->D == 128) return cmp ? launch128<128, MODE_CMP>(p, st, name) : launch128<128, MODE_SWA>(p, st, name);
  return cmp ? launch128<64, MODE_CMP>(p, st, name) : launch128<64, MODE_SWA>(p, st, name);
}

}  // namespace nsa
