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
#include "tma.cuh"

namespace nsa {

namespace {
constexpr int MODE_CMP = 0;
constexpr int MODE_SWA = 1;
}  // namespace

template <int D, int MODE>
__global__ void __launch_bounds__(320, 1)
    dense_dq128_tc_kernel(NsaAttnParams p, const __grid_constant__ CUtensorMap tmq, const __grid_constant__ CUtensorMap tmo,
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
                 s_full = v_free + 16, dp_full = s_full + 16, ds_ready = dp_full + 8, done = ds_ready + 8, tm_slot = done + 8;

  const int tid = threadIdx.x, warp = tid >> 5;
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

  int kv_lo, kv_hi, kv_bos;
  if (MODE == MODE_CMP) {
    kv_lo = 0;
    kv_hi = (tabs_max >= ks - 1) ? min(pc.y_len, (tabs_max - (ks - 1)) / st + 1) : 0;
    kv_bos = pc.y_bos;
  } else {
    kv_lo = (max(0, tabs_min - W) / BN) * BN;   // tiles on a fixed grid of key positions: a row's result does not
    kv_hi = min(tabs_max + 1, pc.x_len);        // depend on which rows share its CTA (shards reproduce the full run)
    kv_bos = pc.x_bos;
  }
  const int ntiles = (kv_hi > kv_lo) ? (kv_hi - kv_lo + BN - 1) / BN : 0;

  if (ntiles == 0) {  // nothing visible for the whole tile: the gradient is zero
    if (tid < 128 && !p.accumulate_dq) {
      const int tok = tid / G, g = tid % G;
      if (tok < ntok) {
        const int64_t q_row = pc.q_start + t0 + tok;
        uint4* o = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.dq) + q_row * p.dq_stride_t + (int64_t)(kh * G + g) * D);
#pragma unroll
        for (int c = 0; c < D / 8; ++c) o[c] = make_uint4(0, 0, 0, 0);
      }
    }
    return;
  }
  if (base & 1023u) {
    if (tid == 0 && p.status) atomicOr(p.status, 8);
    return;
  }
  if (tid == 0) {
    mbar_init(q_full, 1);
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
      // ============================================ TMA producer
      tma::expect_tx(q_full, 2 * Q_BYTES);
#pragma unroll
      for (int sl = 0; sl < SLABS; ++sl) {
        tma::load_3d(sQ + sl * Q_SLAB, &tmq, sl * 64, kh * G, pc.q_start + t0, q_full);
        tma::load_3d(sO + sl * Q_SLAB, &tmo, sl * 64, kh * G, pc.q_start + t0, q_full);
      }
      for (int it = 0; it < ntiles; ++it) {
        const int s = it & 1, row = kv_bos + kv_lo + it * BN;
        if (it >= 2 && !mbar_wait(k_free + 8 * s, ((it >> 1) - 1) & 1, &budget)) timed_out = true;
        tma::expect_tx(k_full + 8 * s, KV_BYTES);
#pragma unroll
        for (int sl = 0; sl < SLABS; ++sl) tma::load_3d(sK + s * KV_BYTES + sl * K_SLAB, &tmk, sl * 64, kh, row, k_full + 8 * s);
        if (it >= 2 && !mbar_wait(v_free + 8 * s, ((it >> 1) - 1) & 1, &budget)) timed_out = true;
        tma::expect_tx(v_full + 8 * s, KV_BYTES);
#pragma unroll
        for (int sl = 0; sl < SLABS; ++sl) tma::load_3d(sV + s * KV_BYTES + sl * K_SLAB, &tmv, sl * 64, kh, row, v_full + 8 * s);
      }
    }
  } else if (warp == 8) {
    if ((tid & 31) == 0) {
      // ============================================ MMA issue
      auto issue_s = [&](int it) {   // S(it) = Q K(it)^T into buffer it & 1
        const uint32_t tK = sK + (it & 1) * KV_BYTES;
        if (!mbar_wait(k_full + 8 * (it & 1), (it >> 1) & 1, &budget)) timed_out = true;
        fence_after_sync();
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t ao = (k >> 2) * Q_SLAB + (k & 3) * 32, bo = (k >> 2) * K_SLAB + (k & 3) * 32;
          mma_ss(tmem + TM_S + 128 * (it & 1), desc_kmajor(sQ + ao), desc_kmajor(tK + bo), IDESC_S, k > 0);
        }
        mma_commit(s_full + 8 * (it & 1));
      };
      if (!mbar_wait(q_full, 0, &budget)) timed_out = true;
      issue_s(0);
      for (int it = 0; it < ntiles; ++it) {
        const int s = it & 1;
        const uint32_t tK = sK + s * KV_BYTES, tV = sV + s * KV_BYTES;
        if (!mbar_wait(v_full + 8 * s, (it >> 1) & 1, &budget)) timed_out = true;
        fence_after_sync();
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t ao = (k >> 2) * Q_SLAB + (k & 3) * 32, bo = (k >> 2) * K_SLAB + (k & 3) * 32;
          mma_ss(tmem + TM_DP, desc_kmajor(sO + ao), desc_kmajor(tV + bo), IDESC_S, k > 0);
        }
        mma_commit(dp_full);
        mma_commit(v_free + 8 * s);
        if (it + 1 < ntiles) issue_s(it + 1);
        // dQ += dS K: k-step u covers keys 16u..16u+15; group h = u / 4 wrote them at columns 64h + 8(u % 4) of dP
        if (!mbar_wait(ds_ready, it & 1, &budget)) timed_out = true;
        fence_after_sync();
#pragma unroll
        for (int u = 0; u < BN / 16; ++u)
          mma_ts(tmem + TM_DQ, tmem + TM_DP + 64 * (u >> 2) + 8 * (u & 3), desc_mnmajor(tK + u * 2048, K_SLAB), IDESC_Q, (it > 0 || u > 0));
        mma_commit(k_free + 8 * s);
      }
      mma_commit(done);
    }
  } else {
    // ============================================ compute groups: column half h; thread = query row
    const int h = warp >> 2, row = tid & 127;
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16) + h * HN;
    const int tok = row / G, g = row % G;
    const bool row_ok = tok < ntok;
    const int t_abs = tabs_min + tok;
    const int64_t q_row = pc.q_start + t0 + tok;
    // keys vis_lo..vis_hi (positions in the sequence's K/V rows) are visible to my row
    int vis_lo = 0, vis_hi = -1;
    float nlse = 0.f, dl = 0.f;
    if (row_ok) {
      if (MODE == MODE_CMP) vis_hi = (t_abs - ks + 1 >= 0) ? (t_abs - ks + 1) / st : -1;
      else { vis_hi = t_abs; vis_lo = t_abs - W; }
      vis_hi = min(vis_hi, kv_hi - 1);
      const int64_t a = q_row * p.lse_stride_t + (int64_t)(kh * G + g) * p.lse_stride_h;
      nlse = -p.lse[a];
      dl = p.delta[a];
    }
    const float c2 = p.sm_scale * 1.4426950408889634f;

    for (int it = 0; it < ntiles; ++it) {
      const int kv0 = kv_lo + it * BN + h * HN;
      const int lo = vis_lo - kv0, hi = vis_hi - kv0;   // visible columns of my half of this tile
      const bool full = lo <= 0 && hi >= HN - 1;
      float x[HN];
      // ---- P = exp2(S c - lse)
      if (!mbar_wait(s_full + 8 * (it & 1), (it >> 1) & 1, &budget)) timed_out = true;
      fence_after_sync();
#pragma unroll
      for (int c = 0; c < HN / 32; ++c) {
        uint32_t sv[32];
        tmem_ld32(lane_base + TM_S + 128 * (it & 1) + c * 32, sv);
        wait_ld();
        if (full) {
#pragma unroll
          for (int i = 0; i < 32; ++i) x[c * 32 + i] = fast_exp2(fmaf(__uint_as_float(sv[i]), c2, nlse));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int col = c * 32 + i;
            x[col] = (col >= lo && col <= hi) ? fast_exp2(fmaf(__uint_as_float(sv[i]), c2, nlse)) : 0.f;
          }
        }
      }
      // ---- dS = P (dP - delta) -> bf16 over the first 32 of my 64 dP columns (already consumed)
      if (!mbar_wait(dp_full, it & 1, &budget)) timed_out = true;
      fence_after_sync();
#pragma unroll
      for (int c = 0; c < HN / 32; ++c) {
        uint32_t dv[32], dd[16];
        tmem_ld32(lane_base + TM_DP + c * 32, dv);
        wait_ld();
#pragma unroll
        for (int i = 0; i < 32; i += 2)
          dd[i >> 1] = pack_bf16(x[c * 32 + i] * (__uint_as_float(dv[i]) - dl), x[c * 32 + i + 1] * (__uint_as_float(dv[i + 1]) - dl));
        tmem_st16(lane_base + TM_DP + c * 16, dd);
      }
      wait_st();
      fence_before_sync();
      mbar_arrive(ds_ready);
    }
    // ---- epilogue: my half of my row of dQ; when adding into an existing dq its old values are fetched before the
    // wait for the last MMA, so that their latency is hidden
    const float sc = p.sm_scale;
    __nv_bfloat16* dq_row = reinterpret_cast<__nv_bfloat16*>(p.dq) + q_row * p.dq_stride_t + (int64_t)(kh * G + g) * D + h * (D / 2);
    uint4 old[D / 16];
#pragma unroll
    for (int c = 0; c < D / 16; ++c)
      old[c] = (p.accumulate_dq && row_ok) ? *reinterpret_cast<const uint4*>(dq_row + c * 8) : make_uint4(0, 0, 0, 0);
    if (!mbar_wait(done, 0, &budget)) timed_out = true;
    fence_after_sync();
    const uint32_t acc = tmem + ((uint32_t)((warp & 3) * 32) << 16) + TM_DQ + h * (D / 2);
#pragma unroll
    for (int c = 0; c < D / 64; ++c) {
      uint32_t o[32];
      tmem_ld32(acc + c * 32, o);
      wait_ld();
      if (row_ok) {
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const uint4 od = old[c * 4 + q4];
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(o[q4 * 8 + e]) * sc;
          f[0] += bf16_lo(od.x); f[1] += bf16_hi(od.x); f[2] += bf16_lo(od.y); f[3] += bf16_hi(od.y);
          f[4] += bf16_lo(od.z); f[5] += bf16_hi(od.z); f[6] += bf16_lo(od.w); f[7] += bf16_hi(od.w);
          uint4 wv;
          wv.x = pack_bf16(f[0], f[1]); wv.y = pack_bf16(f[2], f[3]); wv.z = pack_bf16(f[4], f[5]); wv.w = pack_bf16(f[6], f[7]);
          *reinterpret_cast<uint4*>(dq_row + c * 32 + q4 * 8) = wv;
        }
      }
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
  dim3 grid((p->meta.max_piece_len + TOK - 1) / TOK, p->meta.n_pieces, p->KH);
  dense_dq128_tc_kernel<D, MODE><<<grid, 320, smem, st>>>(*p, tmq, tmo, tmk, tmv);
  return check_launch(name);
}

int launch_dq128(const NsaAttnParams* p, cudaStream_t st, const char* name, bool cmp) {
  if (p->D == 128) return cmp ? launch128<128, MODE_CMP>(p, st, name) : launch128<128, MODE_SWA>(p, st, name);
  return cmp ? launch128<64, MODE_CMP>(p, st, name) : launch128<64, MODE_SWA>(p, st, name);
}

}  // namespace nsa
