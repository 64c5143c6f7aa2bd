// dK/dV of the compressed and sliding-window branches with 64-row K/V tiles (tcgen05 + tensor memory): the fallback of
// dkdv128_tc.cu for head-group sizes that do not divide 128 and for tensors the 128-row TMA boxes cannot address.  (The
// selected branch has its own persistent kernel built on the same tile machinery, slc_bwd_tc.cu.)
//
// One CTA owns a 64-row K/V tile (compressed rows or a 64-key stretch of a sequence) and a slice of the queries that see
// it.  Query rows come in tiles of 128 = (128/G tokens) x (G heads of the kv head), taken from a contiguous token range.
// Two warp groups of 128 threads each work on their own query tile (ping-pong), a ninth warp issues every MMA and six
// more fetch the Q / dO tiles with TMA, one (64 d) x (G heads) x (1 token) box per lane, as soon as a group's buffers
// are free:
//     S    = Q K^T          M = query rows, N = keys      (A, B from shared memory, K-major)
//     dP   = dO V^T
//     P    = exp2(S*c - lse),  dS = P * (dP - delta)      thread i of the group owns row i; bf16 P, dS go to shared memory
//     dV^T += dO^T P        M = value dim, N = keys, contraction over the 128 query rows (A, B MN-major views of the
//     dK^T += Q^T dS        SAME dO / Q / P / dS bytes)
// Accumulating the TRANSPOSED gradients keeps every MMA at M = 128 although a K/V tile has only 64 rows.  At the end
// lane j of the accumulator holds column j of dV (dK): each thread adds its 64 values to the fp32 dV (dK) with atomics
// that are coalesced across a warp.
#include "tma.cuh"

namespace nsa {

constexpr int MODE_CMP = 0;
constexpr int MODE_SWA = 1;

template <int D, int MODE>
__global__ void __launch_bounds__(480, 1)
    dkdv_tc_kernel(NsaAttnParams p, DkdvLaunch L, const __grid_constant__ CUtensorMap tmq, const __grid_constant__ CUtensorMap tmo) {
  using namespace tc;
  constexpr int BK = 64, BQ = 128;
  constexpr uint32_t KV_BYTES = BK * D * 2, Q_BYTES = BQ * D * 2, P_BYTES = BQ * BK * 2;
  constexpr uint32_t Q_SLAB = BQ * 128, K_SLAB = BK * 128;
  constexpr uint32_t A_LBO = (D == 128) ? Q_SLAB : 0;  // D = 64: the second half of M re-reads the only slab (rows 64.. of the result are unused)
  constexpr uint32_t IDESC_SD = make_idesc(BQ, BK, false, false), IDESC_KV = make_idesc(128, BK, true, true);
  constexpr uint32_t TM_DV = 256, TM_DK = 320, TM_COLS = 512;

  extern __shared__ unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sK = base, sV = sK + KV_BYTES;
  const uint32_t sQ0 = sV + KV_BYTES;                 // [2 groups]
  const uint32_t sO0 = sQ0 + 2 * Q_BYTES;             // [2 groups]
  const uint32_t sP0 = sO0 + 2 * Q_BYTES;             // [2 groups]
  const uint32_t sS0 = sP0 + 2 * P_BYTES;             // [2 groups]
  const uint32_t bars = sS0 + 2 * P_BYTES;
  // barriers: in_full[2], sd_done[2], pds_full[2], kv_done[2]; then the tensor-memory address slot
  auto bar = [&](int which, int wg) { return bars + (which * 2 + wg) * 8; };
  const uint32_t tm_slot = bars + 80;

  const int tid = threadIdx.x, warp = tid >> 5;
  const int G = p.QH / p.KH;
  const int TOKQ = BQ / G;
  const int ks = p.hp.kernel_size, st = p.hp.stride, W = p.hp.window;

  int kh, k0, kv_rows, r_lo, r_hi;
  int64_t kv_bos;
  Piece pc;
  {
    kh = blockIdx.z % p.KH;
    pc = load_piece(p.meta, blockIdx.z / p.KH);
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
  }
  if (kv_rows <= 0 || r_hi <= r_lo) return;
  const int n_it = (r_hi - r_lo + TOKQ - 1) / TOKQ;
  const int n_round = (n_it + 1) / 2;

  // ---- set-up
  if (tid == 0) {
    for (int w = 0; w < 2; ++w) {
      mbar_init(bar(0, w), 1);
      mbar_init(bar(1, w), 1);
      mbar_init(bar(2, w), 128);
      mbar_init(bar(3, w), 1);
    }
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc(tm_slot, TM_COLS);
  if (tid < 256) {
    fill_tile_async<D>(sK, reinterpret_cast<const __nv_bfloat16*>(p.k) + (kv_bos + k0) * p.k_stride_t + kh * D, p.k_stride_t, BK,
                       kv_rows, tid, 256);
    fill_tile_async<D>(sV, reinterpret_cast<const __nv_bfloat16*>(p.v) + (kv_bos + k0) * p.v_stride_t + kh * D, p.v_stride_t, BK,
                       kv_rows, tid, 256);
    cp_async_commit();
    if (TOKQ * G < BQ) {  // rows the TMA boxes never write must not hold NaN bit patterns
      for (int i = tid; i < (int)(4 * Q_BYTES / 16); i += 256)
        asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};\n" ::"r"(sQ0 + i * 16), "r"(0) : "memory");
    }
    cp_async_wait<0>();
    fence_proxy_async();
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  uint32_t tmem;
  asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(tmem) : "r"(tm_slot));
  int budget = kWaitBudget;
  bool timed_out = false;

  if (warp == 8) {
    // ================================================= MMA issue (one lane)
    if ((tid & 31) == 0) {
      for (int j = 0; j < n_round; ++j) {
        for (int wg = 0; wg < 2; ++wg) {
          if (!mbar_wait(bar(0, wg), j & 1, &budget)) timed_out = true;
          fence_after_sync();
          const uint32_t tQ = sQ0 + wg * Q_BYTES, tO = sO0 + wg * Q_BYTES;
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            uint32_t ao = (k >> 2) * Q_SLAB + (k & 3) * 32, bo = (k >> 2) * K_SLAB + (k & 3) * 32;
            mma_ss(tmem + 128 * wg, desc_kmajor(tQ + ao), desc_kmajor(sK + bo), IDESC_SD, k > 0);
          }
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            uint32_t ao = (k >> 2) * Q_SLAB + (k & 3) * 32, bo = (k >> 2) * K_SLAB + (k & 3) * 32;
            mma_ss(tmem + 128 * wg + 64, desc_kmajor(tO + ao), desc_kmajor(sV + bo), IDESC_SD, k > 0);
          }
          mma_commit(bar(1, wg));
        }
        for (int wg = 0; wg < 2; ++wg) {
          if (!mbar_wait(bar(2, wg), j & 1, &budget)) timed_out = true;
          fence_after_sync();
          const uint32_t tQ = sQ0 + wg * Q_BYTES, tO = sO0 + wg * Q_BYTES;
          const uint32_t tP = sP0 + wg * P_BYTES, tS = sS0 + wg * P_BYTES;
          const uint32_t first = (j == 0 && wg == 0) ? 0u : 1u;
#pragma unroll
          for (int u = 0; u < BQ / 16; ++u)
            mma_ss(tmem + TM_DV, desc_mnmajor(tO + u * 2048, A_LBO), desc_mnmajor(tP + u * 2048, 0), IDESC_KV, (u > 0) ? 1u : first);
#pragma unroll
          for (int u = 0; u < BQ / 16; ++u)
            mma_ss(tmem + TM_DK, desc_mnmajor(tQ + u * 2048, A_LBO), desc_mnmajor(tS + u * 2048, 0), IDESC_KV, (u > 0) ? 1u : first);
          mma_commit(bar(3, wg));
        }
      }
    }
  } else if (warp >= 9) {
    // ================================================= TMA producer: tile `it` goes to the buffers of group it & 1
    // six producer warps; box b belongs to lane b / 6 of warp 9 + b % 6, so that a small box count still spreads over
    // all of them (each thread's TMA instruction is issued on its own)
    const int lane = (tid & 31) * 6 + (warp - 9);
    constexpr int NP = 192;
    constexpr int SLABS = D / 64;
    const int n_box = TOKQ * SLABS * 2;
    const uint32_t tx = (uint32_t)(TOKQ * G) * D * 2 * 2;
    for (int it = 0; it < 2 * n_round; ++it) {   // an odd tile count still fills group 1's buffers in the last round
      const int wg = it & 1, j = it >> 1;
      const int tok0 = r_lo + it * TOKQ;
      // tensor rows of my first four boxes now, so that the index loads overlap the wait for the buffers
      auto row_of = [&](int b) {
        const int tok = min(tok0 + b / (SLABS * 2), r_hi - 1);   // past the end: a valid row again (its P, dS are zero)
        return pc.q_start + tok;
      };
      int rows[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) rows[u] = (lane + NP * u < n_box) ? row_of(lane + NP * u) : 0;
      if (j > 0 && !mbar_wait(bar(3, wg), (j - 1) & 1, &budget)) timed_out = true;   // dV/dK MMAs of tile it-2 have read them
      if (lane == 0) tma::expect_tx(bar(0, wg), tx);
      __syncwarp();
      auto issue = [&](int b, int row) {
        const int n = b / (SLABS * 2), rest = b - n * (SLABS * 2), sl = rest >> 1, which = rest & 1;
        const uint32_t dst = (which ? sO0 : sQ0) + wg * Q_BYTES + sl * Q_SLAB + n * G * 128;
        tma::load_3d(dst, which ? &tmo : &tmq, sl * 64, kh * G, row, bar(0, wg));
      };
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (lane + NP * u < n_box) issue(lane + NP * u, rows[u]);
      for (int b = lane + 4 * NP; b < n_box; b += NP) issue(b, row_of(b));   // only when G = 1 and D = 128
    }
  } else {
    // ================================================= two warp groups, one query tile each per round
    const int wg = warp >> 2, t = tid & 127;
    const uint32_t tP = sP0 + wg * P_BYTES, tS = sS0 + wg * P_BYTES;
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const float c2 = p.sm_scale * 1.4426950408889634f;
    const int my_n = t / G, my_g = t - my_n * G;
    for (int j = 0; j < n_round; ++j) {
      const int it = 2 * j + wg;
      const int tok0 = r_lo + it * TOKQ;  // first token (range position / list position) of my tile
      if (j > 0 && !mbar_wait(bar(3, wg), (j - 1) & 1, &budget)) timed_out = true;  // my buffers are free again
      // my own row: lse, delta, absolute position
      const bool row_ok = (my_n < TOKQ) && (tok0 + my_n < r_hi);
      float lse = 0.f, dl = 0.f;
      int ta = -1;
      if (row_ok) {
        int64_t q_row = (int64_t)pc.q_start + tok0 + my_n;
        int64_t a = q_row * p.lse_stride_t + (int64_t)(kh * G + my_g) * p.lse_stride_h;
        lse = p.lse[a];
        dl = p.delta[a];
        ta = pc.off + (int)(q_row - pc.q_start);
      }
      // keys kc_lo..kc_hi of the tile are visible to my row
      int kc_lo = 0, kc_hi = -1;
      if (row_ok) {
        if (MODE == MODE_CMP) kc_hi = (ta - ks + 1 >= 0) ? (ta - ks + 1) / st - k0 : -1;
        else kc_hi = ta - k0;
        if (MODE == MODE_SWA) kc_lo = ta - W - k0;
        kc_hi = min(kc_hi, kv_rows - 1);
      }
      const float nlse = -lse;
      if (!mbar_wait(bar(1, wg), j & 1, &budget)) timed_out = true;
      fence_after_sync();
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t sv[32], dv[32];
        tmem_ld32(lane_base + 128 * wg + half * 32, sv);
        tmem_ld32(lane_base + 128 * wg + 64 + half * 32, dv);
        wait_ld();
        uint32_t pp[16], dd[16];
        if (kc_lo <= 0 && kc_hi >= BK - 1) {   // the whole key tile is visible to my row (the usual case)
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float x0 = fast_exp2(fmaf(__uint_as_float(sv[i]), c2, nlse));
            const float x1 = fast_exp2(fmaf(__uint_as_float(sv[i + 1]), c2, nlse));
            pp[i >> 1] = pack_bf16(x0, x1);
            dd[i >> 1] = pack_bf16(x0 * (__uint_as_float(dv[i]) - dl), x1 * (__uint_as_float(dv[i + 1]) - dl));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const int kc = half * 32 + i;
            const float x0 = (kc >= kc_lo && kc <= kc_hi) ? fast_exp2(fmaf(__uint_as_float(sv[i]), c2, nlse)) : 0.f;
            const float x1 = (kc + 1 >= kc_lo && kc + 1 <= kc_hi) ? fast_exp2(fmaf(__uint_as_float(sv[i + 1]), c2, nlse)) : 0.f;
            pp[i >> 1] = pack_bf16(x0, x1);
            dd[i >> 1] = pack_bf16(x0 * (__uint_as_float(dv[i]) - dl), x1 * (__uint_as_float(dv[i + 1]) - dl));
          }
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint32_t off = t * 128 + ((((half * 4 + c) ^ (t & 7))) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(tP + off), "r"(pp[4 * c]), "r"(pp[4 * c + 1]), "r"(pp[4 * c + 2]),
                       "r"(pp[4 * c + 3])
                       : "memory");
          asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(tS + off), "r"(dd[4 * c]), "r"(dd[4 * c + 1]), "r"(dd[4 * c + 2]),
                       "r"(dd[4 * c + 3])
                       : "memory");
        }
      }
      fence_proxy_async();
      fence_before_sync();
      mbar_arrive(bar(2, wg));
    }
    // ---- all MMAs done (the tensor core retires them in issue order, group 1's last commit is the final one)
    if (!mbar_wait(bar(3, wg), (n_round - 1) & 1, &budget)) timed_out = true;
    if (!mbar_wait(bar(3, 1), (n_round - 1) & 1, &budget)) timed_out = true;
    fence_after_sync();
    // group 0 writes dV, group 1 writes dK: lane t = column t of the gradient
    const uint32_t acc = lane_base + (wg == 0 ? TM_DV : TM_DK);
    float* dst = (wg == 0 ? p.dv : p.dk) + (kv_bos + k0) * (wg == 0 ? p.dv_stride_t : p.dk_stride_t) + kh * D + t;
    const int64_t rstride = (wg == 0 ? p.dv_stride_t : p.dk_stride_t);
    const float scale = (wg == 0) ? 1.f : p.sm_scale;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      uint32_t v[32];
      tmem_ld32(acc + half * 32, v);
      wait_ld();
      if (t < D) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          int kc = half * 32 + i;
          if (kc < kv_rows) atomicAdd(dst + (int64_t)kc * rstride, __uint_as_float(v[i]) * scale);
        }
      }
    }
  }
  if (timed_out && p.status) atomicOr(p.status, 2);
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, TM_COLS);
}

template <int D, int MODE>
int launch_dkdv(const NsaAttnParams* p, cudaStream_t st, const char* name, dim3 grid, DkdvLaunch L) {
  size_t smem = (size_t)(2 * 64 + 4 * 128) * D * 2 + 4 * 128 * 64 * 2 + 128 + 1024;
  cudaError_t e = cudaFuncSetAttribute(dkdv_tc_kernel<D, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_error("%s: cudaFuncSetAttribute(%zu B) failed: %s", name, smem, cudaGetErrorString(e));
    return NSA_ERR_CUDA;
  }
  const int G = p->QH / p->KH;
  CUtensorMap tmq, tmo;
  if (p->n_q_rows <= 0 || !tma::make_map(&tmq, p->q, p->n_q_rows, p->QH, D, p->q_stride_t, 1, G) ||
      !tma::make_map(&tmo, p->dout, p->n_q_rows, p->QH, D, p->do_stride_t, 1, G)) {
    set_error("%s: cuTensorMapEncodeTiled failed or is unavailable (q/dout must be 16-byte aligned, n_q_rows set)", name);
    return NSA_ERR_CUDA;
  }
  dkdv_tc_kernel<D, MODE><<<grid, 480, smem, st>>>(*p, L, tmq, tmo);
  return check_launch(name);
}

template int launch_dkdv<128, MODE_CMP>(const NsaAttnParams*, cudaStream_t, const char*, dim3, DkdvLaunch);
template int launch_dkdv<64, MODE_CMP>(const NsaAttnParams*, cudaStream_t, const char*, dim3, DkdvLaunch);
template int launch_dkdv<128, MODE_SWA>(const NsaAttnParams*, cudaStream_t, const char*, dim3, DkdvLaunch);
template int launch_dkdv<64, MODE_SWA>(const NsaAttnParams*, cudaStream_t, const char*, dim3, DkdvLaunch);

}  // namespace nsa
