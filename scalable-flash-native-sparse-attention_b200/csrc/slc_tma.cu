// Selected-block attention over CONTIGUOUS (non-paged) K/V with TMA-staged tiles: forward and dQ.
//
// Every token has its own list of 64-key blocks, so the unit of work is still one warp per (token, kv head) with the
// query heads (in groups of up to 16) as the 16 rows of the warp-level MMA.  What changes against slc_fwd.cu / slc_bwd.cu is how the
// K/V rows reach the MMA: each warp owns a private 64-row K buffer and V buffer in shared memory, its lane 0 fetches a
// selected block with one TMA box per 64-wide slab (128-byte swizzle), and fragments come from ldmatrix.  Fragment-
// direct global loads deliver 64 bytes per L1 wavefront (4 lanes per key row) and saturate the L1 load pipe; the TMA
// copies bypass it.  While S = Q K^T of block i is computed the V tile of block i is in flight, and the K tile of
// block i+1 is requested as soon as S is done.
#include "tma.cuh"

namespace nsa {

namespace {

constexpr int kWarps = 7;

// 16 x 16 A fragments of a [16 heads x D] row-major global matrix (row r at base + r*D), rows >= G clamped
template <int D>
__device__ __forceinline__ void load_a_global(uint32_t (&a)[D / 16][4], const __nv_bfloat16* base, int G, int lane) {
  const int g_ = lane >> 2, c_ = lane & 3;
  const __nv_bfloat16* r0 = base + min(g_, G - 1) * D + 2 * c_;
  const __nv_bfloat16* r1 = base + min(g_ + 8, G - 1) * D + 2 * c_;
#pragma unroll
  for (int k = 0; k < D / 16; ++k) {
    a[k][0] = *reinterpret_cast<const uint32_t*>(r0 + 16 * k);
    a[k][1] = *reinterpret_cast<const uint32_t*>(r1 + 16 * k);
    a[k][2] = *reinterpret_cast<const uint32_t*>(r0 + 16 * k + 8);
    a[k][3] = *reinterpret_cast<const uint32_t*>(r1 + 16 * k + 8);
  }
}
// B fragments from a 64-row tile in slab layout.  nk: operand stored [n = tile row][k = column]
__device__ __forceinline__ void ldb_nk(uint32_t (&b)[4], uint32_t tile, int n0, int ks, int lane) {
  const int r = n0 + (lane & 7) + (lane >> 4) * 8;
  const int c = ks * 2 + ((lane >> 3) & 1);
  ldsm_x4(b[0], b[1], b[2], b[3], tile + tc::slab_off(64, r, c));
}
// kn: operand stored [k = tile row][n = column]
__device__ __forceinline__ void ldb_kn(uint32_t (&b)[4], uint32_t tile, int k0, int n0, int lane) {
  const int r = k0 + (lane & 7) + ((lane >> 3) & 1) * 8;
  const int c = (n0 >> 3) + (lane >> 4);
  ldsm_x4_t(b[0], b[1], b[2], b[3], tile + tc::slab_off(64, r, c));
}

struct WarpPipe {
  uint32_t bufK, bufV, barK, barV;
  int nK, nV;  // completed phases waited so far
};

template <int D>
__device__ __forceinline__ void fetch(uint32_t buf, uint32_t bar, const CUtensorMap* map, int kh, int row) {
  tma::expect_tx(bar, 64 * D * 2);
#pragma unroll
  for (int sl = 0; sl < D / 64; ++sl) tma::load_3d(buf + sl * 64 * 128, map, sl * 64, kh, row, bar);
}

}  // namespace

// ------------------------------------------------------------------------------------------------ forward
template <int D>
__global__ void __launch_bounds__(kWarps * 32, 1)
    slc_fwd_tma_kernel(NsaAttnParams p, const __grid_constant__ CUtensorMap tmk, const __grid_constant__ CUtensorMap tmv) {
  constexpr int KS = D / 16, NT = D / 8, BS = 64;
  constexpr uint32_t TILE = BS * D * 2;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t base = smem_u32(smem_raw);
  WarpPipe wp{base + warp * 2 * TILE, base + warp * 2 * TILE + TILE, base + kWarps * 2 * TILE + warp * 16,
              base + kWarps * 2 * TILE + warp * 16 + 8, 0, 0};
  const int g_ = lane >> 2, c_ = lane & 3;
  // blockIdx.z = (kv head, group of 16 of its query heads): more than 16 query heads per kv head run as several groups
  const int Gall = p.QH / p.KH, HG = (Gall + 15) / 16;
  const int kh = blockIdx.z / HG, hg = blockIdx.z % HG;
  const int G = min(16, Gall - 16 * hg);
  const int64_t hbase = (int64_t)kh * Gall + 16 * hg;   // first query head of my group
  const Piece pc = load_piece(p.meta, blockIdx.y);
  const int tl = (gridDim.x - 1 - blockIdx.x) * kWarps + warp;
  if (tl >= pc.len) return;
  if (base & 1023u) {
    if (lane == 0 && p.status) atomicOr(p.status, 8);
    return;
  }
  const int t_abs = pc.off + tl;
  const int64_t q_row = pc.q_start + tl;
  const int nk = t_abs >= 0 ? t_abs / BS : -1;
  const int n_valid = min(p.hp.top_n, nk + 1);
  const float c2 = p.sm_scale * 1.4426950408889634f;
  if (lane == 0) {
    tc::mbar_init(wp.barK, 1);
    tc::mbar_init(wp.barV, 1);
    tc::fence_mbar_init();
  }
  __syncwarp();
  // my block list: lane i holds entry i; invalid / unused entries drop out of the ballot
  int my_blk = -1;
  if (lane < n_valid) my_blk = __ldg(p.topk + (int64_t)kh * p.topk_stride_h + q_row * p.hp.top_n + lane);
  unsigned todo = __ballot_sync(0xffffffffu, my_blk >= 0 && my_blk <= nk);
  // first row of my block in the K/V tensor: with a paged cache one page-table look-up per lane, all in flight at once (a
  // 64-row block never straddles a page)
  const int my_row = (my_blk >= 0 && my_blk <= nk) ? (int)tok_row(pc, my_blk * BS) : 0;
  const bool paged = pc.x_tab != nullptr;
  int budget = tc::kWaitBudget;
  bool timed_out = false;

  uint32_t qf[KS][4];
  load_a_global<D>(qf, reinterpret_cast<const __nv_bfloat16*>(p.q) + q_row * p.q_stride_t + hbase * D, G, lane);
  float o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

  int cur = -1;
  if (todo) {
    cur = __shfl_sync(0xffffffffu, my_blk, __ffs(todo) - 1);
    const int row = __shfl_sync(0xffffffffu, my_row, __ffs(todo) - 1);
    todo &= todo - 1;
    if (lane == 0) {
      fetch<D>(wp.bufK, wp.barK, &tmk, kh, row);
      fetch<D>(wp.bufV, wp.barV, &tmv, kh, row);
    }
  }
  while (cur >= 0) {
    const int nxt = todo ? __shfl_sync(0xffffffffu, my_blk, __ffs(todo) - 1) : -1;
    const int nxt_row = todo ? __shfl_sync(0xffffffffu, my_row, __ffs(todo) - 1) : 0;
    todo &= todo - 1;
    const int key0 = cur * BS;
    if (!tc::mbar_wait(wp.barK, wp.nK & 1, &budget)) timed_out = true;
    ++wp.nK;
    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < KS; ++kk) {
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t b[4];
        ldb_nk(b, wp.bufK, np * 16, kk, lane);
        mma_bf16(s[2 * np], qf[kk], b[0], b[1]);
        mma_bf16(s[2 * np + 1], qf[kk], b[2], b[3]);
      }
    }
    __syncwarp();
    if (lane == 0 && nxt >= 0) fetch<D>(wp.bufK, wp.barK, &tmk, kh, nxt_row);  // K buffer is free again
    if (cur == nk) {   // the token's own block: keys after it do not take part
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const int key = key0 + nt * 8 + 2 * c_;
        const bool v0 = key <= t_abs, v1 = key + 1 <= t_abs;
        s[nt][0] = v0 ? s[nt][0] : -INFINITY;
        s[nt][1] = v1 ? s[nt][1] : -INFINITY;
        s[nt][2] = v0 ? s[nt][2] : -INFINITY;
        s[nt][3] = v1 ? s[nt][3] : -INFINITY;
      }
    }
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      mx_lo = fmaxf(mx_lo, fmaxf(s[nt][0], s[nt][1]));
      mx_hi = fmaxf(mx_hi, fmaxf(s[nt][2], s[nt][3]));
    }
    mx_lo = warp_max4(mx_lo) * c2;   // c2 > 0: the maximum of the scaled scores
    mx_hi = warp_max4(mx_hi) * c2;
    // Reference maximum: raised only when the block maximum exceeds it by more than 2^8 (then o and l are rescaled); l and
    // the final normalisation use the same reference, so the result is exact, and most blocks skip the rescale.
    float al_lo = 1.f, al_hi = 1.f;
    if (m_lo == -INFINITY) m_lo = mx_lo;
    else if (mx_lo > m_lo + 8.f) { al_lo = fast_exp2(m_lo - mx_lo); m_lo = mx_lo; }
    if (m_hi == -INFINITY) m_hi = mx_hi;
    else if (mx_hi > m_hi + 8.f) { al_hi = fast_exp2(m_hi - mx_hi); m_hi = mx_hi; }
    const float nmu_lo = (m_lo == -INFINITY) ? 0.f : -m_lo, nmu_hi = (m_hi == -INFINITY) ? 0.f : -m_hi;
    float rs_lo = 0.f, rs_hi = 0.f;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      s[nt][0] = fast_exp2(fmaf(s[nt][0], c2, nmu_lo));
      s[nt][1] = fast_exp2(fmaf(s[nt][1], c2, nmu_lo));
      s[nt][2] = fast_exp2(fmaf(s[nt][2], c2, nmu_hi));
      s[nt][3] = fast_exp2(fmaf(s[nt][3], c2, nmu_hi));
      rs_lo += s[nt][0] + s[nt][1];
      rs_hi += s[nt][2] + s[nt][3];
    }
    l_lo = l_lo * al_lo + rs_lo;
    l_hi = l_hi * al_hi + rs_hi;
    if (__any_sync(0xffffffffu, al_lo != 1.f || al_hi != 1.f)) {
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        o[i][0] *= al_lo; o[i][1] *= al_lo; o[i][2] *= al_hi; o[i][3] *= al_hi;
      }
    }
    if (!tc::mbar_wait(wp.barV, wp.nV & 1, &budget)) timed_out = true;
    ++wp.nV;
    if (paged && key0 + BS > pc.x_len) {
      // rows of the page past the sequence's end may hold anything (never-written memory): their probabilities are 0, and
      // 0 * garbage must not reach the sums, so those V rows are cleared
      constexpr int CH = D / 8;
      for (int idx = (pc.x_len - key0) * CH + lane; idx < BS * CH; idx += 32) {
        const int r = idx / CH, c = idx - r * CH;
        asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};\n" ::"r"(wp.bufV + tc::slab_off(BS, r, c)), "r"(0) : "memory");
      }
      __syncwarp();
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const uint32_t a0 = pack_bf16(s[2 * u][0], s[2 * u][1]), a1 = pack_bf16(s[2 * u][2], s[2 * u][3]);
      const uint32_t a2 = pack_bf16(s[2 * u + 1][0], s[2 * u + 1][1]), a3 = pack_bf16(s[2 * u + 1][2], s[2 * u + 1][3]);
#pragma unroll
      for (int np = 0; np < NT / 2; ++np) {
        uint32_t b[4];
        ldb_kn(b, wp.bufV, u * 16, np * 16, lane);
        mma_bf16(o[2 * np], a0, a1, a2, a3, b[0], b[1]);
        mma_bf16(o[2 * np + 1], a0, a1, a2, a3, b[2], b[3]);
      }
    }
    __syncwarp();
    if (lane == 0 && nxt >= 0) fetch<D>(wp.bufV, wp.barV, &tmv, kh, nxt_row);
    cur = nxt;
  }

  l_lo = warp_sum4(l_lo);
  l_hi = warp_sum4(l_hi);
  const float inv_lo = l_lo > 0.f ? 1.f / l_lo : 0.f, inv_hi = l_hi > 0.f ? 1.f / l_hi : 0.f;
  __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(p.o) + q_row * p.o_stride_t + hbase * D + 2 * c_;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    if (g_ < G) *reinterpret_cast<uint32_t*>(op + g_ * D + nt * 8) = pack_bf16(o[nt][0] * inv_lo, o[nt][1] * inv_lo);
    if (g_ + 8 < G) *reinterpret_cast<uint32_t*>(op + (g_ + 8) * D + nt * 8) = pack_bf16(o[nt][2] * inv_hi, o[nt][3] * inv_hi);
  }
  if (c_ == 0 && p.lse) {
    if (g_ < G) p.lse[q_row * p.lse_stride_t + (hbase + g_) * p.lse_stride_h] = l_lo > 0.f ? m_lo + log2f(l_lo) : 0.f;
    if (g_ + 8 < G)
      p.lse[q_row * p.lse_stride_t + (hbase + g_ + 8) * p.lse_stride_h] = l_hi > 0.f ? m_hi + log2f(l_hi) : 0.f;
  }
  if (timed_out && lane == 0 && p.status) atomicOr(p.status, 128);
}

// ------------------------------------------------------------------------------------------------ dQ
template <int D>
__global__ void __launch_bounds__(kWarps * 32, 1)
    slc_dq_tma_kernel(NsaAttnParams p, const __grid_constant__ CUtensorMap tmk, const __grid_constant__ CUtensorMap tmv) {
  constexpr int KS = D / 16, NT = D / 8, BS = 64;
  constexpr uint32_t TILE = BS * D * 2;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t base = smem_u32(smem_raw);
  WarpPipe wp{base + warp * 2 * TILE, base + warp * 2 * TILE + TILE, base + kWarps * 2 * TILE + warp * 16,
              base + kWarps * 2 * TILE + warp * 16 + 8, 0, 0};
  const int g_ = lane >> 2, c_ = lane & 3;
  // blockIdx.z = (kv head, group of 16 of its query heads): more than 16 query heads per kv head run as several groups
  const int Gall = p.QH / p.KH, HG = (Gall + 15) / 16;
  const int kh = blockIdx.z / HG, hg = blockIdx.z % HG;
  const int G = min(16, Gall - 16 * hg);
  const int64_t hbase = (int64_t)kh * Gall + 16 * hg;   // first query head of my group
  const Piece pc = load_piece(p.meta, blockIdx.y);
  const int tl = (gridDim.x - 1 - blockIdx.x) * kWarps + warp;
  if (tl >= pc.len) return;
  if (base & 1023u) {
    if (lane == 0 && p.status) atomicOr(p.status, 8);
    return;
  }
  const int t_abs = pc.off + tl;
  const int64_t q_row = pc.q_start + tl;
  const int nk = t_abs >= 0 ? t_abs / BS : -1;
  const int n_valid = min(p.hp.top_n, nk + 1);
  const float c2 = p.sm_scale * 1.4426950408889634f;
  if (lane == 0) {
    tc::mbar_init(wp.barK, 1);
    tc::mbar_init(wp.barV, 1);
    tc::fence_mbar_init();
  }
  __syncwarp();
  int my_blk = -1;
  if (lane < n_valid) my_blk = __ldg(p.topk + (int64_t)kh * p.topk_stride_h + q_row * p.hp.top_n + lane);
  unsigned todo = __ballot_sync(0xffffffffu, my_blk >= 0 && my_blk <= nk);
  int budget = tc::kWaitBudget;
  bool timed_out = false;

  uint32_t qf[KS][4], of[KS][4];
  load_a_global<D>(qf, reinterpret_cast<const __nv_bfloat16*>(p.q) + q_row * p.q_stride_t + hbase * D, G, lane);
  load_a_global<D>(of, reinterpret_cast<const __nv_bfloat16*>(p.dout) + q_row * p.do_stride_t + hbase * D, G, lane);
  const int h_lo = min(g_, G - 1), h_hi = min(g_ + 8, G - 1);
  const int64_t la = q_row * p.lse_stride_t + (hbase + h_lo) * p.lse_stride_h;
  const int64_t lb = q_row * p.lse_stride_t + (hbase + h_hi) * p.lse_stride_h;
  const float lse_lo = p.lse[la], lse_hi = p.lse[lb], dl_lo = p.delta[la], dl_hi = p.delta[lb];
  float dq[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) dq[i][0] = dq[i][1] = dq[i][2] = dq[i][3] = 0.f;

  int cur = -1;
  if (todo) {
    cur = __shfl_sync(0xffffffffu, my_blk, __ffs(todo) - 1);
    todo &= todo - 1;
    if (lane == 0) {
      fetch<D>(wp.bufK, wp.barK, &tmk, kh, pc.x_bos + cur * BS);
      fetch<D>(wp.bufV, wp.barV, &tmv, kh, pc.x_bos + cur * BS);
    }
  }
  while (cur >= 0) {
    const int nxt = todo ? __shfl_sync(0xffffffffu, my_blk, __ffs(todo) - 1) : -1;
    todo &= todo - 1;
    const int key0 = cur * BS;
    if (!tc::mbar_wait(wp.barK, wp.nK & 1, &budget)) timed_out = true;
    ++wp.nK;
    if (!tc::mbar_wait(wp.barV, wp.nV & 1, &budget)) timed_out = true;
    ++wp.nV;
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
          ldb_nk(b, wp.bufK, half * 32 + np * 16, kk, lane);
          mma_bf16(s[2 * np], qf[kk], b[0], b[1]);
          mma_bf16(s[2 * np + 1], qf[kk], b[2], b[3]);
          ldb_nk(b, wp.bufV, half * 32 + np * 16, kk, lane);
          mma_bf16(dp[2 * np], of[kk], b[0], b[1]);
          mma_bf16(dp[2 * np + 1], of[kk], b[2], b[3]);
        }
      }
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const int key = key0 + half * 32 + nt * 8 + 2 * c_;
        const bool v0 = key <= t_abs, v1 = key + 1 <= t_abs;
        const float p0 = v0 ? fast_exp2(fmaf(s[nt][0], c2, -lse_lo)) : 0.f;
        const float p1 = v1 ? fast_exp2(fmaf(s[nt][1], c2, -lse_lo)) : 0.f;
        const float p2 = v0 ? fast_exp2(fmaf(s[nt][2], c2, -lse_hi)) : 0.f;
        const float p3 = v1 ? fast_exp2(fmaf(s[nt][3], c2, -lse_hi)) : 0.f;
        dp[nt][0] = p0 * (dp[nt][0] - dl_lo);
        dp[nt][1] = p1 * (dp[nt][1] - dl_lo);
        dp[nt][2] = p2 * (dp[nt][2] - dl_hi);
        dp[nt][3] = p3 * (dp[nt][3] - dl_hi);
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const uint32_t a0 = pack_bf16(dp[2 * u][0], dp[2 * u][1]), a1 = pack_bf16(dp[2 * u][2], dp[2 * u][3]);
        const uint32_t a2 = pack_bf16(dp[2 * u + 1][0], dp[2 * u + 1][1]), a3 = pack_bf16(dp[2 * u + 1][2], dp[2 * u + 1][3]);
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
          uint32_t b[4];
          ldb_kn(b, wp.bufK, half * 32 + u * 16, np * 16, lane);
          mma_bf16(dq[2 * np], a0, a1, a2, a3, b[0], b[1]);
          mma_bf16(dq[2 * np + 1], a0, a1, a2, a3, b[2], b[3]);
        }
      }
    }
    __syncwarp();
    if (lane == 0 && nxt >= 0) {
      fetch<D>(wp.bufK, wp.barK, &tmk, kh, pc.x_bos + nxt * BS);
      fetch<D>(wp.bufV, wp.barV, &tmv, kh, pc.x_bos + nxt * BS);
    }
    cur = nxt;
  }

  __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(p.dq) + q_row * p.dq_stride_t + hbase * D + 2 * c_;
  const float sc = p.sm_scale;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    if (g_ < G) {
      uint32_t* dst = reinterpret_cast<uint32_t*>(op + g_ * D + nt * 8);
      float a = dq[nt][0] * sc, b = dq[nt][1] * sc;
      if (p.accumulate_dq) {
        const uint32_t old = *dst;
        a += bf16_lo(old);
        b += bf16_hi(old);
      }
      *dst = pack_bf16(a, b);
    }
    if (g_ + 8 < G) {
      uint32_t* dst = reinterpret_cast<uint32_t*>(op + (g_ + 8) * D + nt * 8);
      float a = dq[nt][2] * sc, b = dq[nt][3] * sc;
      if (p.accumulate_dq) {
        const uint32_t old = *dst;
        a += bf16_lo(old);
        b += bf16_hi(old);
      }
      *dst = pack_bf16(a, b);
    }
  }
  if (timed_out && lane == 0 && p.status) atomicOr(p.status, 256);
}

// returns 1 when not applicable (unaligned tensors; a paged cache in backward or with pages under 64 rows): the
// fragment-direct kernels then run
int launch_slc_tma(const NsaAttnParams* p, cudaStream_t st, bool backward) {
  if (p->n_k_rows <= 0) return 1;
  if (p->meta.kv_table && (backward || p->meta.page_size < 64 || (p->meta.page_size & (p->meta.page_size - 1)))) return 1;
  if ((((uintptr_t)p->k | (uintptr_t)p->v) & 15) || (p->k_stride_t * 2) % 16 || (p->v_stride_t * 2) % 16) return 1;
  const int D = p->D;
  CUtensorMap tmk, tmv;
  if (!tma::make_map(&tmk, p->k, p->n_k_rows, p->KH, D, p->k_stride_t, 64, 1) ||
      !tma::make_map(&tmv, p->v, p->n_k_rows, p->KH, D, p->v_stride_t, 64, 1)) {
    set_error("slc_attn: cuTensorMapEncodeTiled failed or is unavailable");
    return NSA_ERR_CUDA;
  }
  const size_t smem = (size_t)kWarps * 2 * 64 * D * 2 + kWarps * 16;
  dim3 grid((p->meta.max_piece_len + kWarps - 1) / kWarps, p->meta.n_pieces, p->KH * ((p->QH / p->KH + 15) / 16));
  cudaError_t e;
#define NSA_LAUNCH(KERNEL)                                                                              \
  e = cudaFuncSetAttribute(KERNEL, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);             \
  if (e != cudaSuccess) {                                                                               \
    set_error("slc_attn: cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));                      \
    return NSA_ERR_CUDA;                                                                                \
  }                                                                                                     \
  KERNEL<<<grid, kWarps * 32, smem, st>>>(*p, tmk, tmv);
  if (backward) {
    if (D == 128) { NSA_LAUNCH(slc_dq_tma_kernel<128>) } else { NSA_LAUNCH(slc_dq_tma_kernel<64>) }
  } else {
    if (D == 128) { NSA_LAUNCH(slc_fwd_tma_kernel<128>) } else { NSA_LAUNCH(slc_fwd_tma_kernel<64>) }
  }
#undef NSA_LAUNCH
  return check_launch(backward ? "slc_attn_bwd(dq)" : "slc_attn_fwd");
}

}  // namespace nsa
