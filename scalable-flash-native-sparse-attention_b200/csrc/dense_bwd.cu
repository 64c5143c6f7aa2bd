// Backward kernels of the dense-range branches on the Blackwell tensor core (tcgen05 + tensor memory).
//
//  dense_dq_tc_kernel<D,MODE>  dQ of the compressed / sliding-window branch: one CTA per 128-row query tile
//                              (tokens x the G heads of a kv head), loops over its K/V tiles:
//                              S = QK^T, P = exp2(S*c - lse), dP = dO V^T, dS = P*(dP - delta), dQ += dS K.
//  (dK/dV of all three branches live in dkdv_tc.cu; this file launches them.)
// P and dS are rounded to bf16 before the second-stage products, as in the reference kernels
// (flash_nsa/ops/compress_attn.py:311-325, flash_nsa/ops/select_attn.py:262-280).
#include "tc_common.cuh"

namespace nsa {

constexpr int MODE_CMP = 0;
constexpr int MODE_SWA = 1;
constexpr int MODE_SLC = 2;

void launch_delta(const void* o, const void* dout, float* delta, int64_t T, int H, int D, int64_t o_stride_t,
                  int64_t do_stride_t, int64_t lse_stride_t, int64_t lse_stride_h, cudaStream_t st);
int check_attn_common(const NsaAttnParams* p, const char* name, bool need_y);

// ------------------------------------------------------------------------------------------------ dQ
// CTA = 128 threads = one 128-row query tile; thread i owns row i (tensor-memory lane i).  Per 64-row K/V tile:
//   S  = Q K^T (TMEM cols 0..63),  dP = dO V^T (cols 64..127)           A from shared memory (K-major)
//   dS = exp2(S*c - lse) * (dP - delta) -> bf16 -> TMEM cols 0..31 (over S, which has been read)
//   dQ += dS K (cols 128..128+D)                                        A = dS from tensor memory, B = K tile (MN-major)
// K tiles are double-buffered, the V tile single-buffered (it is free again as soon as dP has been read); two CTAs
// share an SM (256 TMEM columns, 112 KB of shared memory each).
template <int D, int MODE>
__global__ void __launch_bounds__(128, 2) dense_dq_tc_kernel(NsaAttnParams p) {
  using namespace tc;
  constexpr int BM = 128, BN = 64, CH = D / 8;
  constexpr uint32_t Q_BYTES = BM * D * 2, KV_BYTES = BN * D * 2, K_SLAB = BN * 128, Q_SLAB = BM * 128;
  constexpr uint32_t TM_S = 0, TM_DP = 64, TM_DQ = 128, TM_COLS = 256;
  constexpr uint32_t IDESC_S = make_idesc(BM, BN, false), IDESC_Q = make_idesc(BM, D, true);

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  const uint32_t sQ = base, sO = sQ + Q_BYTES;
  const uint32_t sK = sO + Q_BYTES;          // 2 stages
  const uint32_t sV = sK + 2 * KV_BYTES;     // 1 stage
  const uint32_t bar_s = sV + KV_BYTES, bar_o = bar_s + 8, tm_slot = bar_o + 8;

  const int tid = threadIdx.x, warp = tid >> 5;
  const int G = p.QH / p.KH;
  const int TOK = BM / G;
  const int tile = gridDim.x - 1 - blockIdx.x;
  const int kh = blockIdx.z;
  const Piece pc = load_piece(p.meta, blockIdx.y);
  const int t0 = tile * TOK;
  if (t0 >= pc.len) return;
  if (base & 1023u) {  // the operand layout needs 1024-byte aligned tiles
    if (tid == 0 && p.status) atomicOr(p.status, 8);
    return;
  }
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

  const int row = tid;
  const int tok = row / G, g = row - tok * G;
  const bool row_ok = tok < ntok;
  const int t_abs = tabs_min + tok;
  const int64_t q_row = pc.q_start + t0 + tok;
  __nv_bfloat16* dq_row = reinterpret_cast<__nv_bfloat16*>(p.dq) + q_row * p.dq_stride_t + (int64_t)(kh * G + g) * D;

  if (ntiles == 0) {
    if (row_ok && !p.accumulate_dq) {
      uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int c = 0; c < CH; ++c) reinterpret_cast<uint4*>(dq_row)[c] = z;
    }
    return;
  }
  if (tid == 0) {
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc(tm_slot, TM_COLS);
  {
    const __nv_bfloat16* qb = reinterpret_cast<const __nv_bfloat16*>(p.q) + (int64_t)(pc.q_start + t0) * p.q_stride_t + (int64_t)kh * G * D;
    const __nv_bfloat16* ob = reinterpret_cast<const __nv_bfloat16*>(p.dout) + (int64_t)(pc.q_start + t0) * p.do_stride_t + (int64_t)kh * G * D;
    for (int i = tid; i < BM * CH; i += 128) {
      int r = i / CH, c = i % CH;
      int tk = r / G, gg = r - tk * G;
      bool ok = tk < ntok;
      cp_async16(sQ + slab_off(BM, r, c), qb + (ok ? (int64_t)tk * p.q_stride_t + gg * D : 0) + c * 8, ok);
      cp_async16(sO + slab_off(BM, r, c), ob + (ok ? (int64_t)tk * p.do_stride_t + gg * D : 0) + c * 8, ok);
    }
  }
  auto load_k = [&](int it) {
    int kv0 = kv_lo + it * BN;
    fill_tile_async<D>(sK + (it & 1) * KV_BYTES, kbase + (int64_t)kv0 * p.k_stride_t, p.k_stride_t, BN, min(BN, kv_hi - kv0), tid, 128);
  };
  auto load_v = [&](int it) {
    int kv0 = kv_lo + it * BN;
    fill_tile_async<D>(sV, vbase + (int64_t)kv0 * p.v_stride_t, p.v_stride_t, BN, min(BN, kv_hi - kv0), tid, 128);
  };
  load_k(0);
  load_v(0);
  cp_async_commit();
  float lse = 0.f, dl = 0.f;
  if (row_ok) {
    int64_t a = q_row * p.lse_stride_t + (int64_t)(kh * G + g) * p.lse_stride_h;
    lse = p.lse[a];
    dl = p.delta[a];
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  uint32_t tmem;
  asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(tmem) : "r"(tm_slot));
  const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
  const float c2 = p.sm_scale * 1.4426950408889634f;
  int budget = kWaitBudget;
  bool timed_out = false;

  for (int it = 0; it < ntiles; ++it) {
    // previous tile's dQ MMA done: the S/dS columns and K stage (it+1)&1 are free
    if (it > 0 && !mbar_wait(bar_o, (it - 1) & 1, &budget)) timed_out = true;
    cp_async_wait<0>();
    fence_proxy_async();
    __syncthreads();
    if (it + 1 < ntiles) load_k(it + 1);
    cp_async_commit();
    const uint32_t tK = sK + (it & 1) * KV_BYTES;
    const int kv0 = kv_lo + it * BN;
    if (tid == 0) {
      fence_after_sync();
#pragma unroll
      for (int k = 0; k < D / 16; ++k) {
        uint32_t ao = (k >> 2) * Q_SLAB + (k & 3) * 32, bo = (k >> 2) * K_SLAB + (k & 3) * 32;
        mma_ss(tmem + TM_S, desc_kmajor(sQ + ao), desc_kmajor(tK + bo), IDESC_S, k > 0);
      }
#pragma unroll
      for (int k = 0; k < D / 16; ++k) {
        uint32_t ao = (k >> 2) * Q_SLAB + (k & 3) * 32, bo = (k >> 2) * K_SLAB + (k & 3) * 32;
        mma_ss(tmem + TM_DP, desc_kmajor(sO + ao), desc_kmajor(sV + bo), IDESC_S, k > 0);
      }
      mma_commit(bar_s);
    }
    if (!mbar_wait(bar_s, it & 1, &budget)) timed_out = true;
    fence_after_sync();
    if (it + 1 < ntiles) load_v(it + 1);  // dP has been computed: the V stage is free
    cp_async_commit();

    uint32_t ds[32];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      uint32_t sv[32], dv[32];
      tmem_ld32(lane_base + TM_S + half * 32, sv);
      tmem_ld32(lane_base + TM_DP + half * 32, dv);
      wait_ld();
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        float x[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int col = kv0 + half * 32 + i + e;
          bool vis;
          if (MODE == MODE_CMP)
            vis = (col * st + ks - 1 <= t_abs) && (col < kv_hi);
          else
            vis = (col <= t_abs) && (col >= t_abs - W) && (col < kv_hi);
          float pv = (vis && row_ok) ? fast_exp2(fmaf(__uint_as_float(sv[i + e]), c2, -lse)) : 0.f;
          x[e] = pv * (__uint_as_float(dv[i + e]) - dl);
        }
        ds[half * 16 + (i >> 1)] = pack_bf16(x[0], x[1]);
      }
    }
    tmem_st32(lane_base + TM_S, ds);
    wait_st();
    fence_before_sync();
    __syncthreads();
    if (tid == 0) {
      fence_after_sync();
#pragma unroll
      for (int u = 0; u < BN / 16; ++u)
        mma_ts(tmem + TM_DQ, tmem + TM_S + u * 8, desc_mnmajor(tK + u * 2048, K_SLAB), IDESC_Q, (it > 0 || u > 0));
      mma_commit(bar_o);
    }
  }
  if (!mbar_wait(bar_o, (ntiles - 1) & 1, &budget)) timed_out = true;
  fence_after_sync();
  cp_async_wait<0>();

  const float sc = p.sm_scale;
#pragma unroll
  for (int c = 0; c < D / 32; ++c) {
    uint32_t o[32];
    tmem_ld32(lane_base + TM_DQ + c * 32, o);
    wait_ld();
    if (row_ok) {
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        float f[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(o[q4 * 8 + e]) * sc;
        uint4* dst = reinterpret_cast<uint4*>(dq_row + c * 32 + q4 * 8);
        if (p.accumulate_dq) {
          uint4 old = *dst;
          f[0] += bf16_lo(old.x); f[1] += bf16_hi(old.x); f[2] += bf16_lo(old.y); f[3] += bf16_hi(old.y);
          f[4] += bf16_lo(old.z); f[5] += bf16_hi(old.z); f[6] += bf16_lo(old.w); f[7] += bf16_hi(old.w);
        }
        uint4 w;
        w.x = pack_bf16(f[0], f[1]); w.y = pack_bf16(f[2], f[3]); w.z = pack_bf16(f[4], f[5]); w.w = pack_bf16(f[6], f[7]);
        *dst = w;
      }
    }
  }
  if (timed_out && p.status) atomicOr(p.status, 4);
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, TM_COLS);
}

template <int D, int MODE>
int launch_dkdv(const NsaAttnParams* p, cudaStream_t st, const char* name, dim3 grid, DkdvLaunch L);  // dkdv_tc.cu
int launch_dkdv128(const NsaAttnParams* p, cudaStream_t st, const char* name, bool cmp, int q_chunk);   // dkdv128_tc.cu
int launch_dq128(const NsaAttnParams* p, cudaStream_t st, const char* name, bool cmp);                  // dense_dq128_tc.cu

template <typename K>
static int set_smem(K kernel, size_t smem, const char* name) {
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_error("%s: cudaFuncSetAttribute failed: %s", name, cudaGetErrorString(e));
    return NSA_ERR_CUDA;
  }
  return NSA_OK;
}

template <int D, int MODE>
static int launch_dq(const NsaAttnParams* p, cudaStream_t st, const char* name) {
  const int G = p->QH / p->KH, TOK = 128 / G;
  size_t smem = (size_t)(2 * 128 + 3 * 64) * D * 2 + 64;
  int rc = set_smem(dense_dq_tc_kernel<D, MODE>, smem, name);
  if (rc) return rc;
  dim3 grid((p->meta.max_piece_len + TOK - 1) / TOK, p->meta.n_pieces, p->KH);
  dense_dq_tc_kernel<D, MODE><<<grid, 128, smem, st>>>(*p);
  return check_launch(name);
}

static int check_bwd(const NsaAttnParams* p, const char* name) {
  NSA_REQUIRE(p->lse && p->dout && p->delta && p->dq && p->dk && p->dv, NSA_ERR_BAD_ARG, "%s: lse, dout, delta, dq, dk, dv are required", name);
  NSA_REQUIRE(p->QH / p->KH <= 64, NSA_ERR_UNSUPPORTED_SHAPE, "%s: more than 64 query heads per kv head", name);
  NSA_REQUIRE(p->dk_stride_t % 2 == 0 && p->dv_stride_t % 2 == 0, NSA_ERR_BAD_ARG, "%s: dk/dv row strides must be even", name);
  return NSA_OK;
}

}  // namespace nsa

using namespace nsa;

extern "C" int nsa_cmp_attn_bwd(const NsaAttnParams* p, void* stream) {
  int rc = check_attn_common(p, "cmp_attn_bwd", true);
  if (rc) return rc;
  if ((rc = check_bwd(p, "cmp_attn_bwd"))) return rc;
  if (p->meta.n_pieces <= 0 || p->meta.max_piece_len <= 0 || p->n_q_rows <= 0) return NSA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int ph = p->phases ? p->phases : 7;
  if (ph & 1)
    launch_delta(p->o, p->dout, p->delta, p->n_q_rows, p->QH, p->D, p->o_stride_t, p->do_stride_t, p->lse_stride_t, p->lse_stride_h, st);
  if ((ph & 2) && p->meta.y_maxlen > 0) {
    rc = launch_dkdv128(p, st, "cmp_attn_bwd(dkdv)", true, 2048);
    if (rc < 0) return rc;
  }
  if ((ph & 2) && p->meta.y_maxlen > 0 && rc == 1) {
    DkdvLaunch L{2048};
    dim3 grid((p->meta.y_maxlen + 63) / 64, (p->meta.max_piece_len + L.q_chunk - 1) / L.q_chunk, p->meta.n_pieces * p->KH);
    rc = (p->D == 128) ? launch_dkdv<128, MODE_CMP>(p, st, "cmp_attn_bwd(dkdv)", grid, L)
                       : launch_dkdv<64, MODE_CMP>(p, st, "cmp_attn_bwd(dkdv)", grid, L);
    if (rc) return rc;
  }
  if (!(ph & 4)) return check_launch("cmp_attn_bwd");
  rc = launch_dq128(p, st, "cmp_attn_bwd(dq)", true);   // contiguous K/V: 128-row tiles, TMA
  if (rc != 1) return rc;
  return (p->D == 128) ? launch_dq<128, MODE_CMP>(p, st, "cmp_attn_bwd(dq)") : launch_dq<64, MODE_CMP>(p, st, "cmp_attn_bwd(dq)");
}

extern "C" int nsa_swa_bwd(const NsaAttnParams* p, void* stream) {
  int rc = check_attn_common(p, "swa_bwd", false);
  if (rc) return rc;
  if ((rc = check_bwd(p, "swa_bwd"))) return rc;
  if (p->meta.n_pieces <= 0 || p->meta.max_piece_len <= 0 || p->n_q_rows <= 0) return NSA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int ph = p->phases ? p->phases : 7;
  if (ph & 1)
    launch_delta(p->o, p->dout, p->delta, p->n_q_rows, p->QH, p->D, p->o_stride_t, p->do_stride_t, p->lse_stride_t, p->lse_stride_h, st);
  if (ph & 2) {
    rc = launch_dkdv128(p, st, "swa_bwd(dkdv)", false, 0);
    if (rc < 0) return rc;
  }
  if ((ph & 2) && rc == 1) {
    DkdvLaunch L{0};
    dim3 grid((p->meta.max_piece_len + p->hp.window + 63) / 64 + 1, 1, p->meta.n_pieces * p->KH);
    rc = (p->D == 128) ? launch_dkdv<128, MODE_SWA>(p, st, "swa_bwd(dkdv)", grid, L) : launch_dkdv<64, MODE_SWA>(p, st, "swa_bwd(dkdv)", grid, L);
    if (rc) return rc;
  }
  if (!(ph & 4)) return check_launch("swa_bwd");
  rc = launch_dq128(p, st, "swa_bwd(dq)", false);
  if (rc != 1) return rc;
  return (p->D == 128) ? launch_dq<128, MODE_SWA>(p, st, "swa_bwd(dq)") : launch_dq<64, MODE_SWA>(p, st, "swa_bwd(dq)");
}
