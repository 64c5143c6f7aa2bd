// Forward of the compressed and sliding-window branches on the Blackwell tensor core (tcgen05 + tensor memory).
//
// CTA = 128 threads = one 128-row query tile: (128/G consecutive tokens) x (the G query heads of one kv head).
// Thread i owns row i: it reads its row of S from tensor-memory lane i, so softmax needs no cross-thread traffic.
//   S  = Q K^T       tcgen05.mma, A = Q tile (smem, K-major), B = K tile (smem, K-major), D = TMEM columns [0,64)
//   P  = exp2(S*c-m) registers -> bf16 -> TMEM columns [64,96)
//   O += P V         tcgen05.mma, A = P (TMEM), B = V tile (smem, MN-major), D = TMEM columns [128,128+D)
// The running maximum is only raised when a row's tile maximum exceeds it by more than 2^8 (the rescale of O in
// tensor memory is then done by the row's own thread); l and the final normalisation use the same reference, so the
// result is exact.  K/V tiles of 64 rows are double-buffered with cp.async in the swizzled operand layout.
// The chain S-MMA -> softmax -> PV-MMA of one CTA is sequential; two CTAs share an SM (256 TMEM columns, ~97 KB of
// shared memory each) so one CTA's MMAs overlap the other's softmax.
#include "tc_common.cuh"

namespace nsa {

constexpr int MODE_CMP = 0;
constexpr int MODE_SWA = 1;
int check_attn_common(const NsaAttnParams* p, const char* name, bool need_y);
int launch_fwd128(const NsaAttnParams* p, cudaStream_t st, const char* name, bool cmp);   // dense_fwd128_tc.cu

template <int D, int MODE>
__global__ void __launch_bounds__(128, 2) dense_fwd_tc_kernel(NsaAttnParams p) {
  using namespace tc;
  constexpr int BM = 128, BN = 64, CH = D / 8, SLABS = D / 64;
  constexpr uint32_t Q_BYTES = BM * D * 2, KV_BYTES = BN * D * 2, K_SLAB = BN * 128;
  constexpr uint32_t TM_S = 0, TM_P = 64, TM_O = 128, TM_COLS = 256;
  constexpr uint32_t IDESC_S = make_idesc(BM, BN, false), IDESC_O = make_idesc(BM, D, true);

  extern __shared__ unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = base;
  const uint32_t sK = sQ + Q_BYTES;             // 2 stages
  const uint32_t sV = sK + 2 * KV_BYTES;        // 2 stages
  const uint32_t bar_s = sV + 2 * KV_BYTES;     // 8 B each
  const uint32_t bar_o = bar_s + 8;
  const uint32_t tm_slot = bar_o + 8;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
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

  int kv_lo, kv_hi;
  const __nv_bfloat16* kbase = reinterpret_cast<const __nv_bfloat16*>(p.k) + kh * D;
  const __nv_bfloat16* vbase = reinterpret_cast<const __nv_bfloat16*>(p.v) + kh * D;
  if (MODE == MODE_CMP) {
    kv_lo = 0;
    kv_hi = (tabs_max >= ks - 1) ? min(pc.y_len, (tabs_max - (ks - 1)) / st + 1) : 0;
  } else {
    kv_lo = max(0, tabs_min - W);
    kv_hi = min(tabs_max + 1, pc.x_len);
  }
  const int ntiles = (kv_hi > kv_lo) ? (kv_hi - kv_lo + BN - 1) / BN : 0;

  // this thread's row
  const int row = tid;
  const int tok = row / G, g = row - tok * G;
  const bool row_ok = tok < ntok;
  const int t_abs = tabs_min + tok;
  const int64_t q_row = pc.q_start + t0 + tok;

  if (ntiles == 0) {  // nothing visible for the whole tile: zeros
    if (row_ok) {
      uint4 z = make_uint4(0, 0, 0, 0);
      uint4* o = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.o) + q_row * p.o_stride_t + (int64_t)(kh * G + g) * D);
#pragma unroll
      for (int c = 0; c < CH; ++c) o[c] = z;
      if (p.lse) p.lse[q_row * p.lse_stride_t + (int64_t)(kh * G + g) * p.lse_stride_h] = 0.f;
    }
    return;
  }

  // ---- set-up: barriers, tensor memory, Q tile, first K/V tile
  if (tid == 0) {
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc(tm_slot, TM_COLS);
  {
    const __nv_bfloat16* qb = reinterpret_cast<const __nv_bfloat16*>(p.q) + (int64_t)(pc.q_start + t0) * p.q_stride_t +
                              (int64_t)kh * G * D;
    for (int i = tid; i < BM * CH; i += 128) {
      int r = i / CH, c = i % CH;
      int tk = r / G, gg = r - tk * G;
      bool ok = tk < ntok;
      cp_async16(sQ + slab_off(BM, r, c), qb + (ok ? (int64_t)tk * p.q_stride_t + gg * D : 0) + c * 8, ok);
    }
  }
  auto load_kv = [&](int it) {
    int kv0 = kv_lo + it * BN;
    int valid = min(BN, kv_hi - kv0);
    fill_kv_tile_async<D, MODE == MODE_CMP>(sK + (it & 1) * KV_BYTES, kbase, p.k_stride_t, pc, kv0, BN, valid, tid, 128);
    fill_kv_tile_async<D, MODE == MODE_CMP>(sV + (it & 1) * KV_BYTES, vbase, p.v_stride_t, pc, kv0, BN, valid, tid, 128);
  };
  load_kv(0);
  cp_async_commit();
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  uint32_t tmem;
  asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(tmem) : "r"(tm_slot));
  const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);  // this warp's 32 lanes

  const float c2 = p.sm_scale * 1.4426950408889634f;
  float m_ref = -INFINITY, l_run = 0.f;
  int budget = kWaitBudget;
  bool timed_out = false;

  for (int it = 0; it < ntiles; ++it) {
    // the previous tile's P.V has finished: its K/V stage and the P columns may be overwritten
    if (it > 0 && !mbar_wait(bar_o, (it - 1) & 1, &budget)) timed_out = true;
    // K/V tile `it` has landed (and is visible to the tensor core); start fetching the next one
    cp_async_wait<0>();
    fence_proxy_async();
    __syncthreads();
    if (it + 1 < ntiles) load_kv(it + 1);
    cp_async_commit();
    const uint32_t tK = sK + (it & 1) * KV_BYTES, tV = sV + (it & 1) * KV_BYTES;
    const int kv0 = kv_lo + it * BN;

    if (tid == 0) {
      fence_after_sync();
#pragma unroll
      for (int k = 0; k < D / 16; ++k) {
        uint32_t koff = (k >> 2) * (BM * 128) + (k & 3) * 32;
        uint32_t boff = (k >> 2) * K_SLAB + (k & 3) * 32;
        mma_ss(tmem + TM_S, desc_kmajor(sQ + koff), desc_kmajor(tK + boff), IDESC_S, k > 0);
      }
      mma_commit(bar_s);
    }
    if (!mbar_wait(bar_s, it & 1, &budget)) timed_out = true;
    fence_after_sync();

    // ---- my row of S
    uint32_t sr[64];
    {
      uint32_t a[32], b[32];
      tmem_ld32(lane_base + TM_S, a);
      tmem_ld32(lane_base + TM_S + 32, b);
      wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        sr[i] = a[i];
        sr[32 + i] = b[i];
      }
    }
    bool full;
    if (MODE == MODE_CMP)
      full = ((kv0 + BN - 1) * st + ks - 1 <= tabs_min) && (kv0 + BN <= kv_hi);
    else
      full = (kv0 + BN - 1 <= tabs_min) && (kv0 >= tabs_max - W) && (kv0 + BN <= kv_hi);
    float mx = -INFINITY;
    if (full) {
#pragma unroll
      for (int i = 0; i < 64; ++i) {
        float v = __uint_as_float(sr[i]) * c2;
        sr[i] = __float_as_uint(v);
        mx = fmaxf(mx, v);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 64; ++i) {
        int col = kv0 + i;
        bool vis;
        if (MODE == MODE_CMP)
          vis = (col * st + ks - 1 <= t_abs) && (col < kv_hi);
        else
          vis = (col <= t_abs) && (col >= t_abs - W) && (col < kv_hi);
        float v = vis ? __uint_as_float(sr[i]) * c2 : -INFINITY;
        sr[i] = __float_as_uint(v);
        mx = fmaxf(mx, v);
      }
    }
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
    const float mu = (m_ref == -INFINITY) ? 0.f : m_ref;
    float rs = 0.f;
    uint32_t pk[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      float e0 = fast_exp2(__uint_as_float(sr[2 * i]) - mu), e1 = fast_exp2(__uint_as_float(sr[2 * i + 1]) - mu);
      rs += e0 + e1;
      pk[i] = pack_bf16(e0, e1);
    }
    l_run = l_run * alpha + rs;
    if (it > 0 && __any_sync(0xffffffffu, need)) {  // rescale my O row (warp-uniform branch, per-lane factor)
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(lane_base + TM_O + c * 32, o);
        wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
        tmem_st32(lane_base + TM_O + c * 32, o);
      }
    }
    tmem_st32(lane_base + TM_P, pk);
    wait_st();
    fence_before_sync();
    __syncthreads();
    if (tid == 0) {
      fence_after_sync();
#pragma unroll
      for (int u = 0; u < BN / 16; ++u)
        mma_ts(tmem + TM_O, tmem + TM_P + u * 8, desc_mnmajor(tV + u * 2048, K_SLAB), IDESC_O, (it > 0 || u > 0));
      mma_commit(bar_o);
    }
  }
  if (!mbar_wait(bar_o, (ntiles - 1) & 1, &budget)) timed_out = true;
  fence_after_sync();
  cp_async_wait<0>();

  // ---- epilogue: my row of O
  const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
  __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.o) + q_row * p.o_stride_t + (int64_t)(kh * G + g) * D;
#pragma unroll
  for (int c = 0; c < D / 32; ++c) {
    uint32_t o[32];
    tmem_ld32(lane_base + TM_O + c * 32, o);
    wait_ld();
    if (row_ok) {
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        uint4 w;
        w.x = pack_bf16(__uint_as_float(o[q4 * 8 + 0]) * inv, __uint_as_float(o[q4 * 8 + 1]) * inv);
        w.y = pack_bf16(__uint_as_float(o[q4 * 8 + 2]) * inv, __uint_as_float(o[q4 * 8 + 3]) * inv);
        w.z = pack_bf16(__uint_as_float(o[q4 * 8 + 4]) * inv, __uint_as_float(o[q4 * 8 + 5]) * inv);
        w.w = pack_bf16(__uint_as_float(o[q4 * 8 + 6]) * inv, __uint_as_float(o[q4 * 8 + 7]) * inv);
        *reinterpret_cast<uint4*>(orow + c * 32 + q4 * 8) = w;
      }
    }
  }
  if (row_ok && p.lse)
    p.lse[q_row * p.lse_stride_t + (int64_t)(kh * G + g) * p.lse_stride_h] = l_run > 0.f ? m_ref + log2f(l_run) : 0.f;
  if (timed_out && p.status) atomicOr(p.status, 1);

  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, TM_COLS);
}

template <int D, int MODE>
static int launch_fwd_tc(const NsaAttnParams* p, cudaStream_t st, const char* name) {
  const int G = p->QH / p->KH;
  const int TOK = 128 / G;
  size_t smem = (size_t)(128 + 4 * 64) * D * 2 + 64 + 1024;
  cudaError_t e = cudaFuncSetAttribute(dense_fwd_tc_kernel<D, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_error("%s: cudaFuncSetAttribute failed: %s", name, cudaGetErrorString(e));
    return NSA_ERR_CUDA;
  }
  dim3 grid((p->meta.max_piece_len + TOK - 1) / TOK, p->meta.n_pieces, p->KH);
  dense_fwd_tc_kernel<D, MODE><<<grid, 128, smem, st>>>(*p);
  return check_launch(name);
}

}  // namespace nsa

using namespace nsa;

extern "C" int nsa_cmp_attn_fwd(const NsaAttnParams* p, void* stream) {
  int rc = check_attn_common(p, "cmp_attn_fwd", true);
  if (rc) return rc;
  NSA_REQUIRE(p->lse, NSA_ERR_BAD_ARG, "cmp_attn_fwd: lse is required");
  if (p->meta.n_pieces <= 0 || p->meta.max_piece_len <= 0) return NSA_OK;
  rc = launch_fwd128(p, (cudaStream_t)stream, "cmp_attn_fwd", true);   // contiguous K/V: 128-row tiles, TMA
  if (rc != 1) return rc;
  if (p->D == 128) return launch_fwd_tc<128, MODE_CMP>(p, (cudaStream_t)stream, "cmp_attn_fwd");
  return launch_fwd_tc<64, MODE_CMP>(p, (cudaStream_t)stream, "cmp_attn_fwd");
}

extern "C" int nsa_swa_fwd(const NsaAttnParams* p, void* stream) {
  int rc = check_attn_common(p, "swa_fwd", false);
  if (rc) return rc;
  NSA_REQUIRE(p->hp.window >= 0, NSA_ERR_BAD_ARG, "swa_fwd: negative window");
  if (p->meta.n_pieces <= 0 || p->meta.max_piece_len <= 0) return NSA_OK;
  rc = launch_fwd128(p, (cudaStream_t)stream, "swa_fwd", false);
  if (rc != 1) return rc;
  if (p->D == 128) return launch_fwd_tc<128, MODE_SWA>(p, (cudaStream_t)stream, "swa_fwd");
  return launch_fwd_tc<64, MODE_SWA>(p, (cudaStream_t)stream, "swa_fwd");
}
