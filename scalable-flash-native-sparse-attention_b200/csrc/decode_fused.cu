// One decode step of NSA for a batch of sequences over a paged KV cache, fused into a single kernel.
// CTA = (sequence, kv head), 8 warps.  The query heads of the kv head are the 16 rows of the warp-level MMA tile and
// every 64-row K/V tile is copied from the cache pages into the warp's private shared-memory buffer with all its
// cp.async copies in flight at once (see warp_tile_smem.cuh); the KV range of each branch is split over the warps and
// their partial softmax states are merged through shared memory:
//   0. the window of 32 tokens ending at the new token is pooled into the new compressed K/V row (when it completes one)
//   1. compressed attention: 64-row tiles of compressed K/V round-robin over the 8 warps  -> cmp_o, lse
//   2. block scores: the same K tiles again, P[j] = sum_heads exp2(s - lse), pooled 4 -> 1 (+ the row before)
//   3. top-n on warp 0: forced blocks + (top_n - forced) rounds of warp-wide arg-max (ties: lowest block index)
//   4. selected blocks on warps 0-4 (the forced ones start before the selection is known), sliding-window tiles on
//      warps 5-7, concurrently with 3
//   5. o = sigmoid(w0) cmp_o + sigmoid(w1) slc_o + sigmoid(w2) swa_o
// Bytes read per (sequence, kv head): compressed K twice and V once, 16 selected blocks and <= 9 window tiles of K and V.
#include <cstdlib>
#include "warp_tile_smem.cuh"

namespace nsa {

template <int D>
__global__ void __launch_bounds__(256, 1) decode_fused_kernel(NsaDecodeParams p) {
  constexpr int CH = D / 8, STATE = 32 + 16 * D;
  constexpr uint32_t TILE_BYTES = 64 * D * 2;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  float* sm = reinterpret_cast<float*>(smem_raw + 8 * TILE_BYTES);   // the first 8 x TILE_BYTES: one K/V tile buffer per warp
  float* state = sm;                        // 8 x STATE floats; reused for the score arrays between phases 1 and 4
  float* cmp_o_s = sm + 8 * STATE;          // [16][D]
  float* lse_s = cmp_o_s + 16 * D;          // [16]
  float* red_v = lse_s + 16;                // [8] arg-max scratch
  int* red_i = reinterpret_cast<int*>(red_v + 8);
  int* sel = red_i + 8;                     // [32]
  float* pcm = state;                       // [y_cap + 8] head-summed probabilities of the compressed rows (index +1)
  float* psl = state + p.y_cap + 8;         // [y_cap/4 + 8] block scores

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g_ = lane >> 2, c_ = lane & 3;
  const int b = blockIdx.x, kh = blockIdx.y;
  const int G = p.QH / p.KH;
  const int ctx = p.context_lens[b];
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.o) + (int64_t)b * p.o_stride_t + (int64_t)kh * G * D;
  if (ctx <= 0) {
    for (int i = tid; i < G * CH; i += 256) reinterpret_cast<uint4*>(out)[i] = make_uint4(0, 0, 0, 0);
    if (p.topk_out && tid < p.hp.top_n) p.topk_out[((int64_t)kh * p.B + b) * p.hp.top_n + tid] = -1;
    return;
  }
  const int t = ctx - 1, nk = t >> 6;
  const int ks = p.hp.kernel_size, st = p.hp.stride, W = p.hp.window;
  const int top_n = p.hp.top_n, ni = p.hp.num_init, nl = p.hp.num_local;
  int Y = ctx >= ks ? (ctx - ks) / st + 1 : 0;
  if (Y > p.y_cap) {
    if (tid == 0 && p.status) atomicOr(p.status, 32);
    Y = p.y_cap;
  }
  const int sh = 31 - __clz(p.page_size), pmask = p.page_size - 1;
  const int32_t* xt = p.kv_table + (int64_t)b * p.kv_table_stride;
  const int32_t* yt = p.cmp_table + (int64_t)b * p.cmp_table_stride;
  auto tokrow = [&](int r) -> int64_t { return ((int64_t)xt[r >> sh] << sh) + (r & pmask); };
  auto cmprow = [&](int j) -> int64_t { return ((int64_t)yt[j >> sh] << sh) + (j & pmask); };
  __nv_bfloat16* kc = reinterpret_cast<__nv_bfloat16*>(p.k_cache) + kh * D;
  __nv_bfloat16* vc = reinterpret_cast<__nv_bfloat16*>(p.v_cache) + kh * D;
  const int64_t cs = p.cache_stride_t;

  // ---- 0. pool the new compressed row (K by threads 0..CH-1, V by the next CH threads)
  {
    const int slot = p.slot_mapping ? p.slot_mapping[b] : -1;
    if (slot >= 0 && ctx >= ks && tid < 2 * CH) {
      __nv_bfloat16* cache = tid < CH ? kc : vc;
      const int c = tid % CH;
      const int start = ((ctx - ks) / st) * st;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int i = 0; i < ks; ++i) {
        uint4 u = *reinterpret_cast<const uint4*>(cache + tokrow(start + i) * cs + c * 8);
        acc[0] += bf16_lo(u.x); acc[1] += bf16_hi(u.x); acc[2] += bf16_lo(u.y); acc[3] += bf16_hi(u.y);
        acc[4] += bf16_lo(u.z); acc[5] += bf16_hi(u.z); acc[6] += bf16_lo(u.w); acc[7] += bf16_hi(u.w);
      }
      const float inv = 1.f / (float)ks;
      uint4 w4;
      w4.x = pack_bf16(acc[0] * inv, acc[1] * inv); w4.y = pack_bf16(acc[2] * inv, acc[3] * inv);
      w4.z = pack_bf16(acc[4] * inv, acc[5] * inv); w4.w = pack_bf16(acc[6] * inv, acc[7] * inv);
      *reinterpret_cast<uint4*>(cache + (int64_t)slot * cs + c * 8) = w4;
    }
    __syncthreads();  // the row is read below by other threads of this CTA (plain loads, no read-only path)
  }

  uint32_t qf[D / 16][4];
  wts::load_q<D>(qf, reinterpret_cast<const __nv_bfloat16*>(p.q) + (int64_t)b * p.q_stride_t + (int64_t)kh * G * D, G, lane);
  const uint32_t buf = smem_u32(smem_raw) + warp * TILE_BYTES;
  const float c2 = p.sm_scale * 1.4426950408889634f;
  const int n_ct = (Y + 63) >> 6;

  // merge the states of warps [w0, w0+nw) for row r, column c: returns the normalised value, optionally the lse
  auto merged = [&](int w0, int nw, int r, int c, float* lse_out) -> float {
    float M = -INFINITY;
    for (int w = 0; w < nw; ++w) M = fmaxf(M, state[(w0 + w) * STATE + r]);
    if (M == -INFINITY) {
      if (lse_out) *lse_out = 0.f;
      return 0.f;
    }
    float L = 0.f, O = 0.f;
    for (int w = 0; w < nw; ++w) {
      const float* sp = state + (w0 + w) * STATE;
      const float f = fast_exp2(sp[r] - M);
      L += sp[16 + r] * f;
      O += sp[32 + r * D + c] * f;
    }
    if (lse_out) *lse_out = L > 0.f ? M + log2f(L) : 0.f;
    return L > 0.f ? O / L : 0.f;
  };

  // ---- 1. compressed attention
  {
    wts::Acc<D> acc;
    acc.init();
    for (int tile = warp; tile < n_ct; tile += 8) {
      const int j0 = tile << 6;
      wts::attend64<D>(acc, qf, buf, kc, vc, cs, cs, [&](int i) { return cmprow(min(j0 + i, Y - 1)); }, [&](int i) { return j0 + i < Y; }, c2, lane);
    }
    wts::store_state<D>(acc, state + warp * STATE, lane);
  }
  __syncthreads();
  for (int idx = tid; idx < 16 * D; idx += 256) {
    const int r = idx / D, c = idx - r * D;
    float l;
    cmp_o_s[idx] = merged(0, 8, r, c, &l);
    if (c == 0) lse_s[r] = l;
  }
  __syncthreads();  // states are dead from here until phase 4: the score arrays live there

  // ---- 2. head-summed probabilities of every compressed row -> pcm[1 + j]
  {
    const float nl_lo = (g_ < G) ? -lse_s[g_] : 0.f, nl_hi = (g_ + 8 < G) ? -lse_s[g_ + 8] : 0.f;
    const bool h_lo = g_ < G, h_hi = g_ + 8 < G;
    if (tid == 0) pcm[0] = 0.f;
    for (int tile = warp; tile < n_ct; tile += 8) {
      const int j0 = tile << 6;
      float s[8][4];
      wts::fill_async<D>(buf, kc, cs, [&](int i) { return cmprow(min(j0 + i, Y - 1)); }, lane);
      wts::fill_wait();
      wts::scores64<D>(s, qf, buf, lane);
      __syncwarp();
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const int col = j0 + nt * 8 + 2 * c_;
        float e0 = (h_lo && col < Y) ? fast_exp2(fmaf(s[nt][0], c2, nl_lo)) : 0.f;
        float e1 = (h_lo && col + 1 < Y) ? fast_exp2(fmaf(s[nt][1], c2, nl_lo)) : 0.f;
        float e2 = (h_hi && col < Y) ? fast_exp2(fmaf(s[nt][2], c2, nl_hi)) : 0.f;
        float e3 = (h_hi && col + 1 < Y) ? fast_exp2(fmaf(s[nt][3], c2, nl_hi)) : 0.f;
        float v0 = e0 + e2, v1 = e1 + e3;
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
          v0 += __shfl_xor_sync(0xffffffffu, v0, o);
          v1 += __shfl_xor_sync(0xffffffffu, v1, o);
        }
        if (g_ == nt) {
          pcm[1 + col] = v0;
          pcm[2 + col] = v1;
        }
      }
    }
  }
  __syncthreads();
  // ---- 3 + 4. selection on warp 0, selected blocks on warps 0-4, sliding window on warps 5-7.
  // The window tiles and the forced blocks do not depend on the selection, so warps 5-7 and 1-3 start on them at once and
  // the memory system stays busy while warp 0 picks the free blocks (pooling 4 -> 1, then rounds of warp-wide arg-max;
  // ties: lowest block index).
  const int n_blk = nk + 1;
  const int n_valid = min(top_n, nk + 1);
  const int n_free = max(0, n_valid - ni - nl);
  {
    wts::Acc<D> acc;
    acc.init();
    auto block_tile = [&](int blk) {
      const int k0 = blk << 6;
      wts::attend64<D>(acc, qf, buf, kc, vc, cs, cs, [&](int x) { return tokrow(min(k0 + x, t)); }, [&](int x) { return k0 + x <= t; }, c2, lane);
    };
    if (warp >= 5) {
      const int lo = max(0, t - W);
      for (int k0 = ((lo >> 6) << 6) + 64 * (warp - 5); k0 <= t; k0 += 192)
        wts::attend64<D>(acc, qf, buf, kc, vc, cs, cs, [&](int x) { return tokrow(min(k0 + x, t)); },
                         [&](int x) { return k0 + x >= lo && k0 + x <= t; }, c2, lane);
    } else {
      if (warp == 0) {
        for (int blk = lane; blk < n_blk; blk += 32) {
          auto at = [&](int j) { return (j >= 0 && j < Y) ? pcm[1 + j] : 0.f; };
          const int j = 4 * blk;
          float pv = at(j - 1) + ((2.f * at(j) + 2.f * at(j + 1)) + (2.f * at(j + 2) + at(j + 3)));
          psl[blk] = (blk >= ni && blk <= nk - nl) ? pv : -1.f;   // forced blocks are not candidates
        }
        sel[lane] = -1;
        __syncwarp();
        for (int r = 0; r < n_free; ++r) {
          float bv = -1.f;
          int bi = 0x7fffffff;
          for (int blk = lane; blk < n_blk; blk += 32) {
            const float v = psl[blk];
            if (v > bv) {  // ascending scan keeps the lowest index among equals
              bv = v;
              bi = blk;
            }
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) {
              bv = ov;
              bi = oi;
            }
          }
          if (lane == 0 && bv >= 0.f) {
            sel[ni + nl + r] = bi;
            psl[bi] = -1.f;
          }
          __syncwarp();
        }
        if (lane < ni) sel[lane] = (lane <= nk) ? lane : -1;
        else if (lane < ni + nl) sel[lane] = (lane <= nk) ? nk - (lane - ni) : -1;
        __syncwarp();
        if (p.topk_out && lane < top_n) p.topk_out[((int64_t)kh * p.B + b) * top_n + lane] = sel[lane];
      } else if (warp - 1 < ni + nl && warp - 1 < n_valid) {
        // forced slot warp-1: initial blocks 0.., then the local blocks nk, nk-1, ..
        const int slot = warp - 1;
        const int blk = slot < ni ? slot : nk - (slot - ni);
        if (blk >= 0 && blk <= nk) block_tile(blk);
      }
      tc::named_barrier(1, 160);   // warps 0-4: the selection is in sel[]
      // forced slots beyond the three head-start warps (other forced-block counts), then the free slots round-robin
      for (int i = 0; i < n_valid; ++i) {
        int owner;
        if (i < ni + nl) owner = (i + 1 <= 3) ? -1 : (i % 5);          // slots 0..2 were taken by warps 1..3 above
        else owner = ((i - ni - nl) + 4) % 5;
        if (owner != warp) continue;
        const int blk = sel[i];
        if (blk >= 0 && blk <= nk) block_tile(blk);
      }
    }
    __syncthreads();  // every read of the score arrays is done: the states may be written again
    wts::store_state<D>(acc, state + warp * STATE, lane);
  }
  __syncthreads();
  // ---- 5. merge + gated combine
  const __nv_bfloat16* wp = reinterpret_cast<const __nv_bfloat16*>(p.w) + (int64_t)b * p.w_stride_t + (int64_t)kh * G * 3;
  for (int idx = tid; idx < G * D; idx += 256) {
    const int r = idx / D, c = idx - r * D;
    const float slc = merged(0, 5, r, c, nullptr), swa = merged(5, 3, r, c, nullptr);
    const float s0 = 1.f / (1.f + __expf(-__bfloat162float(wp[r * 3 + 0])));
    const float s1 = 1.f / (1.f + __expf(-__bfloat162float(wp[r * 3 + 1])));
    const float s2 = 1.f / (1.f + __expf(-__bfloat162float(wp[r * 3 + 2])));
    out[idx] = __float2bfloat16(s0 * cmp_o_s[idx] + s1 * slc + s2 * swa);
  }
}

}  // namespace nsa

using namespace nsa;

namespace nsa {
int launch_decode_ring(const NsaDecodeParams* p, cudaStream_t st);   // decode_ring.cu
int decode_cluster_size_query(const NsaDecodeParams* p);               // decode_ring.cu
}

extern "C" int nsa_decode_cluster_size(const NsaDecodeParams* p) {
  NSA_REQUIRE(p && p->B >= 0 && p->KH > 0 && p->page_size > 0 && p->y_cap > 0, NSA_ERR_BAD_ARG, "decode_cluster_size: bad sizes");
  NSA_REQUIRE(p->D == 64 || p->D == 128, NSA_ERR_UNSUPPORTED_SHAPE, "decode_cluster_size: head dim %d not supported (64 or 128)", p->D);
  static const bool per_warp = [] { const char* e = getenv("NSA_DECODE_PER_WARP_LOADS"); return e && e[0] == '1'; }();
  return per_warp ? 1 : decode_cluster_size_query(p);
}

extern "C" int nsa_decode_fused(const NsaDecodeParams* p, void* stream) {
  NSA_REQUIRE(p && p->q && p->k_cache && p->v_cache && p->w && p->o && p->context_lens && p->kv_table && p->cmp_table, NSA_ERR_BAD_ARG,
              "decode_fused: null pointer");
  NSA_REQUIRE(p->D == 64 || p->D == 128, NSA_ERR_UNSUPPORTED_SHAPE, "decode_fused: head dim %d not supported (64 or 128)", p->D);
  NSA_REQUIRE(p->KH > 0 && p->QH % p->KH == 0 && p->QH / p->KH <= 16, NSA_ERR_UNSUPPORTED_SHAPE,
              "decode_fused: at most 16 query heads per kv head (QH=%d, KH=%d)", p->QH, p->KH);
  NSA_REQUIRE(p->hp.kernel_size == 32 && p->hp.stride == 16 && p->hp.block_size == 64, NSA_ERR_UNSUPPORTED_SHAPE,
              "decode_fused: only kernel_size=32, stride=16, block_size=64 (got %d/%d/%d)", p->hp.kernel_size, p->hp.stride, p->hp.block_size);
  NSA_REQUIRE(p->hp.top_n >= 1 && p->hp.top_n <= 32 && p->hp.num_init + p->hp.num_local <= p->hp.top_n, NSA_ERR_BAD_ARG,
              "decode_fused: bad top_n / forced block counts");
  NSA_REQUIRE(p->page_size >= 64 && (p->page_size & (p->page_size - 1)) == 0, NSA_ERR_UNSUPPORTED_SHAPE,
              "decode_fused: page_size=%d must be a power of two >= 64", p->page_size);
  NSA_REQUIRE(p->y_cap > 0 && p->y_cap % 4 == 0, NSA_ERR_BAD_ARG, "decode_fused: y_cap=%d must be a positive multiple of 4", p->y_cap);
  if (p->B <= 0) return NSA_OK;
  // the TMA-fed kernel (a ring of K/V tiles filled by a producer warp) when the cache can be addressed by bulk tensor loads;
  // NSA_DECODE_PER_WARP_LOADS=1 keeps the kernel below, in which every warp fetches its own tiles
  static const bool per_warp = [] { const char* e = getenv("NSA_DECODE_PER_WARP_LOADS"); return e && e[0] == '1'; }();
  if (!per_warp) {
    const int rc = launch_decode_ring(p, (cudaStream_t)stream);
    if (rc <= 0) return rc;
  }
  const int D = p->D;
  const size_t states = (size_t)8 * (32 + 16 * D) * 4, scores = ((size_t)p->y_cap + 8 + p->y_cap / 4 + 8) * 4;
  NSA_REQUIRE(scores <= states, NSA_ERR_UNSUPPORTED_SHAPE, "decode_fused: y_cap=%d too large for head dim %d (max %d)", p->y_cap, D,
              (int)((states / 4 - 16) * 4 / 5));
  const size_t smem = (size_t)8 * 64 * D * 2 + states + (size_t)16 * D * 4 + 64 + 64 + 128;
  cudaError_t e = (D == 128) ? cudaFuncSetAttribute(decode_fused_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                             : cudaFuncSetAttribute(decode_fused_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_error("decode_fused: cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
    return NSA_ERR_CUDA;
  }
  dim3 grid(p->B, p->KH);
  if (D == 128) decode_fused_kernel<128><<<grid, 256, smem, (cudaStream_t)stream>>>(*p);
  else decode_fused_kernel<64><<<grid, 256, smem, (cudaStream_t)stream>>>(*p);
  return check_launch("decode_fused");
}
