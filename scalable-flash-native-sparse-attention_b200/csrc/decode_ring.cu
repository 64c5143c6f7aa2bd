// One decode step of NSA over a paged KV cache in a single kernel, with the cache tiles streamed by TMA.
//
// CTA = (sequence, kv head): one producer warp and six consumer warps.  The producer walks a job list -- every 64-row K/V
// tile the step has to read, in the order the branches need them -- and copies each job's K and V tile (one bulk tensor
// load per 64-column slab; a 64-row tile never straddles a page) into a ring of five 2-tile slots, as far ahead as the ring
// allows: ~150 KB per SM are in flight all the time, whatever the consumers are doing.  (In decode_fused.cu every warp
// fetches its own tile, K then V into the same buffer, and computes in between: half the bytes in flight, and the kernel
// reached 0.53 of the copy bandwidth.)  Each consumer owns the jobs assigned to it, keeps one running softmax state in
// registers and releases a slot as soon as it has multiplied the tile.  The query heads of the kv head are the 16 rows of
// the warp-level MMA tile, as in warp_tile_smem.cuh.
//
//   0. the window of 32 tokens ending at the new token is pooled into the new compressed K/V row (when it completes one)
//   1. compressed attention: tiles of compressed K/V round-robin over the six consumers            -> cmp_o, lse
//   2. block scores: the same K tiles again (from L2), P[j] = sum_heads exp2(s - lse)               -> pcm[]
//   3. top-n on consumer 0 (pool 4 -> 1 + the row before, then rounds of warp-wide arg-max; ties: lowest block index) WHILE
//   4. consumers 4-5 work through the sliding-window tiles and consumers 1-3 through the forced blocks; then the free
//      blocks round-robin over consumers 0-3 (the producer waits for the selection before it fetches them)
//   5. o = sigmoid(w0) cmp_o + sigmoid(w1) slc_o + sigmoid(w2) swa_o
// Partial softmax states are merged through shared memory after 1 and after 4; that region holds the score arrays in
// between.  Bytes read per (sequence, kv head): compressed K twice and V once, 16 selected blocks and <= 9 window tiles.
#include "tma.cuh"
#include "warp_tile_smem.cuh"

namespace nsa {

constexpr int RING_NC = 6;        // consumer warps
constexpr int JOB_CMP_KV = 0, JOB_CMP_K = 1, JOB_WIN = 2, JOB_SLC = 3;

__host__ __device__ constexpr int job_pack(int type, int cons, int idx) { return type | (cons << 2) | (idx << 5); }

template <int D>
__global__ void __launch_bounds__(32 * (RING_NC + 1), 1)
    decode_ring_kernel(NsaDecodeParams p, int n_slots, int job_cap, const __grid_constant__ CUtensorMap tmk,
                       const __grid_constant__ CUtensorMap tmv) {
  using namespace tc;
  constexpr int CH = D / 8, STATE = 32 + 16 * D, SLABS = D / 64;
  constexpr uint32_t TILE_BYTES = 64 * D * 2, SLAB_BYTES = 64 * 128;
  constexpr int NCT = RING_NC * 32;   // consumer threads
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t ring = smem_u32(smem_raw);                       // n_slots x (K tile, V tile)
  unsigned char* after_ring = smem_raw + (size_t)n_slots * 2 * TILE_BYTES;
  float* state = reinterpret_cast<float*>(after_ring);            // RING_NC x STATE floats; the score arrays between the merges
  const size_t region = (size_t)max(RING_NC * STATE, p.y_cap + 8 + p.y_cap / 4 + 8) * 4;
  float* pcm = state;                       // [y_cap + 8] head-summed probabilities of the compressed rows (index +1)
  float* psl = state + p.y_cap + 8;         // [y_cap/4 + 8] block scores
  float* cmp_o_s = reinterpret_cast<float*>(after_ring + region);  // [16][D] merged output of the compressed branch
  float* lse_s = cmp_o_s + 16 * D;                                // [16]
  int* sel = reinterpret_cast<int*>(lse_s + 16);                  // [32]
  int* jobs = sel + 32;                                           // [job_cap]
  const uint32_t bars = (smem_u32(jobs + job_cap) + 7u) & ~7u;    // full[n_slots], empty[n_slots], sel_ready
  auto full = [&](int s) { return bars + 8 * s; };
  auto empty = [&](int s) { return bars + 8 * (n_slots + s); };
  const uint32_t sel_ready = bars + 16 * n_slots;
  const uint32_t issued = sel_ready + 8;   // number of jobs whose loads have been issued (written by the producer)

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g_ = lane >> 2, c_ = lane & 3;
  const int b = blockIdx.x, kh = blockIdx.y;
  const int G = p.QH / p.KH;
  const int ctx = p.context_lens[b];
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.o) + (int64_t)b * p.o_stride_t + (int64_t)kh * G * D;
  if (ring & 1023u) {   // the swizzled tile layout needs 1 KB alignment of the ring
    if (tid == 0 && p.status) atomicOr(p.status, 8);
    return;
  }
  if (ctx <= 0) {
    for (int i = tid; i < G * CH; i += blockDim.x) reinterpret_cast<uint4*>(out)[i] = make_uint4(0, 0, 0, 0);
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

  const int n_ct = (Y + 63) >> 6;
  const int lo = max(0, t - W);
  const int w_k0 = (lo >> 6) << 6;                       // first window tile
  const int n_wt = ((t - w_k0) >> 6) + 1;                // window tiles
  const int n_valid = min(top_n, nk + 1);
  const int nf = min(ni + nl, n_valid);                  // forced slots
  const int n_free = n_valid - nf;
  const int n_jobs = 2 * n_ct + nf + n_wt + n_free;

  // ---- set-up: barriers, the job list, the new compressed row
  if (tid == 0) {
    for (int s = 0; s < n_slots; ++s) {
      mbar_init(full(s), 1);
      mbar_init(empty(s), 1);
    }
    mbar_init(sel_ready, 1);
    asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(issued), "r"(0) : "memory");
    fence_mbar_init();
    // job list: (type, consumer, index).  Phase 4 is ordered so that the ring always holds work for both consumer groups:
    // forced blocks (consumers 1-3), two window tiles (4-5), then two selected blocks for every further window tile.
    int n = 0;
    for (int i = 0; i < n_ct; ++i) jobs[n++] = job_pack(JOB_CMP_KV, i % RING_NC, i);
    for (int i = 0; i < n_ct; ++i) jobs[n++] = job_pack(JOB_CMP_K, i % RING_NC, i);
    for (int s = 0; s < nf; ++s) jobs[n++] = job_pack(JOB_SLC, 1 + s % 3, s);
    int wi = 0, fi = 0;
    for (; wi < min(n_wt, 2); ++wi) jobs[n++] = job_pack(JOB_WIN, 4 + (wi & 1), wi);
    while (wi < n_wt || fi < n_free) {
      for (int u = 0; u < 2 && fi < n_free; ++u, ++fi) jobs[n++] = job_pack(JOB_SLC, fi & 3, nf + fi);
      if (wi < n_wt) { jobs[n++] = job_pack(JOB_WIN, 4 + (wi & 1), wi); ++wi; }
    }
  }
  {
    const int slot = p.slot_mapping ? p.slot_mapping[b] : -1;
    if (slot >= 0 && ctx >= ks && tid < 2 * CH) {   // K by threads 0..CH-1, V by the next CH threads
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
      fence_proxy_async_global();   // the row is read below by bulk tensor loads of this CTA
    }
  }
  __syncthreads();
  int budget = kWaitBudget;
  bool timed_out = false;

  if (warp == RING_NC) {
    // ================================================= producer (one lane)
    if (lane == 0) {
      for (int j = 0; j < n_jobs; ++j) {
        const int job = jobs[j], type = job & 3, idx = job >> 5;
        const int s = j % n_slots;
        if (j >= n_slots && !mbar_wait(empty(s), ((j / n_slots) - 1) & 1, &budget)) timed_out = true;
        int row;
        if (type == JOB_CMP_KV || type == JOB_CMP_K) {
          row = (int)cmprow(idx << 6);
        } else if (type == JOB_WIN) {
          row = (int)tokrow(w_k0 + (idx << 6));
        } else {
          if (idx >= nf && idx == nf && !mbar_wait(sel_ready, 0, &budget)) timed_out = true;   // first free block: the list is there
          const int blk = idx >= nf ? sel[idx] : (idx < ni ? idx : nk - (idx - ni));
          row = (int)tokrow(max(0, min(blk, nk)) << 6);
        }
        const uint32_t dst = ring + (uint32_t)s * 2 * TILE_BYTES;
        tma::expect_tx(full(s), type == JOB_CMP_K ? TILE_BYTES : 2 * TILE_BYTES);
#pragma unroll
        for (int sl = 0; sl < SLABS; ++sl) {
          tma::load_3d(dst + sl * SLAB_BYTES, &tmk, sl * 64, kh, row, full(s));
          if (type != JOB_CMP_K) tma::load_3d(dst + TILE_BYTES + sl * SLAB_BYTES, &tmv, sl * 64, kh, row, full(s));
        }
        asm volatile("st.release.cta.shared::cta.b32 [%0], %1;\n" ::"r"(issued), "r"(j + 1) : "memory");
      }
    }
  } else {
    // ================================================= consumers
    const int cw = warp, ctid = tid;       // consumer warp 0..5, consumer thread 0..191
    uint32_t qf[D / 16][4];
    wts::load_q<D>(qf, reinterpret_cast<const __nv_bfloat16*>(p.q) + (int64_t)b * p.q_stride_t + (int64_t)kh * G * D, G, lane);
    const float c2 = p.sm_scale * 1.4426950408889634f;
    // A slot is used by different consumers in turn, so a consumer can get to its wait while the slot's barrier is still
    // one or more phases behind, where a parity test means nothing.  It therefore first waits until the producer has
    // issued its job (the barrier is then in that job's phase, open or complete), and only then for the data.
    auto wait_job = [&](int j) {
      int seen = 0;
      for (int i = 0; i < budget; ++i) {
        asm volatile("ld.acquire.cta.shared::cta.b32 %0, [%1];\n" : "=r"(seen) : "r"(issued) : "memory");
        if (seen > j) break;
      }
      if (seen <= j) {
        timed_out = true;
        budget = 8;
      }
      if (!mbar_wait(full(j % n_slots), (j / n_slots) & 1, &budget)) timed_out = true;
    };
    auto release = [&](int j) {
      __syncwarp();
      if (lane == 0) {
        fence_proxy_async();
        mbar_arrive(empty(j % n_slots));
      }
    };
    // merge the states of consumers [w0, w0+nw) for row r, column c: the normalised value, optionally the lse
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

    int j = 0;
    // ---- 1. compressed attention
    {
      wts::Acc<D> acc;
      acc.init();
      for (; j < n_ct; ++j) {
        if (((jobs[j] >> 2) & 7) != cw) continue;
        const int j0 = (jobs[j] >> 5) << 6;
        wait_job(j);
        const uint32_t bk = ring + (uint32_t)(j % n_slots) * 2 * TILE_BYTES;
        wts::attend64_smem<D>(acc, qf, bk, bk + TILE_BYTES, [&](int i) { return j0 + i < Y; }, min(64, Y - j0), c2, lane);
        release(j);
      }
      wts::store_state<D>(acc, state + cw * STATE, lane);
    }
    named_barrier(1, NCT);
    for (int idx = ctid; idx < 16 * D; idx += NCT) {
      const int r = idx / D, c = idx - r * D;
      float l;
      cmp_o_s[idx] = merged(0, RING_NC, r, c, &l);
      if (c == 0) lse_s[r] = l;
    }
    named_barrier(1, NCT);   // the states are dead until phase 4 is over: the score arrays live there

    // ---- 2. head-summed probabilities of every compressed row -> pcm[1 + j]
    {
      const float nl_lo = (g_ < G) ? -lse_s[g_] : 0.f, nl_hi = (g_ + 8 < G) ? -lse_s[g_ + 8] : 0.f;
      const bool h_lo = g_ < G, h_hi = g_ + 8 < G;
      if (ctid == 0) pcm[0] = 0.f;
      for (; j < 2 * n_ct; ++j) {
        if (((jobs[j] >> 2) & 7) != cw) continue;
        const int j0 = (jobs[j] >> 5) << 6;
        wait_job(j);
        float s[8][4];
        wts::scores64<D>(s, qf, ring + (uint32_t)(j % n_slots) * 2 * TILE_BYTES, lane);
        release(j);
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
    named_barrier(1, NCT);

    // ---- 3 + 4. selection on consumer 0; window tiles on consumers 4-5, selected blocks on consumers 0-3
    const int n_blk = nk + 1;
    if (cw == 0) {
      for (int blk = lane; blk < n_blk; blk += 32) {
        auto at = [&](int jj) { return (jj >= 0 && jj < Y) ? pcm[1 + jj] : 0.f; };
        const int jj = 4 * blk;
        float pv = at(jj - 1) + ((2.f * at(jj) + 2.f * at(jj + 1)) + (2.f * at(jj + 2) + at(jj + 3)));
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
      __syncwarp();
      if (lane == 0) mbar_arrive(sel_ready);
    }
    {
      wts::Acc<D> acc;
      acc.init();
      bool have_sel = cw == 0;
      for (; j < n_jobs; ++j) {
        const int job = jobs[j];
        if (((job >> 2) & 7) != cw) continue;
        const int type = job & 3, idx = job >> 5;
        int k0;
        if (type == JOB_WIN) {
          k0 = w_k0 + (idx << 6);
        } else {
          if (idx >= nf && !have_sel) {
            if (!mbar_wait(sel_ready, 0, &budget)) timed_out = true;
            have_sel = true;
          }
          const int blk = idx >= nf ? sel[idx] : (idx < ni ? idx : nk - (idx - ni));
          k0 = max(0, min(blk, nk)) << 6;
          if (blk < 0 || blk > nk) k0 = -1;   // an unused slot: its tile was fetched (block 0) but takes no part
        }
        wait_job(j);
        const uint32_t bk = ring + (uint32_t)(j % n_slots) * 2 * TILE_BYTES;
        if (k0 >= 0) {
          if (type == JOB_WIN)
            wts::attend64_smem<D>(acc, qf, bk, bk + TILE_BYTES, [&](int x) { return k0 + x >= lo && k0 + x <= t; }, min(64, t - k0 + 1), c2, lane);
          else
            wts::attend64_smem<D>(acc, qf, bk, bk + TILE_BYTES, [&](int x) { return k0 + x <= t; }, min(64, t - k0 + 1), c2, lane);
        }
        release(j);
      }
      named_barrier(1, NCT);   // every read of the score arrays is done: the states may be written again
      wts::store_state<D>(acc, state + cw * STATE, lane);
    }
    named_barrier(1, NCT);
    // ---- 5. merge + gated combine
    const __nv_bfloat16* wp = reinterpret_cast<const __nv_bfloat16*>(p.w) + (int64_t)b * p.w_stride_t + (int64_t)kh * G * 3;
    for (int idx = ctid; idx < G * D; idx += NCT) {
      const int r = idx / D, c = idx - r * D;
      const float slc = merged(0, 4, r, c, nullptr), swa = merged(4, 2, r, c, nullptr);
      const float s0 = 1.f / (1.f + __expf(-__bfloat162float(wp[r * 3 + 0])));
      const float s1 = 1.f / (1.f + __expf(-__bfloat162float(wp[r * 3 + 1])));
      const float s2 = 1.f / (1.f + __expf(-__bfloat162float(wp[r * 3 + 2])));
      out[idx] = __float2bfloat16(s0 * cmp_o_s[idx] + s1 * slc + s2 * swa);
    }
  }
  if (timed_out && p.status) atomicOr(p.status, 2048);
}

// returns 1 when the configuration is not covered (decode_fused_kernel then runs), 0 on launch, < 0 on error
int launch_decode_ring(const NsaDecodeParams* p, cudaStream_t st) {
  const int D = p->D;
  if (p->cache_rows <= 0 || (p->cache_stride_t * 2) % 16 || (((uintptr_t)p->k_cache | (uintptr_t)p->v_cache) & 15)) return 1;
  const size_t tile = (size_t)64 * D * 2;
  const size_t region = (size_t)max(RING_NC * (32 + 16 * D), p->y_cap + 8 + p->y_cap / 4 + 8) * 4;
  const int job_cap = 2 * ((p->y_cap + 63) / 64) + 2 * p->hp.top_n + p->hp.window / 64 + 8;
  const size_t fixed = region + ((size_t)16 * D + 16 + 32 + job_cap) * 4 + 8 + 16 * 8 + 16 + 1024;
  int n_slots = (int)((227 * 1024 - fixed) / (2 * tile));
  if (n_slots > 5) n_slots = 5;
  if (n_slots < 3) return 1;
  const size_t smem = (size_t)n_slots * 2 * tile + fixed;
  CUtensorMap tmk, tmv;
  if (!tma::make_map(&tmk, p->k_cache, p->cache_rows, p->KH, D, p->cache_stride_t, 64, 1) ||
      !tma::make_map(&tmv, p->v_cache, p->cache_rows, p->KH, D, p->cache_stride_t, 64, 1))
    return 1;
  cudaError_t e = (D == 128) ? cudaFuncSetAttribute(decode_ring_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                             : cudaFuncSetAttribute(decode_ring_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_error("decode_fused: cudaFuncSetAttribute(%zu B) failed: %s", smem, cudaGetErrorString(e));
    return NSA_ERR_CUDA;
  }
  dim3 grid(p->B, p->KH);
  if (D == 128) decode_ring_kernel<128><<<grid, 32 * (RING_NC + 1), smem, st>>>(*p, n_slots, job_cap, tmk, tmv);
  else decode_ring_kernel<64><<<grid, 32 * (RING_NC + 1), smem, st>>>(*p, n_slots, job_cap, tmk, tmv);
  return check_launch("decode_fused");
}

}  // namespace nsa
