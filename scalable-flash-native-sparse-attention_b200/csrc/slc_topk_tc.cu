// Block-importance scores + top-n selection on the Blackwell tensor core, operands staged by TMA.
//
// CTA = 128 consecutive query tokens x one kv head.  MMA rows are TOKENS (one query head per MMA), so a thread owns
// one token for the whole kernel and everything after the MMA is thread-local:
//   for each tile of 128 compressed rows, for each query head h of the kv head (in order h = 0..G-1):
//       S_h = Q_h K^T                      tcgen05.mma, Q_h tile [128 tokens x d] and K tile [128 rows x d] loaded by TMA
//       p[c] = exp2(S_h[c]*c - lse_h)      the thread's 128 columns, fp32; rows the token cannot see yet count as 0
//       blk[i] += p[4i] + 2 (p[4i+1] + p[4i+2] + p[4i+3]) + p[4i+4]     31 selection blocks, heads in order
//   merge the 31 block sums into the thread's sorted list of the best free blocks (value descending, block index
//   ascending).
// A tile starts one compressed row early and advances by 124 rows, so the "row before" of its first block is inside
// the tile and tiles are independent.  Three warp groups take three consecutive tiles of the SAME tokens, so one TMA
// load of Q_h feeds three MMAs; each group has one S buffer in tensor memory (the next head's product is issued as soon
// as the group has read the last column), and while one group waits for its product the other two keep the schedulers
// busy: with two groups the kernel was bound by instruction latency at two warps per scheduler.  Warp 12 issues the
// MMAs, warp 13 the TMA loads (14 warps are allocated as 16: 128 registers per thread).  At the end the lists of
// groups 1 and 2 are merged into group 0's.
// Nothing but the [kh, t, top_n] indices is written (optionally the block scores, for inspection).
#include "tma.cuh"

namespace nsa {

namespace {

constexpr int kList = 13;  // free slots per row handled by this kernel: top_n - num_init - num_local

__device__ __forceinline__ bool better(float av, int ai, float bv, int bi) { return av > bv || (av == bv && ai < bi); }

struct TopList {
  float v[kList];
  int i[kList];
  __device__ __forceinline__ void init() {
#pragma unroll
    for (int k = 0; k < kList; ++k) {
      v[k] = -1.f;
      i[k] = 0x7fffffff;
    }
  }
  // Candidate whose index is larger than every index in the list (a group meets its blocks in increasing order), so it
  // loses every tie: it goes behind all entries with v >= cv.  Position by 13 independent compares, then one shift
  // (no dependent chain, and the common "not good enough" case leaves after one compare).
  __device__ __forceinline__ void insert_newer(float cv, int ci) {
    if (!(cv > v[kList - 1])) return;
    int pos = 0;
#pragma unroll
    for (int k = 0; k < kList; ++k) pos += (v[k] >= cv) ? 1 : 0;
#pragma unroll
    for (int k = kList - 1; k >= 0; --k) {
      const bool here = (k == pos), shift = (k > pos);
      if (k > 0) {
        v[k] = here ? cv : (shift ? v[k - 1] : v[k]);
        i[k] = here ? ci : (shift ? i[k - 1] : i[k]);
      } else {
        v[k] = here ? cv : v[k];
        i[k] = here ? ci : i[k];
      }
    }
  }
  __device__ __forceinline__ void insert(float cv, int ci) {
    if (!better(cv, ci, v[kList - 1], i[kList - 1])) return;
    v[kList - 1] = cv;
    i[kList - 1] = ci;
#pragma unroll
    for (int k = kList - 1; k > 0; --k) {
      bool up = better(v[k], i[k], v[k - 1], i[k - 1]);
      float tv = v[k - 1];
      int ti = i[k - 1];
      v[k - 1] = up ? v[k] : tv;
      i[k - 1] = up ? i[k] : ti;
      v[k] = up ? tv : v[k];
      i[k] = up ? ti : i[k];
    }
  }
};

// The list for the half-precision scoring modes, where a score is 16 bits: one sortable word per entry,
// (half bits << 16) | (0xffff - block), so that a larger word means a better entry (higher score, then lower block index).
// Scores are non-negative, so their half bits order like the values; 0 marks an empty entry (a real entry has a block
// index below 0xffff).  With one-word entries the list is maintained by sorting networks instead of insertions: a tile's
// 32 candidate words are sorted (bitonic, 240 max/min pairs on registers with compile-time indices), and the best 16 of
// list and candidates are max(list[j], candidates[15 - j]), a bitonic sequence that 32 more pairs put back in order.  No
// branches, no divergence between the lanes of a warp, no long dependent chains: the per-entry insertion it replaces
// (31 candidates x ~70 dependent instructions, taken whenever ANY lane of the warp needed it) cost a quarter of the
// kernel's time.  The list keeps 16 entries (a power of two for the networks); the first 13 are the result.
struct PackedList {
  static constexpr int N = 16;
  uint32_t k[N];
  __device__ __forceinline__ void init() {
#pragma unroll
    for (int j = 0; j < N; ++j) k[j] = 0u;
  }
  static __device__ __forceinline__ uint32_t key(float rounded_score, int blk) {
    return ((uint32_t)__half_as_ushort(__float2half_rn(rounded_score)) << 16) | (uint32_t)(0xffff - blk);
  }
  template <int LEN>
  static __device__ __forceinline__ void bitonic_merge_desc(uint32_t (&c)[LEN]) {   // c bitonic -> c descending
#pragma unroll
    for (int j = LEN / 2; j > 0; j >>= 1) {
#pragma unroll
      for (int i = 0; i < LEN; ++i) {
        const int l = i ^ j;
        if (l > i) {
          const uint32_t a = c[i], b = c[l];
          c[i] = max(a, b);
          c[l] = min(a, b);
        }
      }
    }
  }
  static __device__ __forceinline__ void sort32_desc(uint32_t (&c)[32]) {
#pragma unroll
    for (int kk = 2; kk <= 32; kk <<= 1) {
#pragma unroll
      for (int j = kk >> 1; j > 0; j >>= 1) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int l = i ^ j;
          if (l > i) {
            const uint32_t a = c[i], b = c[l];
            const bool desc = (i & kk) == 0;
            c[i] = desc ? max(a, b) : min(a, b);
            c[l] = desc ? min(a, b) : max(a, b);
          }
        }
      }
    }
  }
  // b: 16 words in descending order (e.g. the head of a sorted candidate array, or another list)
  __device__ __forceinline__ void merge(const uint32_t* b) {
#pragma unroll
    for (int j = 0; j < N; ++j) k[j] = max(k[j], b[N - 1 - j]);
    bitonic_merge_desc<N>(k);
  }
  __device__ __forceinline__ int block(int j) const { return 0xffff - (int)(k[j] & 0xffffu); }
};

}  // namespace

// PACKED: the scores are rounded to half before they are compared (quant 1 or 2) and the lists hold one word per entry
template <int D, bool PACKED>
__global__ void __launch_bounds__(448, 1) slc_topk_tc_kernel(NsaTopkParams p, const __grid_constant__ CUtensorMap tmq,
                                                             const __grid_constant__ CUtensorMap tmk) {
  using namespace tc;
  constexpr int BM = 128, BN = 128, STEP = 124, NQ = 4, NW = 3, SLABS = D / 64;
  constexpr uint32_t TILE_BYTES = BM * D * 2, SLAB_BYTES = 128 * 128;
  constexpr uint32_t IDESC = make_idesc(BM, BN, false);

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  const uint32_t sQ = base;                       // NQ stages
  const uint32_t sK = sQ + NQ * TILE_BYTES;       // one tile per warp group
  const uint32_t bars = sK + NW * TILE_BYTES;
  const uint32_t q_full = bars, q_free = bars + 8 * NQ, k_full = bars + 16 * NQ, k_free = k_full + 8 * NW;
  const uint32_t s_full = k_free + 8 * NW, s_free = s_full + 8 * NW, tm_slot = s_free + 8 * NW;   // s_*[wg]

  const int tid = threadIdx.x, warp = tid >> 5;
  const int G = p.QH / p.KH;
  const int tile = gridDim.x - 1 - blockIdx.x;
  const int kh = blockIdx.z;
  const Piece pc = load_piece(p.meta, blockIdx.y);
  const int t0 = tile * BM;
  if (t0 >= pc.len) return;
  if (base & 1023u) {
    if (tid == 0 && p.status) atomicOr(p.status, 8);
    return;
  }
  const int ntok = min(BM, pc.len - t0);
  const int ks = p.hp.kernel_size, st = p.hp.stride, bs = p.hp.block_size;
  const int top_n = p.hp.top_n, ni = p.hp.num_init, nl = p.hp.num_local;
  const int tabs_max = pc.off + t0 + ntok - 1;
  const int nvis_max = (tabs_max >= ks - 1) ? min(pc.y_len, (tabs_max - (ks - 1)) / st + 1) : 0;
  const int n_tiles = max(nvis_max / STEP + 1, max(tabs_max, 0) / bs / 31 + 1);
  const int n_rounds = (n_tiles + NW - 1) / NW;   // each round: NW consecutive tiles, one per warp group
  const int N = n_rounds * G;                      // MMA steps per warp group

  if (tid == 0) {
    for (int s = 0; s < NQ; ++s) {
      mbar_init(q_full + 8 * s, 1);
      mbar_init(q_free + 8 * s, 1);
    }
    for (int w = 0; w < NW; ++w) {
      mbar_init(k_full + 8 * w, 1);
      mbar_init(k_free + 8 * w, 1);
      mbar_init(s_full + 8 * w, 1);
      mbar_init(s_free + 8 * w, 128);
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

  if (warp == 4 * NW + 1) {
    if ((tid & 31) == 0) {
      // ============================================ TMA producer: the K tiles of each round, the Q_h tile of every step
      const int q_row0 = pc.q_start + t0;
      auto load_q = [&](int n) {
        const int s = n % NQ;
        if (n >= NQ && !mbar_wait(q_free + 8 * s, ((n / NQ) - 1) & 1, &budget)) timed_out = true;
        tma::expect_tx(q_full + 8 * s, TILE_BYTES);
        const int head = kh * G + (n % G);
#pragma unroll
        for (int sl = 0; sl < SLABS; ++sl) tma::load_3d(sQ + s * TILE_BYTES + sl * SLAB_BYTES, &tmq, sl * 64, head, q_row0, q_full + 8 * s);
      };
      auto load_k = [&](int jr) {
        for (int w = 0; w < NW; ++w) {
          if (jr > 0 && !mbar_wait(k_free + 8 * w, (jr - 1) & 1, &budget)) timed_out = true;
          tma::expect_tx(k_full + 8 * w, TILE_BYTES);
          const int row = pc.y_bos + STEP * (NW * jr + w) - 1;
#pragma unroll
          for (int sl = 0; sl < SLABS; ++sl) tma::load_3d(sK + w * TILE_BYTES + sl * SLAB_BYTES, &tmk, sl * 64, kh, row, k_full + 8 * w);
        }
      };
      // the K tiles of round jr can only be fetched when the last MMA of round jr - 1 is done; by then the Q tiles of the
      // first NQ - 2 steps of round jr are already on their way (their stages were freed earlier)
      load_k(0);
      for (int n = 0; n < N; ++n) {
        load_q(n);
        const int m = n + 2 - NQ;                    // step m - 1 can complete with what has been requested so far
        if (m > 0 && m % G == 0) load_k(m / G);
      }
      for (int jr = max(1, (N + 1 - NQ) / G + 1); jr < n_rounds; ++jr) load_k(jr);
    }
  } else if (warp == 4 * NW) {
    if ((tid & 31) == 0) {
      // ============================================ MMA issue: one S buffer per warp group
      for (int jr = 0; jr < n_rounds; ++jr) {
        for (int h = 0; h < G; ++h) {
          const int n = jr * G + h, s = n % NQ;
          if (!mbar_wait(q_full + 8 * s, (n / NQ) & 1, &budget)) timed_out = true;
          for (int w = 0; w < NW; ++w) {
            if (h == 0 && !mbar_wait(k_full + 8 * w, jr & 1, &budget)) timed_out = true;
            if (n >= 1 && !mbar_wait(s_free + 8 * w, (n - 1) & 1, &budget)) timed_out = true;
            fence_after_sync();
#pragma unroll
            for (int k = 0; k < D / 16; ++k) {
              const uint32_t off = (k >> 2) * SLAB_BYTES + (k & 3) * 32;
              mma_ss(tmem + w * 128, desc_kmajor(sQ + s * TILE_BYTES + off), desc_kmajor(sK + w * TILE_BYTES + off), IDESC, k > 0);
            }
            mma_commit(s_full + 8 * w);
            if (h == G - 1) mma_commit(k_free + 8 * w);
          }
          mma_commit(q_free + 8 * s);
        }
      }
    }
  } else {
    // ============================================ NW warp groups: tiles NW*jr + wg of the same 128 tokens
    const int wg = warp >> 2, t = tid & 127;
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const bool tok_ok = t < ntok;
    const int t_abs = pc.off + t0 + t;
    const int64_t q_row = pc.q_start + t0 + (tok_ok ? t : 0);
    const int nvis = (tok_ok && t_abs >= ks - 1) ? min(pc.y_len, (t_abs - (ks - 1)) / st + 1) : 0;
    const int nk = (tok_ok && t_abs >= 0) ? t_abs / bs : -1;
    const float c2 = p.sm_scale * 1.4426950408889634f;
    const float* lse_p = p.lse + q_row * p.lse_stride_t + (int64_t)kh * G * p.lse_stride_h;
    const int64_t Tq = p.meta.piece_cu[p.meta.n_pieces];
    TopList lst;
    PackedList pl;
    if (PACKED) pl.init(); else lst.init();
    // Pooling is linear, so every head's probabilities go straight into the tile's 31 block sums (block i = columns
    // 4i .. 4i+4 with weights 1 2 2 2 1): 32 accumulators per thread instead of 128.
    float blk[32];

    for (int jr = 0; jr < n_rounds; ++jr) {
      const int j = NW * jr + wg;
      const int row0 = STEP * j - 1;                       // column c is compressed row row0 + c
      const bool full = (row0 >= 0) && (row0 + BN - 1 < nvis);   // no column of this tile is masked for my token
#pragma unroll
      for (int c = 0; c < 32; ++c) blk[c] = 0.f;
      float nlse = -__ldg(lse_p);
      for (int h = 0; h < G; ++h) {
        const int n = jr * G + h;
        const float cur = nlse;
        if (h + 1 < G) nlse = -__ldg(lse_p + (int64_t)(h + 1) * p.lse_stride_h);
        if (!mbar_wait(s_full + 8 * wg, n & 1, &budget)) timed_out = true;
        fence_after_sync();
#pragma unroll
        for (int q8 = 0; q8 < 8; ++q8) {
          uint32_t sv[16];
          tmem_ld16(lane_base + wg * 128 + q8 * 16, sv);
          wait_ld();
          if (q8 == 7) {   // every column of my S buffer has been read: the next head's product may overwrite it
            fence_before_sync();
            mbar_arrive(s_free + 8 * wg);
          }
          float e[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) e[i] = fmaf(__uint_as_float(sv[i]), c2, cur);
#pragma unroll
          for (int i = 0; i < 16; ++i) e[i] = fast_exp2(e[i]);
          if (!full) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int r = row0 + q8 * 16 + i;
              e[i] = (r >= 0 && r < nvis) ? e[i] : 0.f;
            }
          }
#pragma unroll
          for (int c = 0; c < 16; c += 4) {
            const int i = q8 * 4 + (c >> 2);
            blk[i] += fmaf(2.f, (e[c + 1] + e[c + 2]) + e[c + 3], e[c]);
            if (i > 0) blk[i - 1] += e[c];
          }
        }
      }
      // ---- this tile's 31 blocks
      if (PACKED) {
        uint32_t cand[32];
#pragma unroll
        for (int i = 0; i < 31; ++i) {
          float pv = blk[i];
          pv = __half2float(__float2half_rn(p.quant == 2 ? pv * pv * pv : pv));
          const int bi = 31 * j + i;
          if (p.probs && tok_ok && bi < (int)p.probs_stride_t)
            reinterpret_cast<__half*>(p.probs)[((int64_t)kh * Tq + q_row) * p.probs_stride_t + bi] = __float2half_rn(pv);
          cand[i] = (bi >= ni && bi <= nk - nl) ? PackedList::key(pv, bi) : 0u;
        }
        cand[31] = 0u;
        PackedList::sort32_desc(cand);
        pl.merge(cand);
      } else {
#pragma unroll
        for (int i = 0; i < 31; ++i) {
          const float pv = blk[i];
          const int bi = 31 * j + i;
          if (p.probs && tok_ok && bi < (int)p.probs_stride_t)
            reinterpret_cast<float*>(p.probs)[((int64_t)kh * Tq + q_row) * p.probs_stride_t + bi] = pv;
          if (bi >= ni && bi <= nk - nl) lst.insert_newer(pv, bi);
        }
      }
    }
    // ---- merge the other groups' lists into group 0's and write the row
    __syncwarp();
    float* mv = reinterpret_cast<float*>(smem_raw);            // the Q stages are idle now (all MMAs have completed)
    int* mi = reinterpret_cast<int*>(smem_raw + (NW - 1) * 128 * 16 * 4);
    named_barrier(1, 128 * NW);
    if (wg > 0) {
      if (PACKED) {
#pragma unroll
        for (int k = 0; k < PackedList::N; ++k) mi[((wg - 1) * PackedList::N + k) * 128 + t] = (int)pl.k[k];
      } else {
#pragma unroll
        for (int k = 0; k < kList; ++k) {
          mv[((wg - 1) * kList + k) * 128 + t] = lst.v[k];
          mi[((wg - 1) * kList + k) * 128 + t] = lst.i[k];
        }
      }
    }
    named_barrier(1, 128 * NW);
    if (wg == 0) {
#pragma unroll 1
      for (int g = 0; g < NW - 1; ++g) {
        if (PACKED) {
          uint32_t other[PackedList::N];
#pragma unroll
          for (int k = 0; k < PackedList::N; ++k) other[k] = (uint32_t)mi[(g * PackedList::N + k) * 128 + t];
          pl.merge(other);
        } else {
#pragma unroll
          for (int k = 0; k < kList; ++k) lst.insert(mv[(g * kList + k) * 128 + t], mi[(g * kList + k) * 128 + t]);
        }
      }
      if (tok_ok) {
        const int n_free = max(0, min(top_n, nk + 1) - ni - nl);
        int32_t* out = p.topk + ((int64_t)kh * Tq + q_row) * top_n;
        for (int s = 0; s < ni; ++s) out[s] = (s <= nk) ? s : p.ignore_index;
        for (int s = 0; s < nl; ++s) out[ni + s] = (ni + s <= nk) ? nk - s : p.ignore_index;
#pragma unroll
        for (int r = 0; r < kList; ++r) out[ni + nl + r] = (r < n_free) ? (PACKED ? pl.block(r) : lst.i[r]) : p.ignore_index;
      }
    }
  }
  if (timed_out && p.status) atomicOr(p.status, 16);
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

// ---------------------------------------------------------------------------------------------------- host side
// returns 1 when this kernel does not cover the call (caller then uses the warp-MMA kernel), 0 on launch, <0 on error
int launch_slc_topk_tc(const NsaTopkParams* p, int64_t q_rows, int64_t ck_rows, cudaStream_t st) {
  if (p->meta.kv_table || p->meta.cmp_table) return 1;                       // paged rows cannot be fetched as one box
  if (p->hp.top_n - p->hp.num_init - p->hp.num_local != kList) return 1;
  if ((p->q_stride_t * 2) % 16 || (p->ck_stride_t * 2) % 16 || ((uintptr_t)p->q & 15) || ((uintptr_t)p->ck & 15)) return 1;
  if (ck_rows <= 0) return 1;
  CUtensorMap tmq, tmk;
  if (!tma::make_map(&tmq, p->q, q_rows, p->QH, p->D, p->q_stride_t, 128, 1) ||
      !tma::make_map(&tmk, p->ck, ck_rows, p->KH, p->D, p->ck_stride_t, 128, 1)) {
    set_error("slc_topk: cuTensorMapEncodeTiled failed or is unavailable");
    return NSA_ERR_CUDA;
  }
  const int D = p->D;
  size_t smem = (size_t)7 * 128 * D * 2 + 256;
  // block indices must fit the 16 bits of a packed list entry; longer sequences compare (value, index) pairs
  const bool packed = p->quant != 0 && (p->meta.x_maxlen + p->hp.block_size - 1) / p->hp.block_size < 0xffff && p->meta.x_maxlen > 0;
  auto kern = (D == 128) ? (packed ? slc_topk_tc_kernel<128, true> : slc_topk_tc_kernel<128, false>)
                         : (packed ? slc_topk_tc_kernel<64, true> : slc_topk_tc_kernel<64, false>);
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_error("slc_topk: cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
    return NSA_ERR_CUDA;
  }
  dim3 grid((p->meta.max_piece_len + 127) / 128, p->meta.n_pieces, p->KH);
  kern<<<grid, 448, smem, st>>>(*p, tmq, tmk);
  return check_launch("slc_topk");
}

}  // namespace nsa
