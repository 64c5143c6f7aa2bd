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
//   3. top-n (pool 4 -> 1 + the row before; ties: lowest block index): up to 256 blocks by rank counting on the 128
//      threads of consumers 0-3 (rank = number of candidates that beat mine), longer contexts by rounds of arg-max over
//      the same 128 threads (a thread keeps the best of its run of blocks; one warp reduction and one barrier per round)
//   4. the forced blocks (their tiles arrive while the selection runs), then the free blocks, round-robin over consumers
//      0-3 (the producer waits for the selection before it fetches the free ones)
//   W. consumers 4-5 do the sliding-window tiles once their share of 1 is stored: these depend on nothing, and their
//      jobs are spread through the list from phase 2 on (one after every two compressed tiles), so that their loads fill
//      the time in which the others synchronise, merge and select and would leave the memory system idle
//   5. o = sigmoid(w0) cmp_o + sigmoid(w1) slc_o + sigmoid(w2) swa_o
// Partial softmax states are merged through shared memory after 1 and after 4; that region holds the score arrays in
// between.  Bytes read per (sequence, kv head): compressed K twice and V once, 16 selected blocks and <= 9 window tiles.
//
// Few sequences (the grid would leave most SMs idle) run as thread-block CLUSTERS of 2, 4 or 8 CTAs per (sequence, kv
// head), XC = true: CTA r of the cluster takes every CS-th compressed tile, window tile and selected slot.  Three exchanges
// through distributed shared memory: (1) the log-sum-exp of each CTA's share of the compressed rows, read by every CTA to
// form the global one; (2) every tile's 64 head-summed probabilities are stored into the score array of EVERY CTA (16-byte
// remote stores), and each CTA then makes the same selection for itself; (3) every CTA reads the others' normalised partial
// outputs of the three branches with their log-sum-exps (all of a thread's remote loads in flight together), merges them
// and writes its slice of the output row.  An exchange is an mbarrier per CTA on which thread c of every CTA arrives
// remotely for CTA c (bounded waits like every other one here); one hardware cluster barrier after the barrier
// initialisation and one before exit (a CTA's shared memory must outlive every remote access to it).
#include <cstdio>
#include <cstdlib>

#include "tma.cuh"
#include "warp_tile_smem.cuh"

namespace nsa {

// RING_NC consumer warps, of which 0..RING_NS-1 do the compressed and selected branches and the others the window (all share
// the compressed tiles).  Built as 6 / 4 with a ring of five slots, one CTA per SM; 3 / 2 with two slots and two CTAs per SM
// measured the same within 3 % (config 4), so the time is not a matter of how many CTAs an SM holds.
constexpr int RING_WIN_ROWS = 16;   // window tiles at most
constexpr int JOB_CMP_KV = 0, JOB_CMP_K = 1, JOB_WIN = 2, JOB_SLC = 3;

__host__ __device__ constexpr int job_pack(int type, int cons, int idx) { return type | (cons << 2) | (idx << 5); }

// ---- cluster helpers (distributed shared memory)
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_size() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;\n" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t peer_addr(uint32_t local, uint32_t rank) {   // shared::cta address -> the same place in CTA `rank`
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_peer4(uint32_t addr, float4 v) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ float ld_peer(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(addr));
  return v;
}
constexpr int RING_MAX_CLUSTER = 8;
// The same shared-memory word of every CTA of the cluster.  A remote load takes several hundred nanoseconds, so all of
// them are issued before the first value is used (a loop that folds each value as it arrives pays that time per CTA).
__device__ __forceinline__ void ld_all_peers(float (&v)[RING_MAX_CLUSTER], uint32_t local_addr, int CS, float fill) {
#pragma unroll
  for (int c = 0; c < RING_MAX_CLUSTER; ++c) v[c] = fill;
#pragma unroll
  for (int c = 0; c < RING_MAX_CLUSTER; ++c)
    if (c < CS) v[c] = ld_peer(peer_addr(local_addr, c));
}
__device__ __forceinline__ void fence_cluster() { asm volatile("fence.acq_rel.cluster;\n" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_peer(uint32_t peer_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(peer_bar) : "memory");
}
// bounded wait with cluster-scope acquire: what the peers stored before their arrival is visible afterwards
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, int* budget) {
  for (int i = 0; i < *budget; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  *budget = 8;
  return false;
}
__device__ __forceinline__ void cluster_barrier() {   // every thread of every CTA of the cluster
  asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;\n" ::: "memory");
}

template <int D, int RING_NC, int RING_NS, bool XC>
__global__ void __launch_bounds__(32 * (RING_NC + 1), RING_NC <= 3 ? 2 : 1)
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
  float* pcm = state;                       // [y_cap + 8] head-summed probabilities of the compressed rows (index + PO)
  constexpr int PO = 4;                     // row j at pcm[PO + j]: a tile's 64 values start on a 16-byte boundary
  float* psl = state + p.y_cap + 8;         // [y_cap/4 + 8] block scores
  float* cmp_o_s = reinterpret_cast<float*>(after_ring + region);  // [16][D] merged output of the compressed branch
  float* lse_s = cmp_o_s + 16 * D;                                // [16]
  int* sel = reinterpret_cast<int*>(lse_s + 16);                  // [32]
  int* jobs = sel + 32;                                           // [job_cap]
  // first cache row of a job's tile, by type: compressed tiles [ct_cap], window tiles [RING_WIN_ROWS], selected slots [32]
  int* rows = jobs + job_cap;
  int* rows_win = rows + ((p.y_cap + 63) >> 6);
  int* rows_slc = rows_win + RING_WIN_ROWS;
  float* fac = reinterpret_cast<float*>(rows_slc + 32);          // [RING_NC][16] merge weights, then [3][16] gates
  float* lse_x = fac + (RING_NC + 3) * 16;                        // [3][16] this CTA's log-sum-exp of its share: cmp, slc, window
  float* xw = lse_x + 48;                                         // [RING_MAX_CLUSTER][3][16] merge weights of the CTAs' partials
  int* marks = reinterpret_cast<int*>(xw + RING_MAX_CLUSTER * 48);  // [3] end of the phase-1 / phase-2 part of the job list, its length
  const uint32_t bars = (smem_u32(marks + 3) + 7u) & ~7u;         // full[n_slots], empty[n_slots], sel_ready, issued, xbar[3]
  auto full = [&](int s) { return bars + 8 * s; };
  auto empty = [&](int s) { return bars + 8 * (n_slots + s); };
  const uint32_t sel_ready = bars + 16 * n_slots;
  const uint32_t issued = sel_ready + 8;   // number of jobs whose loads have been issued (written by the producer)
  const uint32_t xbar = issued + 8;        // three cluster exchanges, each used once

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g_ = lane >> 2, c_ = lane & 3;
  // the kv heads of a sequence are neighbours in launch order: they read the same token rows (window, forced blocks,
  // compressed rows) at about the same time, 256 bytes each out of the same 2 KB of DRAM
  const int CS = XC ? (int)cluster_size() : 1, cr = XC ? (int)cluster_rank() : 0;   // cluster = CS neighbours in x
  const int kh = XC ? blockIdx.x / CS : blockIdx.x, b = blockIdx.y;
  const int G = p.QH / p.KH;
  const int ctx = p.context_lens[b];
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.o) + (int64_t)b * p.o_stride_t + (int64_t)kh * G * D;
  if (ring & 1023u) {   // the swizzled tile layout needs 1 KB alignment of the ring
    if (tid == 0 && p.status) atomicOr(p.status, 8);
    return;
  }
  if (ctx <= 0) {   // the whole cluster leaves here, before any exchange
    if (cr == 0) {
      for (int i = tid; i < G * CH; i += blockDim.x) reinterpret_cast<uint4*>(out)[i] = make_uint4(0, 0, 0, 0);
      if (p.topk_out && tid < p.hp.top_n) p.topk_out[((int64_t)kh * p.B + b) * p.hp.top_n + tid] = -1;
    }
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

  const int n_ct_all = (Y + 63) >> 6;
  const int n_ct = XC ? (n_ct_all - cr + CS - 1) / CS : n_ct_all;   // this CTA's compressed tiles: cr, cr + CS, ...
  auto ct_row0 = [&](int li) { return (XC ? li * CS + cr : li) << 6; };   // first compressed row of local tile li
  const int lo = max(0, t - W);
  const int w_k0 = (lo >> 6) << 6;                       // first window tile
  const int n_wt = ((t - w_k0) >> 6) + 1;                // window tiles
  const int n_valid = min(top_n, nk + 1);
  const int nf = min(ni + nl, n_valid);                  // forced slots
  const int n_free = n_valid - nf;
  // window tile wi and selected slot s belong to CTA wi % CS and s % CS

  // ---- set-up: barriers, the job list, the new compressed row
  if (tid == RING_NC * 32) {
    tma::prefetch_map(&tmk);
    tma::prefetch_map(&tmv);
  }
  if (tid == 0) {
    for (int s = 0; s < n_slots; ++s) {
      mbar_init(full(s), 1);
      mbar_init(empty(s), 1);
    }
    mbar_init(sel_ready, 1);
    if (XC)
      for (int i = 0; i < 3; ++i) mbar_init(xbar + 8 * i, CS);
    asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(issued), "r"(0) : "memory");
    fence_mbar_init();
  }
  // The first cache row of every tile whose place is known now: the page-table look-ups of all tiles are in flight at
  // once (the rows of the free blocks are filled in by the selection).
  for (int i = tid; i < n_ct + n_wt + nf; i += blockDim.x) {
    if (i < n_ct) rows[i] = (int)cmprow(ct_row0(i));
    else if (i < n_ct + n_wt) rows_win[i - n_ct] = (int)tokrow(w_k0 + ((i - n_ct) << 6));
    else {
      const int sidx = i - n_ct - n_wt;
      rows_slc[sidx] = (int)tokrow(max(0, min(sidx < ni ? sidx : nk - (sidx - ni), nk)) << 6);
    }
  }
  // Job list: (type, consumer, index) in the order the producer fetches them.
  if (tid == 32) {
    int n = 0, wi = 0;
    int wl = 0, sl = 0;   // local counters spread this CTA's jobs over its consumers
    auto win = [&]() {
      while (XC && wi < n_wt && wi % CS != cr) ++wi;
      if (wi < n_wt) {
        jobs[n++] = job_pack(JOB_WIN, RING_NS + wl++ % (RING_NC - RING_NS), wi);
        ++wi;
      }
    };
    auto mine = [&](int slot_idx) { return !XC || slot_idx % CS == cr; };
    for (int i = 0; i < n_ct; ++i) jobs[n++] = job_pack(JOB_CMP_KV, i % RING_NC, i);
    marks[0] = n;
    for (int i = 0; i < n_ct; i += 2) {   // tiles i and i + 1 in the two halves of one slot
      jobs[n++] = job_pack(JOB_CMP_K, (i >> 1) % RING_NC, i);
      win();
    }
    marks[1] = n;
    for (int sidx = 0; sidx < nf; ++sidx)
      if (mine(sidx)) jobs[n++] = job_pack(JOB_SLC, RING_NS > 1 ? 1 + sl++ % (RING_NS - 1) : 0, sidx);
    for (;;) {
      const int before = n;
      win();
      if (n == before) break;
    }
    sl = 0;
    for (int fi = 0; fi < n_free; ++fi)
      if (mine(nf + fi)) jobs[n++] = job_pack(JOB_SLC, sl++ % RING_NS, nf + fi);
    marks[2] = n;
  }
  {
    // The new compressed row: the mean of the last ks token rows, summed in row order like the stand-alone pooling kernel.
    // All threads first bring the ks x (K, V) row slices into shared memory with every load in flight at once (a thread
    // that loads and adds row after row pays a page-table look-up and a cache-row read ks times in a row: 5 us per CTA).
    const int slot = p.slot_mapping ? p.slot_mapping[b] : -1;
    if (slot >= 0 && ctx >= ks) {   // the same for every thread of the CTA (and every CTA of a cluster: each writes the row)
      const int start = ((ctx - ks) / st) * st;
      uint4* stage = reinterpret_cast<uint4*>(state);   // [ks][K chunks, V chunks]: the states are not in use yet
      const int total = min(ks * 2 * CH, 5 * (int)blockDim.x);
      uint4 piece[5];
#pragma unroll
      for (int u = 0; u < 5; ++u) {
        const int idx = tid + u * blockDim.x;
        if (idx < total) {
          const int i = idx / (2 * CH), rem = idx - i * 2 * CH;
          const __nv_bfloat16* cache = rem < CH ? kc : vc;
          piece[u] = *reinterpret_cast<const uint4*>(cache + tokrow(start + i) * cs + (rem % CH) * 8);
        }
      }
#pragma unroll
      for (int u = 0; u < 5; ++u) {
        const int idx = tid + u * blockDim.x;
        if (idx < total) stage[idx] = piece[u];
      }
      __syncthreads();
      if (tid < 2 * CH) {   // K by threads 0..CH-1, V by the next CH threads
        __nv_bfloat16* cache = tid < CH ? kc : vc;
        const int c = tid % CH;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int i = 0; i < ks; ++i) {
          const uint4 u = stage[i * 2 * CH + tid];
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
  }
  __syncthreads();
  if (XC) cluster_barrier();   // every CTA's barriers exist before a peer arrives on them
  const int n_jobs = marks[2];
  int budget = kWaitBudget;
  bool timed_out = false;

  if (warp == RING_NC) {
    // ================================================= producer (one lane)
    if (lane == 0) {
      bool have_sel = false;
      for (int j = 0; j < n_jobs; ++j) {
        const int job = jobs[j], type = job & 3, idx = job >> 5;
        const int s = j % n_slots;
        if (j >= n_slots && !mbar_wait(empty(s), ((j / n_slots) - 1) & 1, &budget)) timed_out = true;
        // the first free block: the selection warp has written the list and the rows of all free blocks
        if (type == JOB_SLC && idx >= nf && !have_sel) {
          if (!mbar_wait(sel_ready, 0, &budget)) timed_out = true;
          have_sel = true;
        }
        const int row = type <= JOB_CMP_K ? rows[idx] : (type == JOB_WIN ? rows_win[idx] : rows_slc[idx]);
        const uint32_t dst = ring + (uint32_t)s * 2 * TILE_BYTES;
        const bool k_pair = type == JOB_CMP_K && idx + 1 < n_ct;
        tma::expect_tx(full(s), (type == JOB_CMP_K && !k_pair) ? TILE_BYTES : 2 * TILE_BYTES);
        const int row2 = k_pair ? rows[idx + 1] : row;
#pragma unroll
        for (int sl = 0; sl < SLABS; ++sl) {
          tma::load_3d(dst + sl * SLAB_BYTES, &tmk, sl * 64, kh, row, full(s));
          if (type != JOB_CMP_K) tma::load_3d(dst + TILE_BYTES + sl * SLAB_BYTES, &tmv, sl * 64, kh, row, full(s));
          else if (k_pair) tma::load_3d(dst + TILE_BYTES + sl * SLAB_BYTES, &tmk, sl * 64, kh, row2, full(s));
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
    // merge weights of the states of consumers [w0, w0+nw) for row r: fac[w][r] = exp2(m_w - M) / L (0 for an empty row);
    // returns the merged log-sum-exp
    auto merge_weights = [&](int w0, int nw, int r) -> float {
      float M = -INFINITY;
      for (int w = 0; w < nw; ++w) M = fmaxf(M, state[(w0 + w) * STATE + r]);
      float L = 0.f;
      if (M != -INFINITY)
        for (int w = 0; w < nw; ++w) L += state[(w0 + w) * STATE + 16 + r] * fast_exp2(state[(w0 + w) * STATE + r] - M);
      const float inv = L > 0.f ? 1.f / L : 0.f;
      for (int w = 0; w < nw; ++w) fac[(w0 + w) * 16 + r] = L > 0.f ? fast_exp2(state[(w0 + w) * STATE + r] - M) * inv : 0.f;
      return L > 0.f ? M + log2f(L) : -INFINITY;
    };
    // cluster exchange k: what this CTA's consumers wrote before it (here or into the peers) is visible to every CTA of the
    // cluster after it
    auto xchg = [&](int k) {
      fence_cluster();
      named_barrier(1, NCT);
      if (ctid < CS) mbar_arrive_peer(peer_addr(xbar + 8 * k, ctid));   // thread c tells CTA c
      if (!mbar_wait_cluster(xbar + 8 * k, 0, &budget)) timed_out = true;
    };

    constexpr int NST = RING_NS * 32;   // threads of consumers 0-3 (named barrier 2)
    const int end_a = marks[0], end_b = marks[1];
    int j = 0;
    // ---- 1. compressed attention (all six consumers)
    {
      wts::Acc<D> ca;
      ca.init();
      for (; j < end_a; ++j) {
        if (((jobs[j] >> 2) & 7) != cw) continue;
        const int j0 = ct_row0(jobs[j] >> 5);
        wait_job(j);
        const uint32_t bk = ring + (uint32_t)(j % n_slots) * 2 * TILE_BYTES;
        wts::attend64_smem<D>(ca, qf, bk, bk + TILE_BYTES, [&](int i) { return j0 + i < Y; }, min(64, Y - j0), c2, lane);
        release(j);
      }
      wts::store_state<D>(ca, state + cw * STATE, lane);
    }
    named_barrier(1, NCT);
    if (ctid < 16) {
      const float l = merge_weights(0, RING_NC, ctid);
      if (XC) lse_x[ctid] = l;
      else lse_s[ctid] = l == -INFINITY ? 0.f : l;
    }
    named_barrier(1, NCT);
    for (int idx = ctid; idx < 16 * D; idx += NCT) {
      const int r = idx / D;
      float o = 0.f;
#pragma unroll
      for (int w = 0; w < RING_NC; ++w) o += state[w * STATE + 32 + idx] * fac[w * 16 + r];
      cmp_o_s[idx] = o;   // normalised by this CTA's own sum
    }
    if (XC) {
      // exchange 1: the log-sum-exp over ALL compressed rows.  Every CTA is past reading its states when it arrives, so the
      // peers may store probabilities into that region afterwards.
      xchg(0);
      if (ctid < 16) {
        float l[RING_MAX_CLUSTER];
        ld_all_peers(l, smem_u32(lse_x + ctid), CS, -INFINITY);
        float M = -INFINITY, L = 0.f;
#pragma unroll
        for (int c = 0; c < RING_MAX_CLUSTER; ++c) M = fmaxf(M, l[c]);
        if (M != -INFINITY) {
#pragma unroll
          for (int c = 0; c < RING_MAX_CLUSTER; ++c) L += fast_exp2(l[c] - M);   // exp2(-inf) = 0 for absent or empty CTAs
        }
        lse_s[ctid] = L > 0.f ? M + log2f(L) : 0.f;
      }
    }
    named_barrier(1, NCT);   // the states are dead until phase 4 is over: the score arrays live there

    // ---- 2. head-summed probabilities of every compressed row -> pcm[PO + j]; consumers 4-5 also start on the window
    wts::Acc<D> acc;   // the state a consumer ends with: selected branch (consumers 0-3) or window (4-5)
    acc.init();
    const float nl_lo = (g_ < G) ? -lse_s[g_] : 0.f, nl_hi = (g_ + 8 < G) ? -lse_s[g_ + 8] : 0.f;
    const bool h_lo = g_ < G, h_hi = g_ + 8 < G;
    auto window_tile = [&](int jj) {
      const int k0 = w_k0 + ((jobs[jj] >> 5) << 6);
      wait_job(jj);
      const uint32_t bk = ring + (uint32_t)(jj % n_slots) * 2 * TILE_BYTES;
      wts::attend64_smem<D>(acc, qf, bk, bk + TILE_BYTES, [&](int x) { return k0 + x >= lo && k0 + x <= t; }, min(64, t - k0 + 1), c2, lane);
      release(jj);
    };
    if (ctid == 0) pcm[PO - 1] = 0.f;
    for (; j < end_b; ++j) {
      const int job = jobs[j];
      if (((job >> 2) & 7) != cw) continue;
      if ((job & 3) == JOB_WIN) {
        window_tile(j);
        continue;
      }
      wait_job(j);
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        const int ti = (job >> 5) + half;   // the slot holds K tiles ti (first half) and ti + 1 (second half)
        if (ti >= n_ct) break;
        const int j0 = ct_row0(ti);
        float s[8][4];
        wts::scores64<D>(s, qf, ring + (uint32_t)(j % n_slots) * 2 * TILE_BYTES + half * TILE_BYTES, lane);
        if (half == 1 || ti + 1 >= n_ct) release(j);
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
            pcm[PO + col] = v0;
            pcm[PO + 1 + col] = v1;
          }
        }
        if (XC) {   // the tile's 64 values into the score array of every other CTA of the cluster: 16 lanes x 16 bytes each
          __syncwarp();
          if (lane < 16) {
            const float4 v = *reinterpret_cast<const float4*>(pcm + PO + j0 + 4 * lane);
            const uint32_t a = smem_u32(pcm + PO + j0 + 4 * lane);
            for (int c = 0; c < CS; ++c)
              if (c != cr) st_peer4(peer_addr(a, c), v);
          }
        }
      }
    }
    if (XC) xchg(1);               // exchange 2: every CTA's pcm[] is complete
    else named_barrier(1, NCT);   // pcm[] is complete

    if (cw >= RING_NS) {
      // ================================ W. the rest of the sliding window
      for (; j < n_jobs; ++j)
        if (((jobs[j] >> 2) & 7) == cw) window_tile(j);
    } else {
      // ---- 3. selection
      const int n_blk = nk + 1;
      const bool by_rank = n_blk <= 2 * NST;   // CTA-uniform
      auto pooled = [&](int blk) -> float {
        auto at = [&](int jj) { return (jj >= 0 && jj < Y) ? pcm[PO + jj] : 0.f; };
        const int jj = 4 * blk;
        const float pv = at(jj - 1) + ((2.f * at(jj) + 2.f * at(jj + 1)) + (2.f * at(jj + 2) + at(jj + 3)));
        return (blk >= ni && blk <= nk - nl) ? pv : -1.f;   // forced blocks are not candidates
      };
      if (by_rank) {
        // every thread owns blocks ctid and ctid + 128; its rank among the candidates is the number of candidates with a
        // larger score, or the same score and a lower index: ranks 0..n_free-1 are the list, in the order the rounds of
        // arg-max would have produced it
        for (int blk = ctid; blk < n_blk; blk += NST) psl[blk] = pooled(blk);
        if (ctid < 32) sel[ctid] = -1;
        named_barrier(2, NST);
        for (int my = ctid; my < n_blk; my += NST) {
          const float v = psl[my];
          if (v < 0.f) continue;
          int rank = 0;
#pragma unroll 4
          for (int o = 0; o < n_blk; ++o) {
            const float u = psl[o];
            rank += (u > v || (u == v && o < my)) ? 1 : 0;
          }
          if (rank < n_free) sel[ni + nl + rank] = my;
        }
        if (ctid < ni) sel[ctid] = (ctid <= nk) ? ctid : -1;
        else if (ctid < ni + nl) sel[ctid] = (ctid <= nk) ? nk - (ctid - ni) : -1;
        named_barrier(2, NST);
      } else {
        // Rounds of arg-max over the 128 threads.  A thread owns `per` CONSECUTIVE blocks and keeps the best of them (ascending
        // scan: the lowest index among equals); a round is one warp reduction (largest score) and a ballot -- the lowest lane
        // that holds that score holds the warp's lowest such block -- then the four warps' candidates through shared memory and
        // one barrier (two sets of places, used in turn).  Only the winner rescans its blocks.  Scores are >= 0, so their bit
        // patterns order like unsigned integers; 0 = no candidate.
        for (int blk = ctid; blk < n_blk; blk += NST) psl[blk] = pooled(blk);
        if (ctid < 32) sel[ctid] = -1;
        named_barrier(2, NST);
        unsigned* wbest = reinterpret_cast<unsigned*>(xw);   // [2][RING_NS][2]: key, block
        const int per = (n_blk + NST - 1) / NST, b0 = ctid * per;
        unsigned key;
        int bi;
        auto local_best = [&]() {
          key = 0u;
          bi = 0x7fffffff;
          for (int blk = b0; blk < min(n_blk, b0 + per); ++blk) {
            const float v = psl[blk];
            const unsigned kk = v >= 0.f ? __float_as_uint(v) + 1u : 0u;
            if (kk > key) {
              key = kk;
              bi = blk;
            }
          }
        };
        local_best();
        for (int r = 0; r < n_free; ++r) {
          const unsigned wkey = __reduce_max_sync(0xffffffffu, key);
          const int wl = __ffs(__ballot_sync(0xffffffffu, key == wkey)) - 1;
          const int wbi = __shfl_sync(0xffffffffu, bi, wl);
          unsigned* slot = wbest + (r & 1) * 2 * RING_NS;
          if (lane == 0) {
            slot[2 * cw] = wkey;
            slot[2 * cw + 1] = (unsigned)wbi;
          }
          named_barrier(2, NST);
          unsigned best = 0u;
          int best_blk = -1;
#pragma unroll
          for (int w = 0; w < RING_NS; ++w)   // ascending warps own ascending blocks: the first of equal scores is the lowest block
            if (slot[2 * w] > best) {
              best = slot[2 * w];
              best_blk = (int)slot[2 * w + 1];
            }
          if (best == 0u) break;   // fewer candidates than slots (the same answer in every thread)
          if (best_blk == bi && key == best) {
            sel[ni + nl + r] = bi;
            psl[bi] = -1.f;
            local_best();
          }
        }
        if (ctid < ni) sel[ctid] = (ctid <= nk) ? ctid : -1;
        else if (ctid < ni + nl) sel[ctid] = (ctid <= nk) ? nk - (ctid - ni) : -1;
        named_barrier(2, NST);
      }
      if (cw == 0) {
        if (cr == 0 && p.topk_out && lane < top_n) p.topk_out[((int64_t)kh * p.B + b) * top_n + lane] = sel[lane];
        // the cache rows of the free blocks, for the producer (an unused slot fetches block 0 and takes no part)
        if (lane >= nf && lane < n_valid) rows_slc[lane] = (int)tokrow(max(0, min(sel[lane], nk)) << 6);
        __syncwarp();
        if (lane == 0) mbar_arrive(sel_ready);
      }
      // ---- 4. the selected blocks
      for (; j < n_jobs; ++j) {
        const int job = jobs[j];
        if (((job >> 2) & 7) != cw) continue;
        const int idx = job >> 5;
        const int blk = idx >= nf ? sel[idx] : (idx < ni ? idx : nk - (idx - ni));
        int k0 = max(0, min(blk, nk)) << 6;
        if (blk < 0 || blk > nk) k0 = -1;   // an unused slot: its tile was fetched (block 0) but takes no part
        wait_job(j);
        const uint32_t bk = ring + (uint32_t)(j % n_slots) * 2 * TILE_BYTES;
        if (k0 >= 0)
          wts::attend64_smem<D>(acc, qf, bk, bk + TILE_BYTES, [&](int x) { return k0 + x <= t; }, min(64, t - k0 + 1), c2, lane);
        release(j);
      }
    }
    named_barrier(1, NCT);   // every read of the score arrays is done: the states may be written again
    wts::store_state<D>(acc, state + cw * STATE, lane);
    named_barrier(1, NCT);
    // ---- 5. merge + gated combine
    const __nv_bfloat16* wp = reinterpret_cast<const __nv_bfloat16*>(p.w) + (int64_t)b * p.w_stride_t + (int64_t)kh * G * 3;
    if (ctid < 16) {
      const float l = merge_weights(0, RING_NS, ctid);
      if (XC) lse_x[16 + ctid] = l;
    } else if (ctid < 32) {
      const float l = merge_weights(RING_NS, RING_NC - RING_NS, ctid - 16);
      if (XC) lse_x[32 + ctid - 16] = l;
    } else if (ctid < 32 + 3 * 16) {
      const int i = ctid - 32, r = i / 3;   // gates: sigmoid of the three logits of head r
      fac[RING_NC * 16 + i] = r < G ? 1.f / (1.f + __expf(-__bfloat162float(wp[i]))) : 0.f;
    }
    named_barrier(1, NCT);
    const float* gate = fac + RING_NC * 16;
    if (!XC) {
      for (int idx = ctid; idx < G * D; idx += NCT) {
        const int r = idx / D;
        float slc = 0.f, swa = 0.f;
#pragma unroll
        for (int w = 0; w < RING_NS; ++w) slc += state[w * STATE + 32 + idx] * fac[w * 16 + r];
#pragma unroll
        for (int w = RING_NS; w < RING_NC; ++w) swa += state[w * STATE + 32 + idx] * fac[w * 16 + r];
        out[idx] = __float2bfloat16(gate[r * 3] * cmp_o_s[idx] + gate[r * 3 + 1] * slc + gate[r * 3 + 2] * swa);
      }
    } else {
      // this CTA's normalised partial outputs, in place: the selected branch over the state of consumer 0, the window over the
      // state of the first window consumer (a thread reads and writes only its own element of every state)
      for (int idx = ctid; idx < G * D; idx += NCT) {
        const int r = idx / D;
        float slc = 0.f, swa = 0.f;
#pragma unroll
        for (int w = 0; w < RING_NS; ++w) slc += state[w * STATE + 32 + idx] * fac[w * 16 + r];
#pragma unroll
        for (int w = RING_NS; w < RING_NC; ++w) swa += state[w * STATE + 32 + idx] * fac[w * 16 + r];
        state[32 + idx] = slc;
        state[RING_NS * STATE + 32 + idx] = swa;
      }
      xchg(2);   // exchange 3: every CTA's partials and their log-sum-exps are in place
      {          // CTA c merges and writes the c-th slice of the output row
        if (ctid < 48) {   // weight of CTA c's partial of branch ctid / 16, head ctid % 16: exp2(lse_c) / sum over the CTAs
          float l[RING_MAX_CLUSTER];
          ld_all_peers(l, smem_u32(lse_x + ctid), CS, -INFINITY);
          float M = -INFINITY, L = 0.f;
#pragma unroll
          for (int c = 0; c < RING_MAX_CLUSTER; ++c) M = fmaxf(M, l[c]);
          if (M != -INFINITY) {
#pragma unroll
            for (int c = 0; c < RING_MAX_CLUSTER; ++c) L += fast_exp2(l[c] - M);
          }
          const float inv = L > 0.f ? 1.f / L : 0.f;
#pragma unroll
          for (int c = 0; c < RING_MAX_CLUSTER; ++c) xw[c * 48 + ctid] = L > 0.f ? fast_exp2(l[c] - M) * inv : 0.f;
        }
        named_barrier(1, NCT);
        const uint32_t a_cmp = smem_u32(cmp_o_s), a_slc = smem_u32(state + 32), a_swa = smem_u32(state + RING_NS * STATE + 32);
        const int chunk = (G * D + CS - 1) / CS;
        for (int idx = cr * chunk + ctid; idx < min(G * D, (cr + 1) * chunk); idx += NCT) {
          const int r = idx / D;
          float pc[RING_MAX_CLUSTER], ps[RING_MAX_CLUSTER], pw[RING_MAX_CLUSTER];   // 3 x CS remote loads in flight
          ld_all_peers(pc, a_cmp + 4 * idx, CS, 0.f);
          ld_all_peers(ps, a_slc + 4 * idx, CS, 0.f);
          ld_all_peers(pw, a_swa + 4 * idx, CS, 0.f);
          float cmp = 0.f, slc = 0.f, swa = 0.f;
#pragma unroll
          for (int c = 0; c < RING_MAX_CLUSTER; ++c) {   // the weights of absent CTAs are 0
            cmp += xw[c * 48 + r] * pc[c];
            slc += xw[c * 48 + 16 + r] * ps[c];
            swa += xw[c * 48 + 32 + r] * pw[c];
          }
          out[idx] = __float2bfloat16(gate[r * 3] * cmp + gate[r * 3 + 1] * slc + gate[r * 3 + 2] * swa);
        }
      }
    }
  }
  if (timed_out && p.status) atomicOr(p.status, 2048);
  if (XC) cluster_barrier();   // a CTA's shared memory outlives every remote access to it
}

template <int D, int NC, int NS, bool XC>
static int launch_shape(NsaDecodeParams p, cudaStream_t st, int max_slots, size_t smem_cap, int cs, bool dry) {
  const size_t tile = (size_t)64 * D * 2;
  const int job_cap = 2 * ((p.y_cap + 63) / 64) + 2 * p.hp.top_n + p.hp.window / 64 + 8;
  const int rows_cap = (p.y_cap + 63) / 64 + RING_WIN_ROWS + 32;
  const size_t region = (size_t)max(NC * (32 + 16 * D), p.y_cap + 8 + p.y_cap / 4 + 8) * 4;
  const size_t fixed = region + ((size_t)16 * D + 16 + 32 + job_cap + rows_cap + (NC + 3) * 16 + 48 + RING_MAX_CLUSTER * 48 + 3) * 4 + 8 +
                       16 * 8 + 16 + 1024;
  if (fixed + 2 * 2 * tile > smem_cap) return 1;
  int n_slots = (int)((smem_cap - fixed) / (2 * tile));
  if (n_slots > max_slots) n_slots = max_slots;
  if (n_slots < 2) return 1;
  const size_t smem = (size_t)n_slots * 2 * tile + fixed;
  CUtensorMap tmk, tmv;
  if (!dry && (!tma::make_map(&tmk, p.k_cache, p.cache_rows, p.KH, D, p.cache_stride_t, 64, 1) ||
               !tma::make_map(&tmv, p.v_cache, p.cache_rows, p.KH, D, p.cache_stride_t, 64, 1)))
    return 1;
  auto kernel = decode_ring_kernel<D, NC, NS, XC>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_error("decode_fused: cudaFuncSetAttribute(%zu B) failed: %s", smem, cudaGetErrorString(e));
    return NSA_ERR_CUDA;
  }
  if (!XC) {
    if (dry) return 0;
    dim3 grid(p.KH, p.B);
    kernel<<<grid, 32 * (NC + 1), smem, st>>>(p, n_slots, job_cap, tmk, tmv);
    return check_launch("decode_fused");
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.KH * cs, p.B);
  cfg.blockDim = dim3(32 * (NC + 1));
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = cs;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  // clusters of this size and shared-memory footprint the GPU holds at once: all of the step's clusters must fit, a second
  // wave would cost more than the split saves
  static struct { size_t smem; int dev, fit; } cache[4] = {{0, -1, 0}, {0, -1, 0}, {0, -1, 0}, {0, -1, 0}};   // per cluster size (this D)
  int dev = 0;
  (void)cudaGetDevice(&dev);
  auto& slot = cache[cs == 2 ? 1 : cs == 4 ? 2 : cs == 8 ? 3 : 0];
  int fit = slot.fit;
  if (slot.smem != smem || slot.dev != dev) {   // the query costs more host time than the launch itself: ask once
    if (cudaOccupancyMaxActiveClusters(&fit, kernel, &cfg) != cudaSuccess) {
      (void)cudaGetLastError();
      fit = 0;
    }
    slot.smem = smem;
    slot.dev = dev;
    slot.fit = fit;
  }
  static const bool debug = getenv("NSA_DECODE_CLUSTER_DEBUG") != nullptr;
  if (debug) fprintf(stderr, "[nsa] decode: %d x %d CTAs as clusters of %d: %d clusters fit\n", p.B, p.KH, cs, fit);
  if (fit < 1 || (int64_t)p.B * p.KH > fit) return 2;
  if (dry) return 0;
  e = cudaLaunchKernelEx(&cfg, kernel, p, n_slots, job_cap, tmk, tmv);
  if (e != cudaSuccess) {
    set_error("decode_fused: cluster launch failed: %s", cudaGetErrorString(e));
    return NSA_ERR_CUDA;
  }
  return check_launch("decode_fused");
}

// CTAs per (sequence, kv head).  The host does not know the context lengths (they are device data); the width of the page
// table bounds them.  Measured (batch 1 / 4 / 16 of 4 kv heads, CUDA graph, against one CTA): clusters of 4 and 8 win from 4K
// tokens on (4K: 0.0247 -> 0.021-0.023 ms, 16K: 0.041 -> 0.029, 128K: 0.109 -> 0.037); clusters of 2 lose at 4K, are even at
// 8K and win from 16K on (0.041 -> 0.036; 128K batch 16: 0.121 -> 0.094), because the three exchanges cost what half of a
// short step saves.  So: the largest size whose grid stays within the SMs, 4 and 8 for tables of 4K tokens or more, 2 for
// 16K or more.  NSA_DECODE_CLUSTER=1|2|4|8 overrides it.
static int forced_cluster_size() {
  static const int forced = [] {
    const char* e = getenv("NSA_DECODE_CLUSTER");
    const int v = e ? atoi(e) : 0;
    return (v == 1 || v == 2 || v == 4 || v == 8) ? v : 0;
  }();
  return forced;
}
static bool cluster_size_ok(const NsaDecodeParams* p, int cs) {
  static const int sms = [] {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    return n;
  }();
  const int64_t ctas = (int64_t)p->B * p->KH;
  const int64_t cap_tokens = (int64_t)p->kv_table_stride * p->page_size;
  if (ctas * cs > sms) return false;
  return cap_tokens >= (cs >= 4 ? 4096 : 16384);
}
static int decode_cluster_size_for(const NsaDecodeParams* p) {
  if (forced_cluster_size()) return forced_cluster_size();
  for (int cs = RING_MAX_CLUSTER; cs > 1; cs >>= 1)
    if (cluster_size_ok(p, cs)) return cs;
  return 1;
}

// dry: everything but the launch; returns the cluster size that a launch would use (0 when the kernel does not cover the
// configuration) instead of a status
static int launch_or_ask(const NsaDecodeParams* p, cudaStream_t st, bool dry) {
  const int D = p->D;
  if (!dry && (p->cache_rows <= 0 || (p->cache_stride_t * 2) % 16 || (((uintptr_t)p->k_cache | (uintptr_t)p->v_cache) & 15))) return 1;
  if (p->hp.window / 64 + 2 > RING_WIN_ROWS || p->hp.top_n > 32) return dry ? 0 : 1;
  const size_t cap = 227 * 1024;
  for (int cs = decode_cluster_size_for(p); cs > 1; cs >>= 1) {   // 2 = no room for clusters of this size: try the next smaller one
    if (!forced_cluster_size() && !cluster_size_ok(p, cs)) continue;
    const int rc = D == 128 ? launch_shape<128, 6, 4, true>(*p, st, 5, cap, cs, dry) : launch_shape<64, 6, 4, true>(*p, st, 5, cap, cs, dry);
    if (rc != 2) return dry ? (rc == 0 ? cs : (rc == 1 ? 0 : rc)) : rc;
  }
  const int rc = D == 128 ? launch_shape<128, 6, 4, false>(*p, st, 5, cap, 1, dry) : launch_shape<64, 6, 4, false>(*p, st, 5, cap, 1, dry);
  return dry ? (rc == 0 ? 1 : (rc == 1 ? 0 : rc)) : rc;
}

// returns 1 when the configuration is not covered (decode_fused_kernel then runs), 0 on launch, < 0 on error
int launch_decode_ring(const NsaDecodeParams* p, cudaStream_t st) { return launch_or_ask(p, st, false); }
// CTAs per (sequence, kv head) a launch with these parameters would use; 1 also when the fallback kernel would run
int decode_cluster_size_query(const NsaDecodeParams* p) {
  const int n = launch_or_ask(p, nullptr, true);
  return n == 0 ? 1 : n;
}

}  // namespace nsa
