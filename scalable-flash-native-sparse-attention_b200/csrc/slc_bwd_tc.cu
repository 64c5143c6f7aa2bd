// Selected-branch backward on the Blackwell tensor core: dK/dV and, fused, dQ.  PERSISTENT: one CTA per SM walks the work
// items of the key-block -> queries index (k2q.cu) in order.
//
// An item is (key block, slice of the list of query rows that selected it).  The index lists its items range-major
// (all items whose query rows lie in local rows [r*R, (r+1)*R), then the next range), and the CTAs take them off that list
// one at a time through a global ticket counter, so at any moment the items in flight are neighbours in the list and all
// CTAs gather q / dO rows of, and reduce into dq rows of, ONE range of R rows: with R sized to a third of L2 those rows are
// fetched from DRAM once per range instead of once per selected block (16 times).  (Items handed out round-robin drift
// apart, because item sizes differ by 30x: after a few ranges the CTAs were spread over two or three ranges and 72 % of the
// dq reductions still missed L2.)  The last CTA to finish puts the ticket counter back to zero for the next launch.
// The same kernel built block-major with each block's whole list in one CTA moved 11x the algorithmic bytes through DRAM.
//
// Per item, as in dkdv_tc.cu: the 64-row K/V tile of the block sits in shared memory; query rows come in tiles of
// 128 = (128/G tokens) x (G heads of the kv head) gathered by six TMA producer warps (one (64 d) x (G heads) x (1 token)
// box per lane); two warp groups of 128 threads work on one tile each (ping-pong), a ninth warp issues every MMA:
//     S    = Q K^T,  dP = dO V^T                       M = query rows, N = keys (A, B K-major from shared memory)
//     P    = exp2(S*c - lse),  dS = P * (dP - delta)    thread i of the group owns row i; bf16 P, dS go to shared memory
//     dV^T += dO^T P,  dK^T += Q^T dS                   transposed accumulators keep M = 128 (A, B MN-major views)
//     dQ_tile = dS K                                    A = the dS bytes read K-major, B = the K tile MN-major
// The group stages dQ_tile as bf16 in its P / dS buffers (free by then, in the layout of a q tile) and adds it into dq with
// one bulk tensor reduction per (token, 64-column slab).  At the end of an item lane j of the dV^T / dK^T accumulators
// holds column j of dV / dK: 64 coalesced fp32 atomics per thread.
//
// Items overlap.  The producer warps own the schedule: their leader draws the ticket of item n+1 as soon as the last loads
// of item n are issued and publishes it through a ticket barrier; once the last MMAs of item n have completed they load
// the K/V tile (TMA) and the first two query tiles of item n+1 while the compute groups still add the last dQ tile and
// flush dV / dK of item n; the first S / dP products of item n+1 run under that flush as well, only its first dV / dK
// products wait until the accumulators have been read (acc_free).  There is no CTA-wide barrier between items.
// Barriers keep counting across items: every pipeline barrier completes the same number of phases per item (one per
// round and group; the dQ hand-over barrier one per tile; ticket, K/V and accumulator barriers one per item), so a role
// derives every parity from the number of rounds and items it has seen.
#include "tma.cuh"

namespace nsa {

__device__ __forceinline__ int find_le_slc(const int32_t* cu, int n, int x) {
  int lo = 0, hi = n;
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (cu[mid] <= x) lo = mid; else hi = mid;
  }
  return lo;
}

template <int D>
__global__ void __launch_bounds__(480, 1)
    slc_bwd_tc_kernel(const NsaAttnParams p, int fuse_dq, const __grid_constant__ CUtensorMap tmq, const __grid_constant__ CUtensorMap tmo,
                      const __grid_constant__ CUtensorMap tmdq, const __grid_constant__ CUtensorMap tmk,
                      const __grid_constant__ CUtensorMap tmv) {
  using namespace tc;
  constexpr int BK = 64, BQ = 128;
  constexpr uint32_t KV_BYTES = BK * D * 2, Q_BYTES = BQ * D * 2, P_BYTES = BQ * BK * 2;
  constexpr uint32_t Q_SLAB = BQ * 128, K_SLAB = BK * 128;
  constexpr uint32_t A_LBO = (D == 128) ? Q_SLAB : 0;  // D = 64: the second half of M re-reads the only slab (rows 64.. of the result are unused)
  constexpr uint32_t IDESC_SD = make_idesc(BQ, BK, false, false), IDESC_KV = make_idesc(128, BK, true, true);
  constexpr uint32_t IDESC_DQ = make_idesc(BQ, D, true, false);
  constexpr uint32_t TM_DV = 256, TM_DK = 320, TM_DQ = 384, TM_COLS = 512;
  constexpr int SLABS = D / 64;

  extern __shared__ unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sK = base, sV = sK + KV_BYTES;
  const uint32_t sQ0 = sV + KV_BYTES;                 // [2 groups]
  const uint32_t sO0 = sQ0 + 2 * Q_BYTES;             // [2 groups]
  const uint32_t sP0 = sO0 + 2 * Q_BYTES;             // [2 groups]
  const uint32_t sS0 = sP0 + 2 * P_BYTES;             // [2 groups]
  const uint32_t bars = sS0 + 2 * P_BYTES;
  // barriers: in_full[2], sd_done[2], pds_full[2], kv_done[2], dq_read[2], ticket_full[2], then kv_full, acc_free; then the
  // tensor-memory address slot and the two ticket slots.  Item n uses ticket barrier / slot n & 1 (phase n >> 1): the leader
  // can be one item ahead of the slowest thread, and with one barrier a thread two phases behind would wait for ever.
  auto bar = [&](int which, int wg) { return bars + (which * 2 + wg) * 8; };
  const uint32_t kv_full = bars + 96, acc_free = bars + 104;
  const uint32_t tm_slot = bars + 112, ticket_slot = bars + 120;

  const int tid = threadIdx.x, warp = tid >> 5;
  const int G = p.QH / p.KH;
  const int TOKQ = BQ / G;
  const bool fuse = fuse_dq != 0;

  // ---- set-up, once per CTA
  if (tid == 0) {
    for (int w = 0; w < 2; ++w) {
      mbar_init(bar(0, w), 1);
      mbar_init(bar(1, w), 1);
      mbar_init(bar(2, w), 128);
      mbar_init(bar(3, w), 1);
      mbar_init(bar(4, w), 128);
    }
    mbar_init(bar(5, 0), 1);
    mbar_init(bar(5, 1), 1);
    mbar_init(kv_full, 1);
    mbar_init(acc_free, 256);
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc(tm_slot, TM_COLS);
  if (tid < 256 && TOKQ * G < BQ) {  // rows the TMA boxes never write must not hold NaN bit patterns
    for (int i = tid; i < (int)(4 * Q_BYTES / 16); i += 256)
      asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};\n" ::"r"(sQ0 + i * 16), "r"(0) : "memory");
    fence_proxy_async();
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  uint32_t tmem;
  asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(tmem) : "r"(tm_slot));
  int budget = kWaitBudget;
  bool timed_out = false;
  int jb = 0;   // rounds completed by this CTA in earlier items: the same number in every thread

  int total_items = 0;
  for (int h = 0; h < p.KH; ++h) total_items += min(__ldg(p.k2q_n_items + h), p.k2q_items_cap);
  int32_t* ticket = p.k2q_n_items + p.KH;   // [0] next item to hand out, [1] CTAs that have finished

  const bool leader = tid == 288;   // lane 0 of the first producer warp draws the tickets
  if (leader) {
    const int g0 = atomicAdd(ticket, 1);
    asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(ticket_slot), "r"(g0) : "memory");
    mbar_arrive(bar(5, 0));
  }

  {
    for (int n = 0;; ++n) {
      // ---- item n of this CTA: its ticket was published by the producer leader (release / acquire through the barrier)
      if (!mbar_wait(bar(5, n & 1), (n >> 1) & 1, &budget)) {   // no ticket: give up (the slot would hold a stale one)
        timed_out = true;
        break;
      }
      int g;
      asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(g) : "r"(ticket_slot + 4 * (n & 1)));
      if (g >= total_items || g < 0) break;
      if (warp >= 9) named_barrier(4, 192);   // the producer warps stay within one item of their leader
      int kh = 0, item_i = g;
      for (;;) {   // item g of the concatenation over kv heads
        const int cnt = min(__ldg(p.k2q_n_items + kh), p.k2q_items_cap);
        if (item_i < cnt) break;
        item_i -= cnt;
        ++kh;
      }
      const int4* items = reinterpret_cast<const int4*>(p.k2q_items) + (int64_t)kh * p.k2q_items_cap;
      const int32_t* list = p.k2q_tokens + (int64_t)kh * p.k2q_stride_h;
      const int4 item = __ldg(items + item_i);
      const int row = item.x, r_lo = item.y;
      const int b = find_le_slc(p.k2q_blk_cu, p.meta.n_pieces, row);
      const int k0 = (row - p.k2q_blk_cu[b]) * BK;
      int kv_row0, kv_rows, ta_base;   // first K/V tensor row of the block, its valid rows, position of local row 0 in the sequence
      {
        const Piece pc = load_piece(p.meta, b);
        kv_row0 = pc.x_bos + k0;
        kv_rows = max(min(BK, pc.x_len - k0), 0);
        ta_base = pc.off - pc.q_start;
      }
      const int r_hi = max(item.z, r_lo + 1);   // nsa_k2q_index writes no empty items; a foreign one still runs one (masked) tile
      const int n_it = (r_hi - r_lo + TOKQ - 1) / TOKQ;
      const int n_round = (n_it + 1) / 2;

      if (warp == 8) {
        // ================================================= MMA issue (one lane)
        if ((tid & 31) == 0) {
          if (!mbar_wait(kv_full, n & 1, &budget)) timed_out = true;   // the item's K/V tile has landed
          // Issue order per round: S, dP of both groups, then dV, dK, dQ of both groups: a group's softmax arithmetic runs
          // under the other group's S, dP.  (Per group S dP dV dK dQ, which would put one group's fetch under the other
          // group's five products, leaves the tensor core idle during that arithmetic and measured 15 % slower.)
          for (int j = 0; j < n_round; ++j) {
            const int jj = jb + j;
            for (int wg = 0; wg < 2; ++wg) {
              if (!mbar_wait(bar(0, wg), jj & 1, &budget)) timed_out = true;
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
              if (!mbar_wait(bar(2, wg), jj & 1, &budget)) timed_out = true;
              // the first dV / dK products of an item overwrite the accumulators: the previous item's flush has read them
              if (j == 0 && wg == 0 && n > 0 && !mbar_wait(acc_free, (n - 1) & 1, &budget)) timed_out = true;
              fence_after_sync();
              const uint32_t tQ = sQ0 + wg * Q_BYTES, tO = sO0 + wg * Q_BYTES;
              const uint32_t tP = sP0 + wg * P_BYTES, tS = sS0 + wg * P_BYTES;
              const uint32_t first_mma = (j == 0 && wg == 0) ? 0u : 1u;
#pragma unroll
              for (int u = 0; u < BQ / 16; ++u)
                mma_ss(tmem + TM_DV, desc_mnmajor(tO + u * 2048, A_LBO), desc_mnmajor(tP + u * 2048, 0), IDESC_KV,
                       (u > 0) ? 1u : first_mma);
#pragma unroll
              for (int u = 0; u < BQ / 16; ++u)
                mma_ss(tmem + TM_DK, desc_mnmajor(tQ + u * 2048, A_LBO), desc_mnmajor(tS + u * 2048, 0), IDESC_KV,
                       (u > 0) ? 1u : first_mma);
              if (fuse) {   // dS K into its own columns, once the previous tile's product has been read out of them
                const int m = 2 * jj + wg;
                if (m > 0 && !mbar_wait(bar(4, 0), (m - 1) & 1, &budget)) timed_out = true;
                fence_after_sync();
#pragma unroll
                for (int u = 0; u < BK / 16; ++u)
                  mma_ss(tmem + TM_DQ, desc_kmajor(tS + u * 32), desc_mnmajor(sK + u * 2048, K_SLAB), IDESC_DQ, u > 0);
              }
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
        const int n_box = TOKQ * SLABS * 2;
        const uint32_t tx = (uint32_t)(TOKQ * G) * D * 2 * 2;
        if (n > 0) {   // every MMA of the previous item has completed: K/V and both groups' buffers are free
          if (!mbar_wait(bar(3, 0), (jb - 1) & 1, &budget)) timed_out = true;
          if (!mbar_wait(bar(3, 1), (jb - 1) & 1, &budget)) timed_out = true;
        }
        if (leader) {
          tma::expect_tx(kv_full, 2 * KV_BYTES);
#pragma unroll
          for (int sl = 0; sl < SLABS; ++sl) {
            tma::load_3d(sK + sl * K_SLAB, &tmk, sl * 64, kh, kv_row0, kv_full);
            tma::load_3d(sV + sl * K_SLAB, &tmv, sl * 64, kh, kv_row0, kv_full);
          }
        }
        for (int it = 0; it < 2 * n_round; ++it) {   // an odd tile count still fills group 1's buffers in the last round
          const int wg = it & 1, j = it >> 1;
          const int tok0 = r_lo + it * TOKQ;
          // tensor rows of my first four boxes now, so that the index loads overlap the wait for the buffers
          auto row_of = [&](int bx) {
            const int tok = min(tok0 + bx / (SLABS * 2), r_hi - 1);   // past the end: a valid row again (its P, dS are zero)
            return __ldg(list + tok);
          };
          int rows[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) rows[u] = (lane + NP * u < n_box) ? row_of(lane + NP * u) : 0;
          if (j > 0 && !mbar_wait(bar(3, wg), (jb + j - 1) & 1, &budget)) timed_out = true;   // dV/dK MMAs of tile it-2 have read them
          if (lane == 0) tma::expect_tx(bar(0, wg), tx);
          __syncwarp();
          auto issue = [&](int bx, int trow) {
            const int n = bx / (SLABS * 2), rest = bx - n * (SLABS * 2), sl = rest >> 1, which = rest & 1;
            const uint32_t dst = (which ? sO0 : sQ0) + wg * Q_BYTES + sl * Q_SLAB + n * G * 128;
            tma::load_3d(dst, which ? &tmo : &tmq, sl * 64, kh * G, trow, bar(0, wg));
          };
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (lane + NP * u < n_box) issue(lane + NP * u, rows[u]);
          for (int bx = lane + 4 * NP; bx < n_box; bx += NP) issue(bx, row_of(bx));   // only when G = 1 and D = 128
          // the boxes of this group's NEXT tile: asked into L2 now, fetched into shared memory when the buffers are free
          if (it + 2 < n_it) {
            const int tok2 = tok0 + 2 * TOKQ;
            for (int bx = lane; bx < n_box; bx += NP) {
              const int n = bx / (SLABS * 2), rest = bx - n * (SLABS * 2), sl = rest >> 1, which = rest & 1;
              if (tok2 + n < r_hi) tma::prefetch_3d(which ? &tmo : &tmq, sl * 64, kh * G, __ldg(list + tok2 + n));
            }
          }
        }
        if (leader) {   // the next item's ticket, while this item is being worked on
          const int g1 = atomicAdd(ticket, 1);
          asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(ticket_slot + 4 * ((n + 1) & 1)), "r"(g1) : "memory");
          mbar_arrive(bar(5, (n + 1) & 1));
        }
      } else {
        // ================================================= two warp groups, one query tile each per round
        const int wg = warp >> 2, t = tid & 127;
        const uint32_t tP = sP0 + wg * P_BYTES, tS = sS0 + wg * P_BYTES;
        const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        const float c2 = p.sm_scale * 1.4426950408889634f;
        const int my_n = t / G, my_g = t - my_n * G;
        // fused dQ: my row of dS K (complete once kv_done has fired) goes, as bf16, into my P and dS buffers (free by
        // then) in the layout of a q tile; one bulk tensor reduction per (token, 64-column slab) then adds the token's
        // [G heads x 64] box into dq.  red_row = tensor row of token t % TOKQ of the tile (threads that own a box).
        const int n_box = TOKQ * SLABS;
        int red_row = -1;
        auto add_dq = [&](int trow) {
          fence_after_sync();
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t v[32];
            tmem_ld32(lane_base + TM_DQ + c * 32, v);
            wait_ld();
            const uint32_t sb = ((c >> 1) ? tS : tP) + t * 128;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint32_t w[4];
#pragma unroll
              for (int u = 0; u < 4; ++u)
                w[u] = pack_bf16(__uint_as_float(v[8 * i + 2 * u]) * p.sm_scale, __uint_as_float(v[8 * i + 2 * u + 1]) * p.sm_scale);
              const uint32_t ch = (c & 1) * 4 + i;
              asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(sb + ((ch ^ (t & 7)) << 4)), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                           : "memory");
            }
          }
          fence_before_sync();
          mbar_arrive(bar(4, 0));             // the dQ columns may take the next tile's product
          fence_proxy_async();
          named_barrier(2 + wg, 128);
          if (t < n_box) {
            if (trow >= 0) {
              for (int bx = t; bx < n_box; bx += 128) {
                const int n = bx % TOKQ, sl = bx / TOKQ;
                tma::reduce_add_3d(&tmdq, sl * 64, kh * G, trow, (sl ? tS : tP) + n * G * 128);
              }
            }
            tma::bulk_commit();
          }
        };

        // my row of a round: its tensor row two rounds ahead, its lse / delta one round ahead, so that neither load is waited for
        auto row_at = [&](int j) {
          const int tok = r_lo + (2 * j + wg) * TOKQ + my_n;
          return (my_n < TOKQ && j < n_round && tok < r_hi) ? __ldg(list + tok) : -1;
        };
        int qrow_cur = row_at(0), qrow_nxt = row_at(1);
        float lse_nxt = 0.f, dl_nxt = 0.f;
        if (qrow_cur >= 0) {
          const int64_t a = (int64_t)qrow_cur * p.lse_stride_t + (int64_t)(kh * G + my_g) * p.lse_stride_h;
          lse_nxt = p.lse[a];
          dl_nxt = p.delta[a];
        }
        for (int j = 0; j < n_round; ++j) {
          const int jj = jb + j;
          const int it = 2 * j + wg;
          const int tok0 = r_lo + it * TOKQ;  // first list position of my tile
          // my own row: lse, delta, absolute position (loaded during the previous round)
          const bool row_ok = qrow_cur >= 0;
          const float lse = lse_nxt, dl = dl_nxt;
          const int ta = row_ok ? ta_base + qrow_cur : -1;
          qrow_cur = qrow_nxt;
          lse_nxt = 0.f;
          dl_nxt = 0.f;
          if (qrow_cur >= 0) {
            const int64_t a = (int64_t)qrow_cur * p.lse_stride_t + (int64_t)(kh * G + my_g) * p.lse_stride_h;
            lse_nxt = p.lse[a];
            dl_nxt = p.delta[a];
          }
          qrow_nxt = row_at(j + 2);
          if (j > 0 && !mbar_wait(bar(3, wg), (jj - 1) & 1, &budget)) timed_out = true;  // my buffers are free again
          if (fuse && j > 0) add_dq(red_row);
          if (fuse && t < n_box) {
            const int tok = tok0 + t % TOKQ;
            red_row = (tok < r_hi) ? __ldg(list + tok) : -1;
          }
          // keys 0..kc_hi of the tile are visible to my row
          const int kc_hi = row_ok ? min(ta - k0, kv_rows - 1) : -1;
          const float nlse = -lse;
          if (!mbar_wait(bar(1, wg), jj & 1, &budget)) timed_out = true;
          fence_after_sync();
          if (fuse && (j > 0 || n > 0)) {   // the reductions of the previous tile (or item) have read my P / dS buffers
            if (t < n_box) tma::bulk_wait_read();
            named_barrier(2 + wg, 128);
          }
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            uint32_t sv[32], dv[32];
            tmem_ld32(lane_base + 128 * wg + half * 32, sv);
            tmem_ld32(lane_base + 128 * wg + 64 + half * 32, dv);
            wait_ld();
            uint32_t pp[16], dd[16];
            if (kc_hi >= BK - 1) {   // the whole key tile is visible to my row (the usual case)
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
                const float x0 = (kc <= kc_hi) ? fast_exp2(fmaf(__uint_as_float(sv[i]), c2, nlse)) : 0.f;
                const float x1 = (kc + 1 <= kc_hi) ? fast_exp2(fmaf(__uint_as_float(sv[i + 1]), c2, nlse)) : 0.f;
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
        // ---- all MMAs of the item done (the tensor core retires them in issue order, group 1's last commit is the final one)
        const int last = (jb + n_round - 1) & 1;
        if (!mbar_wait(bar(3, wg), last, &budget)) timed_out = true;
        if (fuse) add_dq(red_row);
        if (wg == 0 && !mbar_wait(bar(3, 1), last, &budget)) timed_out = true;
        fence_after_sync();
        // group 0 writes dV, group 1 writes dK: lane t = column t of the gradient
        const uint32_t acc = lane_base + (wg == 0 ? TM_DV : TM_DK);
        float* dst = (wg == 0 ? p.dv : p.dk) + (int64_t)kv_row0 * (wg == 0 ? p.dv_stride_t : p.dk_stride_t) + kh * D + t;
        const int64_t rstride = (wg == 0 ? p.dv_stride_t : p.dk_stride_t);
        const float scale = (wg == 0) ? 1.f : p.sm_scale;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t v[32];
          tmem_ld32(acc + half * 32, v);
          wait_ld();
          if (half == 1) {
            fence_before_sync();
            mbar_arrive(acc_free);   // both halves are in registers: the next item's products may overwrite the accumulators
          }
          if (t < D) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int kc = half * 32 + i;
              if (kc < kv_rows) atomicAdd(dst + (int64_t)kc * rstride, __uint_as_float(v[i]) * scale);
            }
          }
        }
      }
      jb += n_round;
    }
  }
  if (warp < 8 && fuse && (tid & 127) < TOKQ * SLABS) tma::bulk_wait_all();   // the reductions have been written
  if (tid == 0) {   // the last CTA to get here leaves both counters at zero for the next launch
    __threadfence();
    if (atomicAdd(ticket + 1, 1) == (int)gridDim.x - 1) {
      ticket[0] = 0;
      ticket[1] = 0;
      __threadfence();
    }
  }
  if (timed_out && p.status) atomicOr(p.status, 2);
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, TM_COLS);
}

static int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  }
  return n;
}

template <int D>
static int launch(const NsaAttnParams* p, cudaStream_t st, const char* name, int fuse) {
  size_t smem = (size_t)(2 * 64 + 4 * 128) * D * 2 + 4 * 128 * 64 * 2 + 160 + 1024;
  cudaError_t e = cudaFuncSetAttribute(slc_bwd_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_error("%s: cudaFuncSetAttribute(%zu B) failed: %s", name, smem, cudaGetErrorString(e));
    return NSA_ERR_CUDA;
  }
  const int G = p->QH / p->KH;
  CUtensorMap tmq, tmo, tmdq, tmk, tmv;
  if (p->n_q_rows <= 0 || p->n_k_rows <= 0 || !tma::make_map(&tmq, p->q, p->n_q_rows, p->QH, D, p->q_stride_t, 1, G) ||
      !tma::make_map(&tmo, p->dout, p->n_q_rows, p->QH, D, p->do_stride_t, 1, G) ||
      !tma::make_map(&tmk, p->k, p->n_k_rows, p->KH, D, p->k_stride_t, 64, 1) ||
      !tma::make_map(&tmv, p->v, p->n_k_rows, p->KH, D, p->v_stride_t, 64, 1)) {
    set_error("%s: cuTensorMapEncodeTiled failed or is unavailable (q, dout, k, v must be 16-byte aligned; n_q_rows, n_k_rows set)", name);
    return NSA_ERR_CUDA;
  }
  if (!fuse) {
    tmdq = tmq;   // unused
  } else if (!tma::make_map(&tmdq, p->dq, p->n_q_rows, p->QH, D, p->dq_stride_t, 1, G)) {
    set_error("%s: cuTensorMapEncodeTiled failed for dq (must be 16-byte aligned with a row stride that is a multiple of 8)", name);
    return NSA_ERR_CUDA;
  }
  slc_bwd_tc_kernel<D><<<sm_count(), 480, smem, st>>>(*p, fuse, tmq, tmo, tmdq, tmk, tmv);
  return check_launch(name);
}

// dK/dV (and dQ when `fuse`) of the selected branch over the work items of the k2q index
int launch_slc_bwd_tc(const NsaAttnParams* p, cudaStream_t st, const char* name, int fuse) {
  return p->D == 128 ? launch<128>(p, st, name, fuse) : launch<64>(p, st, name, fuse);
}

}  // namespace nsa
