// Key-block -> queries index for the selected-attention backward.
// For every (kv head, key block row) the list of local query rows that selected the block, in CSR form:
// count (histogram) -> exclusive scan -> fill.  Memory is O(T*top_n) instead of a dense [KH, blocks, T] table.
// Block rows are laid out piece by piece: row = blk_cu[piece] + block index inside the sequence.
// The order of the rows inside one list is not fixed (the fill uses an atomic cursor).
//
// Range buckets.  With range_rows > 0 the lists are split by the RANGE of the query row (q_row / range_rows): the CSR row
// of (range r, block row b) is the "cell" r * n_blocks_total + b, cells are ordered range-major.  The backward kernel
// walks the cells in that order, so everything that runs at the same time gathers q / dO rows and reduces into dq rows
// of ONE range, which is sized to stay in L2.  With item_rows > 0 the scan also cuts every cell into work items of at
// most item_rows list entries, (block row, first entry, end entry, range), in cell order: the unit of work of the
// persistent backward kernel (one cell of the always-selected first block holds range_rows entries, an average cell a few
// dozen, so cells themselves would not balance).
#include <mutex>
#include "nsa_common.cuh"

namespace nsa {

// Fill cursors for nsa_k2q_index_static: part of the library image, so every GPU that loads the library carries
// these 1 MiB until the process exits.  Shared by all calls on a device.
constexpr int kStaticCursorEntries = 262144;
static __device__ __align__(256) int32_t g_static_cursor[kStaticCursorEntries];

__device__ __forceinline__ int find_piece(const int32_t* cu, int n, int row) {
  int lo = 0, hi = n;  // largest b with cu[b] <= row
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (cu[mid] <= row) lo = mid; else hi = mid;
  }
  return lo;
}

__host__ __device__ __forceinline__ int n_ranges_of(const NsaK2qParams& p) {
  return p.range_rows > 0 ? (int)((p.Tq + p.range_rows - 1) / p.range_rows) : 1;
}
__host__ __device__ __forceinline__ int64_t n_cells_of(const NsaK2qParams& p) { return (int64_t)n_ranges_of(p) * p.n_blocks_total; }

// returns the CSR row (cell) of entry (kh, q_row, slot) or -1 when the slot is unused / out of range
__device__ __forceinline__ int entry_row(const NsaK2qParams& p, int kh, int64_t q_row, int slot) {
  int b = find_piece(p.meta.piece_cu, p.meta.n_pieces, (int)q_row);
  int off = p.meta.piece_off ? p.meta.piece_off[b] : 0;
  int t_abs = off + (int)q_row - p.meta.piece_cu[b];
  int nk = t_abs / p.hp.block_size;
  if (slot >= min(p.hp.top_n, nk + 1)) return -1;
  int blk = p.topk[((int64_t)kh * p.Tq + q_row) * p.hp.top_n + slot];
  if (blk < 0 || blk > nk) return -1;
  const int range = p.range_rows > 0 ? (int)(q_row / p.range_rows) : 0;
  return range * p.n_blocks_total + p.blk_cu[b] + blk;
}

__global__ void k2q_zero_kernel(NsaK2qParams p) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nc = n_cells_of(p);
  int64_t n_off = (int64_t)p.KH * (nc + 1), n_cur = (int64_t)p.KH * nc;
  if (i < n_off) p.offsets[i] = 0;
  if (i < n_cur) p.cursor[i] = 0;
  if (i < 2 && p.n_items) p.n_items[p.KH + i] = 0;   // ticket counters of the backward kernel
}

// Threads are slot-major (thread i = slot i / Tq of token i % Tq), so a warp holds one slot of 32 consecutive tokens: the
// forced slots (initial block, local blocks) then name the same block row in every lane, and one atomic per distinct
// row per warp (match + leader) replaces up to 32 atomics on one address.
__global__ void k2q_count_kernel(NsaK2qParams p) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int kh = blockIdx.y;
  const int lane = threadIdx.x & 31;
  int row = -1;
  if (i < p.Tq * p.hp.top_n) row = entry_row(p, kh, i % p.Tq, (int)(i / p.Tq));
  const unsigned grp = __match_any_sync(0xffffffffu, row);
  if (row >= 0 && lane == __ffs(grp) - 1) atomicAdd(p.offsets + (int64_t)kh * (n_cells_of(p) + 1) + row + 1, __popc(grp));
}

// inclusive scan over the 1024 threads of the CTA; `sums` is a 32-entry shared array (free again when the call returns)
__device__ __forceinline__ int block_scan_1024(int v, int* sums) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  int x = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane >= o) x += y;
  }
  if (lane == 31) sums[w] = x;
  __syncthreads();
  if (w == 0) {
    int s = sums[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int y = __shfl_up_sync(0xffffffffu, s, o);
      if (lane >= o) s += y;
    }
    sums[lane] = s;
  }
  __syncthreads();
  const int total = x + (w > 0 ? sums[w - 1] : 0);
  __syncthreads();
  return total;
}

// in-place inclusive scan of offsets[kh][1..n] (offsets[kh][0] stays 0): one CTA of 1024 threads per kv head.  With work
// items asked for, the same pass scans the item counts of the cells and writes each cell's items.
__global__ void k2q_scan_kernel(NsaK2qParams p) {
  __shared__ int sums[32];
  __shared__ int carry_s, carry_items;
  const int kh = blockIdx.x;
  const int64_t nc = n_cells_of(p);
  int* a = p.offsets + (int64_t)kh * (nc + 1) + 1;
  const int n = (int)nc, tid = threadIdx.x;
  const bool want_items = p.items != nullptr && p.item_rows > 0;
  int4* items = want_items ? reinterpret_cast<int4*>(p.items) + (int64_t)kh * p.items_cap : nullptr;
  if (tid == 0) { carry_s = 0; carry_items = 0; }
  __syncthreads();
  for (int base = 0; base < n; base += 1024) {
    const int i = base + tid;
    const int v = i < n ? a[i] : 0;
    const int c0 = carry_s, ci0 = carry_items;
    const int end = block_scan_1024(v, sums) + c0;
    if (i < n) a[i] = end;
    int n_it = 0, it_end = 0;
    if (want_items) {
      n_it = v > 0 ? (v + p.item_rows - 1) / p.item_rows : 0;
      it_end = block_scan_1024(n_it, sums) + ci0;
      const int start = end - v;
      const int row = i % max(p.n_blocks_total, 1), range = i / max(p.n_blocks_total, 1);
      for (int u = 0; u < n_it; ++u) {
        const int slot = it_end - n_it + u;
        const int lo = start + u * p.item_rows;
        if (slot < p.items_cap) items[slot] = make_int4(row, lo, min(end, lo + p.item_rows), range);
      }
    }
    __syncthreads();
    if (tid == 1023) { carry_s = end; carry_items = it_end; }
    __syncthreads();
  }
  if (want_items && tid == 0 && p.n_items) p.n_items[kh] = min(carry_items, p.items_cap);
}

__global__ void k2q_fill_kernel(NsaK2qParams p) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int kh = blockIdx.y;
  const int lane = threadIdx.x & 31;
  int row = -1;
  int64_t q_row = 0;
  if (i < p.Tq * p.hp.top_n) {
    q_row = i % p.Tq;
    row = entry_row(p, kh, q_row, (int)(i / p.Tq));
  }
  const unsigned grp = __match_any_sync(0xffffffffu, row);
  const int leader = __ffs(grp) - 1;
  int base = 0;
  const int64_t nc = n_cells_of(p);
  if (row >= 0 && lane == leader) base = atomicAdd(p.cursor + (int64_t)kh * nc + row, __popc(grp));
  base = __shfl_sync(0xffffffffu, base, leader);
  if (row < 0) return;
  const int pos = p.offsets[(int64_t)kh * (nc + 1) + row] + base + __popc(grp & ((1u << lane) - 1));
  p.tokens[(int64_t)kh * (p.Tq * p.hp.top_n) + pos] = (int)q_row;
}

}  // namespace nsa

using namespace nsa;

static int k2q_launch(const NsaK2qParams* p, cudaStream_t st);

extern "C" int nsa_k2q_index(const NsaK2qParams* p, void* stream) {
  NSA_REQUIRE(p && p->topk && p->offsets && p->tokens && p->cursor && p->blk_cu && p->meta.piece_cu, NSA_ERR_BAD_ARG,
              "k2q_index: null pointer");
  NSA_REQUIRE(p->KH > 0 && p->n_blocks_total >= 0 && p->hp.top_n > 0 && p->hp.block_size > 0, NSA_ERR_BAD_ARG, "k2q_index: bad sizes");
  NSA_REQUIRE(p->range_rows >= 0 && p->item_rows >= 0, NSA_ERR_BAD_ARG, "k2q_index: range_rows / item_rows must not be negative");
  NSA_REQUIRE(p->item_rows == 0 || (p->items && p->n_items && p->items_cap > 0), NSA_ERR_BAD_ARG,
              "k2q_index: item_rows > 0 needs items, n_items and items_cap");
  NSA_REQUIRE((((uintptr_t)p->items) & 15) == 0, NSA_ERR_BAD_ARG, "k2q_index: items must be 16-byte aligned");
  NSA_REQUIRE(n_cells_of(*p) < (1ll << 31), NSA_ERR_UNSUPPORTED_SHAPE, "k2q_index: ranges x block rows exceeds 2^31");
  return k2q_launch(p, (cudaStream_t)stream);
}

// Device address of g_static_cursor on the CURRENT device, looked up once per device.  In host code the array's
// name is only a handle for the runtime, never a pointer a kernel may dereference.
static int static_cursor_ptr(int32_t** out) {
  static std::mutex mu;
  static int32_t* ptrs[64] = {nullptr};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    set_error("k2q_index_static: cudaGetDevice failed or device ordinal %d out of range", dev);
    return NSA_ERR_CUDA;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (!ptrs[dev]) {
    void* sym = nullptr;
    e = cudaGetSymbolAddress(&sym, g_static_cursor);
    if (e != cudaSuccess || !sym) {
      set_error("k2q_index_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return NSA_ERR_CUDA;
    }
    ptrs[dev] = static_cast<int32_t*>(sym);
  }
  *out = ptrs[dev];
  return NSA_OK;
}

extern "C" int nsa_k2q_index_static(const NsaK2qParams* p, void* stream) {
  NSA_REQUIRE(p && p->topk && p->offsets && p->tokens && p->blk_cu && p->meta.piece_cu, NSA_ERR_BAD_ARG,
              "k2q_index_static: null pointer");
  NSA_REQUIRE(p->KH > 0 && p->n_blocks_total >= 0 && p->hp.top_n > 0 && p->hp.block_size > 0, NSA_ERR_BAD_ARG,
              "k2q_index_static: bad sizes");
  NSA_REQUIRE(p->range_rows >= 0 && p->item_rows >= 0, NSA_ERR_BAD_ARG, "k2q_index_static: range_rows / item_rows must not be negative");
  NSA_REQUIRE(p->item_rows == 0 || (p->items && p->n_items && p->items_cap > 0), NSA_ERR_BAD_ARG,
              "k2q_index_static: item_rows > 0 needs items, n_items and items_cap");
  NSA_REQUIRE((((uintptr_t)p->items) & 15) == 0, NSA_ERR_BAD_ARG, "k2q_index_static: items must be 16-byte aligned");
  const int64_t need = (int64_t)p->KH * n_cells_of(*p);
  NSA_REQUIRE(need <= kStaticCursorEntries, NSA_ERR_UNSUPPORTED_SHAPE,
              "k2q_index_static: KH * ranges * n_blocks_total = %lld exceeds the built-in scratch of %d entries; use nsa_k2q_index "
              "with caller-provided scratch", (long long)need, kStaticCursorEntries);
  NsaK2qParams q = *p;
  int rc = static_cursor_ptr(&q.cursor);
  if (rc) return rc;
  return k2q_launch(&q, (cudaStream_t)stream);
}

static int k2q_launch(const NsaK2qParams* p, cudaStream_t st) {
  int64_t nz = (int64_t)p->KH * (n_cells_of(*p) + 1);
  k2q_zero_kernel<<<(unsigned)((nz + 255) / 256), 256, 0, st>>>(*p);
  int64_t n = p->Tq * p->hp.top_n;
  if (n > 0 && p->n_blocks_total > 0) {
    dim3 grid((unsigned)((n + 255) / 256), p->KH);
    k2q_count_kernel<<<grid, 256, 0, st>>>(*p);
    k2q_scan_kernel<<<p->KH, 1024, 0, st>>>(*p);
    k2q_fill_kernel<<<grid, 256, 0, st>>>(*p);
  }
  return check_launch("k2q_index");
}
