"""Block-importance scores and top-n block selection, and the key-block -> queries index used by the
selected-attention backward.  Python surface of flash_nsa/ops/topk.py."""
import torch

from ..utils import NSAHelper, cdiv
from ._common import S, call, check_bf16_3d, hyper, is_cp, local_rows, ptr, seq_meta, status_word


@torch.no_grad()
def slc_topk_indices(q, k, lse, sm_scale=None, return_slc_prob=False, align=True, ignore_index=None, fp32=False,
                     maybe_efficient_version=False, scale_slc_p=True):
    """q [t,qh,d], k = compressed keys [rows,kh,d], lse [qh,t] of the compressed branch ->
    (topk [kh,t,top_n] int32, block scores or None).

    Selection compares, per (kv head, token), the pooled block scores.  As in the reference (topk.py:632-776) there are
    two paths.  `maybe_efficient_version=True` with kernel 32 / stride 16 / block 64 (what every module passes): scores in
    fp32 when `fp32`, otherwise rounded to half after cubing (`scale_slc_p`, while the padded block count is <= 2048) or
    without cubing.  Otherwise the general path, for any kernel_size / stride / block_size: per-row probabilities (summed
    over the kv head's query heads) rounded to half unless `fp32`, pooled in fp32 with the weights
    overlap(row window, block) / stride.  Unused slots hold `ignore_index` (default: number of blocks of the longest
    sequence).  Scores are never materialised unless `return_slc_prob`."""
    check_bf16_3d("q", q)
    check_bf16_3d("k", k)
    T, QH, D = q.shape
    KH = k.size(1)
    assert QH % KH == 0
    if sm_scale is None:
        sm_scale = D ** -0.5
    helper = NSAHelper
    num_slc_blocks = cdiv(helper.x_maxlen, NSAHelper.block_size)
    pad_blocks = max(1 << max(num_slc_blocks - 1, 0).bit_length(), 8) if align else max(num_slc_blocks, 8)
    assert ignore_index is None or ignore_index >= num_slc_blocks
    ignore_index = num_slc_blocks if ignore_index is None else ignore_index
    std = (NSAHelper.kernel_size, NSAHelper.stride, NSAHelper.block_size) == (32, 16, 64)
    general = not (maybe_efficient_version and std)
    if fp32:
        quant = 0
    elif general:
        quant = 3
    elif scale_slc_p and pad_blocks <= 2048:
        quant = 2
    else:
        quant = 1
    topk = torch.empty(KH, T, NSAHelper.top_n, dtype=torch.int32, device=q.device)
    probs = None
    if return_slc_prob:
        probs = torch.zeros(KH, T, pad_blocks, device=q.device, dtype=torch.float32 if quant in (0, 3) else torch.float16)
    if T == 0:
        return topk, probs
    p = S["NsaTopkParams"]()
    p.meta, p.hp = seq_meta(helper), hyper()
    p.q, p.ck, p.lse, p.topk, p.probs = ptr(q), ptr(k), ptr(lse), ptr(topk), ptr(probs)
    p.q_stride_t, p.ck_stride_t = q.stride(0), k.stride(0)
    p.status = ptr(status_word(q.device))
    assert lse.dtype == torch.float32 and lse.is_contiguous() and tuple(lse.shape) == (QH, T)
    p.lse_stride_t, p.lse_stride_h = 1, lse.stride(0)
    p.probs_stride_t = pad_blocks if probs is not None else 0
    p.sm_scale = float(sm_scale)
    p.QH, p.KH, p.D = QH, KH, D
    p.ignore_index, p.quant = ignore_index, quant
    p.q_rows, p.ck_rows = T, k.size(0)
    call("nsa_slc_topk", p, q)
    return topk, probs


class K2qIndex(tuple):
    """(offsets, tokens) of the key-block -> queries index, plus what the backward kernel needs: `items` [kh, cap, 4] =
    (block row, first entry, end entry, range) and `n_items` [kh] when work items were asked for, `range_rows` and
    `n_ranges`.  Unpacks as `offsets, tokens = index` like the plain form."""

    def __new__(cls, offsets, tokens, items=None, n_items=None, range_rows=0, n_ranges=1, cursor=None):
        self = super().__new__(cls, (offsets, tokens))
        self.offsets, self.tokens, self.items, self.n_items = offsets, tokens, items, n_items
        self.range_rows, self.n_ranges = range_rows, n_ranges
        self._cursor = cursor      # scratch of the build: kept until the index goes away (the build is asynchronous)
        return self


def backward_index_sizes(G, D, rows, max_blocks=None, top_n=16):
    """(range_rows, item_rows) that slc_attn_bwd asks for.  A range keeps q + dO + dq of the rows that the running CTAs
    touch in L2, but it also cuts every block's list into one cell per range, and a cell is worth running only when it fills
    whole query tiles: with `max_blocks` key blocks in the longest sequence a range of r rows gives cells of about
    r * top_n / max_blocks rows.  So the range is the power of two that gives >= 128 rows per cell, at least 4096 rows, and
    no ranges at all once that needs more than 32 MiB of q per range (measured on B200, one kv head of 16 heads, d = 128:
    64K tokens 2.85 ms without ranges / 2.63 with 8192-row ranges; one shard of 8 at 1M tokens 6.1 ms without / 19.3 with
    4096-row ranges).  An item holds at most 64 query tiles of 128 / G tokens (32: 2 % slower at 64K, 16: 9 %)."""
    per_row = G * D * 2
    cap = 1 << (((32 << 20) // per_row).bit_length() - 1)
    if max_blocks is None:
        want = cap // 2
    else:
        want = 1 << max(0, (128 * max_blocks + top_n - 1) // top_n - 1).bit_length()
    range_rows = max(want, min(4096, cap))
    if want > cap or rows <= range_rows:
        range_rows = 0
    return range_rows, 64 * max(128 // G, 1)


@torch.no_grad()
def get_bind_from_find(topk, helper=NSAHelper, range_rows=0, item_rows=0):
    """topk [kh,t,top_n] -> K2qIndex (offsets [kh, cells+1], tokens [kh, t*top_n]): for every (kv head, key block) the
    list of local query rows that selected it, `tokens[h, offsets[h,b]:offsets[h,b+1]]` (order inside a list not fixed).
    Block rows are laid out per piece (sequence, or shard piece under context parallelism) with k_cu_seqlens /
    cp_k_cu_seqlens.  `range_rows` > 0 splits every list by the range `row // range_rows` of the query row (cell =
    range * blocks + block row, range-major); `item_rows` > 0 also returns the work items of the backward kernel."""
    KH, T, top_n = topk.shape
    cp = is_cp(helper)
    blk_cu = helper.cp_k_cu_seqlens if cp else helper.k_cu_seqlens
    n_blocks = helper.cp_k_len if cp else helper.k_len
    n_ranges = cdiv(T, range_rows) if range_rows > 0 else 1
    n_cells = n_ranges * n_blocks
    dev = topk.device
    offsets = torch.empty(KH, n_cells + 1, dtype=torch.int32, device=dev)
    tokens = torch.empty(KH, max(T * top_n, 1), dtype=torch.int32, device=dev)
    cursor = torch.empty(KH, max(n_cells, 1), dtype=torch.int32, device=dev)
    p = S["NsaK2qParams"]()
    p.meta, p.hp = seq_meta(helper), hyper()
    p.hp.top_n = top_n
    p.topk, p.offsets, p.tokens, p.cursor, p.blk_cu = ptr(topk), ptr(offsets), ptr(tokens), ptr(cursor), ptr(blk_cu)
    p.Tq, p.KH, p.n_blocks_total = T, KH, n_blocks
    p.range_rows, p.item_rows = range_rows, item_rows
    items = n_items = None
    if item_rows > 0:
        cap = T * top_n // item_rows + min(n_cells, T * top_n) + 1
        items = torch.empty(KH, cap, 4, dtype=torch.int32, device=dev)
        n_items = torch.zeros(KH + 2, dtype=torch.int32, device=dev)   # + the backward kernel's two ticket counters
        p.items, p.n_items, p.items_cap = ptr(items), ptr(n_items), cap
    call("nsa_k2q_index", p, topk)
    return K2qIndex(offsets, tokens, items, n_items, range_rows, n_ranges, cursor)


@torch.no_grad()
def k2q_index_into(topk, offsets, tokens, helper=NSAHelper):
    """Builds the same index as `get_bind_from_find`, but into tensors the caller already owns and without any
    scratch allocation: the fill cursors live inside the kernel library.  Meant for callers that must not allocate
    device memory where they call this (a server whose memory pool already owns the whole GPU, a no-allocation
    region of a runtime).  `offsets` is int32 [kh, blocks+1], `tokens` int32 [kh, >= t*top_n]; kh * blocks must not
    exceed 262144.  Calls on one GPU share the library's scratch, so do not run two of them concurrently on
    different streams; issue the first call on a device outside stream capture."""
    KH, T, top_n = topk.shape
    cp = is_cp(helper)
    blk_cu = helper.cp_k_cu_seqlens if cp else helper.k_cu_seqlens
    n_blocks = helper.cp_k_len if cp else helper.k_len
    assert offsets.dtype == torch.int32 and tuple(offsets.shape) == (KH, n_blocks + 1) and offsets.is_contiguous()
    assert tokens.dtype == torch.int32 and tokens.size(0) == KH and tokens.size(1) == T * top_n and tokens.is_contiguous()
    p = S["NsaK2qParams"]()
    p.meta, p.hp = seq_meta(helper), hyper()
    p.hp.top_n = top_n
    p.topk, p.offsets, p.tokens, p.cursor, p.blk_cu = ptr(topk), ptr(offsets), ptr(tokens), 0, ptr(blk_cu)
    p.Tq, p.KH, p.n_blocks_total = T, KH, n_blocks
    call("nsa_k2q_index_static", p, topk)
    return offsets, tokens
