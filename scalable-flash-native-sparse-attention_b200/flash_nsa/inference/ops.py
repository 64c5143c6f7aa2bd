"""Per-step paged-KV ops behind nsa_prefill / nsa_decode (Python surface of flash_nsa/inference/{compress_kv,
compress_attn,topk,select_attn,combine}.py).  Hyper-parameters arrive as arguments here (the reference's inference
functions do not read NSAHelper)."""
import torch

from .. import _lib
from ..ops._common import S, call, ptr, status_word
from ..ops.combine import combine_fwd


def _i32(t):
    assert t.dtype == torch.int32 and t.is_contiguous() or t.dim() == 2, "int32 tensors expected for lengths / tables"
    return t


def _hyper(kernel_size=32, stride=16, block_size=64, window=512, top_n=16, num_init=1, num_local=2):
    h = S["NsaHyper"]()
    h.kernel_size, h.stride, h.block_size, h.window = kernel_size, stride, block_size, window
    h.top_n, h.num_init, h.num_local = top_n, num_init, num_local
    return h


_STEP_TENSORS = None   # inside one_step(): the length tables of the step, built once and shared by its ops


class one_step:
    """Scope of one prefill / decode step: the ops called inside it share the piece tables they derive from the step's
    context_lens / x_cu_seqlens (about ten tiny launches per op otherwise).  The caller must not change those tensors inside."""

    def __enter__(self):
        global _STEP_TENSORS
        self.prev, _STEP_TENSORS = _STEP_TENSORS, {}
        return self

    def __exit__(self, *exc):
        global _STEP_TENSORS
        _STEP_TENSORS = self.prev
        return False


class _PagedMeta:
    """Piece table of an inference step, built with device-side ops only (no synchronisation)."""

    def __init__(self, context_lens, x_cu_seqlens, x_maxlen, kv_table, cmp_table, page_size, kernel_size, stride):
        dev = context_lens.device
        B = context_lens.numel()
        key = (context_lens.data_ptr(), B, None if x_cu_seqlens is None else x_cu_seqlens.data_ptr(), kernel_size, stride)
        shared = _STEP_TENSORS.get(key) if _STEP_TENSORS is not None else None
        if shared is not None:
            self.piece_cu, self.piece_off, self.x_cu, self.y_cu = shared
            if x_cu_seqlens is None:
                x_maxlen = 1
        else:
            ctx = context_lens.to(torch.int32)
            if x_cu_seqlens is None:      # decode: one row per sequence
                self.piece_cu = torch.arange(B + 1, dtype=torch.int32, device=dev)
                x_len = torch.ones(B, dtype=torch.int32, device=dev)
                x_maxlen = 1
            else:
                self.piece_cu = x_cu_seqlens.to(torch.int32).contiguous()
                x_len = self.piece_cu[1:] - self.piece_cu[:-1]
            self.piece_off = (ctx - x_len).contiguous()                     # position of the first new token; -1 for padding rows
            zero = torch.zeros(1, dtype=torch.int32, device=dev)
            self.x_cu = torch.cat([zero, torch.cumsum(ctx, 0, dtype=torch.int32)]).contiguous()
            y_len = torch.clamp((ctx - kernel_size) // stride + 1, min=0).to(torch.int32)
            self.y_cu = torch.cat([zero, torch.cumsum(y_len, 0, dtype=torch.int32)]).contiguous()
            if _STEP_TENSORS is not None:
                _STEP_TENSORS[key] = (self.piece_cu, self.piece_off, self.x_cu, self.y_cu)
        self.kv_table = kv_table
        self.cmp_table = cmp_table
        m = S["NsaSeqMeta"]()
        m.piece_cu, m.piece_seq, m.piece_off = ptr(self.piece_cu), 0, ptr(self.piece_off)
        m.x_cu, m.y_cu = ptr(self.x_cu), ptr(self.y_cu)
        m.n_pieces = m.n_seq = B
        m.max_piece_len = int(x_maxlen)
        m.x_maxlen, m.y_maxlen = 0, 0          # only used by training-side grids
        m.page_size = page_size
        if kv_table is not None:
            assert kv_table.dtype == torch.int32 and kv_table.stride(-1) == 1
            m.kv_table, m.kv_table_stride = ptr(kv_table), kv_table.stride(0)
        if cmp_table is not None:
            assert cmp_table.dtype == torch.int32 and cmp_table.stride(-1) == 1
            m.cmp_table, m.cmp_table_stride = ptr(cmp_table), cmp_table.stride(0)
        self.struct = m


def _flat(cache):
    """[pages, page, h, d] -> ([pages*page, h, d] view, page_size)"""
    assert cache.dim() == 4 and cache.is_contiguous() and cache.dtype in (torch.bfloat16, torch.float16)
    return cache.view(-1, cache.size(2), cache.size(3)), cache.size(1)


def _attn_params(q, kf, vf, meta, hp, sm_scale, o, lse, lse_head_major, topk=None):
    T, QH, D = q.shape
    assert q.dtype in (torch.bfloat16, torch.float16) and kf.dtype == q.dtype and vf.dtype == q.dtype
    assert q.stride(-1) == 1 and q.stride(1) == D
    KH = kf.size(1)
    p = S["NsaAttnParams"]()
    p.meta, p.hp = meta.struct, hp
    p.q, p.k, p.v, p.o, p.lse = ptr(q), ptr(kf), ptr(vf), ptr(o), ptr(lse)
    p.q_stride_t, p.k_stride_t, p.v_stride_t, p.o_stride_t = q.stride(0), kf.stride(0), vf.stride(0), o.stride(0)
    if lse_head_major:
        p.lse_stride_t, p.lse_stride_h = 1, lse.stride(0)
    else:
        p.lse_stride_t, p.lse_stride_h = lse.stride(0), 1
    if topk is not None:
        assert topk.dtype == torch.int32 and topk.is_contiguous()
        p.topk, p.topk_stride_h = ptr(topk), topk.stride(0)
        p.hp.top_n = topk.size(-1)
    p.sm_scale = float(sm_scale)
    p.QH, p.KH, p.D = QH, KH, D
    p.status = ptr(status_word(q.device))
    p.n_q_rows, p.n_k_rows = T, kf.size(0)   # the cache as one flat [pages * page_size, kh, d] tensor: the TMA-fed kernels map it
    return p


# ------------------------------------------------------------------------------------------------ pooling into the cache
def _pool(cache0, cache1, slot_mapping, block_table, y_cu_seqlens, y_maxlen, context_lens, kernel_size, stride, decode):
    f0, page = _flat(cache0)
    p = S["NsaPagedPoolParams"]()
    p.cache0 = ptr(f0)
    p.cache1 = ptr(_flat(cache1)[0]) if cache1 is not None else 0
    p.slot_mapping, p.kv_table = ptr(slot_mapping), ptr(block_table)
    p.y_cu, p.context_lens = ptr(y_cu_seqlens), ptr(context_lens)
    p.row_stride = f0.stride(0)
    p.B = block_table.size(0)
    p.H, p.D = f0.size(1), f0.size(2)
    p.page_size, p.table_stride = page, block_table.stride(0)
    p.y_maxlen = int(y_maxlen) if y_maxlen is not None else 0
    p.kernel_size, p.stride, p.decode = kernel_size, stride, int(decode)
    assert slot_mapping.dtype == torch.int32 and block_table.dtype == torch.int32
    call("nsa_paged_mean_pool", p, cache0)


def zero_cache_tails(k_cache, v_cache, lens, block_table, compressed=None):
    """Clear the cache rows [lens[b], next multiple of 128) of every sequence (rows of the kind `block_table` lists: token
    rows with the context lengths, compressed rows with the compressed-row counts).  The TMA-fed prefill kernels read whole
    128-row tiles of a page, and what lies past a sequence's end may be never-written memory (0 * NaN); those rows belong
    to no one yet, so clearing them changes nothing a later step reads.  `compressed=(kernel_size, stride)`: `lens` are
    token counts and the rows are the compressed rows they give."""
    f0, page = _flat(k_cache)
    p = S["NsaPagedPoolParams"]()
    p.cache0, p.cache1 = ptr(f0), ptr(_flat(v_cache)[0])
    p.kv_table, p.context_lens = ptr(block_table), ptr(lens)
    p.row_stride = f0.stride(0)
    p.B = block_table.size(0)
    p.H, p.D = f0.size(1), f0.size(2)
    p.page_size, p.table_stride = page, block_table.stride(0)
    if compressed is not None:
        p.kernel_size, p.stride, p.decode = int(compressed[0]), int(compressed[1]), 2
    assert lens.dtype == torch.int32 and block_table.dtype == torch.int32 and lens.numel() >= p.B
    call("nsa_paged_zero_tails", p, k_cache)


def mean_pooling_prefill(x, y_cu_seqlens, y_maxlen, slot_mapping, block_table, kernel_size=32, stride=16):
    """Pool every compressed row that has a slot (slot_mapping != -1) from the paged tokens, in place."""
    _pool(x, None, slot_mapping, block_table, y_cu_seqlens, y_maxlen, None, kernel_size, stride, False)
    return x


def kv_mean_pooling_prefill(k, v, y_cu_seqlens, y_maxlen, slot_mapping, block_table, kernel_size=32, stride=16):
    """K and V caches in one launch (the reference pools them one after the other, inference/__init__.py:76-77)."""
    assert k.shape == v.shape
    _pool(k, v, slot_mapping, block_table, y_cu_seqlens, y_maxlen, None, kernel_size, stride, False)


def mean_pooling_decode(x, slot_mapping, block_table, context_lens=None, kernel_size=32, stride=16):
    _pool(x, None, slot_mapping, block_table, None, None, context_lens, kernel_size, stride, True)
    return x


def kv_mean_pooling_decode(k, v, slot_mapping, block_table, context_lens=None, kernel_size=32, stride=16):
    """K and V in one launch: the window ending at the newest token, when it completes a compressed row."""
    assert k.shape == v.shape
    _pool(k, v, slot_mapping, block_table, None, None, context_lens, kernel_size, stride, True)


# ------------------------------------------------------------------------------------------------ compressed attention
def cmp_attn_prefill(q, k, v, x_cu_seqlens, x_maxlen, block_tables, context_lens, kernel_size=32, stride=16, sm_scale=None):
    """-> (o [t,qh,d], lse [qh,t]); `block_tables` are the pages of the compressed rows."""
    T, QH, D = q.shape
    sm_scale = D ** -0.5 if sm_scale is None else sm_scale
    kf, page = _flat(k)
    vf, _ = _flat(v)
    meta = _PagedMeta(context_lens, x_cu_seqlens, x_maxlen, None, block_tables, page, kernel_size, stride)
    o = torch.empty(T, QH, D, device=q.device, dtype=q.dtype)
    lse = torch.empty(QH, T, device=q.device, dtype=torch.float32)
    if T:
        if x_maxlen >= 64 and page >= 128:   # the 128-row-tile kernel will run: the rows after each sequence's last compressed row
            zero_cache_tails(k, v, context_lens, block_tables, compressed=(kernel_size, stride))
        call("nsa_cmp_attn_fwd", _attn_params(q, kf, vf, meta, _hyper(kernel_size, stride), sm_scale, o, lse, True), q)
    return o, lse


def cmp_attn_decode(q, k, v, block_tables, context_lens, out=None, num_splits=0, max_num_splits=4, kernel_size=32, stride=16,
                    sm_scale=None, tma=True, bench=False):
    """-> (o [b,qh,d], lse [b,qh])"""
    B, QH, D = q.shape
    sm_scale = D ** -0.5 if sm_scale is None else sm_scale
    kf, page = _flat(k)
    vf, _ = _flat(v)
    meta = _PagedMeta(context_lens, None, 1, None, block_tables, page, kernel_size, stride)
    o = torch.empty(B, QH, D, device=q.device, dtype=q.dtype) if out is None else out
    lse = torch.empty(B, QH, device=q.device, dtype=torch.float32)
    if B:
        call("nsa_cmp_attn_fwd", _attn_params(q, kf, vf, meta, _hyper(kernel_size, stride), sm_scale, o, lse, False), q)
    return o, lse


# ------------------------------------------------------------------------------------------------ top-n
def _topk(q, k, lse, lse_head_major, meta_args, block_size, top_n, num_inital, num_local, kernel_size, stride, sm_scale,
          fixed_num_slc_blocks=2048, y_maxlen=0):
    T, QH, D = q.shape
    kf, page = _flat(k)
    KH = kf.size(1)
    meta = _PagedMeta(*meta_args, page, kernel_size, stride)
    meta.struct.x_maxlen = int(fixed_num_slc_blocks) * block_size   # bound of the sequence length (general-size kernel)
    topk = torch.empty(KH, T, top_n, dtype=torch.int32, device=q.device)
    ck_rows = 0
    x_maxlen = meta_args[2]
    if (y_maxlen and x_maxlen >= 64 and (kernel_size, stride, block_size) == (32, 16, 64) and top_n - num_inital - num_local == 13
            and QH // KH <= 64 and T):
        # a prefill chunk: the compressed K rows of the batch are few (tokens / 16), so they are copied out of their pages
        # into one contiguous buffer and the tcgen05 scoring kernel runs on that (its tiles cannot follow a page table)
        B = meta_args[0].numel()
        ck_rows = B * int(y_maxlen)
        gathered = torch.empty(ck_rows, KH, D, dtype=kf.dtype, device=kf.device)
        g = S["NsaPagedPoolParams"]()
        g.cache0, g.cache1 = ptr(kf), ptr(gathered)
        g.kv_table, g.y_cu = ptr(meta.cmp_table), ptr(meta.y_cu)
        g.row_stride, g.B, g.H, g.D = kf.stride(0), B, KH, D
        g.page_size, g.table_stride, g.y_maxlen = page, meta.cmp_table.stride(0), int(y_maxlen)
        call("nsa_paged_gather_rows", g, q)
        kf = gathered
        meta.struct.cmp_table, meta.struct.cmp_table_stride = 0, 0
    p = S["NsaTopkParams"]()
    p.meta, p.hp = meta.struct, _hyper(kernel_size, stride, block_size, 0, top_n, num_inital, num_local)
    p.q, p.ck, p.lse, p.topk, p.probs = ptr(q), ptr(kf), ptr(lse), ptr(topk), 0
    p.q_stride_t, p.ck_stride_t = q.stride(0), kf.stride(0)
    p.q_rows, p.ck_rows = T, ck_rows
    p.status = ptr(status_word(q.device))
    if lse_head_major:
        p.lse_stride_t, p.lse_stride_h = 1, lse.stride(0)
    else:
        p.lse_stride_t, p.lse_stride_h = lse.stride(0), 1
    p.sm_scale = float(D ** -0.5 if sm_scale is None else sm_scale)
    p.QH, p.KH, p.D = QH, KH, D
    p.ignore_index, p.quant = -1, 0        # block scores stay in fp32 here (the reference rounds per-row scores to half)
    if T:
        call("nsa_slc_topk", p, q)
    return topk


@torch.no_grad()
def topk_prefill(q, k, lse, x_cu_seqlens, x_maxlen, y_maxlen, block_tables, context_lens, fixed_y_maxlen=8192,
                 fixed_num_slc_blocks=2048, kernel_size=32, stride=16, block_size=64, top_n=16, num_inital=1, num_local=2,
                 sm_scale=None, fp32=False):
    """-> topk [kh,t,top_n] int32, unused slots = -1"""
    return _topk(q, k, lse, True, (context_lens, x_cu_seqlens, x_maxlen, None, block_tables), block_size, top_n, num_inital,
                 num_local, kernel_size, stride, sm_scale, fixed_num_slc_blocks, y_maxlen=y_maxlen)


@torch.no_grad()
def topk_decode(q, k, lse, block_tables, context_lens, kernel_size=32, stride=16, block_size=64, top_n=16, num_inital=1,
                num_local=2, fixed_num_slc_blocks=2048, fixed_y_maxlen=8192, sm_scale=None, persistent=False, workers=4):
    """-> topk [kh,b,top_n] int32, unused slots = -1; lse is [b,qh]"""
    return _topk(q, k, lse, False, (context_lens, None, 1, None, block_tables), block_size, top_n, num_inital, num_local,
                 kernel_size, stride, sm_scale, fixed_num_slc_blocks)


# ------------------------------------------------------------------------------------------------ selected + window attention
def _token_branch(fn, q, k, v, meta_args, hp, sm_scale, topk=None):
    T, QH, D = q.shape
    sm_scale = D ** -0.5 if sm_scale is None else sm_scale
    kf, page = _flat(k)
    vf, _ = _flat(v)
    meta = _PagedMeta(*meta_args, page, hp.kernel_size, hp.stride)
    o = torch.empty(T, QH, D, device=q.device, dtype=q.dtype)
    lse = torch.empty(T, QH, device=q.device, dtype=torch.float32)
    if T:
        call(fn, _attn_params(q, kf, vf, meta, hp, sm_scale, o, lse, False, topk), q)
    return o, lse


def slc_attn_prefill(q, k, v, topk, x_cu_seqlens, x_maxlen, block_tables, context_lens, block_size=64, top_n=16, sm_scale=None):
    return _token_branch("nsa_slc_attn_fwd", q, k, v, (context_lens, x_cu_seqlens, x_maxlen, block_tables, None),
                         _hyper(block_size=block_size, top_n=top_n), sm_scale, topk)


def slc_attn_decode(q, k, v, topk, block_tables, context_lens, block_size=64, top_n=16, num_splits=4, out=None, sm_scale=None,
                    bench=False):
    return _token_branch("nsa_slc_attn_fwd", q, k, v, (context_lens, None, 1, block_tables, None),
                         _hyper(block_size=block_size, top_n=top_n), sm_scale, topk)


def swa_prefill(q, k, v, x_cu_seqlens, x_maxlen, block_tables, context_lens, window_size=512, sm_scale=None):
    """Sliding-window attention of the new tokens over the paged cache (the reference calls flash-attn here,
    flash_nsa/inference/__init__.py:125-155)."""
    if q.size(0) and x_maxlen >= 64 and k.size(1) >= 128:   # the 128-row-tile kernel will run (see zero_cache_tails)
        zero_cache_tails(k, v, context_lens, block_tables)
    return _token_branch("nsa_swa_fwd", q, k, v, (context_lens, x_cu_seqlens, x_maxlen, block_tables, None),
                         _hyper(window=window_size), sm_scale)[0]


def fused_slc_swa_attn_decode(q, k, v, topk, block_tables, context_lens, out=None, num_splits=0, max_num_splits=4, block_size=64,
                              top_n=16, window_size=512, sm_scale=None, bench=False):
    """-> (slc_o, swa_o), each [b,qh,d].  Two launches here (selected blocks, window)."""
    slc_o, _ = slc_attn_decode(q, k, v, topk, block_tables, context_lens, block_size, top_n, sm_scale=sm_scale)
    swa_o, _ = _token_branch("nsa_swa_fwd", q, k, v, (context_lens, None, 1, block_tables, None), _hyper(window=window_size),
                             sm_scale)
    return slc_o, swa_o


# ------------------------------------------------------------------------------------------------ combine
def combine_prefill(a, b, c, w, out=None):
    return combine_fwd(a, b, c, w, out=out)


def combine_decode(a, b, c, w, out=None):
    return combine_fwd(a, b, c, w, out=out)


# ------------------------------------------------------------------------------------------------ fused decode step
def decode_fused_supported(q, k, kernel_size, stride, block_size, top_n, num_init_blocks, num_local_blocks):
    QH, KH, D = q.size(1), k.size(2), q.size(2)
    page = k.size(1)
    return (kernel_size == 32 and stride == 16 and block_size == 64 and QH % KH == 0 and QH // KH <= 16 and D in (64, 128)
            and top_n <= 32 and num_init_blocks + num_local_blocks <= top_n and page >= 64 and page & (page - 1) == 0)


def decode_cluster_size(B, KH, page_size, table_width, D=128, fixed_y_maxlen=8192):
    """CTAs the one-launch decode step gives each (sequence, kv head) for a batch of B sequences whose page table has
    `table_width` columns: 1, or 2 / 4 / 8 (a thread-block cluster) for few sequences with room for long contexts."""
    from .._lib import lib
    import ctypes
    p = S["NsaDecodeParams"]()
    p.B, p.KH, p.QH, p.D, p.page_size, p.kv_table_stride = B, KH, KH, D, page_size, table_width
    p.hp = _hyper()
    p.y_cap = min((int(fixed_y_maxlen) + 3) // 4 * 4, ((8 * (32 + 16 * D) - 16) * 4 // 5) // 4 * 4)
    n = lib().nsa_decode_cluster_size(ctypes.byref(p))
    assert n > 0, lib().nsa_last_error().decode()
    return n


def nsa_decode_fused(q, k, v, w, context_lens, block_tables, cmp_slot_mapping, cmp_block_tables, fixed_y_maxlen=8192,
                     kernel_size=32, stride=16, block_size=64, top_n=16, num_init_blocks=1, num_local_blocks=2, window_size=512,
                     sm_scale=None, return_topk=False):
    """The whole decode step in ONE launch (pooling of the new compressed row, the three branches, top-n, combine).
    `fixed_y_maxlen` bounds the compressed rows of a sequence (it sizes a shared-memory array; 8192 = 128K tokens)."""
    B, QH, D = q.shape
    kf, page = _flat(k)
    vf, _ = _flat(v)
    KH = kf.size(1)
    assert q.dtype in (torch.bfloat16, torch.float16) and kf.dtype == q.dtype and vf.dtype == q.dtype and w.dtype == q.dtype
    assert q.stride(-1) == 1 and q.stride(1) == D and w.stride(-1) == 1 and w.stride(1) == 3
    o = torch.empty(B, QH, D, device=q.device, dtype=q.dtype)
    topk = torch.empty(KH, B, top_n, dtype=torch.int32, device=q.device) if return_topk else None
    p = S["NsaDecodeParams"]()
    p.q, p.k_cache, p.v_cache, p.w, p.o = ptr(q), ptr(kf), ptr(vf), ptr(w), ptr(o)
    p.context_lens, p.kv_table, p.cmp_table = ptr(context_lens), ptr(block_tables), ptr(cmp_block_tables)
    p.slot_mapping, p.topk_out, p.status = ptr(cmp_slot_mapping), ptr(topk), ptr(status_word(q.device))
    p.hp = _hyper(kernel_size, stride, block_size, window_size, top_n, num_init_blocks, num_local_blocks)
    p.q_stride_t, p.o_stride_t, p.w_stride_t, p.cache_stride_t = q.stride(0), o.stride(0), w.stride(0), kf.stride(0)
    p.sm_scale = float(D ** -0.5 if sm_scale is None else sm_scale)
    p.B, p.QH, p.KH, p.D = B, QH, KH, D
    p.page_size, p.kv_table_stride, p.cmp_table_stride = page, block_tables.stride(0), cmp_block_tables.stride(0)
    fit = ((8 * (32 + 16 * D) - 16) * 4 // 5) // 4 * 4        # what the kernel's shared-memory score array can hold
    p.y_cap = min((int(fixed_y_maxlen) + 3) // 4 * 4, fit)
    p.cache_rows = kf.size(0)
    for t_ in (context_lens, block_tables, cmp_block_tables, cmp_slot_mapping):
        assert t_.dtype == torch.int32
    if B:
        call("nsa_decode_fused", p, q)
    return (o, topk) if return_topk else o
