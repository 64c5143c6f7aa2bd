"""Paged-KV inference entry points: `nsa_prefill` (chunked prefill) and `nsa_decode`, plus the per-step ops.
Same signatures as flash_nsa/inference/__init__.py:21-257 of the reference.

The KV cache is `k, v: [pages, page_size, kh, d]`; token p of a sequence lives at page `block_tables[b, p // page_size]`;
the compressed (mean-pooled) rows live in the SAME tensors, in the pages listed by `cmp_block_tables`, and are written in
place at the flat rows given by `cmp_slot_mapping` (-1 = already pooled / nothing new).  All kernels are the training
forward kernels running on a piece table with the paged-row lookup switched on: a prefill chunk or a decode token is a
"piece" whose first row sits at position context_len - new_tokens of its sequence.  No host synchronisation happens in
any of these calls, shapes depend only on the arguments, so a decode step can be captured in a CUDA graph.
"""
from ..ops._common import poll_status, post_status
from .ops import (mean_pooling_prefill, kv_mean_pooling_prefill, mean_pooling_decode, kv_mean_pooling_decode, cmp_attn_prefill, cmp_attn_decode,
                  topk_prefill, topk_decode, slc_attn_prefill, slc_attn_decode, fused_slc_swa_attn_decode, swa_prefill,
                  combine_prefill, combine_decode, nsa_decode_fused, decode_fused_supported, zero_cache_tails, one_step)


def store_kvcache(key, value, k_cache, v_cache, slot_mapping):
    """Write the new tokens' K/V rows into the paged cache: key/value [n, kh, d], caches [pages, page_size, kh, d],
    slot_mapping int32 [n] = flat cache row per token (-1 = skip).  The caller-side op of the serving engine
    (nano-vllm/nanovllm/layers/attention.py:147-154)."""
    from ..ops._common import S, call, ptr
    N, H, D = key.shape
    row = H * D
    assert key.stride(-1) == 1 and value.stride(-1) == 1 and key.stride(1) == D and value.stride(1) == D
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.size(-1) * k_cache.size(-2) == row
    assert slot_mapping.numel() == N and slot_mapping.dtype.is_signed and slot_mapping.element_size() == 4
    p = S["NsaStoreKvParams"]()
    p.key, p.value, p.k_cache, p.v_cache, p.slot_mapping = ptr(key), ptr(value), ptr(k_cache), ptr(v_cache), ptr(slot_mapping)
    p.key_stride, p.value_stride, p.N, p.row_elems = key.stride(0), value.stride(0), N, row
    if N > 0:
        call("nsa_store_kvcache", p, key)


def nsa_prefill(q, k, v, w, x_cu_seqlens, y_cu_seqlens, x_maxlen, y_maxlen, context_lens, block_tables, cmp_slot_mapping,
                cmp_block_tables, fixed_y_maxlen=8192, fixed_num_slc_blocks=2048, kernel_size=32, stride=16, block_size=64,
                top_n=16, num_init_blocks=1, num_local_blocks=2, window_size=512, sm_scale=None):
    """q [t,qh,d] new tokens (t = sum of chunk lengths), k/v caches already holding those tokens, w [t,qh,3] ->
    o [t,qh,d].  Mutates the caches: pooled rows are written at cmp_slot_mapping."""
    assert k.size(1) % 128 == 0
    if sm_scale is None:
        sm_scale = q.size(-1) ** -0.5
    poll_status(q.device)      # a pipeline time-out of an earlier call raises here, without synchronising
    hp = dict(kernel_size=kernel_size, stride=stride)
    with one_step():   # the four attention ops share the length tables derived from context_lens / x_cu_seqlens
        kv_mean_pooling_prefill(k, v, y_cu_seqlens, y_maxlen, block_table=block_tables, slot_mapping=cmp_slot_mapping, **hp)
        cmp_o, lse = cmp_attn_prefill(q, k, v, x_cu_seqlens, x_maxlen, block_tables=cmp_block_tables, context_lens=context_lens,
                                      sm_scale=sm_scale, **hp)
        topk = topk_prefill(q, k, lse, x_cu_seqlens, x_maxlen, y_maxlen, block_tables=cmp_block_tables, context_lens=context_lens,
                            fixed_y_maxlen=fixed_y_maxlen, fixed_num_slc_blocks=fixed_num_slc_blocks, sm_scale=sm_scale,
                            block_size=block_size, top_n=top_n, num_inital=num_init_blocks, num_local=num_local_blocks, **hp)
        slc_o, _ = slc_attn_prefill(q, k, v, topk, x_cu_seqlens, x_maxlen, block_tables=block_tables, context_lens=context_lens,
                                    block_size=block_size, top_n=top_n, sm_scale=sm_scale)
        swa_o = swa_prefill(q, k, v, x_cu_seqlens, x_maxlen, block_tables=block_tables, context_lens=context_lens,
                            window_size=window_size, sm_scale=sm_scale)
    o = combine_prefill(cmp_o, slc_o, swa_o, w)
    post_status(q.device)
    return o


def nsa_decode(q, k, v, w, context_lens, block_tables, cmp_slot_mapping, cmp_block_tables, cmp_num_splits=0, slc_num_splits=0,
               fixed_y_maxlen=8192, fixed_num_slc_blocks=2048, kernel_size=32, stride=16, block_size=64, top_n=16,
               num_init_blocks=1, num_local_blocks=2, window_size=512, sm_scale=None):
    """One new token per sequence: q [b,qh,d], w [b,qh,3] -> o [b,qh,d].  Rows with context_len == 0 (graph padding)
    produce zeros.  Runs as one fused launch when the configuration allows (kernel 32 / stride 16 / block 64, at most 16
    query heads per kv head), otherwise as the sequence of per-branch ops.  The split arguments are accepted for source
    compatibility (the fused kernel splits the KV ranges over the warps of a CTA by itself)."""
    assert k.size(1) % 128 == 0
    if sm_scale is None:
        sm_scale = q.size(-1) ** -0.5
    poll_status(q.device)      # as in nsa_prefill; skipped while the step is being captured into a CUDA graph
    if decode_fused_supported(q, k, kernel_size, stride, block_size, top_n, num_init_blocks, num_local_blocks):
        o = nsa_decode_fused(q, k, v, w, context_lens, block_tables, cmp_slot_mapping, cmp_block_tables, fixed_y_maxlen,
                             kernel_size, stride, block_size, top_n, num_init_blocks, num_local_blocks, window_size, sm_scale)
    else:
        o = nsa_decode_unfused(q, k, v, w, context_lens, block_tables, cmp_slot_mapping, cmp_block_tables, cmp_num_splits,
                               slc_num_splits, fixed_y_maxlen, fixed_num_slc_blocks, kernel_size, stride, block_size, top_n,
                               num_init_blocks, num_local_blocks, window_size, sm_scale)
    post_status(q.device)
    return o


def nsa_decode_unfused(q, k, v, w, context_lens, block_tables, cmp_slot_mapping, cmp_block_tables, cmp_num_splits=0,
                       slc_num_splits=0, fixed_y_maxlen=8192, fixed_num_slc_blocks=2048, kernel_size=32, stride=16, block_size=64,
                       top_n=16, num_init_blocks=1, num_local_blocks=2, window_size=512, sm_scale=None):
    """The decode step as the sequence of per-branch ops (the reference's structure); used for configurations the fused
    kernel does not cover and as a cross-check of it."""
    if sm_scale is None:
        sm_scale = q.size(-1) ** -0.5
    hp = dict(kernel_size=kernel_size, stride=stride)
    with one_step():
        kv_mean_pooling_decode(k, v, block_table=block_tables, slot_mapping=cmp_slot_mapping, context_lens=context_lens, **hp)
        cmp_o, lse = cmp_attn_decode(q, k, v, block_tables=cmp_block_tables, context_lens=context_lens, num_splits=cmp_num_splits,
                                     sm_scale=sm_scale, **hp)
        topk = topk_decode(q, k, lse, fixed_y_maxlen=fixed_y_maxlen, fixed_num_slc_blocks=fixed_num_slc_blocks,
                           block_tables=cmp_block_tables, context_lens=context_lens, block_size=block_size, top_n=top_n,
                           num_inital=num_init_blocks, num_local=num_local_blocks, sm_scale=sm_scale, **hp)
        slc_o, swa_o = fused_slc_swa_attn_decode(q, k, v, topk, num_splits=slc_num_splits, block_tables=block_tables,
                                                 context_lens=context_lens, block_size=block_size, top_n=top_n,
                                                 window_size=window_size, sm_scale=sm_scale)
    return combine_decode(cmp_o, slc_o, swa_o, w)
