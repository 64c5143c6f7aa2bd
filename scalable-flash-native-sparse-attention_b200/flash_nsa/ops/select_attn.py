"""Attention over the selected key blocks.  Python surface of flash_nsa/ops/select_attn.py."""
import torch

from ..utils import NSAHelper
from ._common import attn_params, call, is_cp, ptr
from .topk import backward_index_sizes, get_bind_from_find


def slc_attn_fwd(q, k, v, topk, sm_scale=None, o=None, helper=NSAHelper):
    """q [t,qh,d], k/v [tokens,kh,d], topk [kh,t,top_n] -> (o, lse [t,qh] fp32 base 2)."""
    T, QH, D = q.shape
    if sm_scale is None:
        sm_scale = D ** -0.5
    if o is None:
        o = torch.empty(T, QH, v.size(-1), device=q.device, dtype=q.dtype)
    lse = torch.empty(T, QH, device=q.device, dtype=torch.float32)
    if T > 0:
        call("nsa_slc_attn_fwd", attn_params(q, k, v, helper, sm_scale, o=o, lse=lse, topk=topk), q)
    return o, lse


def slc_attn_bwd(q, k, v, topk, o, lse, do, dq=None, dk=None, dv=None, sm_scale=None, fuse_dqdkdv=False,
                 dkdv_dtype=torch.float, dkdv_repeat=True, async_dq=False, helper=NSAHelper, delta=None,
                 accumulate_dq=None, two_kernel_dq=False, range_rows=None, item_rows=None):
    """-> (dq, dk, dv).  Given `dq` (bf16) / `dk`,`dv` (fp32 [tokens,kh,d]) the results are added into them;
    otherwise dq is new and dk/dv come back in k's dtype.  dK/dV and dQ come from ONE block-major kernel whatever
    `fuse_dqdkdv` says (the reference's fuse_dqdkdv=True form, flash_nsa/ops/select_attn.py:148-335,646): per key block and
    query tile it adds dS K into dq with bf16 reductions, so the last bits of dq depend on the order of those adds.
    `two_kernel_dq=True` (not in the reference) runs the block-major dK/dV kernel and then the token-major dQ kernel, which
    accumulates a token's dq in fp32 in a fixed order.  `range_rows` / `item_rows` override the sizes of the key-block ->
    queries index (default: backward_index_sizes); they change the order of the work, not the result."""
    T, QH, D = q.shape
    if sm_scale is None:
        sm_scale = D ** -0.5
    if not (do.stride(-1) == 1 and do.stride(1) == do.size(-1)):
        do = do.contiguous()
    acc_dq = (dq is not None) if accumulate_dq is None else bool(accumulate_dq)   # False with a given dq: overwrite it
    if dq is None:
        dq = torch.empty_like(q)
    own = dk is None
    if own:
        dk = torch.zeros(k.shape, device=k.device, dtype=torch.float32)
        dv = torch.zeros(v.shape, device=v.device, dtype=torch.float32)
    have_delta = delta is not None   # sum_d o * do per (token, head), laid out like lse (e.g. from combine_bwd)
    if not have_delta:
        delta = torch.empty_like(lse)
    if T > 0:
        auto_r, auto_i = backward_index_sizes(QH // k.size(1), D, T, helper.cp_k_maxlen if is_cp(helper) else helper.k_maxlen,
                                              topk.size(-1))
        range_rows = auto_r if range_rows is None else range_rows
        item_rows = auto_i if item_rows is None else item_rows
        index = get_bind_from_find(topk, helper=helper, range_rows=range_rows, item_rows=item_rows)
        p = attn_params(q, k, v, helper, sm_scale, o=o, lse=lse, dout=do, delta=delta, dq=dq, dk=dk, dv=dv, topk=topk)
        attach_k2q(p, index, helper)
        p.accumulate_dq = int(acc_dq)
        if two_kernel_dq:
            p.phases = 2 if have_delta else 3
            call("nsa_slc_attn_bwd", p, q)
            p.phases = 4
        elif have_delta:
            p.phases = 6
        call("nsa_slc_attn_bwd", p, q)
    if own:
        dk, dv = dk.to(k.dtype), dv.to(v.dtype)
    if async_dq:
        return dq, dk, dv, (lambda: None)
    return dq, dk, dv


def attach_k2q(p, index, helper=NSAHelper):
    """Point an NsaAttnParams at a key-block -> queries index built by get_bind_from_find (the tensors must stay alive
    until the launch has been enqueued)."""
    offsets, tokens = index[0], index[1]
    assert getattr(index, "items", None) is not None, "the backward needs an index built with item_rows > 0"
    p.k2q_offsets, p.k2q_tokens = ptr(offsets), ptr(tokens)
    p.k2q_stride_h = tokens.stride(0)
    p.n_blocks_total = helper.cp_k_len if is_cp(helper) else helper.k_len
    p.k2q_blk_cu = ptr(helper.cp_k_cu_seqlens if is_cp(helper) else helper.k_cu_seqlens)
    p.k2q_items, p.k2q_n_items, p.k2q_items_cap = ptr(index.items), ptr(index.n_items), index.items.size(1)


class _SlcAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, topk, sm_scale):
        if sm_scale is None:
            sm_scale = q.size(-1) ** -0.5
        o, lse = slc_attn_fwd(q, k, v, topk, sm_scale)
        ctx.save_for_backward(q, k, v, o, lse, topk)
        ctx.sm_scale = sm_scale
        ctx.helper = NSAHelper.get_bwd_helper()
        return o

    @staticmethod
    def backward(ctx, do, *args):
        q, k, v, o, lse, topk = ctx.saved_tensors
        dq, dk, dv = slc_attn_bwd(q, k, v, topk, o, lse, do, sm_scale=ctx.sm_scale, helper=ctx.helper)
        return dq, dk, dv, None, None


def select_attn(q, k, v, topk, sm_scale=None):
    """q [t,qh,d], k/v [t,kh,d], topk [kh,t,top_n] -> o [t,qh,d]"""
    return _SlcAttention.apply(q, k, v, topk, sm_scale)
