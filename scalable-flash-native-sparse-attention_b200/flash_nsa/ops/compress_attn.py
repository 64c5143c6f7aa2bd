"""Attention over the compressed keys/values (block-causal), with base-2 log-sum-exp.
Python surface of flash_nsa/ops/compress_attn.py."""
import torch

from ..utils import NSAHelper
from ._common import attn_params, call


def cmp_attn_fwd(q, k, v, sm_scale=None, o=None, helper=NSAHelper):
    """q [t,qh,d] (local rows), k/v [compressed rows, kh, d] -> (o [t,qh,d], lse [qh,t] fp32, base 2)."""
    T, QH, D = q.shape
    if sm_scale is None:
        sm_scale = D ** -0.5
    if o is None:
        o = torch.empty(T, QH, v.size(-1), device=q.device, dtype=q.dtype)
    lse = torch.empty(QH, T, device=q.device, dtype=torch.float32)
    if T > 0:
        call("nsa_cmp_attn_fwd", attn_params(q, k, v, helper, sm_scale, o=o, lse=lse, lse_is_head_major=True, need_y=True), q)
    return o, lse


def cmp_attn_bwd(q, k, v, o, lse, do, dq=None, sm_scale=None, fuse_dqdkdv=False, dkdv_dtype=torch.float,
                 dkdv_repeat=False, async_dq=False, helper=NSAHelper, delta=None):
    """Returns (dq, dk, dv).  With `dq` given the result is added into it; dk/dv come back in k's dtype.
    `async_dq=True` additionally returns a callable (a no-op here: dq is produced by the same launch sequence)."""
    T, QH, D = q.shape
    if sm_scale is None:
        sm_scale = D ** -0.5
    if not (do.stride(-1) == 1 and do.stride(1) == do.size(-1)):
        do = do.contiguous()
    acc_dq = dq is not None
    if dq is None:
        dq = torch.empty_like(q)
    dk = torch.zeros(k.shape, device=k.device, dtype=torch.float32)
    dv = torch.zeros(v.shape, device=v.device, dtype=torch.float32)
    have_delta = delta is not None   # sum_d o * do per (head, token), laid out like lse (e.g. from combine_bwd)
    if not have_delta:
        delta = torch.empty_like(lse)
    if T > 0 and k.size(0) > 0:
        p = attn_params(q, k, v, helper, sm_scale, o=o, lse=lse, lse_is_head_major=True, dout=do, delta=delta, dq=dq,
                        dk=dk, dv=dv, need_y=True)
        p.accumulate_dq = int(acc_dq)
        if have_delta:
            p.phases = 6
        call("nsa_cmp_attn_bwd", p, q)
    elif not acc_dq:
        dq.zero_()
    dk, dv = dk.to(k.dtype), dv.to(v.dtype)
    if async_dq:
        return dq, dk, dv, (lambda: None)
    return dq, dk, dv


class _CmpAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, sm_scale):
        if sm_scale is None:
            sm_scale = q.size(-1) ** -0.5
        o, lse = cmp_attn_fwd(q, k, v, sm_scale)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.sm_scale = sm_scale
        ctx.helper = NSAHelper.get_bwd_helper()
        ctx.mark_non_differentiable(lse)
        return o, lse

    @staticmethod
    def backward(ctx, do, *args):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = cmp_attn_bwd(q, k, v, o, lse, do, sm_scale=ctx.sm_scale, helper=ctx.helper)
        return dq, dk, dv, None


def compress_attn(q, k, v, sm_scale=None):
    """q [t,qh,d], k/v [total compressed rows, kh, d] -> (o, lse)"""
    return _CmpAttention.apply(q, k, v, sm_scale)
