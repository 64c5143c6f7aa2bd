"""Sliding-window attention (keys t-window .. t, causal), own kernels instead of the reference's flash-attn
calls.  Python surface of flash_nsa/ops/sliding_window_attention.py."""
import torch

from ..utils import NSAHelper
from ._common import attn_params, call


def swa_fwd(q, k, v, sm_scale=None, out=None, helper=NSAHelper):
    """-> (o [t,qh,d], lse [t,qh] fp32 base 2).  Under context parallelism q is the local shard and k/v the
    gathered sequence; rows know their absolute position, so no k-slicing tables are needed."""
    T, QH, D = q.shape
    if sm_scale is None:
        sm_scale = D ** -0.5
    if out is None:
        out = torch.empty(T, QH, v.size(-1), device=q.device, dtype=q.dtype)
    lse = torch.empty(T, QH, device=q.device, dtype=torch.float32)
    if T > 0:
        call("nsa_swa_fwd", attn_params(q, k, v, helper, sm_scale, o=out, lse=lse), q)
    return out, lse


def swa_bwd(q, k, v, out, lse, dout, sm_scale=None, helper=NSAHelper, dq=None, dk=None, dv=None):
    """-> (dq bf16, dk, dv).  Given fp32 `dk`/`dv` the result is added into them (and they are returned),
    otherwise new tensors in k's dtype are returned; given `dq` the result is added into it."""
    T, QH, D = q.shape
    if sm_scale is None:
        sm_scale = D ** -0.5
    if not (dout.stride(-1) == 1 and dout.stride(1) == dout.size(-1)):
        dout = dout.contiguous()
    acc_dq = dq is not None
    if dq is None:
        dq = torch.empty_like(q)
    own = dk is None
    if own:
        dk = torch.zeros(k.shape, device=k.device, dtype=torch.float32)
        dv = torch.zeros(v.shape, device=v.device, dtype=torch.float32)
    delta = torch.empty_like(lse)
    p = attn_params(q, k, v, helper, sm_scale, o=out, lse=lse, dout=dout, delta=delta, dq=dq, dk=dk, dv=dv)
    p.accumulate_dq = int(acc_dq)
    if T > 0:
        call("nsa_swa_bwd", p, q)
    if own:
        return dq, dk.to(k.dtype), dv.to(v.dtype)
    return dq, dk, dv


def two_stage_swa_fwd(q, k, v, out, sm_scale=None, stage=1, helper=NSAHelper):
    """Context-parallel entry kept for source compatibility.  Stage 1 (local-only rows, used by the
    reference to hide the all-gather) does nothing here; stage 2 computes every row against the gathered K/V."""
    if stage == 1:
        return [None, None]
    _, lse = swa_fwd(q, k, v, sm_scale, out=out, helper=helper)
    return [lse, None]


def two_stage_swa_bwd(q, k, v, out, lse, dout, dq, dk, dv, sm_scale=None, stage=1, helper=NSAHelper):
    if stage == 1:
        return
    swa_bwd(q, k, v, out, lse[0], dout, sm_scale, helper=helper, dq=dq, dk=dk, dv=dv)


class _SWA(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, sm_scale):
        if sm_scale is None:
            sm_scale = q.size(-1) ** -0.5
        o, lse = swa_fwd(q, k, v, sm_scale)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.sm_scale = sm_scale
        ctx.helper = NSAHelper.get_bwd_helper()
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = swa_bwd(q, k, v, o, lse, do, ctx.sm_scale, helper=ctx.helper)
        return dq, dk, dv, None


def swa_varlen_func(q, k, v, sm_scale=None):
    """Causal attention of token t over keys t-window_size .. t of its own sequence."""
    return _SWA.apply(q, k, v, sm_scale)
