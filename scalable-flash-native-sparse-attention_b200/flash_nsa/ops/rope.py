"""Rotary position embedding applied to q and k in one launch.  Python surface of flash_nsa/ops/rope.py:

    e1 = x1 * cos1 - x2 * sin1,   e2 = x2 * cos2 + x1 * sin2      (x1, x2: first and second half of a head)

i.e. x * cos + rotate_half(x) * sin with cos, sin of the full head width."""
import torch

from ._common import S, call, ptr


def _launch(q, k, qe, ke, cos, sin, backward):
    B, N, QH, D = q.shape
    p = S["NsaRopeParams"]()
    p.q, p.k, p.qe, p.ke, p.cos, p.sin = ptr(q), ptr(k), ptr(qe), ptr(ke), ptr(cos), ptr(sin)
    p.q_stride_b, p.q_stride_n, p.q_stride_h = q.stride(0), q.stride(1), q.stride(2)
    p.k_stride_b, p.k_stride_n, p.k_stride_h = k.stride(0), k.stride(1), k.stride(2)
    p.qe_stride_b, p.qe_stride_n, p.qe_stride_h = qe.stride(0), qe.stride(1), qe.stride(2)
    p.ke_stride_b, p.ke_stride_n, p.ke_stride_h = ke.stride(0), ke.stride(1), ke.stride(2)
    p.cos_stride_b, p.cos_stride_n = cos.stride(0), cos.stride(1)
    p.B, p.N, p.QH, p.KH, p.D = B, N, QH, k.size(2), D
    p.backward = int(backward)
    if q.numel() + k.numel() > 0:
        call("nsa_rope", p, q)


def _check(q, k, cos, sin):
    assert q.dim() == 4 and k.dim() == 4 and q.shape[:2] == k.shape[:2] and q.size(-1) == k.size(-1)
    assert q.size(1) == cos.size(1)
    assert q.dtype in (torch.bfloat16, torch.float16) and k.dtype == q.dtype and cos.dtype == q.dtype and sin.dtype == q.dtype
    assert cos.shape == sin.shape and cos.stride() == sin.stride() and cos.size(-1) == q.size(-1)
    for t in (q, k, cos, sin):
        assert t.stride(-1) == 1


class _FusedApplyRope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, cos, sin, inplace):
        _check(q, k, cos, sin)
        if inplace:
            # written into the storage of q and k, which the caller gives up (as in the reference, the inputs are returned
            # without being marked dirty: they are usually views of a projection output, which autograd does not let a
            # two-output function modify, and nothing upstream needs their old values)
            qe, ke = q, k
        else:
            qe = torch.empty(q.shape, device=q.device, dtype=q.dtype)
            ke = torch.empty(k.shape, device=k.device, dtype=k.dtype)
        _launch(q, k, qe, ke, cos, sin, False)
        ctx.save_for_backward(cos, sin)
        return qe, ke

    @staticmethod
    def backward(ctx, dqe, dke):
        cos, sin = ctx.saved_tensors
        if dqe.stride(-1) != 1:
            dqe = dqe.contiguous()
        if dke.stride(-1) != 1:
            dke = dke.contiguous()
        dq, dk = torch.empty_like(dqe), torch.empty_like(dke)
        _launch(dqe, dke, dq, dk, cos, sin, True)
        return dq, dk, None, None, None


def fused_apply_rope(q, k, cos, sin, inplace=False):
    """q [b,s,qh,d], k [b,s,kh,d], cos/sin [b,s,d] (or [1,s,d], or with a singleton head axis) -> (qe, ke)."""
    if cos.dim() == 4:
        cos = cos.squeeze(-2)
    if sin.dim() == 4:
        sin = sin.squeeze(-2)
    if cos.size(0) != q.size(0):
        b = q.size(0)
        _, s, d = cos.shape
        cos = cos.expand(b, s, d)
        sin = sin.expand(b, s, d)
    return _FusedApplyRope.apply(q, k, cos, sin, inplace)
