"""Gated sum of the three branch outputs, o = sum_i sigmoid(w_i) * branch_i.
Python surface of flash_nsa/ops/combine.py."""
import math

import torch

from ._common import S, call, ptr


def _params(a, b, c, w):
    T, H, D = a.shape
    p = S["NsaCombineParams"]()
    p.a, p.b, p.c, p.w = ptr(a), ptr(b), ptr(c), ptr(w)
    p.a_stride_t, p.b_stride_t, p.c_stride_t, p.w_stride_t = a.stride(0), b.stride(0), c.stride(0), w.stride(0)
    p.T, p.H, p.D = T, H, D
    return p


def _check(a, b, c, w):
    T, H, D = a.shape
    assert a.shape == b.shape and a.shape == c.shape
    assert list(w.shape) == [T, H, 3], f"w.shape: {w.shape}, expected: [{T}, {H}, 3]"
    assert math.log2(D).is_integer()
    for name, t in (("a", a), ("b", b), ("c", c)):
        assert t.dtype == a.dtype and t.stride(-1) == 1 and t.stride(1) == D, f"{name}: one 16-bit dtype, contiguous heads"
    assert a.dtype in (torch.bfloat16, torch.float16) and w.dtype == a.dtype and w.stride(-1) == 1 and w.stride(1) == 3


def combine_fwd(a, b, c, w, out=None):
    _check(a, b, c, w)
    T, H, D = a.shape
    if out is None:
        out = torch.empty(T, H, D, device=a.device, dtype=a.dtype)
    assert out.stride(-1) == 1 and out.stride(1) == D
    p = _params(a, b, c, w)
    p.y, p.y_stride_t = ptr(out), out.stride(0)
    call("nsa_combine_fwd", p, a)
    return out


def combine_bwd(a, b, c, w, dout, dw=None, deltas=None):
    """Returns (da, db, dc, dw).  `deltas`: optional three fp32 [T,H] tensors (any strides, e.g. a transposed view)
    that receive sum_d x * dx per (token, head): the row term a branch backward otherwise computes in a pass of its
    own."""
    _check(a, b, c, w)
    if not (dout.stride(-1) == 1 and dout.stride(1) == dout.size(-1)):
        dout = dout.contiguous()
    da, db, dc = torch.empty(a.shape, device=a.device, dtype=a.dtype), torch.empty(a.shape, device=a.device, dtype=a.dtype), \
        torch.empty(a.shape, device=a.device, dtype=a.dtype)
    dw = torch.empty(w.shape, device=w.device, dtype=w.dtype) if dw is None else dw
    assert dw.stride(-1) == 1 and dw.stride(1) == 3
    p = _params(a, b, c, w)
    p.dy, p.dy_stride_t = ptr(dout), dout.stride(0)
    p.da, p.db, p.dc, p.dw, p.dw_stride_t = ptr(da), ptr(db), ptr(dc), ptr(dw), dw.stride(0)
    if deltas is not None:
        T, H, _ = a.shape
        for name, t in zip(("delta_a", "delta_b", "delta_c"), deltas):
            assert t.dtype == torch.float32 and list(t.shape) == [T, H], f"{name}: fp32 [T,H] (a transposed view is fine)"
            setattr(p, name, ptr(t))
            setattr(p, name + "_stride_t", t.stride(0))
            setattr(p, name + "_stride_h", t.stride(1))
    call("nsa_combine_bwd", p, a)
    return da, db, dc, dw


class _FusedSigmoidCombine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, c, w):
        ctx.save_for_backward(a, b, c, w)
        return combine_fwd(a, b, c, w)

    @staticmethod
    def backward(ctx, dout):
        a, b, c, w = ctx.saved_tensors
        return combine_bwd(a, b, c, w, dout)


def fused_sigmoid_combine(a, b, c, w):
    """a, b, c: [t,h,d]; w: [t,h,3] -> [t,h,d]"""
    return _FusedSigmoidCombine.apply(a, b, c, w)
