"""Gate activations of the learned compression: swiglu and sigmoid-mul on a packed [.., 2K] tensor
(gate | up).  Python surface of flash_nsa/ops/act.py."""
import torch

from ._common import S, call, ptr


def _params(x, y, dy, dx, kind):
    p = S["NsaActParams"]()
    p.x, p.y, p.dy, p.dx = ptr(x), ptr(y), ptr(dy), ptr(dx)
    p.K = x.size(-1) // 2
    p.M = x.numel() // x.size(-1)
    p.kind = kind
    return p


def _fwd(x, kind):
    assert x.dtype in (torch.bfloat16, torch.float16) and x.is_contiguous() and x.size(-1) % 16 == 0
    y = torch.empty(*x.shape[:-1], x.size(-1) // 2, device=x.device, dtype=x.dtype)
    call("nsa_act_fwd", _params(x, y, None, None, kind), x)
    return y


def _bwd(x, dy, kind):
    """The gradient is written in place of x, as the reference does (flash_nsa/ops/act.py:56-57, 171-172)."""
    dy = dy.contiguous()
    call("nsa_act_bwd", _params(x, None, dy, x, kind), x)
    return x


def swiglu_fwd(x):
    return _fwd(x, 0)


def swiglu_bwd(x, dy):
    return _bwd(x, dy, 0)


def sigmoid_mul_fwd(x):
    return _fwd(x, 1)


def sigmoid_mul_bwd(x, dy):
    return _bwd(x, dy, 1)


class _Act(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, kind):
        ctx.save_for_backward(x)
        ctx.kind = kind
        return _fwd(x, kind)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        return _bwd(x, dy, ctx.kind), None


def swiglu_impl(x: torch.Tensor) -> torch.Tensor:
    return _Act.apply(x, 0)


def sigmoid_mul_impl(x: torch.Tensor) -> torch.Tensor:
    return _Act.apply(x, 1)
