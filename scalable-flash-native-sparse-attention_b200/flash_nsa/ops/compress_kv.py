"""KV compression: window mean pooling and window gather (im2col) with their backward passes.
Python surface of flash_nsa/ops/compress_kv.py (mean_pooling, construct_block and the *_fwd/_bwd functions)."""
from typing import Optional

import torch

from ..utils import NSAHelper
from ._common import S, call, check_bf16_3d, hyper, ptr, seq_meta


def _pool_params(x, y, dx, helper, accumulate):
    p = S["NsaPoolParams"]()
    p.meta, p.hp = seq_meta(helper, cp=False), hyper()
    p.x, p.y, p.dx = ptr(x), ptr(y), ptr(dx)
    p.x_stride_t = x.stride(0) if x is not None else 0
    p.y_stride_t = y.stride(0)
    p.dx_stride_t = dx.stride(0) if dx is not None else 0
    p.H, p.D = y.size(1), y.size(2)
    p.accumulate = int(accumulate)
    return p


def mean_pooling_fwd(x, helper=NSAHelper):
    check_bf16_3d("x", x)
    T, H, D = x.shape
    y = torch.empty(helper.y_len, H, D, device=x.device, dtype=x.dtype)
    call("nsa_mean_pool_fwd", _pool_params(x, y, None, helper, False), x)
    return y


def mean_pooling_bwd(x, dy, dx: Optional[torch.Tensor] = None, helper=NSAHelper):
    """With `dx` (fp32 [T,H,D]) the pooled gradient is added into it; without, a new tensor in x's dtype is returned."""
    dy = dy.contiguous()
    check_bf16_3d("dy", dy)
    if dx is not None:
        assert dx.dtype == torch.float32 and dx.stride(-1) == 1 and dx.stride(1) == dx.size(-1)
        call("nsa_mean_pool_bwd", _pool_params(None, dy, dx, helper, True), dy)
        return dx
    out = torch.empty(x.shape, device=x.device, dtype=torch.float32)
    call("nsa_mean_pool_bwd", _pool_params(None, dy, out, helper, False), dy)
    return out.to(x.dtype)


def _block_params(x, y, dx, helper, accumulate):
    p = S["NsaBlockParams"]()
    p.meta, p.hp = seq_meta(helper, cp=False), hyper()
    p.x, p.y, p.dx = ptr(x), ptr(y), ptr(dx)
    p.x_stride_t = x.stride(0) if x is not None else 0
    p.dx_stride_t = dx.stride(0) if dx is not None else 0
    p.H, p.D = y.size(1), y.size(3)
    p.accumulate = int(accumulate)
    return p


def construct_block_fwd(x, helper=NSAHelper):
    check_bf16_3d("x", x)
    T, H, D = x.shape
    y = torch.empty(helper.y_len, H, NSAHelper.kernel_size, D, device=x.device, dtype=x.dtype)
    call("nsa_construct_block_fwd", _block_params(x, y, None, helper, False), x)
    return y


def construct_block_bwd(x, dy, dx: Optional[torch.Tensor] = None, helper=NSAHelper):
    dy = dy.contiguous()
    assert dy.dtype in (torch.bfloat16, torch.float16) and dy.dim() == 4
    if dx is not None:
        assert dx.dtype == torch.float32
        call("nsa_construct_block_bwd", _block_params(None, dy, dx, helper, True), dy)
        return dx
    out = torch.empty(x.shape, device=x.device, dtype=torch.float32)
    call("nsa_construct_block_bwd", _block_params(None, dy, out, helper, False), dy)
    return out.to(x.dtype)


class _MeanPooling(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        ctx.save_for_backward(x)
        ctx.helper = NSAHelper.get_bwd_helper()
        return mean_pooling_fwd(x)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        return mean_pooling_bwd(x, dy, helper=ctx.helper)


class _ConstructBlock(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        ctx.save_for_backward(x)
        ctx.helper = NSAHelper.get_bwd_helper()
        return construct_block_fwd(x)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        return construct_block_bwd(x, dy, helper=ctx.helper)


def mean_pooling(x: torch.Tensor) -> torch.Tensor:
    """[t,h,d] -> [total compressed rows, h, d]: mean over windows of kernel_size tokens every stride tokens."""
    return _MeanPooling.apply(x)


def construct_block(x: torch.Tensor) -> torch.Tensor:
    """[t,h,d] -> [total compressed rows, h, kernel_size, d]: the windows themselves."""
    return _ConstructBlock.apply(x)
