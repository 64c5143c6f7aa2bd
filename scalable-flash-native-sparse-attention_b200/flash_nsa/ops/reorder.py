"""Chunk reorder between sequential order and the rank-major zig-zag order of cp_mode=2.
Python surface of flash_nsa/ops/reorder.py."""
import torch

from ._common import S, call, ptr


def reorder(x, world_size, shuffle_mode="shuffle", inplace=False, out=None):
    """`out` (same shape and dtype, not aliasing x) receives the result when given; the kernel runs on the current stream."""
    assert shuffle_mode in ("shuffle", "unshuffle")
    assert x.is_contiguous() and x.size(0) % (2 * world_size) == 0
    chunk_bytes = x.numel() * x.element_size() // (2 * world_size)
    assert chunk_bytes % 16 == 0
    if out is not None:
        assert not inplace and out.shape == x.shape and out.dtype == x.dtype and out.is_contiguous() and out.data_ptr() != x.data_ptr()
    y = torch.empty_like(x) if out is None else out
    p = S["NsaReorderParams"]()
    p.x, p.y, p.chunk_bytes, p.world_size, p.unshuffle = ptr(x), ptr(y), chunk_bytes, world_size, int(shuffle_mode == "unshuffle")
    if x.numel():
        call("nsa_reorder", p, x)
    if inplace:
        x.copy_(y)
        return x
    return y
