"""Splitting a packed batch over the context-parallel ranks, and the rule that picks the shard layout
(flash_nsa/get_batch.py:11-56), without the Megatron imports: the group size and rank are arguments (or come from a
torch.distributed process group).

cp_mode 1: the token axis is cut into cp_size contiguous chunks, rank r takes chunk r.
cp_mode 2: it is cut into 2 * cp_size chunks, rank r takes chunks r and 2 * cp_size - 1 - r (balanced for one long
causal sequence, whose cost grows with the position)."""
from typing import Any, Dict, Optional, Sequence

import torch


def get_cp_mode_from_cu_seqlens(cu_seqlens, cp_size: int, threshold: Optional[float] = None) -> int:
    """cp_mode 2 when the longest sequence is at least `threshold` tokens (default 1.5 x the tokens per rank), else 1."""
    cu = torch.as_tensor(cu_seqlens).cpu()
    total = int(cu[-1])
    if threshold is None:
        threshold = total // cp_size * 1.5
    max_len = int((cu[1:] - cu[:-1]).max())
    return 2 if max_len >= threshold else 1


def split_for_cp_rank(val: torch.Tensor, cp_size: int, cp_rank: int, cp_mode: int, dim: int = -1) -> torch.Tensor:
    """This rank's part of `val` along the token axis `dim`."""
    n = val.size(dim)
    assert n % (cp_size * cp_mode) == 0, f"{n} tokens do not split into {cp_size * cp_mode} chunks"
    chunks = val.chunk(cp_size * cp_mode, dim=dim)
    if cp_mode == 1:
        return chunks[cp_rank].contiguous()
    return torch.cat([chunks[cp_rank], chunks[2 * cp_size - 1 - cp_rank]], dim=dim)


def get_batch_on_this_cp_rank_for_nsa(batch: Dict[str, Any], cp_size: Optional[int] = None, cp_rank: Optional[int] = None,
                                      cp_mode: Optional[int] = None, process_group=None,
                                      keys: Sequence[str] = ("input_ids", "labels", "position_ids")) -> Dict[str, Any]:
    """Replace batch[key] ([b, s] with the tokens on the last axis) by this rank's shard and record batch["cp_mode"].
    cp_mode None = choose it from batch["cu_seqlens"]; cp_size / cp_rank default to the process group's (or the default
    group's) size and rank; with one rank the batch is returned unchanged."""
    if cp_size is None or cp_rank is None:
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized():
            cp_size = dist.get_world_size(process_group) if cp_size is None else cp_size
            cp_rank = dist.get_rank(process_group) if cp_rank is None else cp_rank
        else:
            cp_size, cp_rank = cp_size or 1, cp_rank or 0
    if cp_size <= 1:
        return batch
    if cp_mode is None:
        cp_mode = get_cp_mode_from_cu_seqlens(batch["cu_seqlens"], cp_size)
    batch["cp_mode"] = cp_mode
    for key in keys:
        if key in batch and batch[key] is not None:
            batch[key] = split_for_cp_rank(batch[key], cp_size, cp_rank, cp_mode, dim=-1)
    return batch
