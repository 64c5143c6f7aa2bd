"""HF-style demo attention layer: q / k / v / gate projections, rotary embedding, HFNSACore, output projection.

Drop-in for the reference's demo layer (flash_nsa/layers/hf_level_nsa.py:8-59): same constructor, same forward arguments
and the same parameter names (`q_proj`, `k_proj`, `v_proj`, `combine_proj`, `o_proj`, `nsa.*`), so a state dict of one
loads into the other.  The forward is organised for one pass over the activations: the four input projections run as a
single GEMM over the row-concatenated weights (hidden_states is read once instead of four times), everything after it
works on the packed token axis [b*s, heads, dim] that the NSA core wants, and the equal-length `cu_seqlens` of an
un-packed batch is built once per (batch, length, device) and reused.
"""
from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import NSAConfig
from ..modules.hf_level_nsa import HFNSACore
from ..ops.rope import fused_apply_rope


class HFNSA(nn.Module):
    def __init__(self, config: NSAConfig) -> None:
        super().__init__()
        hidden = config.hidden_size
        self.hidden_size = hidden
        self.num_heads, self.num_kv_heads = config.num_heads, config.num_kv_heads
        self.qk_head_dim, self.v_head_dim = config.qk_head_dim, config.v_head_dim
        # (name, heads, width per head) of the four input projections, in the order their outputs are concatenated
        self._inputs = (("q_proj", self.num_heads, self.qk_head_dim), ("k_proj", self.num_kv_heads, self.qk_head_dim),
                        ("v_proj", self.num_kv_heads, self.v_head_dim), ("combine_proj", self.num_heads, 3))
        for name, heads, width in self._inputs:
            setattr(self, name, nn.Linear(hidden, heads * width, bias=False))
        self.o_proj = nn.Linear(self.num_heads * self.v_head_dim, hidden, bias=False)
        self.nsa = HFNSACore(config)
        self._equal_len_cu: Dict[Tuple[int, int, torch.device], torch.Tensor] = {}

    def _project(self, x: torch.Tensor):
        """x [tokens, hidden] -> q, k, v, gate logits as [tokens, heads, width] views of ONE GEMM's output."""
        weight = torch.cat([getattr(self, name).weight for name, _, _ in self._inputs], dim=0)
        fused = F.linear(x, weight)
        outs, col = [], 0
        for _, heads, width in self._inputs:
            outs.append(fused[:, col:col + heads * width].unflatten(-1, (heads, width)))
            col += heads * width
        return outs

    def _cu_seqlens(self, batch: int, length: int, device: torch.device) -> torch.Tensor:
        key = (batch, length, device)
        if key not in self._equal_len_cu:
            self._equal_len_cu[key] = torch.arange(0, (batch + 1) * length, length, dtype=torch.int32, device=device)
        return self._equal_len_cu[key]

    def forward(self, hidden_states: torch.Tensor, position_embeddings: Tuple[torch.Tensor, torch.Tensor],
                cu_seqlens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """hidden_states [b, s, hidden]; position_embeddings = (cos, sin), each [b or 1, s, qk_head_dim]; cu_seqlens
        describes the packed token axis b*s (default: b sequences of length s)."""
        batch, length, _ = hidden_states.shape
        q, k, v, gate = self._project(hidden_states.reshape(batch * length, self.hidden_size))
        cos, sin = position_embeddings
        # the rope op takes [b, s, heads, dim]; q and k are strided column slices of the fused output, its results are
        # fresh contiguous tensors, so going back to the packed token axis is a view
        q, k = fused_apply_rope(q.unflatten(0, (batch, length)), k.unflatten(0, (batch, length)), cos, sin, inplace=False)
        if cu_seqlens is None:
            cu_seqlens = self._cu_seqlens(batch, length, hidden_states.device)
        attn = self.nsa(q.flatten(0, 1), k.flatten(0, 1), v.contiguous(), gate.contiguous(), cu_seqlens)
        return self.o_proj(attn.reshape(batch, length, self.num_heads * self.v_head_dim))
