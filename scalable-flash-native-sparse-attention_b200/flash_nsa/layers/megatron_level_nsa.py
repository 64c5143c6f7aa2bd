"""Demo attention layer around NSACore with one fused q/k/v/gate projection, sequence-first activations
(flash_nsa/layers/megatron_level_nsa.py:9-114).  With Megatron-Core importable the projections are its tensor-parallel
linears and the context-parallel group comes from its parallel state; otherwise plain nn.Linear and a single GPU.
The fused projection is split into q, k, v, gate (and alignment padding); the k slice has num_kv_heads * qk_head_dim
columns."""
import torch
import torch.nn as nn

from ..config import NSAConfig
from ..modules.megatron_level_nsa import NSACore
from ..ops.rope import fused_apply_rope


def _cdiv(a, b):
    return -(-a // b)


class NSA(nn.Module):
    def __init__(self, config: NSAConfig):
        super().__init__()
        self.config = config
        self.hidden_size = config.hidden_size
        self.num_heads = config.num_heads
        self.num_kv_heads = config.num_kv_heads
        self.qk_head_dim = config.qk_head_dim
        self.v_head_dim = config.v_head_dim
        try:
            from megatron.core import parallel_state
            self.tp_size = parallel_state.get_tensor_model_parallel_world_size()
            cp_process_group = parallel_state.get_context_parallel_group()
            pp_size = parallel_state.get_pipeline_model_parallel_world_size()
            assert self.num_heads % self.tp_size == 0 and self.num_kv_heads % self.tp_size == 0
        except Exception:
            self.tp_size, cp_process_group, pp_size = 1, None, 1
        self.nsa = NSACore(config, process_group=cp_process_group, pp_size=pp_size)
        self.num_heads_per_rank = self.num_heads // self.tp_size
        self.num_kv_heads_per_rank = self.num_kv_heads // self.tp_size
        output_dim = self.num_heads * (self.qk_head_dim + 3) + self.num_kv_heads * (self.qk_head_dim + self.v_head_dim)
        per_rank = _cdiv(_cdiv(output_dim, self.tp_size), 8) * 8          # 16-byte aligned rows per rank
        output_dim = per_rank * self.tp_size
        split = [self.num_heads_per_rank * self.qk_head_dim, self.num_kv_heads_per_rank * self.qk_head_dim,
                 self.num_kv_heads_per_rank * self.v_head_dim, self.num_heads_per_rank * 3]
        self.split_size = split + [per_rank - sum(split)]
        try:
            from megatron.core.tensor_parallel import ColumnParallelLinear, RowParallelLinear
            self.qkvw_proj = ColumnParallelLinear(self.hidden_size, output_dim, config=config, init_method=config.init_method,
                                                  bias=False)
            self.o_proj = RowParallelLinear(self.v_head_dim * self.num_heads, self.hidden_size, config=config,
                                            init_method=config.init_method, bias=False)
        except Exception:
            self.qkvw_proj = nn.Linear(self.hidden_size, output_dim, bias=False)
            self.o_proj = nn.Linear(self.num_heads * self.v_head_dim, self.hidden_size, bias=False)

    def forward(self, hidden_states, rotary_pos_emb, extra_kwargs=None):
        """hidden_states [s, b, hidden] (sequence first); rotary_pos_emb = (cos, sin), batch- or sequence-first;
        extra_kwargs: cu_seqlens (required), cu_seqlens_np, cp_mode."""
        extra_kwargs = extra_kwargs or {}
        s, b, _ = hidden_states.shape
        qkvw = self.qkvw_proj(hidden_states)
        if not isinstance(qkvw, torch.Tensor):
            qkvw = qkvw[0]
        q, k, v, w, _ = qkvw.split(self.split_size, -1)
        q = q.view(*q.shape[:2], self.num_heads_per_rank, self.qk_head_dim)
        k = k.view(*k.shape[:2], self.num_kv_heads_per_rank, self.qk_head_dim)
        v = v.view(*v.shape[:2], self.num_kv_heads_per_rank, self.v_head_dim)
        combine_weight = w.view(*w.shape[:2], self.num_heads_per_rank, 3)
        cos, sin = rotary_pos_emb
        if cos.dim() == 4:
            cos, sin = cos.squeeze(-2), sin.squeeze(-2)
        if cos.size(0) != b and cos.size(0) != 1:   # sequence first -> batch first
            cos, sin = cos.transpose(0, 1), sin.transpose(0, 1)
        # the rotated q and k are new contiguous batch-first tensors, so flattening them is a view
        q, k = fused_apply_rope(q.transpose(0, 1), k.transpose(0, 1), cos, sin, inplace=False)
        q, k = q.flatten(0, 1), k.flatten(0, 1)
        v = v.transpose(0, 1).flatten(0, 1)
        combine_weight = combine_weight.transpose(0, 1).flatten(0, 1)
        cu_seqlens = extra_kwargs.get("cu_seqlens", None)
        assert cu_seqlens is not None
        o = self.nsa(q, k, v, combine_weight, cu_seqlens=cu_seqlens, cu_seqlens_np=extra_kwargs.get("cu_seqlens_np", None),
                     cp_mode=extra_kwargs.get("cp_mode", None))
        o = o.view(b, -1, self.num_heads_per_rank * self.v_head_dim).transpose(0, 1).contiguous()
        out = self.o_proj(o)
        return out[0] if not isinstance(out, torch.Tensor) else out
