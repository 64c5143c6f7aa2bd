"""HFNSACore: the seven NSA steps as independent autograd ops (drop-in for
flash_nsa/modules/hf_level_nsa.py:62-158)."""
import math

import torch

from ..config import NSAConfig
from ..ops.act import sigmoid_mul_impl, swiglu_impl
from ..ops.combine import fused_sigmoid_combine
from ..ops.compress_attn import compress_attn
from ..ops.compress_kv import construct_block, mean_pooling
from ..ops.select_attn import select_attn
from ..ops.sliding_window_attention import swa_varlen_func
from ..ops.topk import slc_topk_indices
from ..utils import NSAHelper


class CompressKV(torch.nn.Module):
    """mean: window mean.  linear / swiglu / sigmoid-mul: windows flattened to [.., kernel_size*d], one
    bias-free Linear shared by all heads (`fc`), then the gate activation."""

    def __init__(self, config: NSAConfig, head_dim=128, version=None):
        super().__init__()
        assert version in ["mean", "sigmoid-mul", "swiglu", "linear"]
        self.head_dim = head_dim
        self.kernel_size = getattr(config, "kernel_size", 32)
        self.stride = getattr(config, "stride", 32)
        self.version = version
        if version != "mean":
            out_features = head_dim if version == "linear" else 2 * head_dim
            self.fc = torch.nn.Linear(self.kernel_size * head_dim, out_features, bias=False)

    def forward(self, x):
        if self.version == "mean":
            return mean_pooling(x)
        hidden = self.fc(torch.flatten(construct_block(x), start_dim=-2, end_dim=-1))
        if self.version == "linear":
            return hidden
        if self.version == "sigmoid-mul":
            return sigmoid_mul_impl(hidden)
        return swiglu_impl(hidden)


class HFNSACore(torch.nn.Module):
    def __init__(self, config: NSAConfig):
        super().__init__()
        self.config = config
        self.qk_head_dim = config.qk_head_dim if config.qk_head_dim is not None else config.head_dim
        self.v_head_dim = config.v_head_dim if config.v_head_dim is not None else config.head_dim
        self.kernel_size = getattr(config, "kernel_size", 32)
        self.stride = getattr(config, "stride", 16)
        self.block_size = getattr(config, "block_size", 64)
        self.top_n = getattr(config, "top_n", 16)
        self.num_local_blocks = getattr(config, "num_local_blocks", 1)
        self.num_init_blocks = getattr(config, "num_init_blocks", 2)
        self.window_size = getattr(config, "window_size", 512)
        self.sm_scale = self.qk_head_dim ** -0.5
        assert math.log2(self.stride).is_integer(), "stride must be a power of 2, like 8, 16 etc."
        assert self.kernel_size % self.stride == 0
        assert self.block_size % self.stride == 0
        NSAHelper.set_hyperparameters(kernel_size=self.kernel_size, stride=self.stride, block_size=self.block_size,
                                      window_size=self.window_size, top_n=self.top_n,
                                      num_init_blocks=self.num_init_blocks, num_local_blocks=self.num_local_blocks)
        self.compress_k = CompressKV(config, head_dim=self.qk_head_dim, version=config.cmp_k_method)
        self.compress_v = CompressKV(config, head_dim=self.v_head_dim, version=config.cmp_v_method)

    def forward(self, q, k, v, combine_weight, cu_seqlens, bench=False, print_result=True):
        """q [t,qh,d], k [t,kh,d], v [t,kh,vd], combine_weight [t,qh,3], cu_seqlens int32 [batch+1] -> o [t,qh,vd].
        With bench=True also returns a dict of per-step CUDA-event times in ms."""
        assert cu_seqlens is not None
        NSAHelper.init_cu_seqlens(cu_seqlens)
        steps = {
            "cmp_k": lambda: self.compress_k(k),
            "cmp_v": lambda: self.compress_v(v),
        }
        cmp_k = steps["cmp_k"]()
        cmp_v = steps["cmp_v"]()
        cmp_o, cmp_lse = compress_attn(q, cmp_k, cmp_v, sm_scale=self.sm_scale)
        topk, _ = slc_topk_indices(q, cmp_k, cmp_lse, sm_scale=self.sm_scale, maybe_efficient_version=True, scale_slc_p=True)
        slc_o = select_attn(q, k, v, topk, sm_scale=self.sm_scale)
        swa_o = swa_varlen_func(q, k, v, self.sm_scale)
        combine_o = fused_sigmoid_combine(cmp_o, slc_o, swa_o, combine_weight)
        if not bench:
            return combine_o
        steps.update({
            "cmp_o": lambda: compress_attn(q, cmp_k, cmp_v, sm_scale=self.sm_scale),
            "top_k": lambda: slc_topk_indices(q, cmp_k, cmp_lse, sm_scale=self.sm_scale, maybe_efficient_version=True),
            "slc_o": lambda: select_attn(q, k, v, topk, sm_scale=self.sm_scale),
            "swa_o": lambda: swa_varlen_func(q, k, v, self.sm_scale),
            "combine": lambda: fused_sigmoid_combine(cmp_o, slc_o, swa_o, combine_weight),
        })
        times = {}
        with torch.no_grad():
            for name, fn in steps.items():
                for _ in range(3):
                    fn()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(10):
                    fn()
                e1.record()
                torch.cuda.synchronize()
                times[name] = e0.elapsed_time(e1) / 10
        if print_result:
            print("forward time (ms):")
            for name, ms in times.items():
                print(f"  {name:8s} {ms:.3f}")
        return combine_o, times
