from .compress_kv import (construct_block, construct_block_bwd, construct_block_fwd, mean_pooling, mean_pooling_bwd,
                          mean_pooling_fwd)
from .act import sigmoid_mul_bwd, sigmoid_mul_fwd, sigmoid_mul_impl, swiglu_bwd, swiglu_fwd, swiglu_impl
from .combine import combine_bwd, combine_fwd, fused_sigmoid_combine
from .compress_attn import cmp_attn_bwd, cmp_attn_fwd, compress_attn
from .topk import get_bind_from_find, slc_topk_indices
from .select_attn import select_attn, slc_attn_bwd, slc_attn_fwd
from .sliding_window_attention import (swa_bwd, swa_fwd, swa_varlen_func, two_stage_swa_bwd, two_stage_swa_fwd)
from .reorder import reorder
from .rope import fused_apply_rope
