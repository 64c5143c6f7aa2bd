"""flash_nsa for B200: Native Sparse Attention on hand-written sm_100a CUDA kernels.

Same import surface as the reference package (flash_nsa/__init__.py:1-23)."""
from .utils import NSAHelper
from .config import NSAConfig

from .modules.hf_level_nsa import HFNSACore
from .ops.select_attn import select_attn
from .ops.topk import slc_topk_indices
from .ops.compress_attn import compress_attn
from .ops.compress_kv import mean_pooling, construct_block
from .ops.sliding_window_attention import swa_varlen_func
from .ops.combine import fused_sigmoid_combine

from .modules.megatron_level_nsa import NSACore, flash_nsa_varlen_func, cp_flash_nsa_varlen_func

from .layers.megatron_level_nsa import NSA
from .layers.hf_level_nsa import HFNSA

from .inference import nsa_prefill, nsa_decode
from .ops._common import check_status
