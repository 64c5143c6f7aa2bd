"""NSACore: the whole NSA path as ONE autograd function, with selective recompute and the context-parallel
variant (drop-in for flash_nsa/modules/megatron_level_nsa.py)."""
import math
from typing import Callable, Union

import numpy as np
import torch

from ..comm import Comm
from ..config import NSAConfig
from ..ops._common import poll_status, post_status
from ..ops.act import sigmoid_mul_bwd, sigmoid_mul_fwd, swiglu_bwd, swiglu_fwd
from ..ops.combine import combine_bwd, combine_fwd
from ..ops.compress_attn import cmp_attn_bwd, cmp_attn_fwd
from ..ops.compress_kv import construct_block_bwd, construct_block_fwd, mean_pooling_bwd, mean_pooling_fwd
from ..ops.select_attn import slc_attn_bwd, slc_attn_fwd
from ..ops.sliding_window_attention import swa_bwd, swa_fwd
from ..ops.topk import slc_topk_indices
from ..utils import NSAHelper


def wgrad_accum(input, grad_output, main_grad):
    """main_grad [out, in] fp32 += grad_output [rows, out]^T @ input [rows, in] (bf16 operands) in ONE launch of the tcgen05
    accumulate GEMM; returns False when the shapes are not its (out, in multiples of 128, aligned rows)."""
    from ..ops._common import S, call, ptr, status_word
    rows, n_in = input.shape
    n_out = grad_output.size(1)
    ok = (input.is_cuda and input.dtype in (torch.bfloat16, torch.float16) and grad_output.dtype == input.dtype and main_grad.dtype == torch.float32
          and tuple(main_grad.shape) == (n_out, n_in) and n_out % 128 == 0 and n_in % 128 == 0
          and input.stride(1) == 1 and grad_output.stride(1) == 1 and main_grad.stride(1) == 1
          and input.stride(0) % 8 == 0 and grad_output.stride(0) % 8 == 0 and main_grad.stride(0) % 4 == 0
          and input.data_ptr() % 16 == 0 and grad_output.data_ptr() % 16 == 0 and main_grad.data_ptr() % 16 == 0)
    if not ok:
        return False
    p = S["NsaWgradParams"]()
    p.dy, p.x, p.main_grad, p.status = ptr(grad_output), ptr(input), ptr(main_grad), ptr(status_word(input.device))
    p.rows, p.dy_stride, p.x_stride, p.grad_stride = rows, grad_output.stride(0), input.stride(0), main_grad.stride(0)
    p.n_out, p.n_in = n_out, n_in
    call("nsa_wgrad_accum", p, input)
    return True


def weight_grad(input, grad_output, weight):
    """dW = grad_output^T @ input, accumulated into `weight.main_grad` when the trainer provides one
    (flash_nsa/modules/megatron_level_nsa.py:20-44, which uses apex's wgrad_gemm_accum_fp32 or its Triton GEMM for this)."""
    input = input.reshape(-1, input.size(-1))
    grad_output = grad_output.reshape(-1, grad_output.size(-1))
    main_grad = getattr(weight, "main_grad", None)
    if main_grad is not None:
        if not wgrad_accum(input, grad_output, main_grad):
            # shapes outside the fused kernel (e.g. 64 output columns): a library GEMM, then the add
            main_grad.addmm_(grad_output.t().to(main_grad.dtype), input.to(main_grad.dtype))
        if hasattr(weight, "grad_added_to_main_grad"):
            weight.grad_added_to_main_grad = True
            return torch.empty(main_grad.shape, dtype=input.dtype, device=input.device, requires_grad=False)
        return None
    return torch.matmul(grad_output.t(), input)


def compress_kv_fwd(x, weight, version, helper=NSAHelper):
    """-> (block_x or None, hidden_state or None, compressed x)"""
    if version == "mean":
        return None, None, mean_pooling_fwd(x, helper=helper)
    block_x = construct_block_fwd(x, helper=helper)
    hidden = torch.matmul(torch.flatten(block_x, start_dim=-2, end_dim=-1), weight.t().to(x.dtype))
    if version == "linear":
        out = hidden
    elif version == "sigmoid-mul":
        out = sigmoid_mul_fwd(hidden)
    else:
        out = swiglu_fwd(hidden)
    return block_x, hidden, out


def compress_kv_bwd(x, weight, block_x, hidden_state, dout, dx, version, helper=NSAHelper, async_dw=False):
    """Adds the compression's input gradient into the fp32 `dx`; returns (dx, dW or a callable giving dW)."""
    if version == "mean":
        mean_pooling_bwd(x, dout, dx, helper=helper)
        return dx, None
    if version == "linear":
        dhidden = dout
    elif version == "sigmoid-mul":
        dhidden = sigmoid_mul_bwd(hidden_state, dout)
    else:
        dhidden = swiglu_bwd(hidden_state, dout)
    dblock = torch.matmul(dhidden, weight.to(dhidden.dtype)).view(*block_x.shape)
    dx = construct_block_bwd(x, dblock, dx, helper=helper)

    def func():
        return weight_grad(block_x.flatten(-2, -1), dhidden, weight)

    return (dx, func) if async_dw else (dx, func())


def _empty(t):
    return isinstance(t, torch.Tensor) and t.numel() == 0


class NSAFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, combine_weight, cmp_k_weight, cmp_v_weight, sm_scale=None):
        if sm_scale is None:
            sm_scale = q.size(-1) ** -0.5
        H = NSAHelper
        block_k, hidden_k, cmp_k = compress_kv_fwd(k, cmp_k_weight, H.cmp_k_method)
        block_v, hidden_v, cmp_v = compress_kv_fwd(v, cmp_v_weight, H.cmp_v_method)
        cmp_o, cmp_lse = cmp_attn_fwd(q, cmp_k, cmp_v, sm_scale=sm_scale)
        topk, _ = slc_topk_indices(q, cmp_k, cmp_lse, sm_scale=sm_scale, maybe_efficient_version=True, scale_slc_p=True)
        slc_o, slc_lse = slc_attn_fwd(q, k, v, topk, sm_scale=sm_scale)
        swa_o, swa_lse = swa_fwd(q, k, v, sm_scale=sm_scale)
        combine_o = combine_fwd(cmp_o, slc_o, swa_o, combine_weight)

        cmp_tensors = [block_k, hidden_k, cmp_k, block_v, hidden_v, cmp_v]
        if H.recompute_cmp_kv:
            H.clear_tensor_data(*cmp_tensors)
        if H.recompute_cmp_o:
            H.clear_tensor_data(cmp_o, cmp_lse)
        if H.recompute_slc_o:
            H.clear_tensor_data(slc_o, slc_lse)
        if H.recompute_swa_o:
            H.clear_tensor_data(swa_o, swa_lse)
        ctx.save_for_backward(q, k, v, combine_weight, cmp_k_weight, cmp_v_weight, *cmp_tensors, cmp_o, cmp_lse, slc_o,
                              slc_lse, swa_o, swa_lse, topk)
        ctx.sm_scale = sm_scale
        ctx.helper = H.get_bwd_helper()
        ctx.methods = (H.cmp_k_method, H.cmp_v_method)
        return combine_o

    @staticmethod
    def backward(ctx, do):
        (q, k, v, combine_weight, cmp_k_weight, cmp_v_weight, block_k, hidden_k, cmp_k, block_v, hidden_v, cmp_v,
         cmp_o, cmp_lse, slc_o, slc_lse, swa_o, swa_lse, topk) = ctx.saved_tensors
        sm_scale, helper = ctx.sm_scale, ctx.helper
        km, vm = ctx.methods
        if _empty(cmp_k):
            block_k, hidden_k, cmp_k = compress_kv_fwd(k, cmp_k_weight, km, helper)
            block_v, hidden_v, cmp_v = compress_kv_fwd(v, cmp_v_weight, vm, helper)
        if _empty(cmp_o):
            cmp_o, cmp_lse = cmp_attn_fwd(q, cmp_k, cmp_v, sm_scale=sm_scale, helper=helper)
        if _empty(slc_o):
            slc_o, slc_lse = slc_attn_fwd(q, k, v, topk, sm_scale=sm_scale, helper=helper)
        if _empty(swa_o):
            swa_o, swa_lse = swa_fwd(q, k, v, sm_scale=sm_scale, helper=helper)

        # the combine backward also yields each branch's delta = sum_d o * do, so the branches skip their delta pass
        deltas = [torch.empty_like(cmp_lse), torch.empty_like(slc_lse), torch.empty_like(swa_lse)]
        dcmp_o, dslc_o, dswa_o, dcombine_weight = combine_bwd(cmp_o, slc_o, swa_o, combine_weight, do,
                                                               deltas=[deltas[0].t(), deltas[1], deltas[2]])
        dq = torch.empty_like(q)
        dk = torch.zeros(k.shape, device=k.device, dtype=torch.float32)
        dv = torch.zeros(v.shape, device=v.device, dtype=torch.float32)
        # the window branch writes dq, the selected branch adds its part with global bf16 reductions, the compressed one
        # adds last in its row-per-thread epilogue; every branch adds into the fp32 dk/dv
        _swa_bwd_into(q, k, v, swa_o, swa_lse, dswa_o, dq, dk, dv, sm_scale, helper, delta=deltas[2], accumulate_dq=False)
        slc_attn_bwd(q, k, v, topk, slc_o, slc_lse, dslc_o, dq, dk, dv, sm_scale=sm_scale, helper=helper, delta=deltas[1],
                     accumulate_dq=True)
        _, dcmp_k, dcmp_v = cmp_attn_bwd(q, cmp_k, cmp_v, cmp_o, cmp_lse, dcmp_o, dq, sm_scale=sm_scale, helper=helper,
                                         delta=deltas[0])
        _, dwk = compress_kv_bwd(k, cmp_k_weight, block_k, hidden_k, dcmp_k, dk, version=km, helper=helper)
        _, dwv = compress_kv_bwd(v, cmp_v_weight, block_v, hidden_v, dcmp_v, dv, version=vm, helper=helper)
        return dq, dk, dv, dcombine_weight, dwk, dwv, None


def _swa_bwd_into(q, k, v, o, lse, dout, dq, dk, dv, sm_scale, helper, delta=None, accumulate_dq=False):
    """Sliding-window backward that writes (or adds into) dq (bf16) and adds into dk/dv (fp32)."""
    from ..ops._common import attn_params, call
    if not (dout.stride(-1) == 1 and dout.stride(1) == dout.size(-1)):
        dout = dout.contiguous()
    have_delta = delta is not None
    if not have_delta:
        delta = torch.empty_like(lse)
    p = attn_params(q, k, v, helper, sm_scale, o=o, lse=lse, dout=dout, delta=delta, dq=dq, dk=dk, dv=dv)
    p.accumulate_dq = int(accumulate_dq)
    if have_delta:
        p.phases = 6
    if q.size(0) > 0:
        call("nsa_swa_bwd", p, q)


class CPNSAFunction(torch.autograd.Function):
    """Context-parallel NSA: q/k/v are this rank's token shard; K and V of `kv_head_stride` kv heads at a time
    are all-gathered over the process group, all branches run with local queries against the gathered
    sequence, and dK/dV go back through a reduce-scatter in fp32."""

    @staticmethod
    def forward(ctx, chunk_q, chunk_k, chunk_v, combine_weight, cmp_k_weight, cmp_v_weight, sm_scale=None):
        H = NSAHelper
        t, qh, d = chunk_q.shape
        kh, vd = chunk_k.size(1), chunk_v.size(-1)
        G = qh // kh
        if sm_scale is None:
            sm_scale = d ** -0.5
        stride = min(H.kv_head_stride, kh)
        assert kh % stride == 0
        W = H.world_size
        comm = Comm(H.process_group, t, W, stride, d, vd, chunk_k.dtype, chunk_k.device, H.cp_mode, with_grads=False)
        saved = []
        combine_o = torch.empty(t, qh, vd, dtype=chunk_q.dtype, device=chunk_q.device)
        comm.all_gather(chunk_k[:, 0:stride], Comm.KEY)
        comm.all_gather(chunk_v[:, 0:stride], Comm.VALUE)
        for h0 in range(0, kh, stride):
            q = chunk_q[:, h0 * G:(h0 + stride) * G]
            w_i = combine_weight[:, h0 * G:(h0 + stride) * G]
            k = comm.wait(Comm.KEY)
            v = comm.wait(Comm.VALUE)
            if h0 + stride < kh:
                # the next group's gather goes out NOW, before this group's kernels are enqueued: the collective starts
                # when the work queued so far is done, so it runs under the kernels below (it fills the other buffer pair)
                comm.all_gather(chunk_k[:, h0 + stride:h0 + 2 * stride], Comm.KEY)
                comm.all_gather(chunk_v[:, h0 + stride:h0 + 2 * stride], Comm.VALUE)
            block_k, hidden_k, cmp_k = compress_kv_fwd(k, cmp_k_weight, H.cmp_k_method)
            block_v, hidden_v, cmp_v = compress_kv_fwd(v, cmp_v_weight, H.cmp_v_method)
            cmp_o, cmp_lse = cmp_attn_fwd(q, cmp_k, cmp_v, sm_scale=sm_scale)
            topk, _ = slc_topk_indices(q, cmp_k, cmp_lse, sm_scale=sm_scale, maybe_efficient_version=True, scale_slc_p=True)
            slc_o, slc_lse = slc_attn_fwd(q, k, v, topk, sm_scale=sm_scale)
            swa_o, swa_lse = swa_fwd(q, k, v, sm_scale=sm_scale)
            comm.release()  # the gathered K/V of this head group are no longer read by later launches
            combine_fwd(cmp_o, slc_o, swa_o, w_i, out=combine_o[:, h0 * G:(h0 + stride) * G])
            # the compressed tensors cover the GLOBAL sequence: they are never kept, backward rebuilds them
            if H.recompute_cmp_o:
                cmp_o, cmp_lse = None, None
            if H.recompute_slc_o:
                slc_o, slc_lse = None, None
            if H.recompute_swa_o:
                swa_o, swa_lse = None, None
            del block_k, hidden_k, cmp_k, block_v, hidden_v, cmp_v
            saved.append([cmp_o, cmp_lse, slc_o, slc_lse, swa_o, swa_lse, topk])
        flat, layout = [], []
        for group in saved:
            layout.append([x is not None for x in group])
            flat += [x for x in group if x is not None]
        ctx.save_for_backward(chunk_q, chunk_k, chunk_v, combine_weight, cmp_k_weight, cmp_v_weight, *flat)
        ctx.layout = layout
        ctx.sm_scale = sm_scale
        ctx.helper = H.get_bwd_helper()
        ctx.stride = stride
        ctx.methods = (H.cmp_k_method, H.cmp_v_method)
        return combine_o

    @staticmethod
    def backward(ctx, do, *args):
        H = NSAHelper
        tensors = ctx.saved_tensors
        chunk_q, chunk_k, chunk_v, combine_weight, cmp_k_weight, cmp_v_weight = tensors[:6]
        flat = list(tensors[6:])
        helper, sm_scale, stride = ctx.helper, ctx.sm_scale, ctx.stride
        km, vm = ctx.methods
        t, qh, d = chunk_q.shape
        kh, vd = chunk_k.size(1), chunk_v.size(-1)
        G = qh // kh
        W = H.world_size
        comm = Comm(H.process_group, t, W, stride, d, vd, chunk_k.dtype, chunk_k.device, helper.cp_mode, with_grads=True)
        chunk_dq = torch.empty_like(chunk_q)
        chunk_dk = torch.empty_like(chunk_k)
        chunk_dv = torch.empty_like(chunk_v)
        dcombine_weight = torch.empty_like(combine_weight)
        dwk = torch.zeros_like(cmp_k_weight) if cmp_k_weight is not None else None
        dwv = torch.zeros_like(cmp_v_weight) if cmp_v_weight is not None else None
        if not (do.stride(-1) == 1 and do.stride(1) == do.size(-1)):
            do = do.contiguous()
        comm.all_gather(chunk_k[:, 0:stride], Comm.KEY)
        comm.all_gather(chunk_v[:, 0:stride], Comm.VALUE)
        for gi, h0 in enumerate(range(0, kh, stride)):
            group = [flat.pop(0) if present else None for present in ctx.layout[gi]]
            cmp_o, cmp_lse, slc_o, slc_lse, swa_o, swa_lse, topk = group
            q = chunk_q[:, h0 * G:(h0 + stride) * G]
            do_i = do[:, h0 * G:(h0 + stride) * G]
            w_i = combine_weight[:, h0 * G:(h0 + stride) * G]
            dq = chunk_dq[:, h0 * G:(h0 + stride) * G]
            k = comm.wait(Comm.KEY)
            v = comm.wait(Comm.VALUE)
            if h0 + stride < kh:   # next group's K/V: issued before this group's kernels, runs under them
                comm.all_gather(chunk_k[:, h0 + stride:h0 + 2 * stride], Comm.KEY)
                comm.all_gather(chunk_v[:, h0 + stride:h0 + 2 * stride], Comm.VALUE)
            block_k, hidden_k, cmp_k = compress_kv_fwd(k, cmp_k_weight, km, helper)
            block_v, hidden_v, cmp_v = compress_kv_fwd(v, cmp_v_weight, vm, helper)
            if cmp_o is None:
                cmp_o, cmp_lse = cmp_attn_fwd(q, cmp_k, cmp_v, sm_scale=sm_scale, helper=helper)
            if slc_o is None:
                slc_o, slc_lse = slc_attn_fwd(q, k, v, topk, sm_scale=sm_scale, helper=helper)
            if swa_o is None:
                swa_o, swa_lse = swa_fwd(q, k, v, sm_scale=sm_scale, helper=helper)
            deltas = [torch.empty_like(cmp_lse), torch.empty_like(slc_lse), torch.empty_like(swa_lse)]
            dcmp_o, dslc_o, dswa_o, _ = combine_bwd(cmp_o, slc_o, swa_o, w_i, do_i,
                                                     dw=dcombine_weight[:, h0 * G:(h0 + stride) * G],
                                                     deltas=[deltas[0].t(), deltas[1], deltas[2]])
            dk, dv = comm.grad_buffers()  # zero-filled fp32 [t*W, stride, d]
            _swa_bwd_into(q, k, v, swa_o, swa_lse, dswa_o, dq, dk, dv, sm_scale, helper, delta=deltas[2], accumulate_dq=False)
            slc_attn_bwd(q, k, v, topk, slc_o, slc_lse, dslc_o, dq, dk, dv, sm_scale=sm_scale, helper=helper, delta=deltas[1],
                         accumulate_dq=True)
            _, dcmp_k, dcmp_v = cmp_attn_bwd(q, cmp_k, cmp_v, cmp_o, cmp_lse, dcmp_o, dq, sm_scale=sm_scale, helper=helper,
                                             delta=deltas[0])
            _, fk = compress_kv_bwd(k, cmp_k_weight, block_k, hidden_k, dcmp_k, dk, version=km, helper=helper, async_dw=True)
            dk_local = comm.reduce_scatter(Comm.GRAD_KEY)
            _, fv = compress_kv_bwd(v, cmp_v_weight, block_v, hidden_v, dcmp_v, dv, version=vm, helper=helper, async_dw=True)
            dv_local = comm.reduce_scatter(Comm.GRAD_VALUE)
            comm.release()
            if isinstance(fk, Callable):
                g = fk()
                if dwk is not None and g is not None:
                    dwk += g
            if isinstance(fv, Callable):
                g = fv()
                if dwv is not None and g is not None:
                    dwv += g
            comm.wait(Comm.GRAD_KEY)
            comm.wait(Comm.GRAD_VALUE)
            chunk_dk[:, h0:h0 + stride].copy_(dk_local)
            chunk_dv[:, h0:h0 + stride].copy_(dv_local)
        return chunk_dq, chunk_dk, chunk_dv, dcombine_weight, dwk, dwv, None


def flash_nsa_varlen_func(q, k, v, combine_weight, cmp_k_weight, cmp_v_weight, sm_scale=None):
    """Requires NSAHelper.init_cu_seqlens(cu_seqlens) beforehand."""
    return NSAFunction.apply(q, k, v, combine_weight, cmp_k_weight, cmp_v_weight, sm_scale)


def cp_flash_nsa_varlen_func(q, k, v, combine_weight, cmp_k_weight, cmp_v_weight, sm_scale=None):
    return CPNSAFunction.apply(q, k, v, combine_weight, cmp_k_weight, cmp_v_weight, sm_scale)


class NSACore(torch.nn.Module):
    def __init__(self, config: NSAConfig, process_group=None, pp_size=1):
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
        self.cmp_k_method = getattr(config, "cmp_k_method", "mean")
        self.cmp_v_method = getattr(config, "cmp_v_method", "mean")
        self.cp_mode = getattr(config, "cp_mode", 2)
        self.kv_head_stride = getattr(config, "kv_head_stride", 1)
        self.use_overlap_swa = getattr(config, "use_overlap_swa", False)
        self.sm_scale = self.qk_head_dim ** -0.5
        assert math.log2(self.stride).is_integer(), "stride must be power of 2, like 8, 16, 32, 64, etc."
        assert self.kernel_size % self.stride == 0
        assert self.block_size % self.stride == 0
        self.process_group = process_group
        NSAHelper.set_hyperparameters(kernel_size=self.kernel_size, stride=self.stride, block_size=self.block_size,
                                      window_size=self.window_size, top_n=self.top_n,
                                      num_init_blocks=self.num_init_blocks, num_local_blocks=self.num_local_blocks)
        NSAHelper.set_recompute(recompute_cmp_kv=getattr(config, "recompute_cmp_kv", False),
                                recompute_cmp_o=getattr(config, "recompute_cmp_o", False),
                                recompute_slc_o=getattr(config, "recompute_slc_o", False),
                                recompute_swa_o=getattr(config, "recompute_swa_o", False))
        NSAHelper.set_context_parallel(process_group=process_group, kv_head_stride=self.kv_head_stride,
                                       use_overlap_swa=self.use_overlap_swa)
        NSAHelper.set_cmp_kv_method(cmp_k_method=self.cmp_k_method, cmp_v_method=self.cmp_v_method)
        NSAHelper.set_pipeline_parallel_world_size(pp_size=pp_size)
        self.cmp_k_weight = None
        self.cmp_v_weight = None
        dev = torch.cuda.current_device() if torch.cuda.is_available() else "cpu"
        if self.cmp_k_method != "mean":
            out = self.qk_head_dim if self.cmp_k_method == "linear" else self.qk_head_dim * 2
            self.cmp_k_weight = torch.nn.Parameter(torch.randn(out, self.kernel_size * self.qk_head_dim, device=dev))
            setattr(self.cmp_k_weight, "sequence_parallel", getattr(config, "sequence_parallel", True))
        if self.cmp_v_method != "mean":
            out = self.v_head_dim if self.cmp_v_method == "linear" else self.v_head_dim * 2
            self.cmp_v_weight = torch.nn.Parameter(torch.randn(out, self.kernel_size * self.v_head_dim, device=dev))
            setattr(self.cmp_v_weight, "sequence_parallel", getattr(config, "sequence_parallel", True))

    def forward(self, q, k, v, combine_weight, cu_seqlens, cu_seqlens_np: np.ndarray = None,
                cp_mode: Union[int, None] = None):
        """q [t,qh,d], k [t,kh,d], v [t,kh,vd], combine_weight [t,qh,3]; with a process group of more than one
        rank the tensors are this rank's token shard and cu_seqlens describes the GLOBAL packed batch."""
        assert cu_seqlens is not None
        cp_mode = cp_mode if cp_mode is not None else self.cp_mode
        NSAHelper.init_cu_seqlens(cu_seqlens, x_cu_seqlens_np=cu_seqlens_np, cp_mode=cp_mode)
        # a pipeline time-out reported by the kernels of an EARLIER call raises here (no synchronisation: the status word is
        # copied to pinned host memory behind each forward and looked at when the next one starts)
        poll_status(q.device)
        if NSAHelper.world_size <= 1:
            o = flash_nsa_varlen_func(q, k, v, combine_weight, self.cmp_k_weight, self.cmp_v_weight, self.sm_scale)
        else:
            o = cp_flash_nsa_varlen_func(q, k, v, combine_weight, self.cmp_k_weight, self.cmp_v_weight, self.sm_scale)
        post_status(q.device)
        return o
