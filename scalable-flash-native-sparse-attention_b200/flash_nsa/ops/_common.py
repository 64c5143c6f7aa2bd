"""Helpers shared by the op wrappers: parameter-struct filling and argument checks."""
import torch

from .. import _lib
from ..utils import NSAHelper

S = _lib.structs


def stream_ptr(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


_empty_stub = {}


def ptr(t):
    """Device address of a tensor for the C ABI; None -> NULL.  An EMPTY tensor has no storage (data_ptr() is 0), but the
    entry points treat NULL as a missing argument, so it gets the address of a small per-device stub instead (nothing is read
    or written through it: every entry point returns before launching when there are no rows)."""
    if t is None:
        return 0
    if t.numel() == 0 and t.is_cuda:
        key = t.device.index
        if key not in _empty_stub:
            _empty_stub[key] = torch.zeros(256, dtype=torch.uint8, device=t.device)
        return _empty_stub[key].data_ptr()
    return t.data_ptr()


def hyper(window=None):
    h = S["NsaHyper"]()
    h.kernel_size, h.stride, h.block_size = NSAHelper.kernel_size, NSAHelper.stride, NSAHelper.block_size
    h.window = NSAHelper.window_size if window is None else window
    h.top_n, h.num_init, h.num_local = NSAHelper.top_n, NSAHelper.num_init_blocks, NSAHelper.num_local_blocks
    return h


def is_cp(helper) -> bool:
    return (getattr(helper, "cp_cu_seqlens", None) is not None and NSAHelper.is_context_parallel_enable
            and getattr(helper, "world_size", 1) > 1)


def seq_meta(helper, cp=None):
    """NsaSeqMeta for the helper's current tables; pieces are the rank's shard pieces under context
    parallelism and whole sequences otherwise."""
    assert helper.x_cu_seqlens is not None, "call NSAHelper.init_cu_seqlens(cu_seqlens) first"
    m = S["NsaSeqMeta"]()
    cp = is_cp(helper) if cp is None else cp
    n_seq = helper.x_cu_seqlens.numel() - 1
    if cp:
        m.piece_cu, m.piece_seq, m.piece_off = ptr(helper.cp_cu_seqlens), ptr(helper.cp_batch_idx), ptr(helper.cp_offset)
        m.n_pieces, m.max_piece_len = helper.cp_batch_idx.numel(), helper.cp_maxlen
    else:
        m.piece_cu, m.piece_seq, m.piece_off = ptr(helper.x_cu_seqlens), 0, 0
        m.n_pieces, m.max_piece_len = n_seq, helper.x_maxlen
    m.x_cu, m.y_cu = ptr(helper.x_cu_seqlens), ptr(helper.y_cu_seqlens)
    m.n_seq, m.x_maxlen, m.y_maxlen = n_seq, helper.x_maxlen, helper.y_maxlen
    return m


def local_rows(helper, cp=None) -> int:
    cp = is_cp(helper) if cp is None else cp
    return helper.cp_len if cp else helper.total_len


HALF_TYPES = (torch.bfloat16, torch.float16)   # one build of the kernel library each


def check_bf16_3d(name, t, last_contig=True):
    assert t.is_cuda, f"{name} must be a CUDA tensor"
    assert t.dtype in HALF_TYPES, f"{name} must be bfloat16 or float16 (got {t.dtype})"
    assert t.dim() == 3, f"{name} must be [t, h, d]"
    assert t.stride(-1) == 1 and t.stride(1) == t.size(-1), f"{name}: heads and head_dim must be contiguous"


_status = {}
_mirror = {}   # device index -> [pinned host copy of the word, event of the last copy or None]

STATUS_BITS = {1: "dense forward", 2: "selected-branch dK/dV", 4: "dense dQ", 8: "misaligned shared memory", 16: "scores + top-n",
               32: "decode: compressed rows exceed y_cap", 64: "dense dK/dV (128-row tiles)", 128: "selected forward",
               256: "selected dQ", 512: "wait self-test", 1024: "weight-gradient GEMM", 2048: "decode (tile ring)"}


def status_word(device):
    """One int32 per device that kernels OR error bits into (bounded waits that gave up)."""
    key = torch.device(device).index
    if key is None:
        key = torch.cuda.current_device()
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
    return _status[key]


def _raise_status(v):
    names = ", ".join(n for b, n in STATUS_BITS.items() if v & b) or "unknown"
    raise _lib.NsaError(f"a kernel gave up waiting on its pipeline (status bits {v:#x}: {names}); the results of the calls since "
                        "the last check are not valid")


def check_status(device="cuda"):
    """Synchronises with the device and raises NsaError if any kernel reported a pipeline time-out since the last check
    (the word is cleared, so the next check starts fresh).  A kernel whose bounded wait ran out still returns, with rc 0
    and garbage results: this is how a caller finds out."""
    d = torch.device(device)
    dev = torch.device("cuda", torch.cuda.current_device()) if d.index is None else d
    w = status_word(dev)
    v = int(w.item())
    m = _mirror.get(dev.index)
    if m is not None:
        m[1] = None
    if v:
        w.zero_()
        _raise_status(v)


def poll_status(device):
    """Non-blocking form used by NSACore.forward / nsa_prefill / nsa_decode: raises if the status word copied to the host at
    the end of an EARLIER call (post_status) has arrived and is non-zero.  Never synchronises; does nothing while the
    current stream is being captured into a CUDA graph."""
    if torch.cuda.is_current_stream_capturing():
        return
    idx = torch.device(device).index
    m = _mirror.get(torch.cuda.current_device() if idx is None else idx)
    if m is None or m[1] is None or not m[1].query():
        return
    m[1] = None
    v = int(m[0][0])
    if v:
        status_word(device).zero_()
        _raise_status(v)


def post_status(device):
    """Enqueue a copy of the status word into pinned host memory behind the work queued so far (no synchronisation)."""
    if torch.cuda.is_current_stream_capturing():
        return
    idx = torch.device(device).index
    idx = torch.cuda.current_device() if idx is None else idx
    m = _mirror.get(idx)
    if m is None:
        m = _mirror[idx] = [torch.zeros(1, dtype=torch.int32).pin_memory(), None]
    if m[1] is not None and not m[1].query():
        return          # the previous copy is still in flight: keep it (its host word must not be overwritten under it)
    m[0].copy_(status_word(torch.device("cuda", idx)), non_blocking=True)
    ev = torch.cuda.Event()
    ev.record()
    m[1] = ev


def call(fn, params, ref_tensor):
    """`ref_tensor`: one of the call's 16-bit tensors (its device gives the stream, its dtype the build of the library);
    entry points without 16-bit data pass any tensor of the call."""
    _lib.call(fn, params, stream_ptr(ref_tensor), f16=ref_tensor.dtype == torch.float16)


def attn_params(q, k, v, helper, sm_scale, *, o=None, lse=None, lse_is_head_major=False, dout=None, delta=None,
                dq=None, dk=None, dv=None, topk=None, cp=None, need_y=False):
    """Fill an NsaAttnParams.  `lse` (and `delta`) are [QH,T] when lse_is_head_major else [T,QH]."""
    check_bf16_3d("q", q)
    check_bf16_3d("k", k)
    check_bf16_3d("v", v)
    T, QH, D = q.shape
    KH = k.size(1)
    assert k.dtype == q.dtype and v.dtype == q.dtype, "q, k and v must share one 16-bit dtype"
    assert k.size(-1) == D and v.size(-1) == D, "this build needs qk_head_dim == v_head_dim"
    assert v.size(1) == KH and v.size(0) == k.size(0) and QH % KH == 0
    p = S["NsaAttnParams"]()
    p.meta, p.hp = seq_meta(helper, cp), hyper()
    p.q, p.k, p.v, p.o, p.lse = ptr(q), ptr(k), ptr(v), ptr(o), ptr(lse)
    p.dout, p.delta, p.dq, p.dk, p.dv, p.topk = ptr(dout), ptr(delta), ptr(dq), ptr(dk), ptr(dv), ptr(topk)
    p.q_stride_t, p.k_stride_t, p.v_stride_t = q.stride(0), k.stride(0), v.stride(0)
    for name, t in (("o", o), ("dout", dout), ("dq", dq)):
        if t is not None:
            assert t.dtype == q.dtype and t.stride(-1) == 1 and t.stride(1) == D, f"{name}: the dtype of q, contiguous heads"
    for name, t in (("dk", dk), ("dv", dv)):
        if t is not None:
            assert t.dtype == torch.float32 and t.stride(-1) == 1 and t.stride(1) == D, f"{name}: fp32, contiguous heads"
    p.o_stride_t = o.stride(0) if o is not None else 0
    p.do_stride_t = dout.stride(0) if dout is not None else 0
    p.dq_stride_t = dq.stride(0) if dq is not None else 0
    p.dk_stride_t = dk.stride(0) if dk is not None else 0
    p.dv_stride_t = dv.stride(0) if dv is not None else 0
    if lse is not None:
        assert lse.dtype == torch.float32 and lse.is_contiguous()
        if lse_is_head_major:
            p.lse_stride_t, p.lse_stride_h = 1, lse.stride(0)
        else:
            p.lse_stride_t, p.lse_stride_h = lse.stride(0), 1
    if topk is not None:
        assert topk.dtype == torch.int32 and topk.is_contiguous() and topk.size(0) == KH and topk.size(1) == T
        p.hp.top_n = topk.size(-1)
        p.topk_stride_h = topk.stride(0)
    p.sm_scale = float(sm_scale)
    p.QH, p.KH, p.D = QH, KH, D
    p.status = ptr(status_word(q.device))
    p.n_q_rows, p.n_k_rows = T, k.size(0)
    return p
