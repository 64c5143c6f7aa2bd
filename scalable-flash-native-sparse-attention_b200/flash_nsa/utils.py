"""Process-wide NSA state: hyper-parameters, varlen metadata and context-parallel shard tables.

Mirrors the reference's `NSAHelper` (flash_nsa/utils.py:49-482): the ops read their sequence metadata
from this class, modules set it up, and `get_bwd_helper()` snapshots it for pipeline-parallel backward.
All derived tables are computed on the host from ONE device->host copy of cu_seqlens.
"""
import numpy as np
import torch


def cdiv(a, b):
    return (a + b - 1) // b


def cu_seqlens_to_seqlens(cu_seqlens):
    return cu_seqlens[1:] - cu_seqlens[:-1]


def seqlens_to_cu_seqlens(seqlens):
    return torch.nn.functional.pad(seqlens.cumsum(-1), [1, 0]).to(torch.int32)


def get_cp_cu_seqlens(cu_seqlens, bos, eos):
    """Cut [bos, eos) at the sequence boundaries inside it (flash_nsa/utils.py:19-32)."""
    bounds, batch = [int(bos)], []
    for idx, val in enumerate(cu_seqlens):
        val = int(val)
        if val >= eos:
            bounds.append(int(eos))
            batch.append(idx - 1)
            break
        if val > bos:
            bounds.append(val)
            batch.append(idx - 1)
    return bounds, batch


def concat_cp_cu_seqlens(cu_seqlens, *parts):
    """Pieces of one or two chunks -> local offsets, sequence ids, in-sequence offsets (flash_nsa/utils.py:34-46)."""
    cp_cu, cp_batch, cp_off = [0], [], []
    for bounds, batch in parts:
        end = cp_cu[-1]
        for i, b in enumerate(batch):
            cp_cu.append(end + bounds[i + 1] - bounds[0])
            cp_batch.append(b)
            cp_off.append(bounds[i] - int(cu_seqlens[b]))
    return cp_cu, cp_batch, cp_off


_VARLEN_FIELDS = [
    "x_cu_seqlens", "x_seqlens", "x_maxlen", "y_cu_seqlens", "y_seqlens", "y_maxlen", "y_len",
    "k_cu_seqlens", "k_seqlens", "k_maxlen", "k_len", "x_cu_seqlens_host", "total_len",
]
_CP_FIELDS = [
    "cp_mode", "seqlen", "cp_bos1", "cp_bos2", "cp_eos1", "cp_eos2", "cp_offset", "cp_batch_idx", "cp_cu_seqlens",
    "cp_seqlens", "cp_maxlen", "atomic_add_dkdv", "cp_k_cu_seqlens", "cp_k_seqlens", "cp_k_maxlen", "cp_k_len",
    "cp_ranges", "cp_len",
]


class NSAHelper:
    is_hopper = True      # kept for source compatibility; this build has a single (sm_100a) code path
    use_tma = True

    kernel_size = 32
    stride = 16
    block_size = 64
    window_size = 512
    top_n = 16
    num_init_blocks = 1
    num_local_blocks = 2

    cmp_k_method = "mean"
    cmp_v_method = "mean"

    recompute_swa_o = False
    recompute_slc_o = False
    recompute_cmp_kv = False
    recompute_cmp_o = False

    is_context_parallel_enable = True
    pp_size = 1

    x_cu_seqlens = x_seqlens = x_maxlen = None
    y_cu_seqlens = y_seqlens = y_maxlen = y_len = None
    k_cu_seqlens = k_seqlens = k_maxlen = k_len = None
    x_cu_seqlens_host = None
    total_len = None

    process_group = None
    rank = 0
    world_size = 1
    cp_mode = 2
    kv_head_stride = 1
    bench_mode = False
    use_overlap_swa = False

    seqlen = cp_bos1 = cp_bos2 = cp_eos1 = cp_eos2 = None
    cp_offset = cp_batch_idx = cp_cu_seqlens = cp_seqlens = cp_maxlen = None
    atomic_add_dkdv = None
    cp_k_cu_seqlens = cp_k_seqlens = cp_k_maxlen = cp_k_len = None
    cp_ranges = None
    cp_len = None

    # ------------------------------------------------------------------ setters (same names as the reference)
    @classmethod
    def set_hyperparameters(cls, kernel_size=32, stride=16, block_size=64, window_size=512, top_n=16,
                            num_init_blocks=1, num_local_blocks=2):
        changed = (cls.kernel_size, cls.stride, cls.block_size) != (kernel_size, stride, block_size)
        cls.kernel_size, cls.stride, cls.block_size = kernel_size, stride, block_size
        cls.window_size, cls.top_n = window_size, top_n
        cls.num_init_blocks, cls.num_local_blocks = num_init_blocks, num_local_blocks
        if changed:
            cls.x_cu_seqlens = None  # derived tables depend on these

    @classmethod
    def set_recompute(cls, recompute_swa_o=False, recompute_slc_o=False, recompute_cmp_kv=False, recompute_cmp_o=False):
        cls.recompute_swa_o, cls.recompute_slc_o = recompute_swa_o, recompute_slc_o
        cls.recompute_cmp_kv, cls.recompute_cmp_o = recompute_cmp_kv, recompute_cmp_o

    @classmethod
    def set_pipeline_parallel_world_size(cls, pp_size):
        cls.pp_size = pp_size

    @classmethod
    def set_context_parallel(cls, process_group=None, kv_head_stride=1, use_overlap_swa=True):
        if process_group is None or not torch.distributed.is_initialized():
            return
        world_size = torch.distributed.get_world_size(process_group)
        if world_size <= 1:
            return
        cls.process_group = process_group
        cls.kv_head_stride = kv_head_stride
        cls.rank = torch.distributed.get_rank(process_group)
        cls.world_size = world_size
        cls.use_overlap_swa = use_overlap_swa
        cls.x_cu_seqlens = None

    @classmethod
    def emulate_context_parallel(cls, rank, world_size, kv_head_stride=1):
        """Put the helper into the state rank `rank` of `world_size` would have, without a process group.
        The ops then expect q-side tensors to be that rank's shard and k/v-side tensors the whole (gathered)
        sequences -- which lets one GPU check every rank's kernels against the unsharded run."""
        cls.process_group = "emulated"
        cls.kv_head_stride = kv_head_stride
        cls.rank, cls.world_size = rank, world_size
        cls.x_cu_seqlens = None

    @classmethod
    def reset_context_parallel(cls):
        cls.process_group, cls.rank, cls.world_size = None, 0, 1
        cls.cp_cu_seqlens = cls.cp_batch_idx = cls.cp_offset = None
        cls.x_cu_seqlens = None

    @classmethod
    def set_cmp_kv_method(cls, cmp_k_method, cmp_v_method):
        cls.cmp_k_method, cls.cmp_v_method = cmp_k_method, cmp_v_method

    @classmethod
    def enable_cp(cls):
        cls.is_context_parallel_enable = True

    @classmethod
    def disable_cp(cls):
        cls.is_context_parallel_enable = False

    @classmethod
    def enable_bench_mode(cls):
        cls.bench_mode = True

    @classmethod
    def disable_bench_mode(cls):
        cls.bench_mode = False

    @classmethod
    def is_use_ampere_ops(cls):
        return False

    # ------------------------------------------------------------------ varlen tables
    @classmethod
    def _need_init(cls, x_cu_seqlens, host):
        if cls.x_cu_seqlens is None or cls.x_cu_seqlens_host is None:
            return True
        if cls.x_cu_seqlens.device != x_cu_seqlens.device:
            return True
        return len(host) != len(cls.x_cu_seqlens_host) or bool((host != cls.x_cu_seqlens_host).any())

    @classmethod
    def _init_xyk_cu_seqlens(cls, x_cu_seqlens, host):
        dev = x_cu_seqlens.device
        x_len = np.diff(host)
        y_len = np.maximum((x_len - cls.kernel_size) // cls.stride + 1, 0)
        k_len = -(-x_len // cls.block_size)
        cls.x_cu_seqlens_host = host.copy()
        cls.total_len = int(host[-1])
        cls.x_cu_seqlens = x_cu_seqlens.to(torch.int32).contiguous()

        def dev_i32(a):
            return torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(dev)

        cls.x_seqlens = dev_i32(x_len)
        cls.x_maxlen = int(x_len.max())
        cls.y_seqlens = dev_i32(y_len)
        cls.y_maxlen = int(y_len.max())
        cls.y_cu_seqlens = dev_i32(np.concatenate([[0], np.cumsum(y_len)]))
        cls.y_len = int(y_len.sum())
        cls.k_seqlens = dev_i32(k_len)
        cls.k_maxlen = int(k_len.max())
        cls.k_cu_seqlens = dev_i32(np.concatenate([[0], np.cumsum(k_len)]))
        cls.k_len = int(k_len.sum())

    @classmethod
    def init_cu_seqlens(cls, x_cu_seqlens: torch.Tensor, x_cu_seqlens_np=None, cp_mode=1):
        host = np.asarray(x_cu_seqlens_np if x_cu_seqlens_np is not None else x_cu_seqlens.cpu().numpy()).astype(np.int64)
        if not cls._need_init(x_cu_seqlens, host) and (cls.process_group is None or cls.cp_mode == cp_mode):
            return
        cls._init_xyk_cu_seqlens(x_cu_seqlens, host)
        if cls.process_group is None:
            return
        cls._init_cp_cu_seqlens(host, cp_mode)

    @classmethod
    def _init_cp_cu_seqlens(cls, host=None, cp_mode=1):
        """Piece table of this rank (flash_nsa/utils.py:284-323).  mode 1: W contiguous chunks;
        mode 2: 2W chunks, rank r owns chunks r and 2W-1-r."""
        assert cp_mode in (1, 2)
        if host is None:
            host = cls.x_cu_seqlens_host
        cls.cp_mode = cp_mode
        S = int(host[-1])
        cls.seqlen = S
        W, r = cls.world_size, cls.rank
        if cp_mode == 2:
            assert S % (2 * W) == 0
            chunk = S // (2 * W)
            cls.cp_bos1, cls.cp_bos2 = chunk * r, chunk * (2 * W - 1 - r)
            cls.cp_eos1, cls.cp_eos2 = cls.cp_bos1 + chunk, cls.cp_bos2 + chunk
            cls.cp_ranges = [(cls.cp_bos1, cls.cp_eos1), (cls.cp_bos2, cls.cp_eos2)]
        else:
            assert S % W == 0
            chunk = S // W
            cls.cp_bos1, cls.cp_eos1 = chunk * r, chunk * r + chunk
            cls.cp_bos2 = cls.cp_eos2 = None
            cls.cp_ranges = [(cls.cp_bos1, cls.cp_eos1)]
        cp_cu, cp_batch, cp_off = concat_cp_cu_seqlens(host, *[get_cp_cu_seqlens(host, b, e) for b, e in cls.cp_ranges])
        dev = cls.x_cu_seqlens.device

        def dev_i32(a):
            return torch.tensor(a, device=dev, dtype=torch.int32)

        cls.cp_cu_seqlens, cls.cp_batch_idx, cls.cp_offset = dev_i32(cp_cu), dev_i32(cp_batch), dev_i32(cp_off)
        cls.atomic_add_dkdv = len(set(cp_batch)) < len(cp_batch)
        lens = np.diff(np.asarray(cp_cu))
        cls.cp_seqlens = dev_i32(lens)
        cls.cp_maxlen = int(lens.max())
        cls.cp_len = int(cp_cu[-1])
        k_lens = -(-(lens + np.asarray(cp_off)) // cls.block_size)
        cls.cp_k_seqlens = dev_i32(k_lens)
        cls.cp_k_cu_seqlens = dev_i32(np.concatenate([[0], np.cumsum(k_lens)]))
        cls.cp_k_maxlen = int(k_lens.max())
        cls.cp_k_len = int(k_lens.sum())

    @classmethod
    def cp_active(cls):
        return cls.cp_cu_seqlens is not None and cls.is_context_parallel_enable and cls.world_size > 1

    # ------------------------------------------------------------------ misc
    @classmethod
    def clear_tensor_data(cls, *tensors):
        for t in tensors:
            if isinstance(t, torch.Tensor):
                t.data = torch.Tensor()

    @classmethod
    def split_d(cls, d):
        p2 = 1 << (d - 1).bit_length()
        if d == p2:
            return d, 0
        d1 = p2 // 2
        return d1, d - d1

    @classmethod
    def get_bwd_helper(cls):
        return cls if cls.pp_size <= 1 else BwdNSAHelper()


class BwdNSAHelper:
    """Frozen copy of the tables a backward pass needs (pipeline parallelism runs backward after the
    global state has moved on to another micro-batch; flash_nsa/utils.py:465-482)."""

    def __init__(self):
        for name in _VARLEN_FIELDS + _CP_FIELDS + ["world_size", "is_context_parallel_enable", "block_size"]:
            setattr(self, name, getattr(NSAHelper, name))

    def cp_active(self):
        return self.cp_cu_seqlens is not None and self.is_context_parallel_enable and self.world_size > 1
