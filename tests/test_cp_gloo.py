"""Host-side logic of the context-parallel path with two CPU processes over gloo: shard tables against the oracle's
restatement of the reference rule, the K/V all-gather (with the zig-zag un-shuffle) and the dK/dV reduce-scatter."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, mode, q):
    try:
        for p in (ROOT, os.path.join(ROOT, "scalable-flash-native-sparse-attention_b200")):
            if p not in sys.path:
                sys.path.insert(0, p)
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from flash_nsa.comm import Comm
        from flash_nsa.utils import NSAHelper
        from oracle import nsa_oracle as O

        cu = [0, 40, 104, 128]
        NSAHelper.set_context_parallel(dist.group.WORLD, kv_head_stride=1)
        NSAHelper.init_cu_seqlens(torch.tensor(cu, dtype=torch.int32), cp_mode=mode)
        meta = O.cp_metadata(cu, rank, world, mode)
        assert NSAHelper.cp_cu_seqlens.tolist() == meta["cp_cu_seqlens"]
        assert NSAHelper.cp_batch_idx.tolist() == meta["cp_batch_idx"]
        assert NSAHelper.cp_offset.tolist() == meta["cp_offset"]
        assert NSAHelper.cp_maxlen == meta["cp_maxlen"]
        assert NSAHelper.atomic_add_dkdv == meta["atomic_add_dkdv"]

        T, H, D = cu[-1], 1, 8
        g = torch.Generator().manual_seed(5)
        k_full = torch.randn(T, H, D, generator=g)
        k_loc = O.cp_local_slice(k_full, meta["ranges"]).contiguous()
        t = k_loc.size(0)
        comm = Comm(dist.group.WORLD, t, world, H, D, D, k_full.dtype, "cpu", cp_mode=mode, with_grads=True)
        comm.all_gather(k_loc, Comm.KEY)
        comm.all_gather(k_loc * 2, Comm.VALUE)
        assert torch.equal(comm.wait(Comm.KEY), k_full)
        assert torch.equal(comm.wait(Comm.VALUE), k_full * 2)
        # second use of the double buffer
        comm.all_gather(k_loc + 1, Comm.KEY)
        assert torch.equal(comm.wait(Comm.KEY), k_full + 1)
        # reduce-scatter: every rank contributes rank+1 times a known global gradient
        dk, dv = comm.grad_buffers()
        dk.copy_(k_full * (rank + 1))
        out = comm.reduce_scatter(Comm.GRAD_KEY)
        comm.wait(Comm.GRAD_KEY)
        want = O.cp_local_slice(k_full * sum(r + 1 for r in range(world)), meta["ranges"])
        assert torch.allclose(out, want, atol=1e-5)
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception as e:  # surface the failure to the parent
        import traceback
        q.put((rank, traceback.format_exc()))


@pytest.mark.parametrize("mode", [1, 2])
def test_two_rank_gloo(mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000 + mode
    procs = [ctx.Process(target=_worker, args=(r, 2, port, mode, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    for rank, msg in res:
        assert msg == "ok", f"rank {rank}: {msg}"
