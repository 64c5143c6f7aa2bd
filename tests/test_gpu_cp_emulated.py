"""Context-parallel kernels on ONE GPU: every rank's shard is run against the gathered K/V and must reproduce the
unsharded run (the scheme of the reference's test_cp.py: gather -> non-CP run -> slice -> compare), for both shard
layouts.  dK/dV of the ranks must add up to the unsharded dK/dV (that sum is what the reduce-scatter computes)."""
import pytest
import torch

from oracle import nsa_oracle as O

pytestmark = pytest.mark.gpu


def _inputs(lens, QH, KH, D, seed):
    g = torch.Generator().manual_seed(seed)
    T = sum(lens)
    cu = [0]
    for L in lens:
        cu.append(cu[-1] + L)
    mk = lambda *s: torch.randn(*s, generator=g).bfloat16().cuda()
    return mk(T, QH, D), mk(T, KH, D), mk(T, KH, D), mk(T, QH, 3), mk(T, QH, D), cu


def _run(q, k, v, w, do, topk=None):
    """All branches fwd + bwd with the current helper state; returns outputs, dq (local) and fp32 dk/dv (global)."""
    from flash_nsa.ops import (mean_pooling_fwd, cmp_attn_fwd, cmp_attn_bwd, slc_topk_indices, slc_attn_fwd, slc_attn_bwd,
                               swa_fwd, swa_bwd, mean_pooling_bwd)
    ck, cv = mean_pooling_fwd(k), mean_pooling_fwd(v)
    cmp_o, cmp_lse = cmp_attn_fwd(q, ck, cv)
    tk, _ = slc_topk_indices(q, ck, cmp_lse, fp32=True, maybe_efficient_version=True)
    if topk is None:
        topk = tk
    slc_o, slc_lse = slc_attn_fwd(q, k, v, topk)
    swa_o, swa_lse = swa_fwd(q, k, v)
    dk = torch.zeros(k.shape, device="cuda")
    dv = torch.zeros(v.shape, device="cuda")
    dq, _, _ = swa_bwd(q, k, v, swa_o, swa_lse, do, dk=dk, dv=dv)
    slc_attn_bwd(q, k, v, topk, slc_o, slc_lse, do, dq, dk, dv)
    _, dck, dcv = cmp_attn_bwd(q, ck, cv, cmp_o, cmp_lse, do, dq)
    mean_pooling_bwd(k, dck, dk)
    mean_pooling_bwd(v, dcv, dv)
    return dict(cmp_o=cmp_o, cmp_lse=cmp_lse, topk=tk, slc_o=slc_o, swa_o=swa_o, dq=dq, dk=dk, dv=dv)


@pytest.mark.parametrize("lens,world,mode", [([1024], 2, 2), ([1024], 4, 1), ([300, 500, 224], 2, 2), ([640, 384], 4, 2),
                                              ([96, 928], 2, 1)])
def test_shards_reproduce_unsharded_run(lens, world, mode):
    from flash_nsa import NSAHelper
    QH, KH, D = 8, 2, 64
    q, k, v, w, do, cu = _inputs(lens, QH, KH, D, seed=sum(lens) + world)
    cu_d = torch.tensor(cu, dtype=torch.int32, device="cuda")
    NSAHelper.reset_context_parallel()
    NSAHelper.set_hyperparameters()
    NSAHelper.init_cu_seqlens(cu_d)
    full = _run(q, k, v, w, do)
    dk_sum = torch.zeros_like(full["dk"])
    dv_sum = torch.zeros_like(full["dv"])
    for rank in range(world):
        NSAHelper.emulate_context_parallel(rank, world)
        NSAHelper.init_cu_seqlens(cu_d, cp_mode=mode)
        meta = O.cp_metadata(cu, rank, world, mode)
        assert NSAHelper.cp_cu_seqlens.tolist() == meta["cp_cu_seqlens"]
        assert NSAHelper.cp_batch_idx.tolist() == meta["cp_batch_idx"]
        assert NSAHelper.cp_offset.tolist() == meta["cp_offset"]
        assert NSAHelper.cp_k_cu_seqlens.tolist() == meta["cp_k_cu_seqlens"]
        rows = torch.cat([torch.arange(b, e) for b, e in meta["ranges"]]).cuda()
        loc = _run(q[rows].contiguous(), k, v, w[rows].contiguous(), do[rows].contiguous(),
                   topk=full["topk"][:, rows].contiguous())
        assert torch.equal(loc["cmp_o"], full["cmp_o"][rows])
        assert torch.equal(loc["cmp_lse"], full["cmp_lse"][:, rows])
        assert torch.equal(loc["topk"], full["topk"][:, rows])
        assert torch.equal(loc["slc_o"], full["slc_o"][rows])
        assert torch.equal(loc["swa_o"], full["swa_o"][rows])
        # dq: same math, but tiles are cut differently at shard boundaries -> bf16 rounding of partial sums may differ
        assert (loc["dq"].float() - full["dq"][rows].float()).abs().max().item() <= 2e-2 * max(1.0, full["dq"].float().abs().max().item())
        dk_sum += loc["dk"]
        dv_sum += loc["dv"]
    NSAHelper.reset_context_parallel()
    for name, a, b in (("dk", dk_sum, full["dk"]), ("dv", dv_sum, full["dv"])):
        assert (a - b).abs().max().item() <= 2e-3 * max(1.0, b.abs().max().item()), name
