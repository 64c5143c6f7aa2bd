"""Compression / selection geometries other than kernel 32 / stride 16 / block 64, and the reference's general scoring
path (per-row probabilities rounded to half, then pooled in fp32).

The scores and the top-n lists of the general kernel are compared with the oracle for several (kernel_size, stride) pairs;
selections as sets with the usual tie policy (a differing row must be a swap of blocks whose oracle scores are within
1e-3 of the row's largest in fp32 mode, 2e-3 in the half-precision mode).  One geometry also runs the whole NSACore
forward + backward against autograd through the oracle, so a valid NSAConfig that is not 32/16/64 works end to end."""
import pytest
import torch

from oracle import nsa_oracle as O
from helpers import topk_mismatch_report

pytestmark = pytest.mark.gpu
TOL = 2e-2


def _mk(lens, QH, KH, D, seed):
    g = torch.Generator().manual_seed(seed)
    T = sum(lens)
    cu = [0]
    for L in lens:
        cu.append(cu[-1] + L)
    mk = lambda *s: torch.randn(*s, generator=g).bfloat16()
    return mk(T, QH, D), mk(T, KH, D), mk(T, KH, D), mk(T, QH, 3), mk(T, QH, D), cu


def _setup(cu, **hp):
    import flash_nsa
    from flash_nsa import NSAHelper
    NSAHelper.reset_context_parallel()
    NSAHelper.set_hyperparameters(**hp)
    NSAHelper.set_recompute()
    NSAHelper.set_cmp_kv_method("mean", "mean")
    NSAHelper.init_cu_seqlens(torch.tensor(cu, dtype=torch.int32, device="cuda"))
    return flash_nsa


@pytest.mark.parametrize("ks,st", [(64, 32), (32, 8), (16, 16), (64, 16), (32, 16)])
@pytest.mark.parametrize("fp32", [True, False])
def test_general_scoring_and_selection(ks, st, fp32):
    lens, QH, KH, D = [900, 333, 70, 20], 16, 2, 64
    q, k, v, w, do, cu = _mk(lens, QH, KH, D, seed=ks + st)
    _setup(cu, kernel_size=ks, stride=st, block_size=64)
    from flash_nsa.ops import mean_pooling_fwd, cmp_attn_fwd, slc_topk_indices
    qd = q.cuda()
    ck, cv = mean_pooling_fwd(k.cuda()), mean_pooling_fwd(v.cuda())
    ck_ref = O.mean_pool(k.float(), cu, ks, st)
    assert (ck.float().cpu() - ck_ref).abs().max().item() <= 8e-3
    cmp_o, lse = cmp_attn_fwd(qd, ck, cv)
    o_ref, lse_ref = O.cmp_attn(q.float(), ck.float().cpu(), cv.float().cpu(), cu, ks, st)
    assert (cmp_o.float().cpu() - o_ref).abs().max().item() <= TOL
    # maybe_efficient_version=False is the general path even for 32/16/64; other geometries take it whatever the flag says
    topk, probs = slc_topk_indices(qd, ck, lse, fp32=fp32, maybe_efficient_version=False, return_slc_prob=True)
    quant = "fp32" if fp32 else "fp16_rows"
    sc = O.slc_scores(q.float(), ck.float().cpu(), lse.float().cpu(), cu, ks, st, 64, quant=quant)
    ref = O.topk_select(sc, cu)
    ign = O.cdiv(max(lens), 64)
    n_diff, n_bad, n_rows = topk_mismatch_report(topk.cpu(), ref, sc, cu, ign, ign, rel_tol=1e-3 if fp32 else 2e-3)
    assert n_bad == 0, (n_diff, n_bad)
    assert n_diff <= max(2, int(2e-2 * n_rows)), (n_diff, n_rows)
    pr = probs.float().cpu()
    for b in range(len(lens)):
        got = pr[:, cu[b]:cu[b + 1], :sc[b].shape[-1]]
        tol = (1e-4 if fp32 else 3e-3) * sc[b].abs().clamp(min=1e-3)
        # a token's own block and later ones get no score in the kernel (no visible row reaches them)
        assert ((got - sc[b]).abs() <= tol).float().mean().item() > 0.999


@pytest.mark.parametrize("QH,KH", [(40, 1), (64, 2)])
def test_general_scoring_with_more_than_16_heads_per_kv_head(QH, KH):
    """Head groups of 16 are summed before the pooling (the reference loops min(G, 16) heads the same way)."""
    ks, st, D = 64, 32, 64
    lens = [300, 70, 513]
    q, k, v, w, do, cu = _mk(lens, QH, KH, D, seed=QH)
    _setup(cu, kernel_size=ks, stride=st, block_size=64)
    from flash_nsa.ops import mean_pooling_fwd, cmp_attn_fwd, slc_topk_indices
    qd = q.cuda()
    ck, cv = mean_pooling_fwd(k.cuda()), mean_pooling_fwd(v.cuda())
    cmp_o, lse = cmp_attn_fwd(qd, ck, cv)
    for fp32 in (True, False):
        topk, _ = slc_topk_indices(qd, ck, lse, fp32=fp32, maybe_efficient_version=False, return_slc_prob=True)
        sc = O.slc_scores(q.float(), ck.float().cpu(), lse.float().cpu(), cu, ks, st, 64, quant="fp32" if fp32 else "fp16_rows")
        ref = O.topk_select(sc, cu)
        ign = O.cdiv(max(lens), 64)
        n_diff, n_bad, n_rows = topk_mismatch_report(topk.cpu(), ref, sc, cu, ign, ign, rel_tol=1e-3 if fp32 else 2e-3)
        assert n_bad == 0, (fp32, n_diff, n_bad)


def test_core_forward_backward_with_another_geometry():
    ks, st = 64, 32
    lens, QH, KH, D = [700, 450], 8, 2, 64
    q, k, v, w, do, cu = _mk(lens, QH, KH, D, seed=4)
    fn = _setup(cu, kernel_size=ks, stride=st, block_size=64)
    cfg = fn.NSAConfig(head_dim=D, num_heads=QH, num_kv_heads=KH, kernel_size=ks, stride=st, block_size=64)
    core = fn.NSACore(cfg)
    leaves = [t.cuda().requires_grad_(True) for t in (q, k, v, w)]
    o = core(*leaves, torch.tensor(cu, dtype=torch.int32, device="cuda"))
    topk_gpu = o.grad_fn.saved_tensors[-1].cpu()
    o.backward(do.cuda())
    ref_leaves = [t.float().requires_grad_(True) for t in (q, k, v, w)]
    # NSACore asks for the 32/16/64 fast path; with another geometry the general path runs in its half-precision row mode
    o_ref = O.nsa_forward(*ref_leaves, cu, kernel_size=ks, stride=st, block_size=64, quant="fp16_rows", topk=topk_gpu)
    (o_ref * do.float()).sum().backward()
    for name, a, b in zip(("o", "dq", "dk", "dv", "dw"), [o] + [t.grad for t in leaves], [o_ref] + [t.grad for t in ref_leaves]):
        err = (a.float().cpu() - b.detach().float()).abs().max().item()
        assert err <= TOL * max(1.0, b.abs().max().item()), (name, err)
