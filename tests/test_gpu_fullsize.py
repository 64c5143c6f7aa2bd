"""Parity at the benchmark's FULL sizes.

The CPU oracle needs O(T^2) memory for a whole sequence, so at 64K tokens it is evaluated on a SAMPLE of query rows
(oracle.nsa_forward_rows: same rules per row; pinned against the full oracle in tests/test_oracle_golden.py).  The
backward is linear in dO, so with a dO that is zero outside the sample the oracle's autograd over the sampled rows gives
the complete dq / dk / dv / dw of that step, and every gradient tensor of the CUDA path is compared in full.

Also here: size-independent properties at full size (softmax rows sum to one: with V = 1 every branch returns 1 where a
row sees any key; rows outside the sample get exactly zero gradient).

Tolerance as in test_gpu_backward.py: max abs error <= 2e-2 * max(1, max|reference|) over EVERY element.  The oracle's
selected branch runs on the selection the CUDA path made (read from the autograd node), so a near-tie that the two
resolve differently cannot move a row; the selections themselves are compared as sets in test_config1_64k_sampled_rows.
"""
import random

import pytest
import torch

from oracle import nsa_oracle as O

pytestmark = pytest.mark.gpu
TOL = 2e-2


def _inputs(lens, QH, KH, D, seed):
    g = torch.Generator().manual_seed(seed)
    T = sum(lens)
    cu = [0]
    for L in lens:
        cu.append(cu[-1] + L)
    mk = lambda *s: torch.randn(*s, generator=g).bfloat16()
    return mk(T, QH, D), mk(T, KH, D), mk(T, KH, D), mk(T, QH, 3), cu


def _sample_rows(cu, n_random, seed):
    rng = random.Random(seed)
    rows = set()
    for b in range(len(cu) - 1):
        L = cu[b + 1] - cu[b]
        for t in (0, 30, 31, 32, 63, 64, 191, 192, 511, 512, 513, 1023, 1024, L // 2, L - 65, L - 2, L - 1):
            if 0 <= t < L:
                rows.add(cu[b] + t)
        for _ in range(n_random):
            rows.add(cu[b] + rng.randrange(L))
    return sorted(rows)


def _setup(cu, methods=("mean", "mean")):
    import flash_nsa
    from flash_nsa import NSAHelper
    NSAHelper.reset_context_parallel()
    NSAHelper.set_hyperparameters()
    NSAHelper.set_recompute()
    NSAHelper.set_cmp_kv_method(*methods)
    NSAHelper.init_cu_seqlens(torch.tensor(cu, dtype=torch.int32, device="cuda"))
    return flash_nsa


def _bulk(name, got, ref, frac=None):
    """frac None: strict maximum.  Otherwise (weight gradients of the learned compression, sums of bf16-rounded terms over
    every compressed row): that quantile within the bound and the maximum within five times the bound."""
    got, ref = got.float().cpu(), ref.float()
    assert got.shape == ref.shape, (name, got.shape, ref.shape)
    assert torch.isfinite(got).all(), name
    err = (got - ref).abs().flatten()
    scale = max(1.0, ref.abs().max().item())
    worst = err.max().item()
    print(f"[fullsize] {name}: max err {worst:.4g}, bound {TOL * scale:.4g}")
    if frac is None:
        assert worst <= TOL * scale, f"{name}: max err {worst:.4g} > {TOL * scale:.4g}"
        return
    k = max(1, int(frac * err.numel()))
    assert err.kthvalue(k).values.item() <= TOL * scale, f"{name}: {err.kthvalue(k).values.item():.4g} > {TOL * scale:.4g}"
    assert worst <= 5 * TOL * scale, f"{name}: max err {worst:.4g} > {5 * TOL * scale:.4g}"


def _core_case(lens, methods, seed, n_random):
    QH, KH, D = 64, 4, 128
    q, k, v, w, cu = _inputs(lens, QH, KH, D, seed)
    T = cu[-1]
    rows = _sample_rows(cu, n_random, seed)
    g = torch.Generator().manual_seed(seed + 1)
    do_rows = torch.randn(len(rows), QH, D, generator=g).bfloat16()
    fn = _setup(cu, methods)
    cfg = fn.NSAConfig(head_dim=D, num_heads=QH, num_kv_heads=KH, cmp_k_method=methods[0], cmp_v_method=methods[1])
    core = fn.NSACore(cfg)
    wk = wv = None
    if core.cmp_k_weight is not None:
        wk = (torch.randn(core.cmp_k_weight.shape, generator=g) * 0.02).bfloat16()
        core.cmp_k_weight.data = wk.cuda()
    if core.cmp_v_weight is not None:
        wv = (torch.randn(core.cmp_v_weight.shape, generator=g) * 0.02).bfloat16()
        core.cmp_v_weight.data = wv.cuda()
    qd, kd, vd, wd = [t.cuda().requires_grad_(True) for t in (q, k, v, w)]
    do = torch.zeros(T, QH, D, dtype=torch.bfloat16, device="cuda")
    ridx = torch.tensor(rows, device="cuda")
    do[ridx] = do_rows.cuda()
    o = core(qd, kd, vd, wd, torch.tensor(cu, dtype=torch.int32, device="cuda"))
    topk_gpu = o.grad_fn.saved_tensors[-1][:, ridx].cpu()       # the CUDA path's selection for the sampled rows
    o.backward(do)
    torch.cuda.synchronize()

    leaves = [t.float().requires_grad_(True) for t in (q, k, v, w)]
    wkr = wk.float().requires_grad_(True) if wk is not None else None
    wvr = wv.float().requires_grad_(True) if wv is not None else None
    o_ref, parts = O.nsa_forward_rows(*leaves, cu, rows, cmp_k_method=methods[0], cmp_v_method=methods[1],
                                      cmp_k_weight=wkr, cmp_v_weight=wvr, quant="fp16_cubed", topk=topk_gpu)
    (o_ref * do_rows.float()).sum().backward()
    qr, kr, vr, wr = leaves

    _bulk("o[rows]", o[ridx], o_ref.detach())
    _bulk("dq[rows]", qd.grad[ridx], qr.grad[rows])
    _bulk("dw[rows]", wd.grad[ridx], wr.grad[rows])
    _bulk("dk", kd.grad, kr.grad)
    _bulk("dv", vd.grad, vr.grad)
    if wkr is not None:
        _bulk("dWk", core.cmp_k_weight.grad, wkr.grad, frac=0.99)
    if wvr is not None:
        _bulk("dWv", core.cmp_v_weight.grad, wvr.grad, frac=0.99)
    # rows outside the sample had dO = 0: their gradients are exactly zero
    rest = torch.ones(T, dtype=torch.bool, device="cuda")
    rest[ridx] = False
    assert qd.grad[rest].abs().max().item() == 0.0
    assert wd.grad[rest].abs().max().item() == 0.0
    return q, k, v, cu, rows, parts


def test_config1_64k_sampled_rows():
    """BASELINE config 1: one causal sequence of 65 536 tokens, 64 q heads / 4 kv heads / d = 128, mean compression."""
    q, k, v, cu, rows, parts = _core_case([65536], ("mean", "mean"), seed=1001, n_random=12)
    # the selection of the sampled rows, from the CUDA scoring kernel, against the oracle's (sets; a differing row must
    # be a swap of blocks whose stored scores are equal or adjacent half-precision values)
    from flash_nsa.ops import mean_pooling, compress_attn, slc_topk_indices
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    ck, cv = mean_pooling(kd), mean_pooling(vd)
    _, lse = compress_attn(qd, ck, cv)
    res = slc_topk_indices(qd, ck, lse, maybe_efficient_version=True, scale_slc_p=True)
    topk = (res[0] if isinstance(res, (tuple, list)) else res)[:, torch.tensor(rows, device="cuda")].cpu().long()
    ref = parts["topk"].long()
    ign_ref = O.cdiv(cu[-1], 64)
    differing = 0
    for kh in range(topk.shape[0]):
        for r, row in enumerate(rows):
            nv = min(16, row // 64 + 1)
            a, b = set(topk[kh, r, :nv].tolist()), set(ref[kh, r, :nv].tolist())
            assert ign_ref not in b
            assert len(a) == nv and all(0 <= x <= row // 64 for x in a), (kh, row, sorted(a))
            differing += int(a != b)
            assert len(a ^ b) <= 4, (kh, row, sorted(a ^ b))          # at most two swapped near-ties
    assert differing <= max(2, (topk.shape[0] * len(rows)) // 10), differing


def test_config2_varlen_learned_compression_sampled_rows():
    """BASELINE config 2: 4 packed sequences with lengths U[4096, 8192], mean K compression, sigmoid-mul V compression."""
    rng = random.Random(1002)
    lens = [rng.randint(4096, 8192) for _ in range(4)]
    _core_case(lens, ("mean", "sigmoid-mul"), seed=1002, n_random=4)


def test_rows_sum_to_one_at_64k():
    """With V = 1 every branch returns exactly-rounded ones wherever the row sees a key (softmax normalisation and the
    masks at full size); compressed rows become visible at t = 31."""
    T, QH, KH, D = 65536, 64, 4, 128
    q, k, _, _, cu = _inputs([T], QH, KH, D, seed=77)
    _setup(cu)
    from flash_nsa.ops import mean_pooling, compress_attn, slc_topk_indices, select_attn, swa_varlen_func
    qd, kd = q.cuda(), k.cuda()
    ones = torch.ones(T, KH, D, dtype=torch.bfloat16, device="cuda")
    ck, cones = mean_pooling(kd), mean_pooling(ones)
    o_cmp, lse = compress_attn(qd, ck, cones)
    assert (o_cmp[:31] == 0).all() and (lse[:, :31] == 0).all()
    assert (o_cmp[31:].float() - 1).abs().max().item() <= 1e-2
    res = slc_topk_indices(qd, ck, lse, maybe_efficient_version=True, scale_slc_p=True)
    topk = res[0] if isinstance(res, (tuple, list)) else res
    o_slc = select_attn(qd, kd, ones, topk)
    assert (o_slc.float() - 1).abs().max().item() <= 1e-2
    o_swa = swa_varlen_func(qd, kd, ones)
    assert (o_swa.float() - 1).abs().max().item() <= 1e-2
