"""Backward parity of the CUDA kernels against autograd through the CPU oracle, and against the gradients the
reference's torch code produced (tests/golden).

Tolerance: max abs error <= 2e-2 * max(1, max|reference gradient|).  Gradients of K/V sum thousands of bf16
products per element (every later query contributes), so their magnitude grows with the sequence length and the
bound scales with it; the reference's own kernels show 0.03-0.5 absolute on such tensors (notebook cell 13).
"""
import numpy as np
import pytest
import torch

from oracle import nsa_oracle as O
from helpers import load_golden, golden_params

pytestmark = pytest.mark.gpu
TOL = 2e-2


def _mk(lens, QH, KH, D, seed):
    g = torch.Generator().manual_seed(seed)
    T = sum(lens)
    cu = [0]
    for L in lens:
        cu.append(cu[-1] + L)
    q = torch.randn(T, QH, D, generator=g).bfloat16()
    k = torch.randn(T, KH, D, generator=g).bfloat16()
    v = torch.randn(T, KH, D, generator=g).bfloat16()
    w = torch.randn(T, QH, 3, generator=g).bfloat16()
    do = torch.randn(T, QH, D, generator=g).bfloat16()
    return q, k, v, w, do, cu


def _setup(cu, **hp):
    import flash_nsa
    from flash_nsa import NSAHelper
    NSAHelper.reset_context_parallel()
    NSAHelper.set_hyperparameters(**hp)
    NSAHelper.set_recompute()
    NSAHelper.set_cmp_kv_method("mean", "mean")
    NSAHelper.init_cu_seqlens(torch.tensor(cu, dtype=torch.int32, device="cuda"))
    return flash_nsa


def _check(name, got, ref, tol=TOL):
    ref = torch.as_tensor(ref).float()
    got = got.float().cpu()
    assert got.shape == ref.shape, (name, got.shape, ref.shape)
    err = (got - ref).abs().max().item()
    bound = tol * max(1.0, ref.abs().max().item())
    assert err <= bound, f"{name}: err {err:.4g} > {bound:.4g}"


CASES = [
    ([320], 4, 1, 64),
    ([17, 32, 47, 48, 130, 1, 700], 4, 1, 64),
    ([200, 333], 16, 1, 128),
    ([1100], 8, 2, 64),
    ([96, 130], 6, 2, 64),
    ([300, 150], 32, 1, 64),   # G = 32: two groups of 16 query heads per kv head in the selected branch
]


def _leaf(*ts):
    return [t.float().clone().requires_grad_(True) for t in ts]


@pytest.mark.parametrize("lens,QH,KH,D", CASES)
def test_branch_backward(lens, QH, KH, D):
    q, k, v, w, do, cu = _mk(lens, QH, KH, D, seed=7 + sum(lens))
    _setup(cu)
    from flash_nsa.ops import (mean_pooling, compress_attn, select_attn, swa_varlen_func, fused_sigmoid_combine)
    dev = lambda *ts: [t.cuda().clone().requires_grad_(True) for t in ts]

    # --- compressed branch, through the pooling (so the pooling backward is covered too)
    qr, kr, vr = _leaf(q, k, v)
    ck, cv = O.mean_pool(kr, cu), O.mean_pool(vr, cu)
    o_ref, lse_ref = O.cmp_attn(qr, ck, cv, cu)
    (o_ref * do.float()).sum().backward()
    qd, kd, vd = dev(q, k, v)
    o, lse = compress_attn(qd, mean_pooling(kd), mean_pooling(vd))
    (o.float() * do.cuda().float()).sum().backward()
    _check("cmp dq", qd.grad, qr.grad)
    _check("cmp dk", kd.grad, kr.grad)
    _check("cmp dv", vd.grad, vr.grad)

    # --- sliding window
    qr, kr, vr = _leaf(q, k, v)
    o_ref, _ = O.swa(qr, kr, vr, cu)
    (o_ref * do.float()).sum().backward()
    qd, kd, vd = dev(q, k, v)
    o = swa_varlen_func(qd, kd, vd)
    (o.float() * do.cuda().float()).sum().backward()
    _check("swa dq", qd.grad, qr.grad)
    _check("swa dk", kd.grad, kr.grad)
    _check("swa dv", vd.grad, vr.grad)

    # --- selected blocks, on the oracle's lists
    with torch.no_grad():
        ckf, cvf = O.mean_pool(k.float(), cu), O.mean_pool(v.float(), cu)
        _, l0 = O.cmp_attn(q.float(), ckf, cvf, cu)
        topk = O.topk_select(O.slc_scores(q.float(), ckf, l0, cu), cu)
    qr, kr, vr = _leaf(q, k, v)
    o_ref, _ = O.slc_attn(qr, kr, vr, topk, cu)
    (o_ref * do.float()).sum().backward()
    qd, kd, vd = dev(q, k, v)
    o = select_attn(qd, kd, vd, topk.cuda())
    (o.float() * do.cuda().float()).sum().backward()
    _check("slc dq", qd.grad, qr.grad)
    _check("slc dk", kd.grad, kr.grad)
    _check("slc dv", vd.grad, vr.grad)

    # --- combine
    a, b, c, wr = _leaf(q, do, (q * 0.5 - do).bfloat16(), w)
    (O.combine(a, b, c, wr) * do.float()).sum().backward()
    ad, bd, cd, wd = dev(q, do, (q * 0.5 - do).bfloat16(), w)
    (fused_sigmoid_combine(ad, bd, cd, wd).float() * do.cuda().float()).sum().backward()
    _check("comb da", ad.grad, a.grad)
    _check("comb db", bd.grad, b.grad)
    _check("comb dc", cd.grad, c.grad)
    _check("comb dw", wd.grad, wr.grad)


def test_selected_backward_one_kernel_equals_two_kernels():
    """The block-major kernel that also adds dS K into dq (bf16 reductions) against the two-kernel form (token-major dQ,
    fp32 accumulation per token): same dk / dv up to the order of their atomics, dq within bf16 rounding of 16 adds."""
    for lens, QH, KH, D in (([1500, 700], 32, 2, 128), ([2100], 8, 2, 64), ([900], 40, 2, 128)):
        q, k, v, w, do, cu = _mk(lens, QH, KH, D, seed=61)
        _setup(cu)
        from flash_nsa.ops import mean_pooling, compress_attn, slc_topk_indices
        from flash_nsa.ops.select_attn import slc_attn_fwd, slc_attn_bwd
        qd, kd, vd, dod = q.cuda(), k.cuda(), v.cuda(), do.cuda()
        ck = mean_pooling(kd)
        _, lse_c = compress_attn(qd, ck, mean_pooling(vd))
        res = slc_topk_indices(qd, ck, lse_c, maybe_efficient_version=True, scale_slc_p=True)
        topk = res[0] if isinstance(res, (tuple, list)) else res
        o, lse = slc_attn_fwd(qd, kd, vd, topk)
        outs = []
        for two in (False, True):
            dq = torch.full_like(qd, 0.25)          # given dq: results are added into it
            dk = torch.zeros(kd.shape, device="cuda", dtype=torch.float32)
            dv = torch.zeros(vd.shape, device="cuda", dtype=torch.float32)
            slc_attn_bwd(qd, kd, vd, topk, o, lse, dod, dq, dk, dv, two_kernel_dq=two)
            outs.append((dq, dk, dv))
        torch.cuda.synchronize()
        for name, a, b in zip(("dq", "dk", "dv"), outs[0], outs[1]):
            scale = max(1.0, b.float().abs().max().item())
            tol = 2e-2 if name == "dq" else 1e-4
            assert (a.float() - b.float()).abs().max().item() <= tol * scale, (name, lens, QH)
        # a dq that bulk tensor reductions cannot address (8-byte aligned only) takes the two-kernel form by itself
        flat = torch.full((qd.numel() + 8,), 0.25, dtype=qd.dtype, device="cuda")
        dq_u = flat[4:4 + qd.numel()].view_as(qd)
        dk = torch.zeros(kd.shape, device="cuda", dtype=torch.float32)
        dv = torch.zeros(vd.shape, device="cuda", dtype=torch.float32)
        slc_attn_bwd(qd, kd, vd, topk, o, lse, dod, dq_u, dk, dv)
        assert torch.equal(dq_u, outs[1][0])
        # a new dq (not given) starts from zero in both forms
        dq0, _, _ = slc_attn_bwd(qd, kd, vd, topk, o, lse, dod)
        assert (dq0.float() - (outs[1][0].float() - 0.25)).abs().max().item() <= 2e-2 * max(1.0, dq0.float().abs().max().item())


@pytest.mark.parametrize("range_rows,item_rows", [(128, 24), (512, 8), (0, 1000), (64, 3)])
def test_selected_backward_does_not_depend_on_how_the_work_is_cut(range_rows, item_rows):
    """The persistent backward kernel walks work items (key block x slice of its query list) range by range; however the
    lists are cut into ranges and items (many small items, items that end inside a query tile, a single range), dk / dv
    agree up to the order of their atomics and dq within the bf16 rounding of its adds, and all match the oracle."""
    lens, QH, KH, D = [900, 333, 70], 32, 2, 128
    q, k, v, w, do, cu = _mk(lens, QH, KH, D, seed=67)
    _setup(cu)
    from flash_nsa.ops.select_attn import slc_attn_fwd, slc_attn_bwd
    ckf = O.mean_pool(k.float(), cu)
    _, l0 = O.cmp_attn(q.float(), ckf, O.mean_pool(v.float(), cu), cu)
    topk = O.topk_select(O.slc_scores(q.float(), ckf, l0, cu), cu)
    qr, kr, vr = _leaf(q, k, v)
    o_ref, _ = O.slc_attn(qr, kr, vr, topk, cu)
    (o_ref * do.float()).sum().backward()
    qd, kd, vd, dod, tk = q.cuda(), k.cuda(), v.cuda(), do.cuda(), topk.cuda()
    o, lse = slc_attn_fwd(qd, kd, vd, tk)
    dq, dk, dv = slc_attn_bwd(qd, kd, vd, tk, o, lse, dod, range_rows=range_rows, item_rows=item_rows)
    _check("dq", dq, qr.grad)
    _check("dk", dk, kr.grad)
    _check("dv", dv, vr.grad)
    dq2, dk2, dv2 = slc_attn_bwd(qd, kd, vd, tk, o, lse, dod)
    assert (dk.float() - dk2.float()).abs().max().item() <= 2e-2 * max(1.0, dk2.float().abs().max().item())
    assert (dq.float() - dq2.float()).abs().max().item() <= 2e-2 * max(1.0, dq2.float().abs().max().item())


def test_k2q_index_is_the_transpose():
    lens = [700, 130]
    q, k, v, w, do, cu = _mk(lens, 4, 2, 64, seed=5)
    _setup(cu)
    from flash_nsa import NSAHelper
    from flash_nsa.ops import get_bind_from_find
    ckf = O.mean_pool(k.float(), cu)
    _, l0 = O.cmp_attn(q.float(), ckf, O.mean_pool(v.float(), cu), cu)
    topk = O.topk_select(O.slc_scores(q.float(), ckf, l0, cu), cu)
    offsets, tokens = get_bind_from_find(topk.cuda())
    offsets, tokens = offsets.cpu(), tokens.cpu()
    k_cu = NSAHelper.k_cu_seqlens.cpu().tolist()
    for kh in range(2):
        for b, L in enumerate(lens):
            for t in range(L):
                pass
        # rebuild the forward lists from the index and compare as sets
        rebuilt = {}
        for row in range(offsets.shape[1] - 1):
            for tok in tokens[kh, offsets[kh, row]:offsets[kh, row + 1]].tolist():
                rebuilt.setdefault(tok, set()).add(row)
        for b, L in enumerate(lens):
            for t in range(L):
                nv = min(16, t // 64 + 1)
                want = {k_cu[b] + int(x) for x in topk[kh, cu[b] + t, :nv].tolist()}
                assert rebuilt.get(cu[b] + t, set()) == want
        assert int(offsets[kh, -1]) == sum(min(16, t // 64 + 1) for L in lens for t in range(L))


def test_k2q_index_with_range_buckets_and_work_items():
    """The form of the index the backward kernel walks: lists split by the range of the query row (cell = range * blocks +
    block row, range-major) and cut into work items of bounded size.  Checked: every cell holds exactly the rows of its
    range that selected its block; the items tile every non-empty cell exactly once, in cell order, none longer than
    item_rows; the plain index is the union over ranges."""
    lens = [700, 130, 333]
    q, k, v, w, do, cu = _mk(lens, 4, 2, 64, seed=6)
    _setup(cu)
    from flash_nsa import NSAHelper
    from flash_nsa.ops import get_bind_from_find
    ckf = O.mean_pool(k.float(), cu)
    _, l0 = O.cmp_attn(q.float(), ckf, O.mean_pool(v.float(), cu), cu)
    topk = O.topk_select(O.slc_scores(q.float(), ckf, l0, cu), cu)
    R, P = 256, 40
    plain = get_bind_from_find(topk.cuda())
    idx = get_bind_from_find(topk.cuda(), range_rows=R, item_rows=P)
    torch.cuda.synchronize()
    T, KH = cu[-1], 2
    n_blocks = NSAHelper.k_len
    assert idx.n_ranges == -(-T // R) and idx.offsets.shape == (KH, idx.n_ranges * n_blocks + 1)
    off, tok, items, n_items = idx.offsets.cpu(), idx.tokens.cpu(), idx.items.cpu(), idx.n_items.cpu()
    p_off, p_tok = plain.offsets.cpu(), plain.tokens.cpu()
    for kh in range(KH):
        union = [[] for _ in range(n_blocks)]
        for cell in range(idx.n_ranges * n_blocks):
            r, row = divmod(cell, n_blocks)
            rows = tok[kh, off[kh, cell]:off[kh, cell + 1]].tolist()
            assert all(r * R <= x < (r + 1) * R for x in rows), (kh, cell)
            union[row] += rows
        for row in range(n_blocks):
            assert sorted(union[row]) == sorted(p_tok[kh, p_off[kh, row]:p_off[kh, row + 1]].tolist()), (kh, row)
        # the items: consecutive slices that cover [0, total) exactly, cell after cell
        pos, cell = 0, 0
        for i in range(int(n_items[kh])):
            row, lo, hi, r = items[kh, i].tolist()
            assert lo == pos and lo < hi <= lo + P
            c = r * n_blocks + row
            assert c >= cell and off[kh, c] <= lo and hi <= off[kh, c + 1]
            cell, pos = c, hi
        assert pos == int(off[kh, -1]) == int(p_off[kh, -1])
        n_expected = sum(-(-int(off[kh, c + 1] - off[kh, c]) // P) for c in range(idx.n_ranges * n_blocks))
        assert int(n_items[kh]) == n_expected
    assert n_items[KH:].tolist() == [0, 0]          # the backward kernel's ticket counters start at zero


@pytest.mark.parametrize("methods", [("mean", "mean"), ("linear", "sigmoid-mul"), ("swiglu", "mean")])
def test_nsa_core_forward_backward(methods):
    """NSACore (one fused autograd function) against autograd through the oracle, learned compression included."""
    lens = [600, 333]
    QH, KH, D = 8, 2, 64
    q, k, v, w, do, cu = _mk(lens, QH, KH, D, seed=17)
    fn = _setup(cu)
    cfg = fn.NSAConfig(head_dim=D, num_heads=QH, num_kv_heads=KH, cmp_k_method=methods[0], cmp_v_method=methods[1])
    core = fn.NSACore(cfg)
    g = torch.Generator().manual_seed(3)
    wk = wv = None
    if core.cmp_k_weight is not None:
        wk = (torch.randn(core.cmp_k_weight.shape, generator=g) * 0.02).bfloat16()
        core.cmp_k_weight.data = wk.cuda()
    if core.cmp_v_weight is not None:
        wv = (torch.randn(core.cmp_v_weight.shape, generator=g) * 0.02).bfloat16()
        core.cmp_v_weight.data = wv.cuda()
    qd, kd, vd, wd = [t.cuda().clone().requires_grad_(True) for t in (q, k, v, w)]
    o = core(qd, kd, vd, wd, torch.tensor(cu, dtype=torch.int32, device="cuda"))
    topk_gpu = o.grad_fn.saved_tensors[-1].cpu()          # the selection the CUDA path made, [KH,T,16]
    (o.float() * do.cuda().float()).sum().backward()

    qr, kr, vr, wr = _leaf(q, k, v, w)
    wkr = wk.float().requires_grad_(True) if wk is not None else None
    wvr = wv.float().requires_grad_(True) if wv is not None else None
    # the oracle's selected branch runs on the CUDA path's own selection, so that a near-tie resolved the other way
    # cannot move a row: every tensor is then held to a strict maximum.  The selection itself is compared below.
    o_ref, parts = O.nsa_forward(qr, kr, vr, wr, cu, cmp_k_method=methods[0], cmp_v_method=methods[1], cmp_k_weight=wkr,
                                 cmp_v_weight=wvr, quant="fp16_cubed", topk=topk_gpu, return_parts=True)
    (o_ref * do.float()).sum().backward()
    T = cu[-1]
    differing = 0
    for b in range(len(lens)):
        for t in range(lens[b]):
            nv = min(16, t // 64 + 1)
            for kh in range(KH):
                a = set(topk_gpu[kh, cu[b] + t, :nv].tolist())
                differing += int(a != set(parts["topk"][kh, cu[b] + t, :nv].tolist()))
                assert len(a) == nv and all(0 <= x <= t // 64 for x in a)
    assert differing <= max(2, KH * T // 50), differing     # learned compression rounds its rows to bf16: a few near-ties flip

    def bulk(name, got, ref, frac=None):
        err = (got.float().cpu() - ref.float()).abs().flatten()
        scale = max(1.0, ref.abs().max().item())
        assert torch.isfinite(got).all(), name
        if frac is None:
            assert err.max().item() <= TOL * scale, f"{name}: max err {err.max().item():.4g} > {TOL * scale:.4g}"
        else:   # weight gradients (sums over every compressed row of bf16-rounded terms): bulk at TOL, tail capped at 5x
            assert err.kthvalue(max(1, int(frac * err.numel()))).values.item() <= TOL * scale, name
            assert err.max().item() <= 5 * TOL * scale, f"{name}: max err {err.max().item():.4g}"

    bulk("o", o, o_ref)
    bulk("dq", qd.grad, qr.grad)
    bulk("dk", kd.grad, kr.grad)
    bulk("dv", vd.grad, vr.grad)
    bulk("dw", wd.grad, wr.grad)
    if wkr is not None:
        bulk("dWk", core.cmp_k_weight.grad, wkr.grad, frac=0.99)
    if wvr is not None:
        bulk("dWv", core.cmp_v_weight.grad, wvr.grad, frac=0.99)


def test_nsa_core_with_empty_and_tiny_sequences_in_the_batch():
    """A packed batch with zero-length sequences, a one-token sequence and one shorter than the compression window (no
    compressed row at all), next to ordinary ones: forward and every gradient against the oracle; then an empty batch."""
    lens = [70, 0, 1, 513, 0, 31]
    QH, KH, D = 8, 2, 64
    q, k, v, w, do, cu = _mk(lens, QH, KH, D, seed=23)
    fn = _setup(cu)
    core = fn.NSACore(fn.NSAConfig(head_dim=D, num_heads=QH, num_kv_heads=KH))
    qd, kd, vd, wd = [t.cuda().clone().requires_grad_(True) for t in (q, k, v, w)]
    o = core(qd, kd, vd, wd, torch.tensor(cu, dtype=torch.int32, device="cuda"))
    topk_gpu = o.grad_fn.saved_tensors[-1].cpu()
    (o.float() * do.cuda().float()).sum().backward()
    qr, kr, vr, wr = _leaf(q, k, v, w)
    o_ref = O.nsa_forward(qr, kr, vr, wr, cu, quant="fp16_cubed", topk=topk_gpu)
    (o_ref * do.float()).sum().backward()
    for name, got, ref in (("o", o, o_ref), ("dq", qd.grad, qr.grad), ("dk", kd.grad, kr.grad), ("dv", vd.grad, vr.grad),
                           ("dw", wd.grad, wr.grad)):
        assert torch.isfinite(got).all(), name
        err = (got.float().cpu() - ref.float()).abs().max().item()
        assert err <= TOL * max(1.0, ref.abs().max().item()), (name, err)
    # no tokens at all: shapes are kept, nothing is launched that could fault
    z = lambda h, d_: torch.zeros(0, h, d_, dtype=torch.bfloat16, device="cuda", requires_grad=True)
    q0, k0, v0, w0 = z(QH, D), z(KH, D), z(KH, D), z(QH, 3)
    o0 = core(q0, k0, v0, w0, torch.tensor([0, 0], dtype=torch.int32, device="cuda"))
    assert o0.shape == (0, QH, D)
    o0.sum().backward()
    assert q0.grad is not None and q0.grad.shape == (0, QH, D)


def test_hf_core_equals_megatron_core():
    """The identity the reference's own test prints (test.py:320-349): both module flavours agree."""
    lens = [500, 400]
    QH, KH, D = 8, 2, 64
    q, k, v, w, do, cu = _mk(lens, QH, KH, D, seed=23)
    fn = _setup(cu)
    cfg = fn.NSAConfig(head_dim=D, num_heads=QH, num_kv_heads=KH)
    cu_d = torch.tensor(cu, dtype=torch.int32, device="cuda")
    outs = []
    for core in (fn.HFNSACore(cfg).cuda(), fn.NSACore(cfg)):
        qd, kd, vd, wd = [t.cuda().clone().requires_grad_(True) for t in (q, k, v, w)]
        o = core(qd, kd, vd, wd, cu_d)
        (o.float() * do.cuda().float()).sum().backward()
        outs.append((o, qd.grad, kd.grad, vd.grad, wd.grad))
    names = ["o", "dq", "dk", "dv", "dw"]
    for name, a, b in zip(names, outs[0], outs[1]):
        scale = max(1.0, a.float().abs().max().item())
        assert (a.float() - b.float()).abs().max().item() <= 3e-2 * scale, name


def test_recompute_flags_do_not_change_results():
    lens = [450]
    QH, KH, D = 8, 2, 64
    q, k, v, w, do, cu = _mk(lens, QH, KH, D, seed=29)
    fn = _setup(cu)
    cu_d = torch.tensor(cu, dtype=torch.int32, device="cuda")
    res = []
    for flag in (False, True):
        cfg = fn.NSAConfig(head_dim=D, num_heads=QH, num_kv_heads=KH, recompute_swa_o=flag, recompute_slc_o=flag,
                           recompute_cmp_kv=flag, recompute_cmp_o=flag)
        core = fn.NSACore(cfg)
        qd, kd, vd, wd = [t.cuda().clone().requires_grad_(True) for t in (q, k, v, w)]
        o = core(qd, kd, vd, wd, cu_d)
        (o.float() * do.cuda().float()).sum().backward()
        res.append((o, qd.grad, wd.grad))
    (o0, dq0, dw0), (o1, dq1, dw1) = res
    assert torch.equal(o0, o1) and torch.equal(dw0, dw1)
    # the selected branch adds its dq with bf16 reductions in global memory, whose order is not fixed from run to run
    assert (dq0.float() - dq1.float()).abs().max().item() <= 2e-2 * max(1.0, dq0.float().abs().max().item())


@pytest.mark.parametrize("name", ["seq320_g4_d64", "seq200_g16_d128"])
def test_against_reference_golden_grads(name):
    g = load_golden(name)
    p = golden_params(g)
    cu = [0, p["T"]]
    _setup(cu)
    step = int(g["row_step"])
    from flash_nsa.ops import mean_pooling, compress_attn, select_attn, fused_sigmoid_combine
    do = g["do"].cuda().float()
    qd, kd, vd = [g[n].cuda().clone().requires_grad_(True) for n in ("q", "k", "v")]
    o, _ = compress_attn(qd, mean_pooling(kd), mean_pooling(vd))
    (o.float() * do).sum().backward()
    _check("cmp dq", qd.grad[::step], g["cmp_dq"])
    _check("cmp dk", kd.grad, g["cmp_dk"])
    _check("cmp dv", vd.grad, g["cmp_dv"])
    ref_topk = torch.from_numpy(g["topk_sorted"].astype(np.int32))
    ref_topk = torch.where(ref_topk < 0, torch.full_like(ref_topk, O.cdiv(p["T"], 64)), ref_topk).contiguous()
    qd, kd, vd = [g[n].cuda().clone().requires_grad_(True) for n in ("q", "k", "v")]
    o = select_attn(qd, kd, vd, ref_topk.cuda())
    (o.float() * do).sum().backward()
    _check("slc dq", qd.grad[::step], g["slc_dq"])
    _check("slc dk", kd.grad, g["slc_dk"])
    _check("slc dv", vd.grad, g["slc_dv"])


def test_compress_weight_grads_accumulate_into_main_grad():
    """With a trainer-provided fp32 `main_grad` on the compression weights (Megatron's gradient-accumulation fusion) the
    weight gradients are added into it and autograd gets a placeholder; the sums equal the plain .grad of a second run."""
    lens = [600, 333]
    QH, KH, D = 8, 2, 64
    q, k, v, w, do, cu = _mk(lens, QH, KH, D, seed=31)
    fn = _setup(cu)
    cfg = fn.NSAConfig(head_dim=D, num_heads=QH, num_kv_heads=KH, cmp_k_method="linear", cmp_v_method="swiglu")
    cu_d = torch.tensor(cu, dtype=torch.int32, device="cuda")
    g = torch.Generator().manual_seed(4)
    res = {}
    for mode in ("plain", "main_grad"):
        core = fn.NSACore(cfg)
        g.manual_seed(4)
        for prm in (core.cmp_k_weight, core.cmp_v_weight):
            prm.data = (torch.randn(prm.shape, generator=g) * 0.02).bfloat16().cuda()
            if mode == "main_grad":
                prm.main_grad = torch.full(prm.shape, 0.5, dtype=torch.float32, device="cuda")
                prm.grad_added_to_main_grad = False
        qd, kd, vd, wd = [t.cuda().clone().requires_grad_(True) for t in (q, k, v, w)]
        o = core(qd, kd, vd, wd, cu_d)
        o.backward(do.cuda())
        if mode == "plain":
            res[mode] = [core.cmp_k_weight.grad.float(), core.cmp_v_weight.grad.float()]
        else:
            assert core.cmp_k_weight.grad_added_to_main_grad and core.cmp_v_weight.grad_added_to_main_grad
            res[mode] = [core.cmp_k_weight.main_grad - 0.5, core.cmp_v_weight.main_grad - 0.5]
    for a, b in zip(res["plain"], res["main_grad"]):
        scale = max(1.0, a.abs().max().item())
        assert (a - b).abs().max().item() <= 1e-2 * scale


@pytest.mark.parametrize("rows,n_out,n_in", [(1000, 128, 2048), (16380, 256, 4096), (63, 128, 128), (4096 * 5 + 17, 128, 4096)])
def test_weight_gradient_accumulate_gemm(rows, n_out, n_in):
    """main_grad += dY^T X in one launch (the fused-accumulate GEMM behind weight_grad) against an fp32 matmul of the same
    bf16 operands, on top of a non-zero buffer, for row counts that are not multiples of the 64-row k-step or of the
    split over CTAs; a strided (column-sliced) dY is taken as it is."""
    from flash_nsa.modules.megatron_level_nsa import wgrad_accum
    g = torch.Generator().manual_seed(rows + n_out)
    wide = torch.randn(rows, n_out + 64, generator=g).bfloat16().cuda()
    dy = wide[:, 64:]                                   # row stride n_out + 64, 16-byte aligned start
    x = torch.randn(rows, n_in, generator=g).bfloat16().cuda()
    acc = torch.full((n_out, n_in), 0.25, dtype=torch.float32, device="cuda")
    assert wgrad_accum(x, dy, acc)
    ref = 0.25 + dy.float().t() @ x.float()
    err = (acc - ref).abs().max().item()
    assert err <= 2e-3 * max(1.0, ref.abs().max().item()), err
    assert wgrad_accum(x, dy, acc)                      # a second call adds again
    assert (acc - (2 * ref - 0.25)).abs().max().item() <= 4e-3 * max(1.0, ref.abs().max().item())
    # shapes the kernel does not take are reported, not mangled
    assert not wgrad_accum(x, dy[:, :64], torch.zeros(64, n_in, device="cuda"))
