"""The CPU oracle against vectors produced by the reference's own torch code (tests/golden)."""
import numpy as np
import pytest
import torch

from oracle import nsa_oracle as O
from helpers import load_golden, golden_params, sorted_valid

CASES = ["seq320_g4_d64", "seq200_g16_d128", "seq1100_g2_d64", "c0_2048_g4_d64"]


def _close(a, b, tol):
    a = torch.as_tensor(a).double()
    b = torch.as_tensor(b).double()
    assert a.shape == b.shape
    err = (a - b).abs().max().item()
    assert err <= tol * max(1.0, b.abs().max().item()), err


@pytest.mark.parametrize("name", CASES)
def test_forward_ops(name):
    g = load_golden(name)
    p = golden_params(g)
    cu = [0, p["T"]]
    step = int(g["row_step"])
    q, k, v = g["q"].double(), g["k"].double(), g["v"].double()
    ck = O.mean_pool(k, cu, p["ks"], p["st"])
    cv = O.mean_pool(v, cu, p["ks"], p["st"])
    _close(ck, g["ck"], 1e-6)
    _close(cv, g["cv"], 1e-6)
    if "blk_k" in g:
        _close(O.construct_block(k, cu, p["ks"], p["st"]), g["blk_k"], 0)
    cmp_o, lse = O.cmp_attn(q, ck, cv, cu, p["ks"], p["st"])
    _close(cmp_o[::step], g["cmp_o"], 2e-6)
    sc = O.slc_scores(q, ck, lse, cu, p["ks"], p["st"], p["bs"])
    topk = O.topk_select(sc, cu, p["top_n"], p["ni"], p["nl"], p["bs"])
    ours = sorted_valid(topk, O.cdiv(p["T"], p["bs"]))
    ref = torch.sort(torch.from_numpy(g["topk_sorted"].astype(np.int64)), -1)[0]   # -1 (= unused slot) first
    assert torch.equal(ours, ref), (ours != ref).any(-1).sum()
    slc_o, _ = O.slc_attn(q, k, v, topk, cu, p["bs"])
    _close(slc_o[::step], g["slc_o"], 2e-6)


@pytest.mark.parametrize("name", CASES[:2])
def test_backward_ops(name):
    g = load_golden(name)
    p = golden_params(g)
    cu = [0, p["T"]]
    step = int(g["row_step"])
    q, k, v, do = [g[n].double().requires_grad_(True) for n in ("q", "k", "v", "do")]
    ck = O.mean_pool(k, cu, p["ks"], p["st"])
    cv = O.mean_pool(v, cu, p["ks"], p["st"])
    cmp_o, lse = O.cmp_attn(q, ck, cv, cu, p["ks"], p["st"])
    (cmp_o * do).sum().backward()
    _close(q.grad[::step], g["cmp_dq"], 2e-6)
    _close(k.grad, g["cmp_dk"], 2e-6)
    _close(v.grad, g["cmp_dv"], 2e-6)
    q.grad = k.grad = v.grad = None
    with torch.no_grad():
        topk = O.topk_select(O.slc_scores(q, ck, lse, cu), cu)
    slc_o, _ = O.slc_attn(q, k, v, topk, cu)
    (slc_o * do).sum().backward()
    _close(q.grad[::step], g["slc_dq"], 2e-6)
    _close(k.grad, g["slc_dk"], 2e-6)
    _close(v.grad, g["slc_dv"], 2e-6)
    if "comb_o" in g:
        w = g["w"].double().requires_grad_(True)
        a, b = cmp_o.detach().requires_grad_(True), slc_o.detach().requires_grad_(True)
        c = (cmp_o * 0.5 - slc_o).detach().requires_grad_(True)
        y = O.combine(a, b, c, w)
        (y * do).sum().backward()
        _close(y, g["comb_o"], 2e-6)
        _close(a.grad, g["comb_da"], 2e-6)
        _close(c.grad, g["comb_dc"], 2e-6)
        _close(w.grad, g["comb_dw"], 2e-6)


def test_misc():
    g = load_golden("misc")
    x, h = g["x"].double(), g["h"].double()
    _close(O.reorder(x, 4, "shuffle"), g["shuffle4"], 0)
    _close(O.reorder(x, 4, "unshuffle"), g["unshuffle4"], 0)
    _close(O.reorder(x, 2, "shuffle"), g["shuffle2"], 0)
    _close(O.act(h, "swiglu"), g["swiglu"], 1e-6)
    _close(O.act(h, "sigmoid-mul"), g["sigmoid_mul"], 1e-6)


def test_varlen_equals_per_sequence():
    """Packed call == per-sequence calls concatenated, including lengths < 32 and odd lengths."""
    gen = torch.Generator().manual_seed(5)
    lens = [17, 32, 47, 48, 130, 1]
    cu = [0]
    for L in lens:
        cu.append(cu[-1] + L)
    T = cu[-1]
    q = torch.randn(T, 4, 32, generator=gen)
    k = torch.randn(T, 2, 32, generator=gen)
    v = torch.randn(T, 2, 32, generator=gen)
    w = torch.randn(T, 4, 3, generator=gen)
    full = O.nsa_forward(q, k, v, w, cu, top_n=4)
    parts = [O.nsa_forward(q[cu[i]:cu[i + 1]], k[cu[i]:cu[i + 1]], v[cu[i]:cu[i + 1]], w[cu[i]:cu[i + 1]],
                           [0, lens[i]], top_n=4) for i in range(len(lens))]
    assert torch.allclose(full, torch.cat(parts), atol=1e-6)
    assert torch.isfinite(full).all()


def test_cp_metadata_matches_reference_rule():
    """Piece table of flash_nsa/utils.py:19-46 on a hand-checked case."""
    cu = [0, 10, 24, 32]
    m = O.cp_metadata(cu, rank=1, world_size=2, cp_mode=2)
    # chunks of 8: rank 1 owns [8,16) and [16,24)
    assert m["ranges"] == [(8, 16), (16, 24)]
    assert m["cp_cu_seqlens"] == [0, 2, 8, 16]
    assert m["cp_batch_idx"] == [0, 1, 1]
    assert m["cp_offset"] == [8, 0, 6]
    assert m["atomic_add_dkdv"] is True
    m1 = O.cp_metadata(cu, rank=0, world_size=2, cp_mode=1)
    assert m1["cp_cu_seqlens"] == [0, 10, 16] and m1["cp_offset"] == [0, 0]


def test_row_subset_matches_full_oracle():
    """nsa_forward_rows (the checker used on full-size inputs) against nsa_forward on a small varlen case: outputs,
    selections and the gradients of a loss that only involves the sampled rows."""
    import torch
    from oracle import nsa_oracle as O
    torch.manual_seed(5)
    lens = [700, 130, 333]
    cu = [0, 700, 830, 1163]
    T, QH, KH, D = cu[-1], 8, 2, 64
    mk = lambda *s: torch.randn(*s, dtype=torch.float64)
    q, k, v, w = mk(T, QH, D), mk(T, KH, D), mk(T, KH, D), mk(T, QH, 3)
    rows = sorted({0, 30, 31, 32, 63, 64, 65, 511, 512, 513, 699, 700, 731, 829, 830, 900, 1162})
    do = mk(len(rows), QH, D)
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v, w)]
    o_full, parts_full = O.nsa_forward(*leaves, cu, return_parts=True)
    (o_full[rows] * do).sum().backward()
    g_full = [t.grad.clone() for t in leaves]
    leaves2 = [t.clone().requires_grad_(True) for t in (q, k, v, w)]
    o_rows, parts = O.nsa_forward_rows(*leaves2, cu, rows)
    (o_rows * do).sum().backward()
    assert torch.equal(parts["topk"], parts_full["topk"][:, rows])
    assert torch.allclose(o_rows, o_full[rows], atol=1e-10, rtol=1e-10)
    for a, b in zip(g_full, [t.grad for t in leaves2]):
        assert torch.allclose(a, b, atol=1e-9, rtol=1e-9)
    # a selection passed in replaces the oracle's own: its own selection (unused slots as -1) reproduces the output, a
    # different one moves only the selected branch; block scores come back per sequence
    tk = parts["topk"].clone()
    tk[tk == O.cdiv(700, 64)] = -1
    o_same, p2 = O.nsa_forward_rows(q, k, v, w, cu, rows, topk=tk)
    assert torch.equal(o_same, o_rows.detach())
    assert [tuple(s.shape) for s in p2["scores"]] == [(KH, 11, 11), (KH, 3, 3), (KH, 3, 6)]
    tk2 = tk.clone()
    r699 = rows.index(699)
    tk2[:, r699, 5] = tk2[:, r699, 4]                      # one block fewer for the row of token 699
    o_less, _ = O.nsa_forward_rows(q, k, v, w, cu, rows, topk=tk2)
    changed = (o_less != o_same).flatten(1).any(1)
    assert changed.nonzero().flatten().tolist() == [r699]
