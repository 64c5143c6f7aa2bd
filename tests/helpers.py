"""Shared helpers for the parity tests."""
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load_golden(name):
    d = dict(np.load(os.path.join(GOLDEN, name + ".npz")))
    for key in ("q", "k", "v", "w", "do", "x", "h"):
        if key in d:
            d[key] = torch.from_numpy(d[key].view(np.int16).copy()).view(torch.bfloat16)
    return d


def golden_params(d):
    T, QH, KH, D, ks, st, bs, top_n, ni, nl = [int(x) for x in d["shape"]]
    return dict(T=T, QH=QH, KH=KH, D=D, ks=ks, st=st, bs=bs, top_n=top_n, ni=ni, nl=nl)


def sorted_valid(topk, ignore):
    """Sort each row with the ignore entries mapped to -1 (they come first)."""
    t = topk.clone().long()
    t[t == ignore] = -1
    return torch.sort(t, -1)[0]


def topk_mismatch_report(idx_a, idx_b, scores, cu, ignore_a, ignore_b, rel_tol):
    """Compare two selections row by row as sets.  A differing row is tolerated only if every
    swapped pair of blocks has near-equal score (relative difference <= rel_tol of the row max).
    Returns (rows_differing, rows_not_explained, total_rows)."""
    KH, T, n = idx_a.shape
    a = sorted_valid(idx_a, ignore_a)
    b = sorted_valid(idx_b, ignore_b)
    diff_rows = (a != b).any(-1).nonzero()
    bad = 0
    for kh, t in diff_rows.tolist():
        seq = max(i for i in range(len(cu) - 1) if cu[i] <= t)
        sc = scores[seq][kh, t - cu[seq]]
        sa = set(a[kh, t].tolist()) - {-1}
        sb = set(b[kh, t].tolist()) - {-1}
        only_a, only_b = sorted(sa - sb), sorted(sb - sa)
        if len(only_a) != len(only_b):
            bad += 1
            continue
        va = torch.sort(sc[only_a])[0]
        vb = torch.sort(sc[only_b])[0]
        scale = float(sc.max().abs()) + 1e-30
        if float((va - vb).abs().max()) > rel_tol * scale:
            bad += 1
    return len(diff_rows), bad, KH * T
