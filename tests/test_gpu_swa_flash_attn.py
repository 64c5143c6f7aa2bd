"""Pins the sliding-window branch to the reference's own arithmetic for it.

The reference computes this branch with flash-attn: `flash_attn_varlen_func(..., causal=True, window_size=(window, -1))`
(flash_nsa/ops/sliding_window_attention.py:26-39, 73-95).  flash-attn is a third-party dependency of the reference, not
part of its tree; where the package is installed next to this build, the same call on the same bf16 inputs is the
reference result for the branch.  Checked against it, on one GPU: this build's window kernels (output and q/k/v
gradients, max abs error <= 2e-2 * max(1, max|ref|)) on a packed batch with sequences shorter than, equal to and far
longer than the window, and the CPU oracle's `swa` (which every other window test is judged by).
Skipped when flash-attn cannot be imported or has no kernel for this GPU."""
import pytest
import torch

from oracle import nsa_oracle as O

pytestmark = pytest.mark.gpu
TOL = 2e-2
WINDOW = 512


def _flash(q, k, v, cu, max_len, do=None):
    try:
        from flash_attn import flash_attn_varlen_func
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"flash-attn is not importable here: {e}")
    q, k, v = [t.detach().clone().requires_grad_(True) for t in (q, k, v)]
    try:
        o = flash_attn_varlen_func(q, k, v, cu, cu, max_len, max_len, causal=True, window_size=(WINDOW, -1))
        if do is not None:
            o.backward(do)
        torch.cuda.synchronize()
    except RuntimeError as e:
        pytest.skip(f"flash-attn has no kernel that runs on this GPU: {str(e)[:200]}")
    return o.detach(), q.grad, k.grad, v.grad


def _mk(lens, QH, KH, D, seed):
    g = torch.Generator().manual_seed(seed)
    T = sum(lens)
    cu = [0]
    for L in lens:
        cu.append(cu[-1] + L)
    mk = lambda *s: torch.randn(*s, generator=g).bfloat16()
    return mk(T, QH, D), mk(T, KH, D), mk(T, KH, D), mk(T, QH, D), cu


def _close(name, got, ref):
    got, ref = got.float().cpu(), ref.float().cpu()
    err = (got - ref).abs().max().item()
    bound = TOL * max(1.0, ref.abs().max().item())
    assert err <= bound, f"{name}: max err {err:.4g} > {bound:.4g}"


@pytest.mark.parametrize("QH,KH,D", [(16, 4, 128), (8, 2, 64)])
def test_window_kernels_match_flash_attn(QH, KH, D):
    from flash_nsa import NSAHelper
    from flash_nsa.ops import swa_varlen_func
    lens = [100, 513, 512, 700, 8192, 1]
    q, k, v, do, cu = _mk(lens, QH, KH, D, seed=41 + D)
    cu_d = torch.tensor(cu, dtype=torch.int32, device="cuda")
    qd, kd, vd, dod = [t.cuda() for t in (q, k, v, do)]
    o_ref, dq_ref, dk_ref, dv_ref = _flash(qd, kd, vd, cu_d, max(lens), dod)
    NSAHelper.reset_context_parallel()
    NSAHelper.set_hyperparameters(window_size=WINDOW)
    NSAHelper.init_cu_seqlens(cu_d)
    leaves = [t.clone().requires_grad_(True) for t in (qd, kd, vd)]
    o = swa_varlen_func(*leaves)
    o.backward(dod)
    _close("o", o, o_ref)
    _close("dq", leaves[0].grad, dq_ref)
    _close("dk", leaves[1].grad, dk_ref)
    _close("dv", leaves[2].grad, dv_ref)


def test_oracle_window_branch_matches_flash_attn():
    """The oracle's restatement of the window mask (keys t-window .. t, 513 keys) against flash-attn itself: outputs and
    gradients of the fp32 oracle on the bf16 inputs agree with flash-attn's bf16 result within the bf16 tolerance."""
    QH, KH, D = 8, 2, 64
    lens = [100, 513, 700, 2048, 1]
    q, k, v, do, cu = _mk(lens, QH, KH, D, seed=7)
    cu_d = torch.tensor(cu, dtype=torch.int32, device="cuda")
    o_ref, dq_ref, dk_ref, dv_ref = _flash(q.cuda(), k.cuda(), v.cuda(), cu_d, max(lens), do.cuda())
    leaves = [t.float().requires_grad_(True) for t in (q, k, v)]
    o, _ = O.swa(*leaves, cu, window=WINDOW)
    (o * do.float()).sum().backward()
    _close("oracle o", o.detach(), o_ref)
    _close("oracle dq", leaves[0].grad, dq_ref)
    _close("oracle dk", leaves[1].grad, dk_ref)
    _close("oracle dv", leaves[2].grad, dv_ref)
    # and the mask itself, exactly: with V = position the window's first key shows through a one-hot-like softmax
    T = 600
    qz = torch.zeros(T, 1, 64)
    pos = torch.arange(T, dtype=torch.float32).view(T, 1, 1).expand(T, 1, 64).contiguous()
    oz, _ = O.swa(qz, torch.zeros(T, 1, 64), pos, [0, T], window=WINDOW)       # uniform weights over the visible keys
    want = torch.tensor([(max(0, t - WINDOW) + t) / 2 for t in range(T)])
    assert (oz[:, 0, 0] - want).abs().max().item() <= 1e-3
