"""Rotary embedding op and the two demo layers (HFNSA, NSA) against the oracle composite.

Tolerances: rope is one rounding per element (<= 2^-8 relative on bf16 values); the layers chain projections, rope, the NSA
core and the output projection, compared with the usual 2e-2 * max(1, max|ref|) bound on 99.5 % of the elements (the block
selection can flip near-ties)."""
import pytest
import torch

from oracle import nsa_oracle as O

pytestmark = pytest.mark.gpu


def _cos_sin(b, s, d, seed):
    g = torch.Generator().manual_seed(seed)
    pos = torch.arange(s, dtype=torch.float32)[None, :, None].expand(b, s, 1)
    inv = 1.0 / (10000 ** (torch.arange(0, d // 2, dtype=torch.float32) / (d // 2)))
    ang = pos * inv[None, None, :] + torch.rand(b, 1, 1, generator=g)
    emb = torch.cat([ang, ang], -1)
    return emb.cos().bfloat16(), emb.sin().bfloat16()


@pytest.mark.parametrize("b,s,qh,kh,d,inplace", [(2, 333, 8, 2, 64, False), (1, 1025, 16, 1, 128, True), (3, 7, 4, 4, 192, False)])
def test_rope_forward_backward(b, s, qh, kh, d, inplace):
    from flash_nsa.ops import fused_apply_rope
    g = torch.Generator().manual_seed(11)
    q = torch.randn(b, s, qh, d, generator=g).bfloat16()
    k = torch.randn(b, s, kh, d, generator=g).bfloat16()
    dqe = torch.randn(b, s, qh, d, generator=g).bfloat16()
    dke = torch.randn(b, s, kh, d, generator=g).bfloat16()
    cos, sin = _cos_sin(b, s, d, 3)
    qr, kr = q.float().requires_grad_(True), k.float().requires_grad_(True)
    qe_ref, ke_ref = O.rope(qr, cos.float(), sin.float()), O.rope(kr, cos.float(), sin.float())
    ((qe_ref * dqe.float()).sum() + (ke_ref * dke.float()).sum()).backward()
    qd, kd = q.cuda().requires_grad_(True), k.cuda().requires_grad_(True)
    qin, kin = (qd * 1, kd * 1) if inplace else (qd, kd)      # in place needs non-leaf inputs
    qe, ke = fused_apply_rope(qin, kin, cos.cuda(), sin.cuda(), inplace=inplace)
    if inplace:
        assert qe.data_ptr() == qin.data_ptr() and ke.data_ptr() == kin.data_ptr()
    ((qe.float() * dqe.cuda().float()).sum() + (ke.float() * dke.cuda().float()).sum()).backward()
    for name, got, ref in (("qe", qe, qe_ref), ("ke", ke, ke_ref), ("dq", qd.grad, qr.grad), ("dk", kd.grad, kr.grad)):
        err = (got.float().cpu() - ref.detach()).abs().max().item()
        assert err <= 2 ** -7 * max(1.0, ref.abs().max().item()), (name, err)


def _ref_layer(x, cos, sin, wq, wk, wv, ww, wo, cu, cfg):
    """fp32 composite: projections, rope, oracle NSA forward, output projection.  x [b,s,hidden]."""
    b, s, _ = x.shape
    q = (x @ wq.t()).view(b, s, cfg.num_heads, cfg.qk_head_dim)
    k = (x @ wk.t()).view(b, s, cfg.num_kv_heads, cfg.qk_head_dim)
    v = (x @ wv.t()).view(b, s, cfg.num_kv_heads, cfg.v_head_dim)
    w = (x @ ww.t()).view(b, s, cfg.num_heads, 3)
    q, k = O.rope(q, cos, sin), O.rope(k, cos, sin)
    o = O.nsa_forward(q.flatten(0, 1), k.flatten(0, 1), v.flatten(0, 1), w.flatten(0, 1), cu, quant="fp16_cubed")
    return o.view(b, s, -1) @ wo.t()


def _bulk(name, got, ref, frac=0.995, tol=2e-2):
    err = (got.float().cpu() - ref.float()).abs().flatten()
    scale = max(1.0, ref.abs().max().item())
    kth = err.kthvalue(max(1, int(frac * err.numel()))).values.item()
    assert kth <= tol * scale, f"{name}: {kth:.4g} > {tol * scale:.4g}"
    assert torch.isfinite(got).all(), name


def test_hfnsa_layer_matches_composite():
    import flash_nsa
    from flash_nsa import NSAHelper
    NSAHelper.reset_context_parallel()
    b, s, hidden = 2, 640, 256
    cfg = flash_nsa.NSAConfig(hidden_size=hidden, head_dim=64, num_heads=8, num_kv_heads=2)
    torch.manual_seed(21)
    layer = flash_nsa.HFNSA(cfg).cuda().bfloat16()
    x = (torch.randn(b, s, hidden) * 0.5).bfloat16()
    cos, sin = _cos_sin(b, s, 64, 5)
    dy = torch.randn(b, s, hidden).bfloat16()
    xd = x.cuda().requires_grad_(True)
    y = layer(xd, (cos.cuda(), sin.cuda()))
    y.backward(dy.cuda())
    ws = [p.detach().float().cpu().requires_grad_(True) for p in (layer.q_proj.weight, layer.k_proj.weight, layer.v_proj.weight,
                                                                  layer.combine_proj.weight, layer.o_proj.weight)]
    xr = x.float().requires_grad_(True)
    y_ref = _ref_layer(xr, cos.float(), sin.float(), *ws, [0, s, 2 * s], cfg)
    (y_ref * dy.float()).sum().backward()
    _bulk("y", y, y_ref.detach())
    _bulk("dx", xd.grad, xr.grad)
    _bulk("dWq", layer.q_proj.weight.grad, ws[0].grad)
    _bulk("dWo", layer.o_proj.weight.grad, ws[4].grad)


def test_nsa_layer_matches_composite():
    import flash_nsa
    from flash_nsa import NSAHelper
    NSAHelper.reset_context_parallel()
    b, s, hidden = 1, 900, 256
    cfg = flash_nsa.NSAConfig(hidden_size=hidden, head_dim=64, num_heads=8, num_kv_heads=2)
    torch.manual_seed(22)
    layer = flash_nsa.NSA(cfg).cuda().bfloat16()
    x = (torch.randn(s, b, hidden) * 0.5).bfloat16()                       # sequence first
    cos, sin = _cos_sin(b, s, 64, 6)
    cu = torch.tensor([0, 400, s], dtype=torch.int32, device="cuda")
    y = layer(x.cuda(), (cos.cuda(), sin.cuda()), {"cu_seqlens": cu})
    W = layer.qkvw_proj.weight.detach().float().cpu()
    sq, sk, sv, sw, _ = layer.split_size
    wq, wk, wv, ww = W[:sq], W[sq:sq + sk], W[sq + sk:sq + sk + sv], W[sq + sk + sv:sq + sk + sv + sw]
    y_ref = _ref_layer(x.float().transpose(0, 1), cos.float(), sin.float(), wq, wk, wv, ww,
                       layer.o_proj.weight.detach().float().cpu(), [0, 400, s], cfg).transpose(0, 1)
    assert y.shape == (s, b, hidden)
    _bulk("y", y, y_ref)
