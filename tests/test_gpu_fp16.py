"""IEEE-half tensors (the reference's ops take fp16 as well as bf16, test.py:14): the second build of the kernel library
(the same sources with the 16-bit element type switched) behind the same Python entry points, against the fp32 oracle on
the same half-rounded inputs.  Tolerances as for bf16 (half has three more mantissa bits, so these pass with room)."""
import pytest
import torch

from oracle import nsa_oracle as O
import test_gpu_backward as TB
import test_gpu_inference as TI

pytestmark = pytest.mark.gpu
TOL = 2e-2


def _half(*ts):
    return [t.float().half() for t in ts]


@pytest.mark.parametrize("QH,KH,D,methods", [(8, 2, 64, ("mean", "mean")), (32, 2, 128, ("linear", "sigmoid-mul")), (16, 4, 128, ("mean", "mean"))])
def test_nsa_core_forward_backward_in_half(QH, KH, D, methods):
    lens = [700, 333, 64]
    q, k, v, w, do, cu = TB._mk(lens, QH, KH, D, seed=23)
    q, k, v, w, do = _half(q, k, v, w, do)
    fn = TB._setup(cu)
    cfg = fn.NSAConfig(head_dim=D, num_heads=QH, num_kv_heads=KH, cmp_k_method=methods[0], cmp_v_method=methods[1])
    core = fn.NSACore(cfg).half()
    g = torch.Generator().manual_seed(3)
    wk = wv = None
    if core.cmp_k_weight is not None:
        wk = (torch.randn(core.cmp_k_weight.shape, generator=g) * 0.02).half()
        core.cmp_k_weight.data = wk.cuda()
    if core.cmp_v_weight is not None:
        wv = (torch.randn(core.cmp_v_weight.shape, generator=g) * 0.02).half()
        core.cmp_v_weight.data = wv.cuda()
    qd, kd, vd, wd = [t.cuda().clone().requires_grad_(True) for t in (q, k, v, w)]
    o = core(qd, kd, vd, wd, torch.tensor(cu, dtype=torch.int32, device="cuda"))
    assert o.dtype == torch.float16
    topk_gpu = o.grad_fn.saved_tensors[-1].cpu()
    (o.float() * do.cuda().float()).sum().backward()
    assert qd.grad.dtype == torch.float16

    qr, kr, vr, wr = TB._leaf(q, k, v, w)
    wkr = wk.float().requires_grad_(True) if wk is not None else None
    wvr = wv.float().requires_grad_(True) if wv is not None else None
    o_ref, parts = O.nsa_forward(qr, kr, vr, wr, cu, cmp_k_method=methods[0], cmp_v_method=methods[1], cmp_k_weight=wkr,
                                 cmp_v_weight=wvr, quant="fp16_cubed", topk=topk_gpu, return_parts=True)
    (o_ref * do.float()).sum().backward()
    differing = 0
    for b in range(len(lens)):
        for t in range(lens[b]):
            nv = min(16, t // 64 + 1)
            for kh in range(KH):
                differing += int(set(topk_gpu[kh, cu[b] + t, :nv].tolist()) != set(parts["topk"][kh, cu[b] + t, :nv].tolist()))
    assert differing <= max(2, KH * cu[-1] // 50), differing

    def bulk(name, got, ref):
        err = (got.float().cpu() - ref.float()).abs()
        assert torch.isfinite(got).all(), name
        assert err.max().item() <= TOL * max(1.0, ref.abs().max().item()), f"{name}: max err {err.max().item():.4g}"

    bulk("o", o, o_ref)
    bulk("dq", qd.grad, qr.grad)
    bulk("dk", kd.grad, kr.grad)
    bulk("dv", vd.grad, vr.grad)
    bulk("dw", wd.grad, wr.grad)


def test_paged_prefill_and_decode_in_half():
    """nsa_prefill of three prompts and one nsa_decode step (the one-launch kernel, here as clusters: the page table is
    4K tokens wide) on half caches."""
    from flash_nsa import nsa_prefill, nsa_decode
    QH, KH, D = 16, 4, 128
    lens = [4100, 1000, 70]
    B = len(lens)
    seqs = TI._seqs(lens, QH, KH, D, seed=41)
    for s in seqs:
        for key in s:
            s[key] = s[key].float().half()
    cache = TI.Cache(lens, KH, D, seed=14)
    cache.k, cache.v = cache.k.half(), cache.v.half()
    end = [L - 1 for L in lens]
    for b, s in enumerate(seqs):
        cache.store(b, s["k"][:end[b]], s["v"][:end[b]])
    cache.cuda()
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")
    y_len = [max((e - 32) // 16 + 1, 0) for e in end]
    x_cu = i32([0] + torch.tensor(end).cumsum(0).tolist())
    y_cu = i32([0] + torch.tensor(y_len).cumsum(0).tolist())
    slots = i32([cache.cmp_slot(b, j) for b in range(B) for j in range(y_len[b])])
    q = torch.cat([seqs[b]["q"][:end[b]] for b in range(B)]).cuda()
    w = torch.cat([seqs[b]["w"][:end[b]] for b in range(B)]).cuda()
    o_pre = nsa_prefill(q, cache.k, cache.v, w, x_cu, y_cu, max(end), max(y_len), i32(end), cache.block_tables, slots,
                        cache.cmp_block_tables)
    assert o_pre.dtype == torch.float16

    def oracle(s, L):   # pooled rows rounded to half, as the kernels store them
        qf, kf, vf, wf = s["q"][:L].float(), s["k"][:L].float(), s["v"][:L].float(), s["w"][:L].float()
        cu = [0, L]
        ck, cv = O.mean_pool(kf, cu).half().float(), O.mean_pool(vf, cu).half().float()
        cmp_o, lse = O.cmp_attn(qf, ck, cv, cu)
        topk = O.topk_select(O.slc_scores(qf, ck, lse, cu), cu)
        return O.combine(cmp_o, O.slc_attn(qf, kf, vf, topk, cu)[0], O.swa(qf, kf, vf, cu)[0], wf)

    refs = [oracle(seqs[b], lens[b]) for b in range(B)]
    off = 0
    for b in range(B):
        assert TI._bulk_ok(o_pre[off:off + end[b]], refs[b][:end[b]]), f"prefill of sequence {b}"
        off += end[b]
    for b, s in enumerate(seqs):     # the newest token of every sequence, then one decode step
        p = lens[b] - 1
        pg = int(cache.block_tables[b, p // TI.PAGE])
        cache.k[pg, p % TI.PAGE] = s["k"][p].cuda()
        cache.v[pg, p % TI.PAGE] = s["v"][p].cuda()
    slot = [cache.cmp_slot(b, (L - 32) // 16) if (L % 16 == 0 and L >= 32) else -1 for b, L in enumerate(lens)]
    qd = torch.stack([seqs[b]["q"][lens[b] - 1] for b in range(B)]).cuda()
    wd = torch.stack([seqs[b]["w"][lens[b] - 1] for b in range(B)]).cuda()
    o_dec = nsa_decode(qd, cache.k, cache.v, wd, i32(lens), cache.block_tables, i32(slot), cache.cmp_block_tables)
    assert o_dec.dtype == torch.float16
    for b in range(B):
        assert TI._bulk_ok(o_dec[b:b + 1], refs[b][-1:]), f"decode of sequence {b}"


def test_mixed_dtypes_are_refused():
    from flash_nsa.ops import compress_attn
    q, k, v, w, do, cu = TB._mk([128], 8, 2, 64, seed=1)
    TB._setup(cu)
    with pytest.raises(AssertionError):
        compress_attn(q.cuda().half(), k.cuda(), v.cuda())
