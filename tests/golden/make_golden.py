"""Generate the golden vectors under tests/golden/ from the reference's own torch code.

Run once, in a container that has the reference checkout:

    python tests/golden/make_golden.py /path/to/reference

It loads flash_nsa/ops/torch_ref.py BY FILE PATH (the package itself needs a GPU to import),
feeds it seeded inputs whose values are exactly representable in bfloat16, and stores inputs
(as bf16 bit patterns) plus the reference outputs (fp32) in .npz files.  The reference functions
run in float64 so that autograd works through torch_cmp_attn (its in-place masking breaks the
fp32 graph); their softmax is still the reference's fp32 softmax.
"""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_ref(root):
    path = os.path.join(root, "flash_nsa", "ops", "torch_ref.py")
    spec = importlib.util.spec_from_file_location("nsa_torch_ref", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def bf16_vals(*shape, gen, scale=1.0):
    x = (torch.randn(*shape, generator=gen) * scale).to(torch.bfloat16)
    return x


def bits(x_bf16):
    return x_bf16.view(torch.int16).numpy().view(np.uint16)


def f32(x):
    return x.detach().to(torch.float32).numpy()


def make_case(ref, name, T, QH, KH, D, seed, rows_keep=None, with_grads=True,
              ks=32, st=16, bs=64, top_n=16, ni=1, nl=2):
    g = torch.Generator().manual_seed(seed)
    q16, k16, v16 = bf16_vals(T, QH, D, gen=g), bf16_vals(T, KH, D, gen=g), bf16_vals(T, KH, D, gen=g)
    w16 = bf16_vals(T, QH, 3, gen=g)
    do16 = bf16_vals(T, QH, D, gen=g)
    q, k, v, w, do = [t.double().requires_grad_(with_grads) for t in (q16, k16, v16, w16, do16)]
    out = dict(q=bits(q16), k=bits(k16), v=bits(v16), w=bits(w16), do=bits(do16),
               shape=np.array([T, QH, KH, D, ks, st, bs, top_n, ni, nl]))

    blk_k = ref.torch_construct_block(k, ks, st)          # [Y,H,ks,D]
    ck, cv = blk_k.mean(-2), ref.torch_construct_block(v, ks, st).mean(-2)
    cmp_o = ref.torch_cmp_attn(q, ck, cv, ks, st)
    topk = ref.torch_topk(q.detach(), ck.detach(), ks, st, bs, top_n, ni, nl)
    slc_o = ref.torch_slc_attn(q, k, v, topk, bs)
    sel = slice(None) if rows_keep is None else slice(0, T, rows_keep)
    out.update(ck=f32(ck), cv=f32(cv), cmp_o=f32(cmp_o[sel]), slc_o=f32(slc_o[sel]),
               topk_sorted=(lambda ts: torch.where(ts > 30000, -1, ts))(torch.sort(topk, -1)[0]).numpy().astype(np.int16),
               row_step=np.array(rows_keep or 1))
    if rows_keep is None:
        out["blk_k"] = f32(blk_k)
    # (sorted ignore entries of torch_topk, 99999999, are stored as -1)
    if with_grads:
        (cmp_o * do).sum().backward()
        out.update(cmp_dq=f32(q.grad[sel]), cmp_dk=f32(k.grad), cmp_dv=f32(v.grad))
        q.grad = k.grad = v.grad = None
        (slc_o * do).sum().backward()
        out.update(slc_dq=f32(q.grad[sel]), slc_dk=f32(k.grad), slc_dv=f32(v.grad))
        q.grad = k.grad = v.grad = None
        a, b, c = [t.detach().clone().requires_grad_(True) for t in (cmp_o, slc_o, cmp_o * 0.5 - slc_o)]
        y = ref.torch_sigmoid_combine(a, b, c, w)
        (y * do).sum().backward()
        if rows_keep is None:
            out.update(comb_o=f32(y), comb_da=f32(a.grad), comb_dc=f32(c.grad), comb_dw=f32(w.grad))
    if not with_grads:
        out.pop("do")
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print(name, {kk: vv.shape for kk, vv in out.items()})


def make_misc(ref):
    g = torch.Generator().manual_seed(7)
    x16 = bf16_vals(96, 2, 16, gen=g)
    h16 = bf16_vals(40, 3, 32, gen=g)
    x = x16.double()
    h = h16.double()
    out = dict(x=bits(x16), h=bits(h16),
               shuffle4=f32(ref.torch_reorder(x, 4, "shuffle")), unshuffle4=f32(ref.torch_reorder(x, 4, "unshuffle")),
               shuffle2=f32(ref.torch_reorder(x, 2, "shuffle")),
               swiglu=f32(ref.torch_swiglu(h)), sigmoid_mul=f32(ref.torch_sigmoid_mul(h)))
    np.savez_compressed(os.path.join(HERE, "misc.npz"), **out)
    print("misc ok")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py /path/to/reference")
    root = sys.argv[1]
    ref = load_ref(root)
    torch.set_num_threads(8)
    make_case(ref, "seq320_g4_d64", T=320, QH=4, KH=1, D=64, seed=11)
    make_case(ref, "seq200_g16_d128", T=200, QH=16, KH=1, D=128, seed=12, rows_keep=4)
    make_case(ref, "seq1100_g2_d64", T=1100, QH=4, KH=2, D=64, seed=13, rows_keep=5, with_grads=False)
    make_case(ref, "c0_2048_g4_d64", T=2048, QH=8, KH=2, D=64, seed=1000, rows_keep=16, with_grads=False)
    make_misc(ref)
