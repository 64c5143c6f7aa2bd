"""This build against the reference's own GPU kernels on the same inputs (run by hand, or through
tests/test_gpu_reference_triton.py).

Both packages are called `flash_nsa`, so each side runs in a process of its own:
    python tests/reference_gpu_compare.py            -> runs both sides of both cases and prints one JSON line per case
    python tests/reference_gpu_compare.py side <ref|ours> <out.pt>              (NSACore forward + backward)
    python tests/reference_gpu_compare.py inference_side <ref|ours> <out.pt>    (paged prefill + one decode step)
The reference package is the pip-installed copy under baseline/_ref (git-ignored; see bench.py --impl reference-gpu)."""
import json
import os
import subprocess
import sys
import tempfile

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LENS = [1500, 2596]          # two packed sequences, 4096 tokens
QH, KH, D = 64, 4, 128


def inputs():
    g = torch.Generator().manual_seed(4242)
    T = sum(LENS)
    mk = lambda *s: torch.randn(*s, generator=g).bfloat16()
    return mk(T, QH, D), mk(T, KH, D), mk(T, KH, D), mk(T, QH, 3), mk(T, QH, D)


def run_side(which, out_path):
    if which == "ref":
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
        import flash_nsa as pkg
        from flash_nsa.config import NSAConfig
        from flash_nsa.modules.megatron_level_nsa import NSACore
        cfg = NSAConfig()
        cfg.qk_head_dim = cfg.v_head_dim = D
        cfg.num_heads, cfg.num_kv_heads = QH, KH
    else:
        sys.path.insert(0, os.path.join(ROOT, "scalable-flash-native-sparse-attention_b200"))
        import flash_nsa as pkg
        from flash_nsa import NSAConfig, NSACore
        cfg = NSAConfig(head_dim=D, num_heads=QH, num_kv_heads=KH)
    dev = torch.device("cuda", 0)
    q, k, v, w, do = [t.to(dev) for t in inputs()]
    for t in (q, k, v, w):
        t.requires_grad_(True)
    core = NSACore(cfg).to(q) if which == "ref" else NSACore(cfg)
    cu = torch.tensor([0, LENS[0], LENS[0] + LENS[1]], dtype=torch.int32, device=dev)
    if which == "ref":
        pkg.NSAHelper.init_cu_seqlens(cu)
    o = core(q, k, v, w, cu)
    o.backward(do)
    torch.cuda.synchronize()
    # the selection itself, from the ops both packages export under the same names
    from flash_nsa.ops.compress_kv import mean_pooling_fwd
    from flash_nsa.ops.compress_attn import cmp_attn_fwd
    from flash_nsa.ops.topk import slc_topk_indices
    pkg.NSAHelper.init_cu_seqlens(cu)
    with torch.no_grad():
        ck, cv = mean_pooling_fwd(k), mean_pooling_fwd(v)
        _, lse = cmp_attn_fwd(q, ck, cv)
        res = slc_topk_indices(q, ck, lse, maybe_efficient_version=True)
    topk = res[0] if isinstance(res, (tuple, list)) else res
    torch.cuda.synchronize()
    torch.save({"o": o.detach().float().cpu(), "dq": q.grad.float().cpu(), "dk": k.grad.float().cpu(), "dv": v.grad.float().cpu(),
                "dw": w.grad.float().cpu(), "topk": topk.to(torch.int64).cpu()}, out_path)


INF_LENS = [700, 1025, 3000]      # contexts of the paged case (prompt = all but the last token, then one decode step)
INF_PAGE = 256     # the reference's window branch over a paged cache (flash-attn) needs pages of a multiple of 256 rows


def run_inference_side(which, out_path):
    """Paged prefill of the prompts and one decode step on caches built from the same seed on both sides."""
    sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref") if which == "ref" else os.path.join(ROOT, "scalable-flash-native-sparse-attention_b200"))
    from flash_nsa.inference import nsa_prefill, nsa_decode
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import test_gpu_inference as TI                  # plain torch helpers (a toy block manager, seeded sequences)
    TI.PAGE = INF_PAGE
    Cache, _seqs = TI.Cache, TI._seqs
    lens, B = INF_LENS, len(INF_LENS)
    seqs = _seqs(lens, QH, KH, D, seed=77)
    cache = Cache([L + 1 for L in lens], KH, D, seed=5)
    end = [L - 1 for L in lens]
    for b, s_ in enumerate(seqs):
        cache.store(b, s_["k"][:end[b]], s_["v"][:end[b]])
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
    for b, s_ in enumerate(seqs):
        p = lens[b] - 1
        pg = int(cache.block_tables[b, p // INF_PAGE])
        cache.k[pg, p % INF_PAGE] = s_["k"][p].cuda()
        cache.v[pg, p % INF_PAGE] = s_["v"][p].cuda()
    slot = [cache.cmp_slot(b, (L - 32) // 16) if (L % 16 == 0 and L >= 32) else -1 for b, L in enumerate(lens)]
    qd = torch.stack([seqs[b]["q"][lens[b] - 1] for b in range(B)]).cuda()
    wd = torch.stack([seqs[b]["w"][lens[b] - 1] for b in range(B)]).cuda()
    o_dec = nsa_decode(qd, cache.k, cache.v, wd, i32(lens), cache.block_tables, i32(slot), cache.cmp_block_tables)
    torch.cuda.synchronize()
    torch.save({"prefill": o_pre.float().cpu(), "decode": o_dec.float().cpu()}, out_path)


def _both(mode, names):
    if not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "flash_nsa")):
        return {"unavailable": "baseline/_ref/flash_nsa is not present"}
    with tempfile.TemporaryDirectory() as tmp:
        res = {}
        for which in ("ref", "ours"):
            path = os.path.join(tmp, which + ".pt")
            r = subprocess.run([sys.executable, os.path.abspath(__file__), mode, which, path], capture_output=True, text=True)
            if r.returncode != 0:
                return {"unavailable": f"{which} side failed: " + (r.stderr.strip().splitlines() or ["?"])[-1][:300]}
            res[which] = torch.load(path)
    out = {}
    for name in names:
        a, b = res["ours"][name], res["ref"][name]
        err = (a - b).abs()
        out[name] = {"max_abs_diff": err.max().item(), "max_abs_ref": b.abs().max().item(),
                     "frac_over_2e-2": (err > 2e-2 * max(1.0, b.abs().max().item())).float().mean().item()}
    return out


def compare_inference():
    out = _both("inference_side", ("prefill", "decode"))
    out.update({"contexts": INF_LENS, "page": INF_PAGE, "heads": [QH, KH, D]})
    return out


def compare():
    if not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "flash_nsa")):
        return {"unavailable": "baseline/_ref/flash_nsa is not present"}
    with tempfile.TemporaryDirectory() as tmp:
        res = {}
        for which in ("ref", "ours"):
            path = os.path.join(tmp, which + ".pt")
            r = subprocess.run([sys.executable, os.path.abspath(__file__), "side", which, path], capture_output=True, text=True)
            if r.returncode != 0:
                return {"unavailable": f"{which} side failed: " + (r.stderr.strip().splitlines() or ["?"])[-1][:300]}
            res[which] = torch.load(path)
    out = {"tokens": sum(LENS), "lens": LENS, "heads": [QH, KH, D]}
    # selections as sets of the valid entries (blocks 0 .. the token's own block) of every (kv head, token) row
    ta, tb = res["ours"]["topk"], res["ref"]["topk"]
    pos = torch.cat([torch.arange(L) for L in LENS])
    nk = (pos // 64).view(1, -1, 1)
    n_blk = int(nk.max()) + 1
    def member(t):      # [kh, rows, n_blk] membership of the valid entries
        valid = (t >= 0) & (t <= nk)
        m = torch.zeros(t.shape[0], t.shape[1], n_blk + 1, dtype=torch.bool)
        m.scatter_(2, torch.where(valid, t, torch.full_like(t, n_blk)), True)
        return m[..., :n_blk]
    sym = (member(ta) ^ member(tb)).sum(-1)          # size of the symmetric difference per (kv head, token) row
    out["topk"] = {"rows": int(sym.numel()), "rows_with_a_different_set": int((sym > 0).sum()),
                   "fraction": (sym > 0).float().mean().item(), "largest_symmetric_difference": int(sym.max())}
    for name in ("o", "dq", "dk", "dv", "dw"):
        a, b = res["ours"][name], res["ref"][name]
        err = (a - b).abs()
        out[name] = {"max_abs_diff": err.max().item(), "max_abs_ref": b.abs().max().item(),
                     "frac_over_2e-2": (err > 2e-2 * max(1.0, b.abs().max().item())).float().mean().item()}
    return out


if __name__ == "__main__":
    if len(sys.argv) >= 4 and sys.argv[1] == "side":
        run_side(sys.argv[2], sys.argv[3])
    elif len(sys.argv) >= 4 and sys.argv[1] == "inference_side":
        run_inference_side(sys.argv[2], sys.argv[3])
    else:
        print(json.dumps(compare()))
        print(json.dumps(compare_inference()))
