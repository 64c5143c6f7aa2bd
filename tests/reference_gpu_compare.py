"""This build against the reference's own GPU kernels on the same inputs (run by hand, or through
tests/test_gpu_reference_triton.py).

Both packages are called `flash_nsa`, so each side runs in a process of its own:
    python tests/reference_gpu_compare.py            -> runs both sides and prints the comparison as one JSON line
    python tests/reference_gpu_compare.py side <ref|ours> <out.pt>
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
    torch.save({"o": o.detach().float().cpu(), "dq": q.grad.float().cpu(), "dk": k.grad.float().cpu(), "dv": v.grad.float().cpu(),
                "dw": w.grad.float().cpu()}, out_path)


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
    for name in ("o", "dq", "dk", "dv", "dw"):
        a, b = res["ours"][name], res["ref"][name]
        err = (a - b).abs()
        out[name] = {"max_abs_diff": err.max().item(), "max_abs_ref": b.abs().max().item(),
                     "frac_over_2e-2": (err > 2e-2 * max(1.0, b.abs().max().item())).float().mean().item()}
    return out


if __name__ == "__main__":
    if len(sys.argv) >= 4 and sys.argv[1] == "side":
        run_side(sys.argv[2], sys.argv[3])
    else:
        print(json.dumps(compare()))
