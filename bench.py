"""Benchmark of the NSA hot path: forward + backward of one NSA layer (NSACore) on packed bf16 inputs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|reference-gpu]

N = 1 : BASELINE config 1 -- one causal sequence of 65 536 tokens, 64 q heads / 4 kv heads / d = 128.
N > 1 : (launched with torchrun) BASELINE config 3 -- one causal sequence of N * 131 072 tokens, sharded
        with the zig-zag layout (cp_mode = 2), K/V all-gathered per kv head over NCCL; weak scaling.  Before
        anything is timed every rank checks the sharded NSACore against the unsharded one (`cp_check`).
--impl reference : the reference's CPU path (its torch restatement in oracle/) timed on the host cores on a
        bounded sample of the same workload.
--impl reference-gpu : the reference package itself (its Triton kernels, installed under baseline/_ref, which is not part
        of this repository's history) on this GPU at config 1, or a line that says why it did not run.  One GPU.

Prints ONE JSON line (rank 0).  Inputs are seeded N(0,1) synthetic tensors, as in the reference's own
benchmarks; there is no dataset on this path.  Every timed region is followed by a check of the kernels'
status word: a pipeline wait that gave up makes the run exit non-zero instead of printing a number.
"""
import argparse
import json
import os
import random
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG_PARENT = os.path.join(ROOT, "scalable-flash-native-sparse-attention_b200")

import numpy as np
import torch

QH, KH, D = 64, 4, 128
H800_TOKENS_PER_S = 65536 / 0.10785   # the reference's published fwd+bwd at 64K on one H800 (34.162 + 73.689 ms)
TOL = 2e-2


def _use_this_build():
    for p in (ROOT, PKG_PARENT):
        if p not in sys.path:
            sys.path.insert(0, p)


# ----------------------------------------------------------------------------------------------- work model
def pair_counts(lens, ks=32, st=16, bs=64, top_n=16, window=512, first=0):
    """(query, key) pairs per q head of each branch, causal-exact; `first` = position of the first query row of every
    sequence (a prefill chunk starts at its prefix length)."""
    cmp_p = slc_p = swa_p = 0
    for L in lens:
        t = np.arange(first, L, dtype=np.int64)
        Y = max((L - ks) // st + 1, 0)
        cmp_p += int(np.where(t >= ks - 1, np.minimum((t - (ks - 1)) // st + 1, Y), 0).sum())
        nk = t // bs
        slc_p += int(((np.minimum(top_n, nk + 1) - 1) * bs + (t % bs) + 1).sum())
        swa_p += int(np.minimum(t + 1, window + 1).sum())
    return cmp_p, slc_p, swa_p


def flops_model(lens, qh=QH, d=D, first=0):
    c, s, w = pair_counts(lens, first=first)
    f = lambda pairs, mm: 2.0 * d * mm * pairs * qh
    return {
        "cmp_fwd": f(c, 2), "topk": f(c, 1), "slc_fwd": f(s, 2), "swa_fwd": f(w, 2),
        "cmp_bwd": f(c, 5), "slc_bwd": f(s, 5), "swa_bwd": f(w, 5),
        # what the two backward kernels of a dense branch execute (S and dP are recomputed in both)
        "cmp_dkdv": f(c, 4), "cmp_dq": f(c, 3), "slc_dkdv": f(s, 4), "slc_dq": f(s, 3), "swa_dkdv": f(w, 4), "swa_dq": f(w, 3),
    }


ALG_KEYS = ("cmp_fwd", "topk", "slc_fwd", "swa_fwd", "cmp_bwd", "slc_bwd", "swa_bwd")


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d.get("bf16_tflops", 1590.0), d.get("hbm_gbs", 6650.0), "measured"
    return 1590.0, 6650.0, "fallback"


def load_traffic():
    """DRAM read + write bytes per launch from the ncu captures summarised under profiles/ (one small JSON beside the .md
    files): {kernel: {"tokens": captured size, "dram_bytes": read+write, "scaling": "linear", "source": "profiles/x.md"}}."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    try:
        with open(path) as f:
            return json.load(f)
    except (OSError, ValueError):
        return {}


# ----------------------------------------------------------------------------------------------- clocks
class ClockSampler:
    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.lines, self.proc = [], None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        rows = [l.split(", ") for ts, l in self.lines if t0 <= ts <= t1 + 0.3] or [l.split(", ") for _, l in self.lines]
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
                for n, v in zip(names, r[2:6]):
                    if v.strip().lower().startswith("active"):
                        reasons.add(n)
            except (ValueError, IndexError):
                continue
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------------------------- reference arm / CPU baseline
def _cpu_model():
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("model name"):
                    return line.split(":", 1)[1].strip()
    except OSError:
        pass
    return "unknown"


def cpu_reference(steps, warmup, threads=None):
    """The reference's torch path (oracle restatement) on the host: forward + backward, fp32, on a bounded sample
    of the headline workload: the benchmark's head configuration (64 q heads / 4 kv heads / d = 128) on one causal sequence
    of 2048 tokens, because that code needs O(heads * T^2) memory and cannot hold 65 536 tokens.  Per-token cost
    grows with the sequence length, so the full-length CPU figure would be lower still."""
    _use_this_build()
    from oracle import nsa_oracle as O
    threads = threads or os.cpu_count()
    torch.set_num_threads(threads)
    T, qh, kh, d = 2048, QH, KH, D
    g = torch.Generator().manual_seed(1000)
    q, k, v = [torch.randn(T, h, d, generator=g, requires_grad=True) for h in (qh, kh, kh)]
    w = torch.randn(T, qh, 3, generator=g, requires_grad=True)
    do = torch.randn(T, qh, d, generator=g)

    def step():
        o = O.nsa_forward(q, k, v, w, [0, T])
        (o * do).sum().backward()
        q.grad = k.grad = v.grad = w.grad = None

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    return {"value": T / dt, "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": f"fwd+bwd of one causal sequence T={T} (not 65536), {qh} q heads / {kh} kv heads, d={d}, fp32 torch on CPU",
            "ms_per_step": dt * 1e3, "steps": steps, "warmup": warmup}


def cpu_config0(reps=5):
    """BASELINE config 0 exactly: the reference's torch path (oracle restatement), FORWARD, one causal sequence T = 2048,
    8 q heads / 2 kv heads / d = 64, fp32, seeded N(0,1) inputs; median of `reps` runs after one warm-up, with one thread
    and with every host core."""
    _use_this_build()
    from oracle import nsa_oracle as O
    T, qh, kh, d = 2048, 8, 2, 64
    g = torch.Generator().manual_seed(1000)
    q, k, v = [torch.randn(T, h, d, generator=g) for h in (qh, kh, kh)]
    w = torch.randn(T, qh, 3, generator=g)
    ms = {}
    all_cores = os.cpu_count()
    with torch.no_grad():
        for n in (1, all_cores):
            torch.set_num_threads(n)
            O.nsa_forward(q, k, v, w, [0, T])
            ts = []
            for _ in range(reps):
                t0 = time.perf_counter()
                O.nsa_forward(q, k, v, w, [0, T])
                ts.append(time.perf_counter() - t0)
            ms[n] = float(np.median(ts)) * 1e3
    torch.set_num_threads(all_cores)
    return {"value": T / (ms[all_cores] * 1e-3), "unit": "tokens/s", "cores": all_cores, "kind": "port",
            "sample": f"BASELINE config 0: forward of one causal sequence T={T}, {qh} q heads / {kh} kv heads, d={d}, fp32 torch "
                      f"on CPU, median of {reps} after 1 warm-up",
            "ms_forward_all_cores": ms[all_cores], "ms_forward_1_thread": ms[1],
            "tokens_per_s_1_thread": T / (ms[1] * 1e-3), "cpu_model": _cpu_model()}


def reference_gpu_arm(args):
    """The reference package's own NSACore (Triton kernels + flash-attn for the window branch) on THIS GPU at config 1,
    timed with CUDA events like the arm of this build; prints its line or why it did not run."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    line = {"impl": "reference-gpu", "metric": "nsa_fwd_bwd_throughput", "unit": "tokens/s", "n_gpus": 1, "higher_is_better": True,
            "dtype": "bf16", "data": "synthetic"}

    def unavailable(why):
        line["unavailable"] = why[:400]
        print(json.dumps(line))

    if not os.path.isdir(os.path.join(ref_dir, "flash_nsa")):
        return unavailable("baseline/_ref/flash_nsa is not present (the reference install does not travel with the repository)")
    sys.path.insert(0, ref_dir)
    try:
        import flash_nsa as ref
        from flash_nsa.config import NSAConfig
        from flash_nsa.modules.megatron_level_nsa import NSACore
        assert os.path.realpath(ref.__file__).startswith(os.path.realpath(ref_dir))
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(dev)
        times = {}
        for T in (4096, args.tokens_per_gpu or 65536):
            g = torch.Generator().manual_seed(1001)
            mk = lambda *s: torch.randn(*s, generator=g).bfloat16().to(dev)
            q, k, v, w, do = mk(T, QH, D), mk(T, KH, D), mk(T, KH, D), mk(T, QH, 3), mk(T, QH, D)
            for t in (q, k, v, w):
                t.requires_grad_(True)
            cfg = NSAConfig()
            cfg.qk_head_dim = cfg.v_head_dim = D
            cfg.num_heads, cfg.num_kv_heads = QH, KH
            core = NSACore(cfg).to(q)
            cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
            ref.NSAHelper.init_cu_seqlens(cu)

            def fwd():
                return core(q, k, v, w, cu)

            def step():
                o = fwd()
                o.backward(do)
                q.grad = k.grad = v.grad = w.grad = None

            for _ in range(max(args.warmup, 3)):
                step()
            torch.cuda.synchronize()
            e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            n = max(1, args.steps)
            e[0].record()
            for _ in range(n):
                step()
            e[1].record()
            with torch.no_grad():
                for _ in range(n):
                    fwd()
            e[2].record()
            torch.cuda.synchronize()
            times[T] = (e[0].elapsed_time(e[1]) / n, e[1].elapsed_time(e[2]) / n)
        T = max(times)
        ms, ms_fwd = times[T]
        line.update({"value": T / (ms * 1e-3), "steps": max(1, args.steps), "warmup": max(args.warmup, 3), "ms_per_step": ms,
                     "ms_forward": ms_fwd, "ms_backward": ms - ms_fwd, "ms_per_step_4k": times[4096][0],
                     "config": {"workload": f"reference NSACore fwd+bwd, one causal sequence of {T} tokens, {QH}/{KH}/{D}", "tokens": T},
                     "versions": {"triton": __import__("triton").__version__, "torch": torch.__version__}})
        try:
            line["decode"] = reference_gpu_decode(dev)
        except Exception as e:  # noqa: BLE001
            line["decode"] = {"unavailable": f"{type(e).__name__}: {(str(e).strip().splitlines() or [''])[0]}"[:300]}
        print(json.dumps(line))
    except BaseException as e:  # noqa: BLE001  (an import error, a JIT failure, an unsupported op: all are "did not run")
        if isinstance(e, KeyboardInterrupt):
            raise
        unavailable(f"{type(e).__name__}: {str(e).strip().splitlines()[0] if str(e).strip() else ''}")


def reference_gpu_decode(dev):
    """The reference's own nsa_decode on the shapes of config 4 (batch 64, contexts U[4096, 8192] with seed 1004, 32 q / 8 kv
    heads, d = 128, page 256, shuffled page tables), of its 4 GiB sweep at 8K, 64K and 128K tokens and of one sequence of 32K /
    128K tokens; caches filled with seeded
    N(0,1) values (the timing does not depend on them), eager and replayed from a CUDA graph."""
    from flash_nsa.inference import nsa_decode

    def timed(fn, n):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / n

    def case(ctx, qh, kh, d, page, seed):
        rng = random.Random(seed)
        B = len(ctx)
        n_tok = [-(-L // page) for L in ctx]
        n_cmp = [-(-max((L - 32) // 16 + 1, 1) // page) for L in ctx]
        total = sum(n_tok) + sum(n_cmp)
        free = list(range(total))
        rng.shuffle(free)
        g = torch.Generator(device=dev).manual_seed(seed)
        kc = torch.randn(total, page, kh, d, device=dev, dtype=torch.bfloat16, generator=g)
        vc = torch.randn(total, page, kh, d, device=dev, dtype=torch.bfloat16, generator=g)
        bt = torch.full((B, max(n_tok)), -1, dtype=torch.int32)
        cbt = torch.full((B, max(n_cmp)), -1, dtype=torch.int32)
        for b in range(B):
            for i in range(n_tok[b]):
                bt[b, i] = free.pop()
            for i in range(n_cmp[b]):
                cbt[b, i] = free.pop()
        q = torch.randn(B, qh, d, device=dev, dtype=torch.bfloat16, generator=g)
        w = torch.randn(B, qh, 3, device=dev, dtype=torch.bfloat16, generator=g)
        args = (q, kc, vc, w, torch.tensor(ctx, dtype=torch.int32, device=dev), bt.to(dev),
                torch.full((B,), -1, dtype=torch.int32, device=dev), cbt.to(dev))
        out = {"ms_eager": timed(lambda: nsa_decode(*args), 20)}
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                nsa_decode(*args)
            out["ms_cuda_graph"] = timed(graph.replay, 50)
        except Exception as e:  # noqa: BLE001
            out["cuda_graph"] = f"not captured: {type(e).__name__}"
        return out

    def prefill_case(prefix, chunk, qh, kh, d, page):
        """The chunked-prefill step of config 4: `chunk` new tokens of one sequence on a `prefix`-token context, K/V of all
        of them already in the (seeded N(0,1)) cache, the compressed rows of the chunk written by the step."""
        from flash_nsa.inference import nsa_prefill
        L1 = prefix + chunk
        ylen = (L1 - 32) // 16 + 1
        n_tok, n_cmp = -(-L1 // page), -(-ylen // page)
        g = torch.Generator(device=dev).manual_seed(prefix)
        kc = torch.randn(n_tok + n_cmp, page, kh, d, device=dev, dtype=torch.bfloat16, generator=g)
        vc = torch.randn(n_tok + n_cmp, page, kh, d, device=dev, dtype=torch.bfloat16, generator=g)
        perm = torch.randperm(n_tok + n_cmp, generator=torch.Generator().manual_seed(prefix)).to(torch.int32)
        bt, cbt = perm[:n_tok].view(1, -1).to(dev), perm[n_tok:].view(1, -1).to(dev)
        slots = [int(perm[n_tok + j // page]) * page + j % page if 16 * j + 31 >= prefix else -1 for j in range(ylen)]
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
        q = torch.randn(chunk, qh, d, device=dev, dtype=torch.bfloat16, generator=g)
        w = torch.randn(chunk, qh, 3, device=dev, dtype=torch.bfloat16, generator=g)
        args = (q, kc, vc, w, i32([0, chunk]), i32([0, ylen]), chunk, ylen, i32([L1]), bt, i32(slots), cbt)
        out = {"ms_eager": timed(lambda: nsa_prefill(*args), 20)}
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                nsa_prefill(*args)
            out["ms_cuda_graph"] = timed(graph.replay, 50)
        except Exception as e:  # noqa: BLE001
            out["cuda_graph"] = f"not captured: {type(e).__name__}"
        return out

    rng = random.Random(1004)
    res = {"config4": case([rng.randint(4096, 8192) for _ in range(64)], 32, 8, 128, 256, 1004)}
    for L in (8192, 65536, 131072):
        res[f"sweep_4gib_{L}"] = case([L] * (1024 * 2048 // L), 64, 4, 128, 256, L)
    for L in (32768, 131072):   # one long sequence: what the reference's split-count arguments are for
        res[f"one_sequence_{L}"] = case([L], 64, 4, 128, 256, L + 1)
    try:
        res["config4_prefill_chunk"] = prefill_case(6144, 2048, 32, 8, 128, 256)
    except Exception as e:  # noqa: BLE001
        res["config4_prefill_chunk"] = {"unavailable": f"{type(e).__name__}: {(str(e).strip().splitlines() or [''])[0]}"[:300]}
    return res


# ----------------------------------------------------------------------------------------------- context-parallel parity check
def cp_check(pg, rank, world):
    """Sharded NSACore (forward + backward over NCCL) against the unsharded NSACore on the same global batch, on every rank:
    both shard layouts, kv_head_stride 1 and 2, packed batches of <= 4K tokens.  Returns {"ok", "max_err", "cases"}; the
    error is relative to the 3e-2 * max(1, max|reference|) bound of the NCCL test (dq tiles are cut differently at shard
    boundaries and dk/dv are summed in another order)."""
    import torch.distributed as dist
    import flash_nsa
    from flash_nsa import NSAHelper
    from flash_nsa.get_batch import split_for_cp_rank
    from flash_nsa.ops._common import check_status
    qh, kh, d = 16, 4, 128
    worst, ok, cases = 0.0, True, 0
    unit = 2 * world * 64
    for mode, lens, stride in ((2, [unit * 2], 1), (1, [unit // 2, unit, unit // 2], 2), (2, [unit + unit // 2, unit // 2], 1),
                               (1, [unit * 2], 1), (2, [unit * 4], 2)):
        g = torch.Generator().manual_seed(100 + mode + len(lens) + stride)
        T = sum(lens)
        cu = [0]
        for L in lens:
            cu.append(cu[-1] + L)
        mk = lambda *s: torch.randn(*s, generator=g).bfloat16().cuda()
        q, k, v, w, do = mk(T, qh, d), mk(T, kh, d), mk(T, kh, d), mk(T, qh, 3), mk(T, qh, d)
        cu_d = torch.tensor(cu, dtype=torch.int32, device="cuda")
        NSAHelper.reset_context_parallel()
        cfg = flash_nsa.NSAConfig(head_dim=d, num_heads=qh, num_kv_heads=kh, cp_mode=mode, kv_head_stride=stride)
        ref_core = flash_nsa.NSACore(cfg)
        leaves = [t.clone().requires_grad_(True) for t in (q, k, v, w)]
        o_ref = ref_core(*leaves, cu_d)
        o_ref.backward(do)
        ref = [o_ref] + [t.grad for t in leaves]
        core = flash_nsa.NSACore(cfg, process_group=pg)
        shard = lambda t: split_for_cp_rank(t, world, rank, mode, dim=0)
        loc = [shard(t).clone().requires_grad_(True) for t in (q, k, v, w)]
        o = core(*loc, cu_d, cp_mode=mode)
        o.backward(shard(do))
        got = [o] + [t.grad for t in loc]
        for name, a, b in zip(("o", "dq", "dk", "dv", "dw"), got, ref):
            b = shard(b.detach())
            err = (a.float() - b.float()).abs().max().item()
            rel = err / (3e-2 * max(1.0, b.float().abs().max().item()))
            worst = max(worst, rel)
            if not (rel <= 1.0):
                ok = False
                print(f"[cp_check] rank {rank} mode {mode} lens {lens} stride {stride}: {name} err {err:.4g} ({rel:.2f} x bound)",
                      file=sys.stderr, flush=True)
        cases += 1
        NSAHelper.reset_context_parallel()
    check_status()
    flag = torch.tensor([1.0 if ok else 0.0, -worst], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=pg)
    return {"ok": bool(flag[0].item() == 1.0), "max_err_over_bound": float(-flag[1].item()), "cases": cases,
            "bound": "3e-2 * max(1, max|unsharded|)", "compared": "o, dq, dk, dv, dw of every rank's shard"}


# ----------------------------------------------------------------------------------------------- GPU arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--tokens-per-gpu", type=int, default=0)
    ap.add_argument("--no-kernel-breakdown", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end pass (profiling runs)")
    ap.add_argument("--no-inference", action="store_true", help="skip the paged decode / chunked prefill measurement")
    ap.add_argument("--no-decode-sweep", action="store_true", help="inference part: config 4 only (profiling runs)")
    ap.add_argument("--no-extras", action="store_true", help="N > 1: skip the strong-scaling and no-recompute side measurements")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        if rank != 0:
            return
        n_steps, n_warm = max(1, min(args.steps, 10)), max(1, min(args.warmup, 2))   # ~3 s per step: bounded to about half a minute
        r = cpu_reference(n_steps, n_warm)
        line = {"impl": "reference", "metric": "nsa_fwd_bwd_throughput", "value": r["value"], "unit": "tokens/s", "n_gpus": args.gpus,
                "steps": n_steps, "warmup": n_warm, "steps_requested": args.steps, "warmup_requested": args.warmup,
                "ms_per_step": r["ms_per_step"], "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": r["sample"]},
                "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
                "e2e": {"value": r["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return
    if args.impl == "reference-gpu":
        if rank == 0:
            reference_gpu_arm(args)
        return

    _use_this_build()
    import flash_nsa
    from flash_nsa import NSAHelper, _lib
    import torch.distributed as dist
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    pg = None
    cp_ok = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        pg = dist.group.WORLD
        cp_ok = cp_check(pg, rank, world)
        if not cp_ok["ok"]:
            if rank == 0:
                print(json.dumps({"metric": "nsa_fwd_bwd_throughput", "n_gpus": world, "cp_check": cp_ok,
                                  "error": "the sharded NSACore does not reproduce the unsharded one; nothing was timed"}))
            dist.destroy_process_group()
            sys.exit(1)
    per_gpu = args.tokens_per_gpu or (65536 if world == 1 else 131072)
    T_total = per_gpu * world
    # Nothing is recomputed in backward at any N: at 131 072 tokens per GPU the saved branch outputs are 6.6 GB of the 180 GB.
    # (The reference's 1M-token run sets all four recompute flags, test_cp.py:511-514, on 80 GB parts: that variant of the
    # step is timed beside it as `recompute_all`.)
    recompute = False
    peak_tf, peak_gbs, peak_src = load_peaks()

    def make_core(recompute_all):
        NSAHelper.reset_context_parallel()
        cfg = flash_nsa.NSAConfig(head_dim=D, num_heads=QH, num_kv_heads=KH, cp_mode=2, kv_head_stride=1,
                                  recompute_cmp_kv=recompute_all, recompute_cmp_o=recompute_all, recompute_slc_o=recompute_all,
                                  recompute_swa_o=recompute_all)
        return flash_nsa.NSACore(cfg, process_group=pg)

    core = make_core(recompute)
    cu_host = np.array([0, T_total], dtype=np.int64)
    cu = torch.tensor(cu_host, dtype=torch.int32, device=dev)

    gen = torch.Generator().manual_seed(1001 + rank)
    host = {name: torch.randn(per_gpu, h, dd, generator=gen).bfloat16().pin_memory()
            for name, h, dd in (("q", QH, D), ("k", KH, D), ("v", KH, D), ("w", QH, 3), ("do", QH, D))}
    q, k, v, w, do = [host[n].to(dev, non_blocking=True) for n in ("q", "k", "v", "w", "do")]
    for t in (q, k, v, w):
        t.requires_grad_(True)

    def run_step(core_, cu_, cu_host_, tensors):
        q_, k_, v_, w_, do_ = tensors
        o = core_(q_, k_, v_, w_, cu_, cu_seqlens_np=cu_host_, cp_mode=2)
        o.backward(do_)
        grads = (q_.grad, k_.grad, v_.grad, w_.grad)
        q_.grad = k_.grad = v_.grad = w_.grad = None
        return o, grads

    def step():
        return run_step(core, cu, cu_host, (q, k, v, w, do))

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        tt = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return tt.item()

    def status_ok(where):
        """Exit non-zero if a kernel of the region just timed reported that a pipeline wait gave up."""
        try:
            flash_nsa.check_status()
        except _lib.NsaError as e:
            print(f"[bench] {where}: {e}", file=sys.stderr, flush=True)
            sys.exit(3)

    def timed(fn, n_steps, n_warm):
        for _ in range(n_warm):
            fn()
        sync_all()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n_steps):
            fn()
        b.record()
        sync_all()
        return max_over_ranks(a.elapsed_time(b) / n_steps)

    for _ in range(args.warmup):
        step()
    sync_all()
    status_ok("warm-up")
    sampler = ClockSampler(local_rank) if rank == 0 else None
    n0 = _lib.launch_count
    t_wall0 = time.time()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    sync_all()
    t_wall1 = time.time()
    launches = (_lib.launch_count - n0) // max(args.steps, 1)
    ms = max_over_ranks(e0.elapsed_time(e1) / args.steps)
    clocks = sampler.stop(t_wall0, t_wall1) if sampler else None
    status_ok("timed steps")

    # ---- end to end: pinned host inputs -> device, the step, results -> pinned host
    out_host = {n: torch.empty_like(host[n]).pin_memory() for n in ("q", "k", "v", "w")}
    o_host = torch.empty(per_gpu, QH, D, dtype=torch.bfloat16).pin_memory()

    # Two device input sets and three streams: while step i computes, the inputs of step i+1 come in over PCIe and the
    # results of step i-1 go out (full duplex), as a training loop that prefetches its next batch does.  Every step
    # still copies all of its inputs from pinned host memory and all of its results back.
    names = ("q", "k", "v", "w", "do")
    sets = [dict(zip(names, (q, k, v, w, do)))]
    sets.append({n: torch.empty_like(t).requires_grad_(n != "do") for n, t in sets[0].items()})
    s_in, s_out, s_main = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_used = [torch.cuda.Event() for _ in range(2)]

    def fetch(i):   # inputs of step i -> set i & 1
        b = i & 1
        s_in.wait_event(ev_used[b])
        with torch.cuda.stream(s_in):
            for n in names:
                sets[b][n].data.copy_(host[n], non_blocking=True)
            ev_in[b].record(s_in)

    def e2e_loop(n_steps):
        for b in range(2):
            ev_used[b].record(s_main)
        fetch(0)
        for i in range(n_steps):
            b = i & 1
            if i + 1 < n_steps:
                fetch(i + 1)
            s_main.wait_event(ev_in[b])
            cur = sets[b]
            o = core(cur["q"], cur["k"], cur["v"], cur["w"], cu, cu_seqlens_np=cu_host, cp_mode=2)
            o.backward(cur["do"])
            grads = [cur[n].grad for n in ("q", "k", "v", "w")]
            for n in ("q", "k", "v", "w"):
                cur[n].grad = None
            ev_used[b].record(s_main)
            s_out.wait_event(ev_used[b])
            with torch.cuda.stream(s_out):
                o_host.copy_(o.detach(), non_blocking=True)
                for n, gt in zip(("q", "k", "v", "w"), grads):
                    out_host[n].copy_(gt, non_blocking=True)
            for t in [o] + grads:
                t.record_stream(s_out)
        s_main.wait_stream(s_out)

    # enough steps to amortise the un-hidden first copy-in / last copy-out (42 ms each at 64K over PCIe): 96 short steps on one
    # GPU (5 s), 16 of the long multi-GPU steps
    n_e2e = 0 if args.no_e2e else (96 if world == 1 else 16)
    if n_e2e:
        e2e_loop(2)
    sync_all()
    e0.record()
    if n_e2e:
        e2e_loop(n_e2e)
    e1.record()
    sync_all()
    ms_e2e = max_over_ranks(e0.elapsed_time(e1) / max(n_e2e, 1)) if n_e2e else float("nan")
    status_ok("end-to-end steps")
    h2d = sum(host[n].numel() * 2 for n in host)
    d2h = o_host.numel() * 2 + sum(out_host[n].numel() * 2 for n in out_host)
    del sets, out_host, o_host

    fm_total = flops_model([T_total])
    alg = sum(fm_total[n] for n in ALG_KEYS)
    # forwards that backward runs again when the recompute flags are on (the compressed-row pooling is negligible)
    executed = alg + (sum(fm_total[n] for n in ("cmp_fwd", "slc_fwd", "swa_fwd")) if recompute else 0.0)

    # ---- per-kernel timing of the dominant kernels (single GPU only), for the roofline object
    roofline, kernels = None, None
    if world == 1 and rank == 0 and not args.no_kernel_breakdown:
        kernels = kernel_breakdown(q, k, v, w, do, [T_total])
        status_ok("kernel breakdown")
        fm = flops_model([T_total])
        top = max((n for n in kernels if n in fm), key=lambda n: kernels[n])
        roofline = roofline_of(top, kernels[top], fm[top], T_total, peak_tf, peak_gbs, peak_src)

    # ---- N > 1: what one step spends where on rank 0, exposed communication, and two side measurements
    extras = {}
    if world > 1:
        extras["kernels_ms"], extras["comm_exposed_ms"] = cp_step_profile(step, sync_all)
        status_ok("profiled step")
        if not args.no_extras:
            core_ra = make_core(True)
            ms_ra = timed(lambda: run_step(core_ra, cu, cu_host, (q, k, v, w, do)), 3, 1)
            status_ok("recompute_all")
            extras["recompute_all"] = {"ms_per_step": ms_ra, "tokens_per_s": T_total / (ms_ra * 1e-3),
                                       "per_gpu_algorithmic_tflops": alg / (ms_ra * 1e-3) / 1e12 / world,
                                       "note": "the same step with the reference's four recompute flags on (the three branch forwards "
                                               "run again in backward), as in its 1M-token run on 80 GB GPUs"}
            core = make_core(recompute)
            extras["strong_128k"] = strong_scaling_128k(make_core, run_step, timed, status_ok, dev, rank, world)

    if world == 1 and not args.no_extras and not args.tokens_per_gpu:
        # the point the multi-GPU runs are set against: the 131 072-token sequence of `strong_128k`, which is also the
        # per-GPU token count of the weak-scaling runs, on this one GPU
        del q, k, v, w, do
        torch.cuda.empty_cache()
        extras["single_gpu_128k"] = single_gpu_128k(make_core, run_step, timed, status_ok, dev)
        extras["varlen_config2"] = varlen_config2(run_step, timed, status_ok, dev)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    value = T_total / (ms * 1e-3)
    flags = {n: recompute for n in ("recompute_cmp_kv", "recompute_cmp_o", "recompute_slc_o", "recompute_swa_o")}
    line = {
        "metric": "nsa_fwd_bwd_throughput", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": value / H800_TOKENS_PER_S if world == 1 else None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": (f"NSA fwd+bwd, one causal sequence of {T_total} tokens, {QH} q heads / {KH} kv heads / d={D}, "
                                f"kernel 32 stride 16 block 64 top-n 16 window 512" + ("" if world == 1 else
                                f", context parallel over {world} GPUs (zig-zag shards, {per_gpu} tokens per GPU)")),
                   "tokens": T_total, "tokens_per_gpu": per_gpu, "l2": "inputs (q alone >= 1 GiB) exceed the 126 MB L2; no explicit flush",
                   "recompute": flags, "algorithmic_tflop_per_step": alg / 1e12, "executed_tflop_per_step": executed / 1e12},
        "achieved_tflops": alg / (ms * 1e-3) / 1e12 / world,
        "per_gpu_algorithmic_tflops": alg / (ms * 1e-3) / 1e12 / world,
        "per_gpu_executed_tflops": executed / (ms * 1e-3) / 1e12 / world,
        "per_gpu_frac_of_peak": alg / (ms * 1e-3) / 1e12 / world / peak_tf, "peak_tflops": peak_tf, "peak_source": peak_src,
        "clocks": clocks, "gpu_launches": launches,
        "e2e": {"value": T_total / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": ms_e2e, "steps": n_e2e,
                "pipeline": "2 input sets, copy-in / compute / copy-out streams; first copy-in and last copy-out are inside the timed region"},
        "status_checked": True,
    }
    if cp_ok is not None:
        line["cp_check"] = cp_ok
    line.update(extras)
    if roofline:
        line["roofline"] = roofline
        line["kernels_ms"] = kernels
    if world == 1 and not args.no_inference:
        line["inference"] = inference_bench(dev, sweep=not args.no_decode_sweep)
        status_ok("inference")
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_config0()
        r = cpu_reference(3, 1)
        line["cpu_baseline_headline_sample"] = {k_: r[k_] for k_ in ("value", "unit", "cores", "kind", "sample", "ms_per_step")}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def roofline_of(name, ms, flops, tokens, peak_tf, peak_gbs, peak_src):
    """Roofline object of one kernel: algorithmic FLOP/s against the measured bf16 peak, and, when an ncu capture of its DRAM
    traffic is on file, that traffic / time against the measured copy bandwidth; `bound` names the larger fraction."""
    ach = flops / (ms * 1e-3) / 1e12
    out = {"kernel": name, "achieved": ach, "peak": peak_tf, "unit": "TFLOP/s", "frac": ach / peak_tf, "tensor_frac": ach / peak_tf,
           "peak_source": peak_src, "ms": ms, "traffic": None}
    t = load_traffic().get(name)
    bound = "tensor"
    if t:
        traffic = t["dram_bytes"] * (tokens / t["tokens"]) if t.get("scaling") == "linear" else (t["dram_bytes"] if t["tokens"] == tokens else None)
        if traffic:
            gbs = traffic / (ms * 1e-3) / 1e9
            out.update({"traffic": traffic, "traffic_source": f"{t['source']}: dram__bytes_read.sum + dram__bytes_write.sum at {t['tokens']} "
                                                              f"tokens" + (f" x {tokens}/{t['tokens']}" if tokens != t["tokens"] else ""),
                        "dram_gbs_from_traffic": gbs, "dram_frac_from_traffic": gbs / peak_gbs, "hbm_peak_gbs": peak_gbs})
            # achieved / peak / frac above are the contraction's FLOPs against the tensor roof, so `bound` stays "tensor"; the
            # DRAM side (measured traffic, not algorithmic bytes) is reported beside it and flagged when it is the busier unit
            out["dram_busier_than_tensor"] = bool(gbs / peak_gbs > ach / peak_tf)
    out["bound"] = bound
    return out


def cp_step_profile(step, sync_all):
    """One extra untimed step on rank 0's own clock: CUDA events around every op call of the context-parallel function give
    the time per kernel family, and events around every Comm.wait() give the time the compute stream stood still for a
    gather or a reduce-scatter (`comm_exposed_ms`)."""
    import flash_nsa.modules.megatron_level_nsa as M
    from flash_nsa.comm import Comm
    records = []

    def wrap(name, fn):
        def inner(*a, **kw):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = fn(*a, **kw)
            e1.record()
            records.append((name, e0, e1))
            return out
        return inner

    families = {"compress_kv_fwd": "pool_fwd", "cmp_attn_fwd": "cmp_fwd", "slc_topk_indices": "topk", "slc_attn_fwd": "slc_fwd",
                "swa_fwd": "swa_fwd", "combine_fwd": "combine_fwd", "combine_bwd": "combine_bwd", "_swa_bwd_into": "swa_bwd",
                "slc_attn_bwd": "slc_bwd_with_k2q", "cmp_attn_bwd": "cmp_bwd", "compress_kv_bwd": "pool_bwd"}
    saved = {n: getattr(M, n) for n in families}
    saved_comm = {n: getattr(Comm, n) for n in ("wait", "reduce_scatter", "grad_buffers")}
    try:
        for n, fam in families.items():
            setattr(M, n, wrap(fam, saved[n]))
        Comm.wait = wrap("comm_wait", saved_comm["wait"])
        Comm.reduce_scatter = wrap("grad_shuffle_and_issue", saved_comm["reduce_scatter"])
        Comm.grad_buffers = wrap("grad_zero_fill", saved_comm["grad_buffers"])
        sync_all()
        step()
        sync_all()
    finally:
        for n, fn in saved.items():
            setattr(M, n, fn)
        for n, fn in saved_comm.items():
            setattr(Comm, n, fn)
    out = {}
    for name, e0, e1 in records:
        out[name] = out.get(name, 0.0) + e0.elapsed_time(e1)
    exposed = out.pop("comm_wait", 0.0)
    return out, exposed


def varlen_config2(run_step, timed, status_ok, dev):
    """BASELINE config 2: four packed sequences with lengths U[4096, 8192] (seed 1002), mean K compression and sigmoid-mul V
    compression with N(0, 0.02) weights, forward + backward through NSACore on one GPU (the reference publishes no time for
    it; tests/test_gpu_fullsize.py checks the same case against the oracle)."""
    import flash_nsa
    from flash_nsa import NSAHelper
    rng = random.Random(1002)
    lens = [rng.randint(4096, 8192) for _ in range(4)]
    T = sum(lens)
    g = torch.Generator().manual_seed(1002)
    mk = lambda h, dd: torch.randn(T, h, dd, generator=g).bfloat16().to(dev)
    q, k, v, w, do = mk(QH, D), mk(KH, D), mk(KH, D), mk(QH, 3), mk(QH, D)
    for t in (q, k, v, w):
        t.requires_grad_(True)
    cu_host = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    cu = torch.tensor(cu_host, dtype=torch.int32, device=dev)
    NSAHelper.reset_context_parallel()
    cfg = flash_nsa.NSAConfig(head_dim=D, num_heads=QH, num_kv_heads=KH, cmp_k_method="mean", cmp_v_method="sigmoid-mul")
    core = flash_nsa.NSACore(cfg)
    if core.cmp_v_weight is not None:
        core.cmp_v_weight.data = (torch.randn(core.cmp_v_weight.shape, generator=g) * 0.02).bfloat16().to(dev)

    def step():
        out = run_step(core, cu, cu_host, (q, k, v, w, do))
        for prm in core.parameters():
            prm.grad = None
        return out

    ms = timed(step, 5, 3)
    status_ok("varlen_config2")
    fm = flops_model(lens)
    alg = sum(fm[n] for n in ALG_KEYS)
    NSAHelper.reset_context_parallel()
    return {"lens": lens, "tokens": T, "ms_per_step": ms, "tokens_per_s": T / (ms * 1e-3), "algorithmic_tflops": alg / (ms * 1e-3) / 1e12,
            "compression": "K mean, V sigmoid-mul (learned, N(0, 0.02) weights)"}


def single_gpu_128k(make_core, run_step, timed, status_ok, dev):
    """One causal sequence of 131 072 tokens on one GPU, no recompute: the single-GPU point of `strong_128k` (efficiency at N
    GPUs = this ms / N / that ms) and the per-GPU token count of the weak-scaling runs."""
    T = 131072
    g = torch.Generator().manual_seed(2001)
    mk = lambda h, dd: torch.randn(T, h, dd, generator=g).bfloat16().to(dev)
    q, k, v, w, do = mk(QH, D), mk(KH, D), mk(KH, D), mk(QH, 3), mk(QH, D)
    for t in (q, k, v, w):
        t.requires_grad_(True)
    cu_host = np.array([0, T], dtype=np.int64)
    cu = torch.tensor(cu_host, dtype=torch.int32, device=dev)
    core = make_core(False)
    ms_step = timed(lambda: run_step(core, cu, cu_host, (q, k, v, w, do)), 3, 2)

    def fwd_only():
        with torch.no_grad():
            core(q, k, v, w, cu, cu_seqlens_np=cu_host, cp_mode=2)

    ms_fwd = timed(fwd_only, 3, 1)
    status_ok("single_gpu_128k")
    fm = flops_model([T])
    alg = sum(fm[n] for n in ALG_KEYS)
    return {"tokens": T, "ms_fwd": ms_fwd, "ms_bwd": ms_step - ms_fwd, "ms_per_step": ms_step, "tokens_per_s": T / (ms_step * 1e-3),
            "algorithmic_tflops": alg / (ms_step * 1e-3) / 1e12,
            "reference_h800_ms": {"fwd": 101.123, "bwd": 213.904}}


def strong_scaling_128k(make_core, run_step, timed, status_ok, dev, rank, world):
    """One causal sequence of 131 072 tokens over the N GPUs of this run (zig-zag shards, kv_head_stride 4 as in the
    reference's figure imgs/cp_degrad1.png, README.md:271), no recompute: forward and backward ms, to be set against the
    single-GPU times of the same sequence divided by N (the reference publishes 90.3 % / 82.3 % on 8 x H800)."""
    import flash_nsa
    from flash_nsa import NSAHelper
    T = 131072
    per = T // world
    g = torch.Generator().manual_seed(2001 + rank)
    mk = lambda h, dd: torch.randn(per, h, dd, generator=g).bfloat16().to(dev)
    q, k, v, w, do = mk(QH, D), mk(KH, D), mk(KH, D), mk(QH, 3), mk(QH, D)
    for t in (q, k, v, w):
        t.requires_grad_(True)
    cu_host = np.array([0, T], dtype=np.int64)
    cu = torch.tensor(cu_host, dtype=torch.int32, device=dev)
    NSAHelper.reset_context_parallel()
    cfg = flash_nsa.NSAConfig(head_dim=D, num_heads=QH, num_kv_heads=KH, cp_mode=2, kv_head_stride=4)
    core = flash_nsa.NSACore(cfg, process_group=torch.distributed.group.WORLD)
    ms_step = timed(lambda: run_step(core, cu, cu_host, (q, k, v, w, do)), 5, 3)

    def fwd_only():
        with torch.no_grad():
            core(q, k, v, w, cu, cu_seqlens_np=cu_host, cp_mode=2)

    ms_fwd = timed(fwd_only, 5, 2)
    status_ok("strong_128k")
    fm = flops_model([T])
    alg = sum(fm[n] for n in ALG_KEYS)
    return {"tokens": T, "tokens_per_gpu": per, "kv_head_stride": 4, "ms_fwd": ms_fwd, "ms_bwd": ms_step - ms_fwd, "ms_per_step": ms_step,
            "per_gpu_algorithmic_tflops": alg / (ms_step * 1e-3) / 1e12 / world,
            "single_gpu_reference_point": "`single_gpu_128k` of the N=1 line (same sequence on one GPU): efficiency = that ms / N / this ms"}


# ----------------------------------------------------------------------------------------------- paged inference (config 4)
class Config4:
    """BASELINE config 4 as tensors on one GPU: a paged KV cache (page 256, randomly permuted page table, 32 q heads /
    8 kv heads / d = 128) holding 64 decode sequences with contexts U[4096, 8192] (seed 1004) and one sequence of a
    6144-token prefix plus a 2048-token chunk.  Token rows are seeded N(0,1); the compressed rows of everything that is
    already in the cache are pooled with the library's own prefill pooling op, as a serving engine would have done on the
    earlier steps.  `check_decode` / `check_prefill` compare results with the CPU oracle run on the un-paged sequences."""

    def __init__(self, dev, B=64, lo=4096, hi=8192, prefix=6144, chunk=2048, seed=1004):
        _use_this_build()
        from flash_nsa.inference import mean_pooling_prefill
        qh, kh, d, page = 32, 8, 128, 256
        self.qh, self.kh, self.d, self.page, self.B, self.dev = qh, kh, d, page, B, dev
        rng = random.Random(seed)
        self.ctx = ctx = [rng.randint(lo, hi) for _ in range(B)]
        n_tok = [-(-L // page) for L in ctx]
        y_len = lambda L: max((L - 32) // 16 + 1, 0)
        n_cmp = [-(-max(y_len(L), 1) // page) for L in ctx]
        self.P, self.Cn = prefix, chunk
        self.L1 = L1 = prefix + chunk
        pre_tok, pre_cmp = -(-L1 // page), -(-y_len(L1) // page)
        total = sum(n_tok) + sum(n_cmp) + pre_tok + pre_cmp
        free = list(range(total))
        rng.shuffle(free)
        g = torch.Generator(device=dev).manual_seed(seed)
        self.kc = torch.randn(total, page, kh, d, device=dev, dtype=torch.bfloat16, generator=g)
        self.vc = torch.randn(total, page, kh, d, device=dev, dtype=torch.bfloat16, generator=g)
        bt = torch.full((B, max(n_tok)), -1, dtype=torch.int32)
        cbt = torch.full((B, max(n_cmp)), -1, dtype=torch.int32)
        for b in range(B):
            for i in range(n_tok[b]):
                bt[b, i] = free.pop()
            for i in range(n_cmp[b]):
                cbt[b, i] = free.pop()
        self.bt_host, self.cbt_host = bt, cbt
        cslot = lambda tab, j: int(tab[j // page]) * page + j % page
        # the row this decode step completes (context a multiple of 16), written by the step itself
        self.new_row = [(L - 32) // 16 if L % 16 == 0 else -1 for L in ctx]
        self.slot = torch.tensor([cslot(cbt[b], j) if j >= 0 else -1 for b, j in enumerate(self.new_row)], dtype=torch.int32, device=dev)
        self.pbt_host = torch.tensor([[free.pop() for _ in range(pre_tok)]], dtype=torch.int32)
        self.pcbt_host = torch.tensor([[free.pop() for _ in range(pre_cmp)]], dtype=torch.int32)
        assert not free
        self.bt, self.cbt, self.pbt, self.pcbt = bt.to(dev), cbt.to(dev), self.pbt_host.to(dev), self.pcbt_host.to(dev)
        self.ctx_d = torch.tensor(ctx, dtype=torch.int32, device=dev)
        self.q = torch.randn(B, qh, d, device=dev, dtype=torch.bfloat16, generator=g)
        self.w = torch.randn(B, qh, 3, device=dev, dtype=torch.bfloat16, generator=g)
        # ---- compressed rows that earlier steps would have written: all rows whose window ends before the newest token
        y_old = [y_len(L - 1) for L in ctx] + [y_len(prefix)]
        y_cu = torch.tensor([0] + np.cumsum(y_old).tolist(), dtype=torch.int32, device=dev)
        tabs = [cbt[b] for b in range(B)] + [self.pcbt_host[0]]
        slots = torch.tensor([cslot(tabs[b], j) for b in range(B + 1) for j in range(y_old[b])], dtype=torch.int32, device=dev)
        width = max(bt.size(1), self.pbt_host.size(1))
        tok_tab = torch.full((B + 1, width), -1, dtype=torch.int32)
        tok_tab[:B, :bt.size(1)] = bt
        tok_tab[B, :self.pbt_host.size(1)] = self.pbt_host[0]
        tok_tab = tok_tab.to(dev)
        for cache in (self.kc, self.vc):
            mean_pooling_prefill(cache, y_cu, max(y_old), slot_mapping=slots, block_table=tok_tab)
        # ---- the chunked-prefill step
        self.xcu = torch.tensor([0, chunk], dtype=torch.int32, device=dev)
        self.ylen = y_len(L1)
        self.ycu = torch.tensor([0, self.ylen], dtype=torch.int32, device=dev)
        pc_host = self.pcbt_host[0].tolist()
        self.pslots_host = [cslot(pc_host, j) if 16 * j + 31 >= prefix else -1 for j in range(self.ylen)]
        self.pslots = torch.tensor(self.pslots_host, dtype=torch.int32, device=dev)
        self.qp = torch.randn(chunk, qh, d, device=dev, dtype=torch.bfloat16, generator=g)
        self.wp = torch.randn(chunk, qh, 3, device=dev, dtype=torch.bfloat16, generator=g)
        self.ctx1 = torch.tensor([L1], dtype=torch.int32, device=dev)

    # -- the two steps, through the public entry points
    def decode(self, return_topk=False):
        from flash_nsa import nsa_decode
        from flash_nsa.inference import nsa_decode_fused
        if return_topk:
            return nsa_decode_fused(self.q, self.kc, self.vc, self.w, self.ctx_d, self.bt, self.slot, self.cbt, return_topk=True)
        return nsa_decode(self.q, self.kc, self.vc, self.w, self.ctx_d, self.bt, self.slot, self.cbt)

    def prefill(self):
        from flash_nsa import nsa_prefill
        return nsa_prefill(self.qp, self.kc, self.vc, self.wp, self.xcu, self.ycu, self.Cn, self.ylen, self.ctx1, self.pbt, self.pslots,
                           self.pcbt)

    # -- checks against the oracle on the un-paged sequences
    def _unpaged(self, table_row, length):
        flat_k, flat_v = self.kc.view(-1, self.kh, self.d), self.vc.view(-1, self.kh, self.d)
        pos = torch.arange(length, device=self.dev)
        rows = table_row.to(self.dev).long()[pos // self.page] * self.page + pos % self.page
        return flat_k[rows].float().cpu(), flat_v[rows].float().cpu()

    @staticmethod
    def _same_selection(got, ref, scores, n_valid):
        """Sets equal, or the swapped blocks' oracle scores within 1e-3 of the row's largest score (tie policy of the fp32
        scoring mode: equal scores go to the lower block index; accumulation order may flip a near-tie)."""
        a, b = set(got[:n_valid].tolist()), set(ref[:n_valid].tolist())
        if a == b:
            return True
        only_a, only_b = sorted(a - b), sorted(b - a)
        if len(only_a) != len(only_b) or min(only_a) < 0 or max(only_a) >= scores.numel():
            return False
        va, vb = torch.sort(scores[only_a])[0], torch.sort(scores[only_b])[0]
        return float((va - vb).abs().max()) <= 1e-3 * (float(scores.max().abs()) + 1e-30)

    def check_decode(self, o, topk, seqs=None):
        """o [B,qh,d], topk [kh,B,16] of ONE decode step on a fresh Config4 against the oracle for the sequences `seqs`
        (default: all).  Returns the worst output error; raises AssertionError on a mismatch."""
        from oracle import nsa_oracle as O
        o, topk = o.float().cpu(), topk.cpu()
        flat_k = self.kc.view(-1, self.kh, self.d)
        worst = 0.0
        flips = 0
        for b in (range(self.B) if seqs is None else seqs):
            L = self.ctx[b]
            k, v = self._unpaged(self.bt_host[b], L)
            qx = self.q[b].float().cpu().unsqueeze(0).expand(L, self.qh, self.d)
            wx = self.w[b].float().cpu().unsqueeze(0).expand(L, self.qh, 3)
            o_ref, parts = O.nsa_forward_rows(qx, k, v, wx, [0, L], [L - 1], topk=topk[:, b:b + 1], round_cmp_to_bf16=True)
            err = (o[b] - o_ref[0]).abs().max().item()
            worst = max(worst, err)
            assert err <= TOL, f"decode sequence {b} (context {L}): output error {err:.4g} > {TOL}"
            nv = min(16, (L - 1) // 64 + 1)
            for h in range(self.kh):
                row = topk[h, b]
                assert len(set(row[:nv].tolist())) == nv and int(row[:nv].min()) >= 0 and int(row[:nv].max()) <= (L - 1) // 64
                same = self._same_selection(row, parts["topk"][h, 0], parts["scores"][0][h, 0], nv)
                assert same, f"decode sequence {b} kv head {h}: selection {sorted(row[:nv].tolist())} vs oracle {sorted(parts['topk'][h, 0, :nv].tolist())}"
                flips += int(set(row[:nv].tolist()) != set(parts["topk"][h, 0, :nv].tolist()))
            j = self.new_row[b]
            if j >= 0:        # the compressed row this step completed, written into the cache in place
                got = flat_k[int(self.slot[b])].float().cpu()
                ref = O.mean_pool(k[16 * j:16 * j + 32], [0, 32])[0]
                assert (got - ref).abs().max().item() <= 8e-3, f"decode sequence {b}: new compressed row"
        return {"max_err": worst, "near_tie_rows": flips}

    def check_prefill(self, o, n_rows=64):
        """o [chunk,qh,d] of the chunked-prefill step against the oracle on `n_rows` sampled rows of the chunk."""
        from oracle import nsa_oracle as O
        from flash_nsa.inference import cmp_attn_prefill, topk_prefill
        rng = random.Random(7)
        local = sorted({0, 1, 63, 64, 127, 128, self.Cn - 65, self.Cn - 1} | {rng.randrange(self.Cn) for _ in range(n_rows)})[:max(n_rows, 8)]
        rows = [self.P + t for t in local]
        # the selection the prefill made: its scoring op again on the same cache (deterministic)
        _, lse = cmp_attn_prefill(self.qp, self.kc, self.vc, self.xcu, self.Cn, block_tables=self.pcbt, context_lens=self.ctx1)
        topk = topk_prefill(self.qp, self.kc, lse, self.xcu, self.Cn, self.ylen, block_tables=self.pcbt, context_lens=self.ctx1)
        topk = topk[:, torch.tensor(local, device=self.dev)].cpu()
        k, v = self._unpaged(self.pbt_host[0], self.L1)
        qx = torch.zeros(self.L1, self.qh, self.d)
        wx = torch.zeros(self.L1, self.qh, 3)
        qx[self.P:], wx[self.P:] = self.qp.float().cpu(), self.wp.float().cpu()
        o_ref, parts = O.nsa_forward_rows(qx, k, v, wx, [0, self.L1], rows, topk=topk, round_cmp_to_bf16=True)
        got = o.float().cpu()[local]
        err = (got - o_ref).abs().max().item()
        assert err <= TOL, f"chunked prefill: output error {err:.4g} > {TOL} on the sampled rows"
        flips = 0
        for r, t in enumerate(rows):
            nv = min(16, t // 64 + 1)
            for h in range(self.kh):
                assert self._same_selection(topk[h, r], parts["topk"][h, r], parts["scores"][0][h, r], nv), f"prefill row {t} kv head {h}"
                flips += int(set(topk[h, r, :nv].tolist()) != set(parts["topk"][h, r, :nv].tolist()))
        # compressed rows the step wrote (windows ending inside the chunk)
        flat_k = self.kc.view(-1, self.kh, self.d)
        ref_rows = O.mean_pool(k, [0, self.L1])
        new = [j for j in range(self.ylen) if self.pslots_host[j] >= 0]
        got_rows = flat_k[torch.tensor([self.pslots_host[j] for j in new], device=self.dev)].float().cpu()
        assert (got_rows - ref_rows[new]).abs().max().item() <= 8e-3, "chunked prefill: pooled rows"
        return {"max_err": err, "rows": len(rows), "near_tie_rows": flips}


def inference_bench(dev, check_seqs=16, sweep=True):
    """BASELINE config 4: fused paged decode of 64 sequences and a chunked prefill of 2048 tokens on a 6144-token prefix.
    Both results are checked against the CPU oracle (un-paged sequences) BEFORE anything is timed: the decode on
    `check_seqs` of the 64 sequences (tests/test_gpu_inference.py checks all 64), the prefill on 64 sampled rows."""
    c4 = Config4(dev)
    o, tk = c4.decode(return_topk=True)
    chk_dec = c4.check_decode(o, tk, seqs=list(range(0, c4.B, max(1, c4.B // check_seqs))))
    assert torch.equal(o, c4.decode())          # the public entry point returns the same tensor (the step is idempotent)
    o_pre = c4.prefill()
    chk_pre = c4.check_prefill(o_pre)

    def timed(fn, n):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    ms_eager = timed(c4.decode, 20)
    graph = torch.cuda.CUDAGraph()
    c4.decode()
    torch.cuda.synchronize()
    with torch.cuda.graph(graph):
        c4.decode()
    ms_graph = timed(graph.replay, 50)
    # bytes a decode step must read: compressed K (twice: attention and scoring) + compressed V, 16 selected blocks and
    # 513 window rows of K and V, per sequence and kv head
    row = c4.kh * c4.d * 2
    alg_bytes = sum(3 * ((L - 32) // 16 + 1) * row + 2 * (16 * 64 + 513) * row for L in c4.ctx)
    ms_pre = timed(c4.prefill, 10)
    del graph
    pgraph = torch.cuda.CUDAGraph()      # the same launches without the host's launch overhead between them
    with torch.cuda.graph(pgraph):
        c4.prefill()
    ms_pre_graph = timed(pgraph.replay, 20)
    del pgraph
    peak_tf, peak_gbs, src = load_peaks()
    fm = flops_model([c4.L1], qh=c4.qh, d=c4.d, first=c4.P)
    pre_flop = sum(fm[n] for n in ("cmp_fwd", "topk", "slc_fwd", "swa_fwd"))
    # bytes the chunk must move at least once: its own q / o / gate rows and the sequence's K/V and compressed K/V
    pre_bytes = c4.Cn * c4.qh * (2 * c4.d + 3) * 2 + 2 * (c4.L1 + c4.ylen) * row
    n_dec, n_chunk = c4.B, c4.Cn
    del c4, o, tk, o_pre              # the sweep below fills its own 4 GiB cache
    torch.cuda.empty_cache()
    sweep = decode_sweep_4gib(dev) if sweep else None
    return {"workload": "decode batch 64, contexts U[4096,8192] (seed 1004), 32 q heads / 8 kv heads / d=128, page 256, shuffled "
                        "page table; chunked prefill 2048 new tokens on a 6144-token prefix",
            "checked_against_oracle": {"decode": chk_dec, "prefill": chk_pre, "tolerance": TOL},
            "decode_ms_eager": ms_eager, "decode_ms_cuda_graph": ms_graph, "decode_tokens_per_s": n_dec / (ms_graph * 1e-3),
            "decode_roofline": {"bound": "hbm", "achieved": alg_bytes / (ms_graph * 1e-3) / 1e9, "peak": peak_gbs, "unit": "GB/s",
                                "frac": alg_bytes / (ms_graph * 1e-3) / 1e9 / peak_gbs, "algorithmic_gb": alg_bytes / 1e9, "peak_source": src},
            "decode_algorithmic_gb": alg_bytes / 1e9, "decode_hbm_gbs": alg_bytes / (ms_graph * 1e-3) / 1e9,
            "decode_hbm_frac": alg_bytes / (ms_graph * 1e-3) / 1e9 / peak_gbs, "hbm_peak_gbs": peak_gbs, "peak_source": src,
            "prefill_chunk_ms": ms_pre, "prefill_tokens_per_s": n_chunk / (ms_pre * 1e-3), "prefill_chunk_ms_cuda_graph": ms_pre_graph,
            "prefill_roofline": {"algorithmic_tflop": pre_flop / 1e12, "tensor_tflops": pre_flop / (ms_pre * 1e-3) / 1e12,
                                 "tensor_frac": pre_flop / (ms_pre * 1e-3) / 1e12 / peak_tf, "algorithmic_gb": pre_bytes / 1e9,
                                 "hbm_frac": pre_bytes / (ms_pre * 1e-3) / 1e9 / peak_gbs,
                                 "bound": "latency / occupancy: 2048 query rows are a few hundred CTAs of short loops, far below both roofs",
                                 "launches": 9},
            "decode_sweep_4gib_64q_4kv": sweep}


def _or_none(fn):
    try:
        return fn()
    except Exception:  # noqa: BLE001  (a descriptive field of the line, never a reason to lose the line)
        return None


def decode_sweep_4gib(dev):
    """The reference's decode micro-benchmark (inference.ipynb cell 46, README.md:291-299): 64 q heads / 4 kv heads / d = 128,
    page 128, K and V caches of 4 GiB in all, batch = 4 GiB / per-sequence KV bytes, every sequence `seqlen` tokens long,
    one nsa_decode step replayed from a CUDA graph.  Cache contents are seeded N(0,1) (the timing does not depend on them;
    results are checked on config 4 and in the tests)."""
    from flash_nsa import nsa_decode
    qh, kh, d, page = 64, 4, 128, 128
    total_tokens = 1024 * 2048
    tok_pages = total_tokens // page
    cmp_pages = tok_pages // 16 + 512
    g = torch.Generator(device=dev).manual_seed(46)
    kc = torch.randn(tok_pages + cmp_pages, page, kh, d, device=dev, dtype=torch.bfloat16, generator=g)
    vc = torch.randn(tok_pages + cmp_pages, page, kh, d, device=dev, dtype=torch.bfloat16, generator=g)
    published = {4096: 0.689377, 8192: 0.420754, 16384: 0.279387, 32768: 0.205926, 65536: 0.172448, 131072: 0.159892}
    out = []
    row = kh * d * 2
    peak_gbs = load_peaks()[1]
    from flash_nsa.inference.ops import decode_cluster_size
    # the reference's six points (batch = 4 GiB / sequence), then few long sequences: the case a cluster per (sequence, kv
    # head) is for
    points = [(L, total_tokens // L) for L in (4096, 8192, 16384, 32768, 65536, 131072)] + [(32768, 1), (131072, 1), (131072, 4)]
    for L, B in points:
        perm = torch.randperm(tok_pages, generator=torch.Generator().manual_seed(L))[:B * (L // page)].to(torch.int32)
        bt = perm.view(B, L // page).to(dev)
        y = (L - 32) // 16 + 1
        per = -(-y // page)
        cperm = (torch.randperm(B * per, generator=torch.Generator().manual_seed(L + 1)) + tok_pages).to(torch.int32)
        cbt = cperm.view(B, per).to(dev)
        ctx = torch.full((B,), L, dtype=torch.int32, device=dev)
        slot = (cbt[:, (y - 1) // page].to(torch.int64) * page + (y - 1) % page).to(torch.int32)   # L is a multiple of 16: a row is completed
        q = torch.randn(B, qh, d, device=dev, dtype=torch.bfloat16, generator=g)
        w = torch.randn(B, qh, 3, device=dev, dtype=torch.bfloat16, generator=g)
        fn = lambda: nsa_decode(q, kc, vc, w, ctx, bt, slot, cbt)
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(30):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / 30
        alg = B * (3 * y * row + 2 * (16 * 64 + 513) * row)
        out.append({"seqlen": L, "batch": B, "ms_cuda_graph": ms, "tokens_per_s": B / (ms * 1e-3), "hbm_frac": alg / (ms * 1e-3) / 1e9 / peak_gbs,
                    "ctas_per_seq_and_kv_head": _or_none(lambda: decode_cluster_size(B, kh, page, bt.stride(0))),
                    "reference_h800_ms_cuda_graph": published[L] if B == total_tokens // L else None})
    return out


def kernel_breakdown(q, k, v, w, do, lens):
    """CUDA-event time (ms) of every kernel family of one forward+backward, each timed alone on the launch stream."""
    from flash_nsa import NSAHelper
    from flash_nsa.ops import (mean_pooling_fwd, mean_pooling_bwd, cmp_attn_fwd, slc_topk_indices, slc_attn_fwd, swa_fwd,
                               combine_fwd, combine_bwd, get_bind_from_find)
    from flash_nsa.ops._common import attn_params, call, ptr, is_cp
    from flash_nsa.ops.select_attn import attach_k2q
    H = NSAHelper
    sm = D ** -0.5
    with torch.no_grad():
        qd, kd, vd, wd = q.detach(), k.detach(), v.detach(), w.detach()
        ck, cv = mean_pooling_fwd(kd), mean_pooling_fwd(vd)
        cmp_o, cmp_lse = cmp_attn_fwd(qd, ck, cv)
        topk, _ = slc_topk_indices(qd, ck, cmp_lse, maybe_efficient_version=True)
        slc_o, slc_lse = slc_attn_fwd(qd, kd, vd, topk)
        swa_o, swa_lse = swa_fwd(qd, kd, vd)
        from flash_nsa.ops.topk import backward_index_sizes
        rr, ir = backward_index_sizes(qd.size(1) // kd.size(1), qd.size(2), qd.size(0), NSAHelper.k_maxlen, topk.size(-1))
        index = get_bind_from_find(topk, range_rows=rr, item_rows=ir)
        dq = torch.empty_like(qd)
        dkf, dvf = torch.zeros(kd.shape, device=kd.device), torch.zeros(vd.shape, device=vd.device)
        dck, dcv = torch.zeros(ck.shape, device=kd.device), torch.zeros(cv.shape, device=kd.device)

        # the combine backward writes the three branches' delta rows as well (the step's branch backwards use them)
        deltas = [torch.empty_like(cmp_lse).t(), torch.empty_like(slc_lse), torch.empty_like(swa_lse)]

        def bwd_call(fn, kk, vv, o, lse, head_major, dk_, dv_, phase, topk_=None):
            delta = torch.empty_like(lse)
            p = attn_params(qd, kk, vv, H, sm, o=o, lse=lse, lse_is_head_major=head_major, dout=do, delta=delta, dq=dq, dk=dk_, dv=dv_,
                            topk=topk_)
            if topk_ is not None:
                attach_k2q(p, index, H)
            call(fn, p, qd)          # delta (and everything else) once, so that the timed phase has valid inputs
            p.phases = phase
            p.accumulate_dq = int(fn != "nsa_swa_bwd")   # as in the step: the window branch writes dq, the others add
            return lambda: call(fn, p, qd)

        fns = {
            "pool_fwd": lambda: mean_pooling_fwd(kd),
            "cmp_fwd": lambda: cmp_attn_fwd(qd, ck, cv),
            "topk": lambda: slc_topk_indices(qd, ck, cmp_lse, maybe_efficient_version=True),
            "slc_fwd": lambda: slc_attn_fwd(qd, kd, vd, topk),
            "swa_fwd": lambda: swa_fwd(qd, kd, vd),
            "combine_fwd": lambda: combine_fwd(cmp_o, slc_o, swa_o, wd),
            "combine_bwd": lambda: combine_bwd(cmp_o, slc_o, swa_o, wd, do, deltas=deltas),
            "k2q_index": lambda: get_bind_from_find(topk, range_rows=rr, item_rows=ir),
            "cmp_dkdv": bwd_call("nsa_cmp_attn_bwd", ck, cv, cmp_o, cmp_lse, True, dck, dcv, 2),
            "cmp_dq": bwd_call("nsa_cmp_attn_bwd", ck, cv, cmp_o, cmp_lse, True, dck, dcv, 4),
            # dK/dV and dQ asked for together run as ONE block-major kernel (dS K added into dq by global reductions)
            "slc_bwd": bwd_call("nsa_slc_attn_bwd", kd, vd, slc_o, slc_lse, False, dkf, dvf, 6, topk),
            "swa_dkdv": bwd_call("nsa_swa_bwd", kd, vd, swa_o, swa_lse, False, dkf, dvf, 2),
            "swa_dq": bwd_call("nsa_swa_bwd", kd, vd, swa_o, swa_lse, False, dkf, dvf, 4),
            "pool_bwd": lambda: mean_pooling_bwd(kd, dck.bfloat16(), dkf),
        }
        out = {}
        for name, fn in fns.items():
            fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(3):
                fn()
            e1.record()
            torch.cuda.synchronize()
            out[name] = e0.elapsed_time(e1) / 3
    return out


if __name__ == "__main__":
    main()
