"""Benchmark of the NSA hot path: forward + backward of one NSA layer (NSACore) on packed bf16 inputs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

N = 1 : BASELINE config 1 -- one causal sequence of 65 536 tokens, 64 q heads / 4 kv heads / d = 128.
N > 1 : (launched with torchrun) BASELINE config 3 -- one causal sequence of N * 131 072 tokens, sharded
        with the zig-zag layout (cp_mode = 2), K/V all-gathered per kv head over NCCL; weak scaling.
--impl reference : the reference's CPU path (its torch restatement in oracle/) timed on the host cores on a
        bounded sample of the same workload.

Prints ONE JSON line (rank 0).  Inputs are seeded N(0,1) synthetic tensors, as in the reference's own
benchmarks; there is no dataset on this path.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "scalable-flash-native-sparse-attention_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

import numpy as np
import torch

QH, KH, D = 64, 4, 128
H800_TOKENS_PER_S = 65536 / 0.10785   # the reference's published fwd+bwd at 64K on one H800 (34.162 + 73.689 ms)


# ----------------------------------------------------------------------------------------------- work model
def pair_counts(lens, ks=32, st=16, bs=64, top_n=16, window=512):
    """(query, key) pairs per q head of each branch, causal-exact."""
    cmp_p = slc_p = swa_p = 0
    for L in lens:
        t = np.arange(L, dtype=np.int64)
        Y = max((L - ks) // st + 1, 0)
        cmp_p += int(np.where(t >= ks - 1, np.minimum((t - (ks - 1)) // st + 1, Y), 0).sum())
        nk = t // bs
        slc_p += int(((np.minimum(top_n, nk + 1) - 1) * bs + (t % bs) + 1).sum())
        swa_p += int(np.minimum(t + 1, window + 1).sum())
    return cmp_p, slc_p, swa_p


def flops_model(lens, qh=QH, d=D):
    c, s, w = pair_counts(lens)
    f = lambda pairs, mm: 2.0 * d * mm * pairs * qh
    return {
        "cmp_fwd": f(c, 2), "topk": f(c, 1), "slc_fwd": f(s, 2), "swa_fwd": f(w, 2),
        "cmp_bwd": f(c, 5), "slc_bwd": f(s, 5), "swa_bwd": f(w, 5),
        # what the two backward kernels of a branch execute (S and dP are recomputed in both)
        "cmp_dkdv": f(c, 4), "cmp_dq": f(c, 3), "slc_dkdv": f(s, 4), "slc_dq": f(s, 3), "swa_dkdv": f(w, 4), "swa_dq": f(w, 3),
    }


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d.get("bf16_tflops", 1590.0), d.get("hbm_gbs", 6650.0), "measured"
    return 1590.0, 6650.0, "fallback"


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
def cpu_reference(steps, warmup, threads=None):
    """The reference's torch path (oracle restatement) on the host: forward + backward, fp32, on a bounded sample
    of the workload: the benchmark's head configuration (64 q heads / 4 kv heads / d = 128) on one causal sequence
    of 2048 tokens, because that code needs O(heads * T^2) memory and cannot hold 65 536 tokens.  Per-token cost
    grows with the sequence length, so the full-length CPU figure would be lower still."""
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
            "ms_per_step": dt * 1e3}


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
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        if rank != 0:
            return
        r = cpu_reference(max(1, min(args.steps, 10)), max(1, min(args.warmup, 2)))
        line = {"impl": "reference", "metric": "nsa_fwd_bwd_throughput", "value": r["value"], "unit": "tokens/s", "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": r["sample"]},
                "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
                "e2e": {"value": r["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    import flash_nsa
    from flash_nsa import NSAHelper, _lib
    import torch.distributed as dist
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    pg = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        pg = dist.group.WORLD
    per_gpu = args.tokens_per_gpu or (65536 if world == 1 else 131072)
    T_total = per_gpu * world
    cfg = flash_nsa.NSAConfig(head_dim=D, num_heads=QH, num_kv_heads=KH, cp_mode=2, kv_head_stride=1,
                              recompute_cmp_kv=world > 1, recompute_cmp_o=world > 1, recompute_slc_o=world > 1,
                              recompute_swa_o=world > 1)
    core = flash_nsa.NSACore(cfg, process_group=pg)
    cu_host = np.array([0, T_total], dtype=np.int64)
    cu = torch.tensor(cu_host, dtype=torch.int32, device=dev)

    gen = torch.Generator().manual_seed(1001 + rank)
    host = {name: torch.randn(per_gpu, h, dd, generator=gen).bfloat16().pin_memory()
            for name, h, dd in (("q", QH, D), ("k", KH, D), ("v", KH, D), ("w", QH, 3), ("do", QH, D))}
    q, k, v, w, do = [host[n].to(dev, non_blocking=True) for n in ("q", "k", "v", "w", "do")]
    for t in (q, k, v, w):
        t.requires_grad_(True)

    def step():
        o = core(q, k, v, w, cu, cu_seqlens_np=cu_host, cp_mode=2)
        o.backward(do)
        grads = (q.grad, k.grad, v.grad, w.grad)
        q.grad = k.grad = v.grad = w.grad = None
        return o, grads

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    sync_all()
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
    ms = e0.elapsed_time(e1) / args.steps
    if world > 1:
        tt = torch.tensor([ms], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms = tt.item()
    clocks = sampler.stop(t_wall0, t_wall1) if sampler else None

    # ---- end to end: pinned host inputs -> device, the step, results -> pinned host
    out_host = {n: torch.empty_like(host[n]) for n in ("q", "k", "v", "w")}
    o_host = torch.empty(per_gpu, QH, D, dtype=torch.bfloat16).pin_memory()
    for n in out_host:
        out_host[n] = out_host[n].pin_memory()

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

    n_e2e = 0 if args.no_e2e else max(16, min(args.steps, 32))   # enough steps to amortise the un-hidden first copy-in / last copy-out
    if n_e2e:
        e2e_loop(2)
    sync_all()
    e0.record()
    if n_e2e:
        e2e_loop(n_e2e)
    e1.record()
    sync_all()
    ms_e2e = e0.elapsed_time(e1) / max(n_e2e, 1) if n_e2e else float("nan")
    if world > 1:
        tt = torch.tensor([ms_e2e], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms_e2e = tt.item()
    h2d = sum(host[n].numel() * 2 for n in host)
    d2h = o_host.numel() * 2 + sum(out_host[n].numel() * 2 for n in out_host)

    # ---- per-kernel timing of the dominant kernels (single GPU only), for the roofline object
    roofline, kernels = None, None
    peak_tf, peak_gbs, peak_src = load_peaks()
    if world == 1 and rank == 0 and not args.no_kernel_breakdown:
        kernels = kernel_breakdown(q, k, v, w, do, [T_total])
        fm = flops_model([T_total])
        top = max((n for n in kernels if n in fm), key=lambda n: kernels[n])
        ach = fm[top] / (kernels[top] * 1e-3) / 1e12
        # DRAM bytes per launch of the kernels that can be the slowest one, from ncu captures at 32K tokens (profiles/),
        # scaled by tokens where the kernel's traffic is linear in tokens (the selected branch); None = not captured
        ncu_traffic_32k = {"slc_bwd": 18.71e9 + 6.28e9, "slc_fwd": 0.6e6 + 508.0e6}
        traffic = ncu_traffic_32k[top] * (T_total / 32768) if top in ncu_traffic_32k else None
        roofline = {"kernel": top, "bound": "tensor", "achieved": ach, "peak": peak_tf, "unit": "TFLOP/s", "frac": ach / peak_tf,
                    "traffic": traffic, "traffic_source": "ncu dram__bytes_read+write at 32K tokens x tokens/32768" if traffic else None,
                    "peak_source": peak_src, "ms": kernels[top]}
        if traffic:   # how close the same launch is to the HBM roof, from the measured DRAM traffic (not algorithmic bytes)
            roofline["dram_gbs_from_traffic"] = traffic / (kernels[top] * 1e-3) / 1e9
            roofline["dram_frac_from_traffic"] = roofline["dram_gbs_from_traffic"] / peak_gbs

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    value = T_total / (ms * 1e-3)
    fm_total = flops_model([T_total])
    alg = sum(fm_total[n] for n in ("cmp_fwd", "topk", "slc_fwd", "swa_fwd", "cmp_bwd", "slc_bwd", "swa_bwd"))
    cpu = cpu_reference(3, 1) if (world == 1 and not args.no_cpu_baseline) else None
    line = {
        "metric": "nsa_fwd_bwd_throughput", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": value / H800_TOKENS_PER_S if world == 1 else None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": (f"NSA fwd+bwd, one causal sequence of {T_total} tokens, {QH} q heads / {KH} kv heads / d={D}, "
                                f"kernel 32 stride 16 block 64 top-n 16 window 512" + ("" if world == 1 else
                                f", context parallel over {world} GPUs (zig-zag shards, {per_gpu} tokens per GPU)")),
                   "tokens": T_total, "l2": "inputs (q alone >= 1 GiB) exceed the 126 MB L2; no explicit flush",
                   "algorithmic_tflop_per_step": alg / 1e12},
        "achieved_tflops": alg / (ms * 1e-3) / 1e12 / world,
        "clocks": clocks, "gpu_launches": launches,
        "e2e": {"value": T_total / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": ms_e2e, "steps": n_e2e,
                "pipeline": "2 input sets, copy-in / compute / copy-out streams; first copy-in and last copy-out are inside the timed region"},
    }
    if roofline:
        line["roofline"] = roofline
        line["kernels_ms"] = kernels
    if world == 1 and not args.no_inference:
        line["inference"] = inference_bench(dev)
    if cpu:
        line["cpu_baseline"] = {k_: cpu[k_] for k_ in ("value", "unit", "cores", "kind", "sample")}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def inference_bench(dev):
    """BASELINE config 4: paged decode (batch 64, contexts U[4096,8192]) and a chunked prefill of 2048 new tokens on a
    6144-token prefix; 32 q heads / 8 kv heads / d = 128, page 256, shuffled page table, seeded N(0,1) cache contents."""
    import random
    from flash_nsa import nsa_decode, nsa_prefill
    qh, kh, d, page = 32, 8, 128, 256
    rng = random.Random(1004)
    B = 64
    ctx = [rng.randint(4096, 8192) for _ in range(B)]
    n_tok = [-(-L // page) for L in ctx]
    n_cmp = [-(-max((L - 32) // 16 + 1, 1) // page) for L in ctx]
    P, Cn = 6144, 2048                     # the chunked-prefill sequence gets page lists of its own
    L1 = P + Cn
    pre_tok, pre_cmp = -(-L1 // page), -(-((L1 - 32) // 16 + 1) // page)
    total = sum(n_tok) + sum(n_cmp) + pre_tok + pre_cmp
    free = list(range(total))
    rng.shuffle(free)
    g = torch.Generator(device=dev).manual_seed(1004)
    kc = torch.randn(total, page, kh, d, device=dev, dtype=torch.bfloat16, generator=g)
    vc = torch.randn(total, page, kh, d, device=dev, dtype=torch.bfloat16, generator=g)
    bt = torch.full((B, max(n_tok)), -1, dtype=torch.int32)
    cbt = torch.full((B, max(n_cmp)), -1, dtype=torch.int32)
    for b in range(B):
        for i in range(n_tok[b]):
            bt[b, i] = free.pop()
        for i in range(n_cmp[b]):
            cbt[b, i] = free.pop()
    slot = torch.tensor([(int(cbt[b, ((L - 32) // 16) // page]) * page + ((L - 32) // 16) % page) if L % 16 == 0 else -1
                         for b, L in enumerate(ctx)], dtype=torch.int32, device=dev)
    pbt = torch.tensor([[free.pop() for _ in range(pre_tok)]], dtype=torch.int32, device=dev)
    pcbt = torch.tensor([[free.pop() for _ in range(pre_cmp)]], dtype=torch.int32, device=dev)
    assert not free
    bt, cbt = bt.to(dev), cbt.to(dev)
    ctx_d = torch.tensor(ctx, dtype=torch.int32, device=dev)
    q = torch.randn(B, qh, d, device=dev, dtype=torch.bfloat16, generator=g)
    w = torch.randn(B, qh, 3, device=dev, dtype=torch.bfloat16, generator=g)

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

    dec = lambda: nsa_decode(q, kc, vc, w, ctx_d, bt, slot, cbt)
    ms_eager = timed(dec, 20)
    graph = torch.cuda.CUDAGraph()
    dec()
    torch.cuda.synchronize()
    with torch.cuda.graph(graph):
        out = dec()
    ms_graph = timed(graph.replay, 50)
    # bytes a decode step must read: compressed K (twice: attention and scoring) + compressed V, 16 selected blocks and
    # 513 window rows of K and V, per sequence and kv head
    row = kh * d * 2
    alg_bytes = sum(3 * ((L - 32) // 16 + 1) * row + 2 * (16 * 64 + 513) * row for L in ctx)
    # chunked prefill: one sequence, 2048 new tokens after 6144 cached ones
    L = L1
    xcu = torch.tensor([0, Cn], dtype=torch.int32, device=dev)
    ylen = (L - 32) // 16 + 1
    ycu = torch.tensor([0, ylen], dtype=torch.int32, device=dev)
    pc_host = pcbt[0].tolist()
    slots = torch.tensor([(pc_host[j // page] * page + j % page) if 16 * j + 31 >= P else -1 for j in range(ylen)],
                         dtype=torch.int32, device=dev)
    qp = torch.randn(Cn, qh, d, device=dev, dtype=torch.bfloat16, generator=g)
    wp = torch.randn(Cn, qh, 3, device=dev, dtype=torch.bfloat16, generator=g)
    ctx1 = torch.tensor([L], dtype=torch.int32, device=dev)
    ms_pre = timed(lambda: nsa_prefill(qp, kc, vc, wp, xcu, ycu, Cn, ylen, ctx1, pbt, slots, pcbt), 10)
    peak_tf, peak_gbs, src = load_peaks()
    return {"workload": "decode batch 64, contexts U[4096,8192] (seed 1004), 32 q heads / 8 kv heads / d=128, page 256, shuffled "
                        "page table; chunked prefill 2048 new tokens on a 6144-token prefix",
            "decode_ms_eager": ms_eager, "decode_ms_cuda_graph": ms_graph, "decode_tokens_per_s": B / (ms_graph * 1e-3),
            "decode_algorithmic_gb": alg_bytes / 1e9, "decode_hbm_gbs": alg_bytes / (ms_graph * 1e-3) / 1e9,
            "decode_hbm_frac": alg_bytes / (ms_graph * 1e-3) / 1e9 / peak_gbs, "hbm_peak_gbs": peak_gbs, "peak_source": src,
            "prefill_chunk_ms": ms_pre, "prefill_tokens_per_s": Cn / (ms_pre * 1e-3)}


def kernel_breakdown(q, k, v, w, do, lens):
    """CUDA-event time (ms) of every kernel family of one forward+backward, each timed alone on the launch stream."""
    from flash_nsa import NSAHelper
    from flash_nsa.ops import (mean_pooling_fwd, mean_pooling_bwd, cmp_attn_fwd, slc_topk_indices, slc_attn_fwd, swa_fwd,
                               combine_fwd, combine_bwd, get_bind_from_find)
    from flash_nsa.ops._common import attn_params, call, ptr, is_cp
    H = NSAHelper
    sm = D ** -0.5
    with torch.no_grad():
        qd, kd, vd, wd = q.detach(), k.detach(), v.detach(), w.detach()
        ck, cv = mean_pooling_fwd(kd), mean_pooling_fwd(vd)
        cmp_o, cmp_lse = cmp_attn_fwd(qd, ck, cv)
        topk, _ = slc_topk_indices(qd, ck, cmp_lse, maybe_efficient_version=True)
        slc_o, slc_lse = slc_attn_fwd(qd, kd, vd, topk)
        swa_o, swa_lse = swa_fwd(qd, kd, vd)
        offsets, tokens = get_bind_from_find(topk)
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
                p.k2q_offsets, p.k2q_tokens, p.k2q_stride_h = ptr(offsets), ptr(tokens), tokens.stride(0)
                p.k2q_blk_cu, p.n_blocks_total = ptr(H.k_cu_seqlens), offsets.size(1) - 1
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
            "k2q_index": lambda: get_bind_from_find(topk),
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
