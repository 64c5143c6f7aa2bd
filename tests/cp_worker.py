"""Worker of tests/test_gpu_cp_multi.py: run with torchrun, one process per GPU.  Every rank builds the same global
batch, runs the unsharded NSACore as the reference, then the context-parallel NSACore on its shard, and compares."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "scalable-flash-native-sparse-attention_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch
import torch.distributed as dist


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    import flash_nsa
    from flash_nsa import NSAHelper
    from oracle import nsa_oracle as O
    QH, KH, D = 16, 2, 128
    ok = True
    for mode, lens, stride in ((2, [2048], 1), (1, [512, 1024, 512], 2), (2, [1536, 512], 1)):
        g = torch.Generator().manual_seed(100 + mode + len(lens))
        T = sum(lens)
        cu = [0]
        for L in lens:
            cu.append(cu[-1] + L)
        mk = lambda *s: torch.randn(*s, generator=g).bfloat16().cuda()
        q, k, v, w, do = mk(T, QH, D), mk(T, KH, D), mk(T, KH, D), mk(T, QH, 3), mk(T, QH, D)
        cu_d = torch.tensor(cu, dtype=torch.int32, device="cuda")

        NSAHelper.reset_context_parallel()
        cfg = flash_nsa.NSAConfig(head_dim=D, num_heads=QH, num_kv_heads=KH, cp_mode=mode, kv_head_stride=stride)
        ref_core = flash_nsa.NSACore(cfg)
        leaves = [t.clone().requires_grad_(True) for t in (q, k, v, w)]
        o_ref = ref_core(*leaves, cu_d)
        o_ref.backward(do)
        ref = [o_ref] + [t.grad for t in leaves]

        core = flash_nsa.NSACore(cfg, process_group=dist.group.WORLD)
        meta = O.cp_metadata(cu, rank, world, mode)
        rows = torch.cat([torch.arange(b, e) for b, e in meta["ranges"]]).cuda()
        loc = [t[rows].clone().requires_grad_(True) for t in (q, k, v, w)]
        o = core(*loc, cu_d, cp_mode=mode)
        o.backward(do[rows])
        got = [o] + [t.grad for t in loc]
        for name, a, b in zip(("o", "dq", "dk", "dv", "dw"), got, ref):
            b = b[rows]
            err = (a.float() - b.float()).abs().max().item()
            bound = 3e-2 * max(1.0, b.float().abs().max().item())
            if not (err <= bound):
                ok = False
                print(f"rank {rank} mode {mode} lens {lens}: {name} err {err:.4g} > {bound:.4g}", flush=True)
        NSAHelper.reset_context_parallel()
    from flash_nsa.ops._common import check_status
    check_status()
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("CP_OK" if flag.item() == 1 else "CP_FAIL", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 1 else 1)


if __name__ == "__main__":
    main()
