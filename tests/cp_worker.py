"""Worker of tests/test_gpu_cp_multi.py: run with torchrun, one process per GPU.  Every rank builds the same global
batches, runs the unsharded NSACore as the reference, then the context-parallel NSACore on its shard over NCCL, and compares
(the check that `bench.py` runs before it times anything at N > 1)."""
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
    from bench import cp_check
    res = cp_check(dist.group.WORLD, rank, world)
    if rank == 0:
        print(res, flush=True)
        print("CP_OK" if res["ok"] else "CP_FAIL", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if res["ok"] else 1)


if __name__ == "__main__":
    main()
